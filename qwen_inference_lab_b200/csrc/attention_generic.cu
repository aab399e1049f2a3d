// Causal grouped-query attention over the paged cache for any head size, page
// size and dtype, on the CUDA cores with float32 arithmetic throughout.
//
// This is the attention of the true 32-bit path, and the one that serves head
// sizes or dtypes the tensor-core kernels do not take.  One block computes one
// (token, query head): scores against the keys of its request from the window's
// start to the token's own position (absolute positions, so a chunk that
// continues a cached prefix is masked correctly; qil/model.py:62-64), softmax
// and the weighted sum of values (qil/model.py:65-68, scale head_dim^-1/2;
// query head h reads kv head h / (Hq/Hkv), qil/paged_attention.py:21).
//
// Keys are walked in tiles of 128 aligned to absolute positions and summed in
// ascending order, so a token's result depends only on its own query and the
// cache contents: not on how the batch was cut or what else is in it.
//
// Two options serve other designs than the reference's.  Values may have another
// size than queries and keys (`v_dim`): a page then holds its key rows
// [kv_head][slot][head_dim] followed by its value rows [kv_head][slot][v_dim],
// which for equal sizes is the layout [2][kv_head][slot][head_dim].  And a bias
// that grows with distance may be taken off the scaled score (`slopes`, one per
// query head): score = q.k * scale - slope_h * (i - j) for the query at position i
// and the key at position j.  With `shared_rows` a page holds its key rows only, and
// a position's value is the first `v_dim` columns of its key.
//
// Further options of the score, all in float32 (`ScoreOptions`):
//   softcap     score <- cap * tanh(score / cap), applied to the scaled product before any bias
//   dist_bias   a learned bias per (query head, distance i - j): float32 [Hq][dist_len], distances beyond the
//               table read its last entry (the caller expands buckets of distances into this table)
//   chunk       position i sees only the j <= i with floor(i / chunk) = floor(j / chunk), chunks counted
//               from position 0 of the sequence
//   sink        one is added to the softmax's denominator: a key of score 0 that has no value; with
//               sink_logits (float32 [Hq]) the added term is exp(sink_logits[h]) instead: a learned score per head
//               that is not scaled and counts once
#include "common.cuh"

struct ScoreOptions {
    float softcap;            // 0: none
    const float* dist_bias;   // null: none
    int dist_len;
    int chunk;                // 0: none
    int sink;                 // 0 or 1
    const float* sink_logits; // null: the sink's score is 0
};

#define GEN_TILE 128
#define GEN_MAX_D 512
#define GEN_DPT (GEN_MAX_D / GEN_TILE)

template <typename T>
__global__ void __launch_bounds__(GEN_TILE)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ kv_cache, T* __restrict__ out,
                         const int* __restrict__ positions, const int* __restrict__ token_row,
                         const int* __restrict__ block_table, int table_stride,
                         int n_q_heads, int n_kv_heads, int head_dim, int v_dim, int page_size, int num_pages,
                         int window, float scale, const float* __restrict__ slopes, ScoreOptions opt, int shared_rows) {
    extern __shared__ long long smem_ll[];
    long long* row_off = smem_ll;                      // [GEN_TILE] element offset of each key row, -1 if none
    long long* val_off = row_off + GEN_TILE;           // [GEN_TILE] element offset of each value row
    float* ks = reinterpret_cast<float*>(val_off + GEN_TILE);  // [GEN_TILE][33]
    float* ps = ks + GEN_TILE * 33;                    // [GEN_TILE]
    float* red = ps + GEN_TILE;                        // [32]
    float* qs = red + 32;                              // [head_dim]

    const int tid = threadIdx.x;
    const int token = blockIdx.x, head = blockIdx.y;
    const int kv_head = head / (n_q_heads / n_kv_heads);
    const int pos = positions[token];
    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (opt.chunk > 0 && pos >= 0) lo = max(lo, pos / opt.chunk * opt.chunk);
    const int* table = block_table + (size_t)token_row[token] * table_stride;
    const float* bias_row = opt.dist_bias != nullptr ? opt.dist_bias + (size_t)head * opt.dist_len : nullptr;

    const float slope = slopes != nullptr ? slopes[head] : 0.f;
    const T* qrow = q + ((size_t)token * n_q_heads + head) * head_dim;
    for (int d = tid; d < head_dim; d += GEN_TILE) qs[d] = to_f32<T>(qrow[d]);

    // the sink is a key of score 0 and weight exp(0 - max) that adds nothing to the sum of values
    float m_run = opt.sink ? (opt.sink_logits != nullptr ? opt.sink_logits[head] : 0.f) : -INFINITY, l_run = opt.sink ? 1.f : 0.f;
    float acc[GEN_DPT];
#pragma unroll
    for (int i = 0; i < GEN_DPT; ++i) acc[i] = 0.f;

    const long long page_elems = (long long)n_kv_heads * page_size * (shared_rows ? head_dim : head_dim + v_dim);
    const long long k_plane = (long long)n_kv_heads * page_size * head_dim;   // a page's key rows come first
    for (int tile = lo / GEN_TILE; tile * GEN_TILE <= pos; ++tile) {
        const int key = tile * GEN_TILE + tid;
        const bool valid = key >= lo && key <= pos;
        long long off = -1, voff = -1;
        if (valid) {
            const int page = key / page_size < table_stride ? table[key / page_size] : -1;
            if (page >= 0 && page < num_pages) {
                const long long row = (long long)kv_head * page_size + (key % page_size);
                off = page * page_elems + row * head_dim;
                voff = shared_rows ? off : page * page_elems + k_plane + row * v_dim;
            }
        }
        __syncthreads();  // previous tile's readers of row_off / ps are done
        row_off[tid] = off;
        val_off[tid] = voff;
        __syncthreads();

        float dot = 0.f;
        for (int d0 = 0; d0 < head_dim; d0 += 32) {
            const int chunk = head_dim - d0 < 32 ? head_dim - d0 : 32;
            for (int idx = tid; idx < GEN_TILE * 32; idx += GEN_TILE) {
                const int kk = idx >> 5, dd = idx & 31;
                const long long ro = row_off[kk];
                ks[kk * 33 + dd] = (ro >= 0 && dd < chunk) ? to_f32<T>(kv_cache[ro + d0 + dd]) : 0.f;
            }
            __syncthreads();
            for (int dd = 0; dd < chunk; ++dd) dot = fmaf(qs[d0 + dd], ks[tid * 33 + dd], dot);
            __syncthreads();
        }
        float score = -INFINITY;
        if (valid && off >= 0) {
            score = dot * scale;
            if (opt.softcap > 0.f) score = opt.softcap * tanhf(score / opt.softcap);
            score -= slope * (float)(pos - key);
            if (bias_row != nullptr) score += bias_row[min(pos - key, opt.dist_len - 1)];
        }
        const float tile_max = block_max(score, red);
        const float m_new = fmaxf(m_run, tile_max);
        const float p = (score == -INFINITY) ? 0.f : expf(score - m_new);
        const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        ps[tid] = p;
        const float tile_sum = block_sum(p, red);   // has __syncthreads inside: ps is visible after it
        l_run = l_run * corr + tile_sum;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < GEN_DPT; ++i) {
            const int d = tid + i * GEN_TILE;
            if (d < v_dim) {
                float a = acc[i] * corr;
                for (int kk = 0; kk < GEN_TILE; ++kk) {
                    const long long vo = val_off[kk];
                    if (vo >= 0) a = fmaf(ps[kk], to_f32<T>(kv_cache[vo + d]), a);
                }
                acc[i] = a;
            }
        }
    }
    T* orow = out + ((size_t)token * n_q_heads + head) * v_dim;
#pragma unroll
    for (int i = 0; i < GEN_DPT; ++i) {
        const int d = tid + i * GEN_TILE;
        if (d < v_dim) orow[d] = from_f32<T>(l_run > 0.f ? acc[i] / l_run : 0.f);
    }
}

extern "C" int qil_attention_generic(
    const void* q, const void* kv_cache, void* out, const int* positions, const int* token_row,
    const int* block_table, int table_stride, int n_tokens, int n_q_heads, int n_kv_heads,
    int head_dim, int v_dim, int page_size, int num_pages, int window, float scale, const float* slopes,
    float softcap, const float* dist_bias, int dist_len, int chunk, int sink, const float* sink_logits, int shared_rows,
    int act_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > GEN_MAX_D || v_dim <= 0 || v_dim > GEN_MAX_D)
        QIL_REFUSE("attention_generic: head sizes %d and %d must lie in 1..%d", head_dim, v_dim, GEN_MAX_D);
    if (shared_rows && v_dim > head_dim) QIL_REFUSE("attention_generic: values of %d out of shared rows of %d", v_dim, head_dim);
    if (n_kv_heads <= 0 || n_q_heads <= 0 || n_q_heads % n_kv_heads)
        QIL_REFUSE("attention_generic: %d query heads do not divide into %d kv heads", n_q_heads, n_kv_heads);
    if (n_q_heads > 65535) QIL_REFUSE("attention_generic: too many heads (%d)", n_q_heads);
    if (page_size <= 0 || window < 0) QIL_REFUSE("attention_generic: page_size %d window %d", page_size, window);
    if (softcap < 0.f || chunk < 0 || (dist_bias != nullptr && dist_len < 1))
        QIL_REFUSE("attention_generic: softcap %g chunk %d distance table of %d", softcap, chunk, dist_len);
    ScoreOptions opt = {softcap, dist_bias, dist_len, chunk, (sink || sink_logits != nullptr) ? 1 : 0, sink_logits};
    dim3 grid(n_tokens, n_q_heads);
    const size_t smem = (size_t)(head_dim + GEN_TILE * 33 + GEN_TILE + 32) * sizeof(float)
                        + 2 * GEN_TILE * sizeof(long long);
    QIL_DISPATCH_1(act_dtype,
        (attention_generic_kernel<T><<<grid, GEN_TILE, smem, stream>>>(
            (const T*)q, (const T*)kv_cache, (T*)out, positions, token_row, block_table, table_stride,
            n_q_heads, n_kv_heads, head_dim, v_dim, page_size, num_pages, window, scale, slopes, opt, shared_rows)));
    QIL_CHECK_LAUNCH();
}
