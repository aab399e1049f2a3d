// Tails of q/k/v projections whose rotation is computed from frequencies, with float32 angles.
//
// The angle of pair i at position p is (float)p * freq[i] (freq: float32 [rot_dims / 2], given by the host, which
// owns the formula); cosine and sine are the accurate float32 functions.  The pair (u, v) becomes
// (u cos a - v sin a, v cos a + u sin a).  Two layouts of the rot_dims rotated dimensions of a vector:
//   layout 0 (halves)       dimension i pairs with dimension i + rot_dims / 2
//   layout 1 (interleaved)  dimension 2 i pairs with dimension 2 i + 1
// Dimensions from rot_dims on pass unchanged.
//
// qk_rotate_store: q [Hq * d], k [Hkv * d], v [Hkv * e] are column ranges of one row-major buffer (a stacked
// projection).  Optionally q and k are first divided by their root mean square over the WHOLE projection (all
// heads at once) and multiplied by a weight per element (float32 arithmetic), or (per_head) every head by its own
// root mean square over its d dimensions, with one weight of d that all heads share; then every head is rotated;
// queries go to q_out, keys and values into the request's page (a page holds its key rows
// [kv_head][slot][d] followed by its value rows [kv_head][slot][e]).
//
// latent_prepare: the tail of a latent attention's projection.  The projection holds per token the queries
// [H][d plain, r rotated] and one row [c latent, r rotated key part].  The latent is divided by its root mean
// square and multiplied by a weight (float32), the key part and every query's rotated part are rotated.  The
// page row of the token becomes the key [c normed latent, r rotated key part] and the value [c normed latent,
// zeros up to value_width] (value_width 0: the page holds key rows only, the value being the key's first c
// columns); the rotated query parts go to columns c .. c + r of every head's row of q_att
// [N][H][c + r] (the first c columns receive the query folded through the key expansion, by another kernel).
// Where the queries come through a latent of their own, the same block norms that latent too: qn_width columns of
// the projection from qn_col on, divided by their root mean square, times qn_w, to qn_out [N][qn_width].
#include "common.cuh"

// The token's angles, once a block: table[i] = cos(pos * freq[i]), table[half + i] = sin(pos * freq[i]), i < half.
// The caller puts a barrier between this and the first rotated_element.
__device__ __forceinline__ void angle_table(float* __restrict__ table, int rot_dims, int pos, const float* __restrict__ freq) {
    const int half = rot_dims >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * freq[i], &table[half + i], &table[i]);
}

__device__ __forceinline__ float rotated_element(const float* __restrict__ vec, int j, int rot_dims, int layout,
                                                 const float* __restrict__ table) {
    // vec: the vector's values in float32 (shared memory); returns element j after rotation
    if (j >= rot_dims) return vec[j];
    const int half = rot_dims >> 1;
    int i, first, second;
    if (layout == 0) { i = j < half ? j : j - half; first = i; second = i + half; }
    else { i = j >> 1; first = 2 * i; second = 2 * i + 1; }
    const float c = table[i], s = table[half + i];
    const float u = vec[first], v = vec[second];
    return j == first ? u * c - v * s : v * c + u * s;
}

// V = 16 / sizeof(T) elements after rotation, from element j0 of a head on, as one 16-byte store.
template <typename T>
__device__ __forceinline__ void store_rotated16(T* __restrict__ dst, const float* __restrict__ head_vals, int j0, int rot_dims,
                                                int layout, const float* __restrict__ table) {
    constexpr int V = 16 / (int)sizeof(T);
    uint4 packed;
    T* out = reinterpret_cast<T*>(&packed);
#pragma unroll
    for (int k = 0; k < V; ++k) out[k] = from_f32<T>(rotated_element(head_vals, j0 + k, rot_dims, layout, table));
    *reinterpret_cast<uint4*>(dst) = packed;
}

// `wide`: every row, column and head starts on a 16-byte boundary, so loads and stores move 16 bytes each.
template <typename T, typename W>
__global__ void __launch_bounds__(256)
qk_rotate_store_kernel(const T* __restrict__ proj, int ld, int q_col, int k_col, int v_col, T* __restrict__ q_out,
                       T* __restrict__ pages, const W* __restrict__ q_norm_w, const W* __restrict__ k_norm_w, float eps,
                       const float* __restrict__ freq, int rot_dims, int layout, const int* __restrict__ positions,
                       const int* __restrict__ token_row, const int* __restrict__ block_table, int table_stride,
                       int n_q_heads, int n_kv_heads, int d, int e, int page_size, int num_pages, int wide, int per_head) {
    constexpr int V = 16 / (int)sizeof(T);
    extern __shared__ __align__(16) float vals[];   // [Hq * d + Hkv * d]: q then k, normed, float32;  then [rot_dims]: the angles
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const int token = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[token];
    const int q_width = n_q_heads * d, k_width = n_kv_heads * d, v_width = n_kv_heads * e;
    const T* row = proj + (size_t)token * ld;
    const float* table = vals + q_width + k_width;
    angle_table(vals + q_width + k_width, rot_dims, pos, freq);
    float sq = 0.f, sk = 0.f;
    if (wide) {
        auto load = [&](int column, int width, float* dst, float& sum) {
            for (int c = tid; c < width / V; c += 256) {
                const uint4 raw = *reinterpret_cast<const uint4*>(row + column + c * V);
                const T* x = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int k = 0; k < V; ++k) { const float f = to_f32<T>(x[k]); dst[c * V + k] = f; sum = fmaf(f, f, sum); }
            }
        };
        load(q_col, q_width, vals, sq);
        load(k_col, k_width, vals + q_width, sk);
    } else {
        for (int i = tid; i < q_width; i += 256) { const float x = to_f32<T>(row[q_col + i]); vals[i] = x; sq = fmaf(x, x, sq); }
        for (int i = tid; i < k_width; i += 256) { const float x = to_f32<T>(row[k_col + i]); vals[q_width + i] = x; sk = fmaf(x, x, sk); }
    }
    if (q_norm_w != nullptr && per_head) {
        // a warp per head: the head's sum of squares by a fixed tree over the lanes, whatever else the step holds
        __syncthreads();
        const int lane = tid & 31, warp = tid >> 5;
        for (int head = warp; head < n_q_heads + n_kv_heads; head += 8) {
            float* v = vals + head * d;
            const W* w = head < n_q_heads ? q_norm_w : k_norm_w;
            float ss = 0.f;
            for (int j = lane; j < d; j += 32) ss = fmaf(v[j], v[j], ss);
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)d + eps);
            for (int j = lane; j < d; j += 32) v[j] = v[j] * r * to_f32<W>(w[j]);
        }
    } else if (q_norm_w != nullptr) {
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        const float rq = 1.0f / sqrtf(sq / (float)q_width + eps);
        const float rk = k_width > 0 ? 1.0f / sqrtf(sk / (float)k_width + eps) : 0.f;
        for (int i = tid; i < q_width; i += 256) vals[i] = vals[i] * rq * to_f32<W>(q_norm_w[i]);
        for (int i = tid; i < k_width; i += 256) vals[q_width + i] = vals[q_width + i] * rk * to_f32<W>(k_norm_w[i]);
    }
    __syncthreads();
    T* q_dst = q_out + (size_t)token * q_width;
    if (wide) {
        for (int c = tid; c < q_width / V; c += 256) {
            const int head = c * V / d, j = c * V - head * d;
            store_rotated16<T>(q_dst + c * V, vals + head * d, j, rot_dims, layout, table);
        }
    } else {
        for (int i = tid; i < q_width; i += 256) {
            const int head = i / d, j = i - head * d;
            q_dst[i] = from_f32<T>(rotated_element(vals + head * d, j, rot_dims, layout, table));
        }
    }
    if (n_kv_heads == 0) return;
    const int index = pos / page_size;
    const int page = (pos >= 0 && index < table_stride) ? block_table[(size_t)token_row[token] * table_stride + index] : -1;
    if (page < 0 || page >= num_pages) return;      // never write outside the pool
    const int slot = pos % page_size;
    T* page_base = pages + (size_t)page * n_kv_heads * page_size * (d + e);
    if (wide) {
        for (int c = tid; c < k_width / V; c += 256) {
            const int head = c * V / d, j = c * V - head * d;
            store_rotated16<T>(page_base + ((size_t)head * page_size + slot) * d + j, vals + q_width + head * d, j, rot_dims,
                               layout, table);
        }
        T* values = page_base + (size_t)n_kv_heads * page_size * d;
        for (int c = tid; c < v_width / V; c += 256) {
            const int head = c * V / e, j = c * V - head * e;
            *reinterpret_cast<uint4*>(values + ((size_t)head * page_size + slot) * e + j) =
                *reinterpret_cast<const uint4*>(row + v_col + c * V);
        }
        return;
    }
    for (int i = tid; i < k_width; i += 256) {
        const int head = i / d, j = i - head * d;
        page_base[((size_t)head * page_size + slot) * d + j] =
            from_f32<T>(rotated_element(vals + q_width + head * d, j, rot_dims, layout, table));
    }
    T* v_base = page_base + (size_t)n_kv_heads * page_size * d;
    for (int i = tid; i < v_width; i += 256) {
        const int head = i / e, j = i - head * e;
        v_base[((size_t)head * page_size + slot) * e + j] = row[v_col + i];
    }
}

extern "C" int qil_qk_rotate_store(const void* proj, int ld, int q_col, int k_col, int v_col, void* q_out, void* pages,
                                   const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps, const float* freq,
                                   int rot_dims, int layout, const int* positions, const int* token_row,
                                   const int* block_table, int table_stride, int n_tokens, int n_q_heads, int n_kv_heads,
                                   int d, int e, int page_size, int num_pages, int act_dtype, int per_head,
                                   cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_q_heads <= 0 || n_kv_heads < 0 || d <= 0 || e <= 0 || page_size <= 0)
        QIL_REFUSE("qk_rotate_store: heads %d/%d sizes %d/%d page %d", n_q_heads, n_kv_heads, d, e, page_size);
    if (rot_dims < 0 || rot_dims > d || (rot_dims & 1) || (rot_dims > 0 && freq == nullptr) || (layout != 0 && layout != 1))
        QIL_REFUSE("qk_rotate_store: %d rotated dimensions of %d, layout %d", rot_dims, d, layout);
    if ((q_norm_w == nullptr) != (k_norm_w == nullptr) && n_kv_heads > 0)
        QIL_REFUSE("qk_rotate_store: give both norm weights or neither");
    const size_t smem = ((size_t)(n_q_heads + n_kv_heads) * d + rot_dims) * sizeof(float);
    if (smem > 160 * 1024) QIL_REFUSE("qk_rotate_store: %d values of q and k per token are too many", (n_q_heads + n_kv_heads) * d);
    cudaError_t err = cudaSuccess;
    QIL_DISPATCH_2(act_dtype, norm_dtype, {
        constexpr int V = 16 / (int)sizeof(T);
        const int wide = (d % V == 0 && e % V == 0 && ld % V == 0 && q_col % V == 0 && k_col % V == 0 && v_col % V == 0 &&
                          (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)pages) & 15) == 0) ? 1 : 0;
        if (smem > 48 * 1024)
            err = cudaFuncSetAttribute(qk_rotate_store_kernel<T, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err == cudaSuccess)
            qil_launch_chained(qk_rotate_store_kernel<T, W>, dim3(n_tokens), dim3(256), smem, stream,
                               (const T*)proj, ld, q_col, k_col, v_col, (T*)q_out, (T*)pages, (const W*)q_norm_w,
                               (const W*)k_norm_w, eps, freq, rot_dims, layout, positions, token_row, block_table,
                               table_stride, n_q_heads, n_kv_heads, d, e, page_size, num_pages, wide, per_head);
    });
    if (err != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(err)); return (int)err; }
    QIL_CHECK_LAUNCH();
}

template <typename T, typename W>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const T* __restrict__ proj, int ld, int q_col, int kv_col, T* __restrict__ q_att, T* __restrict__ pages,
                      const W* __restrict__ norm_w, float eps, const float* __restrict__ freq, int rot_dims, int layout,
                      const int* __restrict__ positions, const int* __restrict__ token_row,
                      const int* __restrict__ block_table, int table_stride, int n_heads, int d, int r, int c,
                      int value_width, int page_size, int num_pages, int qn_col, int qn_width,
                      const W* __restrict__ qn_w, T* __restrict__ qn_out) {
    extern __shared__ float vals[];          // [c + r]: the latent row;  [H * r]: the queries' rotated parts;  [rot_dims]: the angles
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const int token = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[token];
    const T* row = proj + (size_t)token * ld;
    float* q_rot = vals + c + r;
    const float* table = q_rot + n_heads * r;
    angle_table(q_rot + n_heads * r, rot_dims, pos, freq);
    float ss = 0.f;
    for (int i = tid; i < c + r; i += 256) {
        const float x = to_f32<T>(row[kv_col + i]);
        vals[i] = x;
        if (i < c) ss = fmaf(x, x, ss);
    }
    for (int i = tid; i < n_heads * r; i += 256) {
        const int head = i / r, j = i - head * r;
        q_rot[i] = to_f32<T>(row[q_col + head * (d + r) + d + j]);
    }
    ss = block_sum(ss, scratch);              // has barriers inside: vals and q_rot are complete after it
    const float scale = 1.0f / sqrtf(ss / (float)c + eps);
    const int width = c + r;
    T* q_dst = q_att + (size_t)token * n_heads * width;
    for (int i = tid; i < n_heads * r; i += 256) {
        const int head = i / r, j = i - head * r;
        q_dst[head * width + c + j] = from_f32<T>(rotated_element(q_rot + head * r, j, rot_dims, layout, table));
    }
    if (qn_out != nullptr) {                   // the queries' own latent, normed (every thread of the block gets here)
        float sq = 0.f;
        for (int i = tid; i < qn_width; i += 256) { const float x = to_f32<T>(row[qn_col + i]); sq = fmaf(x, x, sq); }
        sq = block_sum(sq, scratch);
        const float q_scale = 1.0f / sqrtf(sq / (float)qn_width + eps);
        T* dst = qn_out + (size_t)token * qn_width;
        for (int i = tid; i < qn_width; i += 256) dst[i] = from_f32<T>(to_f32<T>(row[qn_col + i]) * q_scale * to_f32<W>(qn_w[i]));
    }
    const int index = pos / page_size;
    const int page = (pos >= 0 && index < table_stride) ? block_table[(size_t)token_row[token] * table_stride + index] : -1;
    if (page < 0 || page >= num_pages) return;      // never write outside the pool
    const int slot = pos % page_size;
    T* key = pages + (size_t)page * page_size * (width + value_width) + (size_t)slot * width;
    T* value = pages + (size_t)page * page_size * (width + value_width) + (size_t)page_size * width + (size_t)slot * value_width;
    for (int i = tid; i < width; i += 256) {
        if (i < c) {
            const T z = from_f32<T>(vals[i] * scale * to_f32<W>(norm_w[i]));
            key[i] = z;
            if (value_width > 0) value[i] = z;
        } else {
            key[i] = from_f32<T>(rotated_element(vals + c, i - c, rot_dims, layout, table));
        }
    }
    for (int i = c + tid; i < value_width; i += 256) value[i] = from_f32<T>(0.f);
}

extern "C" int qil_latent_prepare(const void* proj, int ld, int q_col, int kv_col, void* q_att, void* pages,
                                  const void* norm_w, int norm_dtype, float eps, const float* freq, int rot_dims, int layout,
                                  const int* positions, const int* token_row, const int* block_table, int table_stride,
                                  int n_tokens, int n_heads, int d, int r, int c, int value_width, int page_size,
                                  int num_pages, int act_dtype, int qn_col, int qn_width, const void* qn_w, void* qn_out,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (qn_out != nullptr && (qn_w == nullptr || qn_width <= 0 || qn_col < 0 || qn_col + qn_width > ld))
        QIL_REFUSE("latent_prepare: the queries' latent in columns %d .. %d of %d", qn_col, qn_col + qn_width, ld);
    if (n_heads <= 0 || d <= 0 || r < 0 || c <= 0 || page_size <= 0 || (value_width != 0 && (value_width < c || value_width > c + r)))
        QIL_REFUSE("latent_prepare: heads %d sizes %d/%d latent %d values %d page %d", n_heads, d, r, c, value_width, page_size);
    if (rot_dims < 0 || rot_dims > r || (rot_dims & 1) || (rot_dims > 0 && freq == nullptr) || (layout != 0 && layout != 1))
        QIL_REFUSE("latent_prepare: %d rotated dimensions of %d, layout %d", rot_dims, r, layout);
    const size_t smem = (size_t)(c + r + n_heads * r + rot_dims) * sizeof(float);
    if (smem > 160 * 1024) QIL_REFUSE("latent_prepare: %d values per token are too many", c + r + n_heads * r);
    cudaError_t err = cudaSuccess;
    QIL_DISPATCH_2(act_dtype, norm_dtype, {
        if (smem > 48 * 1024)
            err = cudaFuncSetAttribute(latent_prepare_kernel<T, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err == cudaSuccess)
            qil_launch_chained(latent_prepare_kernel<T, W>, dim3(n_tokens), dim3(256), smem, stream,
                               (const T*)proj, ld, q_col, kv_col, (T*)q_att, (T*)pages, (const W*)norm_w, eps, freq,
                               rot_dims, layout, positions, token_row, block_table, table_stride, n_heads, d, r, c,
                               value_width, page_size, num_pages, qn_col, qn_width, (const W*)qn_w, (T*)qn_out);
    });
    if (err != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(err)); return (int)err; }
    QIL_CHECK_LAUNCH();
}

// Products per head: y[n][h][j] = (sum_i w[h][j][i] * x[n][h][i]) (* sigmoid(gate[n][h])), j < n_out, i < n_in
// (gate_each: a gate per output, gate[n][h * n_out + j], instead of one per head).
// x, y and gate are given by the address of head 0's first element of token 0, a row stride and a head stride
// (in elements), so they may be column ranges of wider buffers.  float32 sums in ascending i within a lane's
// share, then a fixed tree over the lanes: a row's result does not depend on the other rows of the launch.
#define HP_TOKENS 8
template <typename T, typename W>
__global__ void __launch_bounds__(256)
head_product_kernel(const T* __restrict__ x, long long x_row, int x_head, const W* __restrict__ w, T* __restrict__ y,
                    long long y_row, int y_head, const T* __restrict__ gate, long long gate_row, int n_tokens,
                    int n_in, int n_out, int gate_each) {
    extern __shared__ float xs[];             // [HP_TOKENS][n_in]
    qil_wait_for_producer();
    qil_release_consumer();
    const int head = blockIdx.y, t0 = blockIdx.x * HP_TOKENS, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int nt = n_tokens - t0 < HP_TOKENS ? n_tokens - t0 : HP_TOKENS;
    for (int i = tid; i < HP_TOKENS * n_in; i += 256) {
        const int t = i / n_in, k = i - t * n_in;
        xs[i] = t < nt ? to_f32<T>(x[(size_t)(t0 + t) * x_row + (size_t)head * x_head + k]) : 0.f;
    }
    __syncthreads();
    const W* wh = w + (size_t)head * n_out * n_in;
    for (int j = blockIdx.z * 8 + warp; j < n_out; j += 8 * gridDim.z) {
        float acc[HP_TOKENS];
#pragma unroll
        for (int t = 0; t < HP_TOKENS; ++t) acc[t] = 0.f;
        const W* wr = wh + (size_t)j * n_in;
        for (int k = lane; k < n_in; k += 32) {
            const float wv = to_f32<W>(wr[k]);
#pragma unroll
            for (int t = 0; t < HP_TOKENS; ++t) acc[t] = fmaf(wv, xs[t * n_in + k], acc[t]);
        }
#pragma unroll
        for (int t = 0; t < HP_TOKENS; ++t) acc[t] = warp_sum(acc[t]);
        if (lane < nt) {
            float v = 0.f;
#pragma unroll
            for (int t = 0; t < HP_TOKENS; ++t) if (t == lane) v = acc[t];
            if (gate != nullptr) {
                const float g = to_f32<T>(gate[(size_t)(t0 + lane) * gate_row + (gate_each ? head * n_out + j : head)]);
                v *= 1.f / (1.f + expf(-g));
            }
            y[(size_t)(t0 + lane) * y_row + (size_t)head * y_head + j] = from_f32<T>(v);
        }
    }
}

extern "C" int qil_head_product(const void* x, long long x_row, int x_head, const void* w, void* y, long long y_row,
                                int y_head, const void* gate, long long gate_row, int n_tokens, int n_heads, int n_in,
                                int n_out, int act_dtype, int weight_dtype, int gate_each, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_heads <= 0 || n_heads > 65535 || n_in <= 0 || n_out <= 0)
        QIL_REFUSE("head_product: %d heads of %d -> %d", n_heads, n_in, n_out);
    const size_t smem = (size_t)HP_TOKENS * n_in * sizeof(float);
    if (smem > 160 * 1024) QIL_REFUSE("head_product: %d inputs per head are too many", n_in);
    const int tiles = (n_tokens + HP_TOKENS - 1) / HP_TOKENS;
    // few token tiles (a decode step): the outputs of a head are spread over several blocks
    int split = 1;
    while (split < 16 && (long long)tiles * n_heads * split < 296 && split * 16 <= n_out) split <<= 1;
    cudaError_t err = cudaSuccess;
    QIL_DISPATCH_2(act_dtype, weight_dtype, {
        if (smem > 48 * 1024)
            err = cudaFuncSetAttribute(head_product_kernel<T, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err == cudaSuccess)
            qil_launch_chained(head_product_kernel<T, W>, dim3(tiles, n_heads, split), dim3(256), smem, stream,
                               (const T*)x, x_row, x_head, (const W*)w, (T*)y, y_row, y_head, (const T*)gate, gate_row,
                               n_tokens, n_in, n_out, gate_each);
    });
    if (err != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(err)); return (int)err; }
    QIL_CHECK_LAUNCH();
}

// y[n, h * width + j] *= sigmoid(gate[n, h]): a gate per token and head on rows laid out head by head (float32 math,
// one rounding).  For steps whose per-head products ran as one batched library product.
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ y, long long y_row, int width, const T* __restrict__ gate, long long gate_row, int n_heads) {
    qil_wait_for_producer();
    qil_release_consumer();
    const size_t token = blockIdx.x;
    const int per_row = n_heads * width;
    for (int i = threadIdx.x; i < per_row; i += 256) {
        const float g = to_f32<T>(gate[token * gate_row + i / width]);
        T* at = y + token * y_row + i;
        *at = from_f32<T>(to_f32<T>(*at) / (1.f + expf(-g)));
    }
}

extern "C" int qil_head_gate(void* y, long long y_row, int width, const void* gate, long long gate_row, int n_tokens,
                             int n_heads, int act_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_heads <= 0 || width <= 0) QIL_REFUSE("head_gate: %d heads of %d", n_heads, width);
    QIL_DISPATCH_1(act_dtype, {
        qil_launch_chained(head_gate_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (T*)y, y_row, width, (const T*)gate,
                           gate_row, n_heads);
    });
    QIL_CHECK_LAUNCH();
}
