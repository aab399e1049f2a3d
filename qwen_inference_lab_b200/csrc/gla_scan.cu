// Gated linear attention with a decay per key channel, as a scan over the tokens of every segment.
//
// Per head, with a state S [d, e] (d key channels, e value channels) kept in float32 per request:
//
//   a_t = sigmoid(z_t)^(1/tau),  z_t = A2 low_t + b           (float32; low_t is the low-rank projection;
//                                                             a kernel of its own, once per layer and step)
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T
//   o_t = S_t^T (q_t * q_scale)
//   y_t = o_t / sqrt(mean_e(o_t^2) + eps) * w  *  silu(g_t)   (norm over the head's e values, gate from a projection)
//
// One block owns one (segment, head, tile of value columns): a thread holds a slice of one column of S in
// registers for the whole segment, reads the state slot of the segment's request at the start and writes
// it back at the end, so a prompt portion goes on from what the portions before it left, and a single
// decoded token is a segment of length one.  When one tile holds all of a head's value columns the norm
// and the gate are applied by the same block; otherwise o goes to a float32 scratch buffer and a row
// kernel norms and gates it.  Tokens are taken in their order with float32 arithmetic, so the
// result does not depend on how a sequence was cut into segments.  Tokens are staged in batches of
// GLA_TB: one barrier pair per batch instead of per token.
//
// Long segments are cut into chunks that run side by side (the `mode` of the entry point): mode 1 scans
// every chunk from a zero state and leaves the chunk's own state and the product of its decays; a carry
// kernel walks a segment's chunks in order, S_in(c+1) = P(c) S_in(c) + S_own(c), leaving every chunk's
// incoming state in place of its own and the last one in the request's slot; mode 2 scans every chunk
// again from its incoming state and writes the outputs.  Twice the arithmetic, all chunks at once.  The
// carry rounds differently from the token-by-token scan: results then depend on the cut in the last bits.
//
// q, k, v, g and low are column ranges of one row-major buffer (the stacked projection), given as
// pointers to their first column and the common row stride.
//
// Two options serve linear attention with a fixed decay per head, S_t = decay_h S_(t-1) + k_t v_t^T:
// `head_decay` (float32 [heads]) stands in for the per-token decays, and `qkv_act` 1 applies silu to q, k
// and v as they are read (in float32).  Such a design norms all heads' outputs together: `force_raw` sends
// the un-normed outputs to the float32 scratch buffer whatever the sizes, and lin_norm_gate_whole
// finishes them (one norm over a token's whole row, times sigmoid of the gate).
#include "common.cuh"

#define GLA_TB 8

__device__ __forceinline__ float decay_from_logit(float z, float inv_tau) {
    // sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau);  log_sigmoid(z) = min(z, 0) - log1p(exp(-|z|))
    const float log_sigmoid = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
    return expf(log_sigmoid * inv_tau);
}

#define GLA_R 32          // rows of a column that one thread holds
#define GLA_THREADS 256
#ifndef GLA_MIN_BLOCKS
#define GLA_MIN_BLOCKS 2  // blocks per multiprocessor the scan is compiled for
#endif

// alpha[t, c] = sigmoid(b_c + sum_j A2[c, j] low[t, j])^(1/tau) for every token and key channel: float32, once
// per layer and step (the scan's blocks all read it).
template <typename T, typename W>
__global__ void __launch_bounds__(256)
gla_decay_kernel(const T* __restrict__ low, int ld, const W* __restrict__ a2, const W* __restrict__ a2_bias, int rank,
                 float inv_tau, int channels, float* __restrict__ alpha) {
    extern __shared__ float s_low[];        // [rank]
    qil_wait_for_producer();
    qil_release_consumer();
    const size_t token = blockIdx.x;
    for (int j = threadIdx.x; j < rank; j += 256) s_low[j] = to_f32<T>(low[token * ld + j]);
    __syncthreads();
    for (int c = threadIdx.x; c < channels; c += 256) {
        float z = to_f32<W>(a2_bias[c]);
        const W* a2_row = a2 + (size_t)c * rank;
        for (int j = 0; j < rank; ++j) z = fmaf(to_f32<W>(a2_row[j]), s_low[j], z);
        alpha[token * channels + c] = decay_from_logit(z, inv_tau);
    }
}

template <typename T, typename W>
__device__ __forceinline__ void gla_norm_gate_rows(const float* o_rows, int o_stride, int nb, size_t first_token,
                                                   const T* g, int ld, const W* norm_w, float eps, int n_heads,
                                                   int head, int e, T* out, int lane, int warp, int warps) {
    for (int tb = warp; tb < nb; tb += warps) {
        const float* o = o_rows + (size_t)tb * o_stride;
        float ss = 0.f;
        for (int c = lane; c < e; c += 32) ss = fmaf(o[c], o[c], ss);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)e + eps);
        const size_t token = first_token + tb;
        for (int c = lane; c < e; c += 32) {
            const float gate = to_f32<T>(g[token * ld + head * e + c]);
            const float y = o[c] * scale * to_f32<W>(norm_w[c]);
            out[(token * n_heads + head) * e + c] = from_f32<T>(y * (gate / (1.f + expf(-gate))));
        }
    }
}

__device__ __forceinline__ float scan_input(float x, int act) { return act == 1 ? x / (1.f + expf(-x)) : x; }

#define GLA_WHOLE 0        // from the state slot, outputs, state written back
#define GLA_OWN_STATE 1    // from zero, no outputs; the chunk's state and the product of its decays are written
#define GLA_FROM_STATE 2   // from the given state, outputs, nothing written back

template <typename T, typename W, bool FUSED, int MODE>
__global__ void __launch_bounds__(GLA_THREADS, GLA_MIN_BLOCKS)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                const float* __restrict__ alpha, const float* __restrict__ head_decay, int qkv_act, int ld, float q_scale,
                const W* __restrict__ norm_w, float eps, float* __restrict__ state, float* __restrict__ decay_product, const int* __restrict__ seg_start,
                const int* __restrict__ seg_len, const int* __restrict__ seg_row, int n_heads, int d, int e,
                int ds_count, int tile_cols, float* __restrict__ o_raw, T* __restrict__ out) {
    constexpr int R = GLA_R;
    extern __shared__ float smem[];
    // q, k and the decays of a token: ds_count blocks of R values, each followed by four unused floats, so that
    // the threads of a quarter warp (which differ in their block) read their 16-byte pieces from different banks
    const int stride = ds_count * (R + 4);
    float* sq = smem;                    // [TB][stride]
    float* sk = sq + GLA_TB * stride;    // [TB][stride]
    float* sa = sk + GLA_TB * stride;    // [TB][stride]
    float* sv = sa + GLA_TB * stride;    // [TB][tile_cols]
    float* so = sv + GLA_TB * tile_cols; // [TB][tile_cols]
    float* sp = so + GLA_TB * tile_cols; // [d]: the product of the decays so far (GLA_OWN_STATE)
    qil_wait_for_producer();
    qil_release_consumer();
    const int tiles = (e + tile_cols - 1) / tile_cols;
    const int head = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * tile_cols, seg = blockIdx.y;
    const int first = seg_start[seg], count = seg_len[seg], row = seg_row[seg];
    const int tid = threadIdx.x, threads = blockDim.x;
    const int local = tid / ds_count, ds = tid % ds_count, col = col0 + local;
    const bool owner = local < tile_cols && col < e;
    float* slot = state + ((size_t)row * n_heads + head) * d * e;

    float S[R];           // rows ds * R .. ds * R + R - 1 of the column (rows past d stay zero)
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int dd = ds * R + r;
        S[r] = (MODE != GLA_OWN_STATE && owner && dd < d) ? slot[(size_t)dd * e + col] : 0.f;
    }
    if (MODE == GLA_OWN_STATE)
        for (int dd = tid; dd < d; dd += threads) sp[dd] = 1.f;
    const int lane = tid & 31, warp = tid >> 5, warps = threads >> 5;
    for (int t0 = 0; t0 < count; t0 += GLA_TB) {
        const int nb = count - t0 < GLA_TB ? count - t0 : GLA_TB;
        __syncthreads();
        for (int i = tid; i < nb * ds_count * R; i += threads) {
            const int tb = i / (ds_count * R), dd = i % (ds_count * R);
            const int to = tb * stride + (dd / R) * (R + 4) + dd % R;
            const bool real = dd < d;           // rows past d: zeros, which keep their (zero) state rows zero
            const size_t at = (size_t)(first + t0 + tb) * ld + head * d + dd;
            if (MODE != GLA_OWN_STATE) sq[to] = real ? scan_input(to_f32<T>(q[at]), qkv_act) * q_scale : 0.f;
            sk[to] = real ? scan_input(to_f32<T>(k[at]), qkv_act) : 0.f;
            sa[to] = !real ? 0.f : head_decay != nullptr ? head_decay[head]
                                                         : alpha[(size_t)(first + t0 + tb) * n_heads * d + head * d + dd];
        }
        for (int i = tid; i < nb * tile_cols; i += threads) {
            const int tb = i / tile_cols, c = col0 + i % tile_cols;
            sv[i] = c < e ? scan_input(to_f32<T>(v[(size_t)(first + t0 + tb) * ld + head * e + c]), qkv_act) : 0.f;
        }
        __syncthreads();
        if (MODE == GLA_OWN_STATE) {
            for (int dd = tid; dd < d; dd += threads) {       // the same thread every batch: no barrier needed
                float product = sp[dd];
                for (int tb = 0; tb < nb; ++tb) product *= sa[tb * stride + (dd / R) * (R + 4) + dd % R];
                sp[dd] = product;
            }
        }
        for (int tb = 0; tb < nb; ++tb) {
            const float vc = owner ? sv[tb * tile_cols + local] : 0.f;
            float o = 0.f;
            const float4* a4 = reinterpret_cast<const float4*>(sa + tb * stride + ds * (R + 4));
            const float4* k4 = reinterpret_cast<const float4*>(sk + tb * stride + ds * (R + 4));
            const float4* q4 = reinterpret_cast<const float4*>(sq + tb * stride + ds * (R + 4));
#pragma unroll
            for (int r4 = 0; r4 < R / 4; ++r4) {
                const float4 a = a4[r4], kk = k4[r4];
                S[4 * r4 + 0] = fmaf(a.x, S[4 * r4 + 0], kk.x * vc);
                S[4 * r4 + 1] = fmaf(a.y, S[4 * r4 + 1], kk.y * vc);
                S[4 * r4 + 2] = fmaf(a.z, S[4 * r4 + 2], kk.z * vc);
                S[4 * r4 + 3] = fmaf(a.w, S[4 * r4 + 3], kk.w * vc);
                if (MODE != GLA_OWN_STATE) {
                    const float4 qq = q4[r4];
                    o = fmaf(S[4 * r4 + 0], qq.x, o);
                    o = fmaf(S[4 * r4 + 1], qq.y, o);
                    o = fmaf(S[4 * r4 + 2], qq.z, o);
                    o = fmaf(S[4 * r4 + 3], qq.w, o);
                }
            }
            if (MODE == GLA_OWN_STATE) continue;
            for (int step = 1; step < ds_count; step <<= 1) o += __shfl_xor_sync(0xffffffffu, o, step);
            if (owner && ds == 0) {
                if (FUSED) so[tb * tile_cols + local] = o;
                else o_raw[((size_t)(first + t0 + tb) * n_heads + head) * e + col] = o;
            }
        }
        if (FUSED && MODE != GLA_OWN_STATE) {
            __syncthreads();
            gla_norm_gate_rows<T, W>(so, tile_cols, nb, (size_t)(first + t0), g, ld, norm_w, eps, n_heads, head, e, out,
                                     lane, warp, warps);
        }
    }
    if (MODE == GLA_FROM_STATE) return;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int dd = ds * R + r;
        if (owner && dd < d) slot[(size_t)dd * e + col] = S[r];
    }
    if (MODE == GLA_OWN_STATE && col0 == 0)
        for (int dd = tid; dd < d; dd += threads) decay_product[((size_t)row * n_heads + head) * d + dd] = sp[dd];
}

// The carry over a long segment's chunks: chunk_state [chunks, heads, d, e] holds every chunk's own state on
// entry and its incoming state on exit; the state after the last chunk goes to the request's slot.
// carry: int32 [n, 3] = (state slot, first chunk, chunks).
__global__ void __launch_bounds__(256)
gla_carry_kernel(float* __restrict__ chunk_state, const float* __restrict__ decay_product, float* __restrict__ slots,
                 const int* __restrict__ carry, int n_heads, int d, int e) {
    qil_wait_for_producer();
    qil_release_consumer();
    const size_t per_state = (size_t)n_heads * d * e;
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= per_state) return;
    const int row = carry[3 * blockIdx.y], first = carry[3 * blockIdx.y + 1], chunks = carry[3 * blockIdx.y + 2];
    const size_t channel = i / e;                 // head * d + key channel
    float s = slots[(size_t)row * per_state + i];
    // four chunks at a time: their loads are all under way before the first is used (a thread reads and writes
    // only its own element of every chunk, so the order of loads and stores between chunks is free)
    for (int c0 = first; c0 < first + chunks; c0 += 4) {
        float own[4], decay[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const bool real = c0 + u < first + chunks;
            own[u] = real ? chunk_state[(size_t)(c0 + u) * per_state + i] : 0.f;
            decay[u] = real ? decay_product[(size_t)(c0 + u) * n_heads * d + channel] : 1.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (c0 + u >= first + chunks) break;
            chunk_state[(size_t)(c0 + u) * per_state + i] = s;
            s = fmaf(decay[u], s, own[u]);
        }
    }
    slots[(size_t)row * per_state + i] = s;
}

// The norm and the gate for heads whose value columns were spread over several blocks: one block per token.
template <typename T, typename W>
__global__ void __launch_bounds__(256)
gla_norm_gate_kernel(const float* __restrict__ o_raw, const T* __restrict__ g, int ld, const W* __restrict__ norm_w,
                     float eps, int n_heads, int e, T* __restrict__ out) {
    qil_wait_for_producer();
    qil_release_consumer();
    const size_t token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int head = warp; head < n_heads; head += 8)
        gla_norm_gate_rows<T, W>(o_raw + (token * n_heads + head) * e, 0, 1, token, g, ld, norm_w, eps, n_heads, head, e,
                                 out, lane, 0, 1);
}

template <typename T, typename W, bool FUSED, int MODE>
static cudaError_t gla_launch(dim3 grid, int threads, size_t smem, cudaStream_t stream, const void* q, const void* k,
                              const void* v, const void* g, const float* alpha, const float* head_decay, int qkv_act,
                              int ld, float q_scale, const void* norm_w, float eps, float* state,
                              float* decay_product, const int* seg_start, const int* seg_len, const int* seg_row, int n_heads, int d, int e,
                              int ds_count, int tile_cols, float* o_raw, void* out) {
    cudaError_t err = cudaFuncSetAttribute(gla_scan_kernel<T, W, FUSED, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    return qil_launch_chained(gla_scan_kernel<T, W, FUSED, MODE>, grid, dim3(threads), smem, stream,
                              (const T*)q, (const T*)k, (const T*)v, (const T*)g, alpha, head_decay, qkv_act, ld, q_scale,
                              (const W*)norm_w, eps, state, decay_product,
                              seg_start, seg_len,
                              seg_row, n_heads, d, e, ds_count, tile_cols, o_raw, (T*)out);
}

// o_raw: float32 [tokens, heads * e] of scratch, needed only when a head's value columns do not fit one
// block (qil_gla_scan_needs_scratch).
extern "C" int qil_gla_scan_needs_scratch(int d, int e) {
    int ds_count = 1;
    while (ds_count * GLA_R < d) ds_count <<= 1;
    return ds_count > 32 ? -1 : (e > GLA_THREADS / ds_count ? 1 : 0);
}

extern "C" int qil_gla_scan(const void* q, const void* k, const void* v, const void* g, const float* alpha,
                            const float* head_decay, int qkv_act, int force_raw, int ld, float q_scale, const void* norm_w, float eps, float* state, const int* seg_start, const int* seg_len,
                            const int* seg_row, int n_segments, int n_tokens, int n_heads, int d, int e, float* o_raw,
                            void* out, int mode, float* decay_product, int act_dtype, int weight_dtype,
                            cudaStream_t stream) {
    // mode: GLA_WHOLE; GLA_OWN_STATE (state: the chunks' states, seg_row: the chunk's index there, decay_product
    // [chunks, heads, d]); GLA_FROM_STATE (state and seg_row as before; the states are read only)
    if (n_segments <= 0) return 0;
    if (mode < 0 || mode > 2 || (mode == GLA_OWN_STATE && decay_product == nullptr)) QIL_REFUSE("gla_scan: mode %d", mode);
    if (n_heads <= 0 || d <= 0 || e <= 0 || (alpha == nullptr) == (head_decay == nullptr) || n_segments > 65535)
        QIL_REFUSE("gla_scan: heads %d sizes %d/%d segments %d", n_heads, d, e, n_segments);
    // a thread holds GLA_R rows of one column; ds_count threads (a power of two within a warp) share a column
    int ds_count = 1;
    while (ds_count * GLA_R < d) ds_count <<= 1;
    if (ds_count > 32) QIL_REFUSE("gla_scan: %d key channels per head are more than %d", d, 32 * GLA_R);
    const int tile_cols = e < GLA_THREADS / ds_count ? e : GLA_THREADS / ds_count;
    const int tiles = (e + tile_cols - 1) / tile_cols;
    const bool fused = tiles == 1 && !force_raw;
    if (!fused && o_raw == nullptr && mode != GLA_OWN_STATE) QIL_REFUSE("gla_scan: %d value columns per head need the scratch buffer", e);
    const int threads = (tile_cols * ds_count + 31) / 32 * 32;
    const size_t smem = ((size_t)GLA_TB * (3 * ds_count * (GLA_R + 4) + 2 * tile_cols) + d) * sizeof(float);
    dim3 grid(n_heads * tiles, n_segments);
    cudaError_t err = cudaSuccess;
#define QIL_GLA_GO(F, M)                                                                                         \
    QIL_DISPATCH_2(act_dtype, weight_dtype,                                                                      \
        (err = gla_launch<T, W, F, M>(grid, threads, smem, stream, q, k, v, g, alpha, head_decay, qkv_act, ld,              \
                                      q_scale, norm_w, eps, state, decay_product, seg_start, seg_len, seg_row, n_heads, \
                                      d, e, ds_count, tile_cols, o_raw, out)))
    if (mode == GLA_OWN_STATE) QIL_GLA_GO(false, GLA_OWN_STATE);
    else if (mode == GLA_WHOLE) { if (fused) QIL_GLA_GO(true, GLA_WHOLE); else QIL_GLA_GO(false, GLA_WHOLE); }
    else { if (fused) QIL_GLA_GO(true, GLA_FROM_STATE); else QIL_GLA_GO(false, GLA_FROM_STATE); }
#undef QIL_GLA_GO
    if (mode == GLA_OWN_STATE) {
        if (err != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(err)); return (int)err; }
        QIL_CHECK_LAUNCH();
    }
    if (err != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(err)); return (int)err; }
    QIL_CHECK_LAUNCH();
}

extern "C" int qil_gla_carry(float* chunk_state, const float* decay_product, float* slots, const int* carry,
                             int n_carries, int n_heads, int d, int e, cudaStream_t stream) {
    if (n_carries <= 0) return 0;
    const size_t per_state = (size_t)n_heads * d * e;
    qil_launch_chained(gla_carry_kernel, dim3((unsigned)((per_state + 255) / 256), n_carries), dim3(256), 0, stream,
                       chunk_state, (const float*)decay_product, slots, carry, n_heads, d, e);
    QIL_CHECK_LAUNCH();
}

// The norm and the gate over o_raw (what qil_gla_scan leaves when a head's value columns do not fit one block),
// once per step after all scans of the layer.
extern "C" int qil_gla_norm_gate(const float* o_raw, const void* g, int ld, const void* norm_w, float eps, int n_tokens,
                                 int n_heads, int e, void* out, int act_dtype, int weight_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    QIL_DISPATCH_2(act_dtype, weight_dtype,
        qil_launch_chained(gla_norm_gate_kernel<T, W>, dim3(n_tokens), dim3(256), 0, stream, o_raw, (const T*)g, ld,
                           (const W*)norm_w, eps, n_heads, e, (T*)out));
    QIL_CHECK_LAUNCH();
}

// alpha float32 [n_tokens, channels] from the low-rank projection (columns of a row-major buffer of stride ld).
extern "C" int qil_gla_decay(const void* low, int ld, const void* a2, const void* a2_bias, int rank, float tau,
                             int n_tokens, int channels, float* alpha, int act_dtype, int weight_dtype,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || channels <= 0 || !(tau > 0.f) || rank > 8192) QIL_REFUSE("gla_decay: rank %d channels %d tau %g", rank, channels, (double)tau);
    QIL_DISPATCH_2(act_dtype, weight_dtype,
        qil_launch_chained(gla_decay_kernel<T, W>, dim3(n_tokens), dim3(256), rank * sizeof(float), stream, (const T*)low, ld,
                           (const W*)a2, (const W*)a2_bias, rank, 1.f / tau, channels, alpha));
    QIL_CHECK_LAUNCH();
}

// out[n][i] = o_raw[n][i] / sqrt(mean_i(o_raw[n]^2) + eps) * w[i] * sigmoid(g[n][i]) over a token's whole row of
// `width` = heads * e values: the finish of a linear attention whose heads are normed together.
template <typename T, typename W>
__global__ void __launch_bounds__(256)
lin_norm_gate_whole_kernel(const float* __restrict__ o_raw, const T* __restrict__ g, int ld, const W* __restrict__ norm_w,
                           float eps, int width, T* __restrict__ out) {
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const size_t token = blockIdx.x;
    const float* o = o_raw + token * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) ss = fmaf(o[i], o[i], ss);
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += 256) {
        const float gate = to_f32<T>(g[token * ld + i]);
        out[token * width + i] = from_f32<T>(o[i] * scale * to_f32<W>(norm_w[i]) * (1.f / (1.f + expf(-gate))));
    }
}

extern "C" int qil_lin_norm_gate_whole(const float* o_raw, const void* g, int ld, const void* norm_w, float eps,
                                       int n_tokens, int width, void* out, int act_dtype, int weight_dtype,
                                       cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0) QIL_REFUSE("lin_norm_gate_whole: width %d", width);
    QIL_DISPATCH_2(act_dtype, weight_dtype,
        qil_launch_chained(lin_norm_gate_whole_kernel<T, W>, dim3(n_tokens), dim3(256), 0, stream, o_raw, (const T*)g, ld,
                           (const W*)norm_w, eps, width, (T*)out));
    QIL_CHECK_LAUNCH();
}
