// Mixture of experts: a float32 router with a softmax over the chosen experts, the grouping of
// (token, chosen expert) pairs by expert, the experts' products over the grouped rows, and the sum of a
// token's weighted expert outputs onto the residual stream.
//
//   route     logits = x R^T + b in float32; the `top` largest (ties: the lower index); weights =
//             softmax over those logits alone.  One block per token, every dot product by one warp with a
//             fixed tree: a token's choice never depends on the rest of the batch.
//   group     pairs p = token * top + slot sorted by expert, and a list of row tiles (expert, first
//             row, rows) for the products.  One block; no host round trip, so the launch sizes of what
//             follows depend on the number of tokens only.
//   gate_up   for every row tile: h = act(A W_gate[e]^T, A W_up[e]^T) with A the tokens' rows gathered
//             through the pair list; both products share the loads of A; h is written in grouped order.
//   down      y[p] = weight[p] * (h W_down[e]^T), float32, written at the pair's own place.
//   combine   out[t] = residual[t] + sum over slots of y[t * top + slot], in slot order.
//
// In float32 the products run on the CUDA cores with float32 FMA, each output element summing over k in
// ascending order with one accumulator: a pair's result does not depend on which rows share its tile.
// bfloat16 rows and weights whose width is a multiple of 8 take the tensor cores (further down).
// The activation is the clamped swish of gated_activation.cu (kind 2) or silu (kind 0).
//
// Other designs of routing and experts, as options of the same kernels:
//   route, mode 1   scores = softmax over all outputs of the router; the choice goes by score + correction[e],
//                   the weights are the chosen scores alone, divided by their sum (+ 1e-20), times weight_scale.
//   route, mode 2   as mode 1, but the chosen scores are the weights as they are (times weight_scale): no division.
//                   One more row behind the router's (`gate_logit`) is a dot product that is handed out as it is:
//                   the logit of a gate, one number per token, for an expert that every token uses.
//   experts         without a gate matrix: h = act(A W_up[e]^T) with act the squared relu (kind 3), silu or gelu.
//   identity        router outputs from `n_experts` on name no expert: grouping skips them and combine adds
//                   weight * x, the token's own row.
//   combine         out = residual + col_scale * (sum + sigmoid(gate_logit[t]) * extra[t]): a learned scale per
//                   feature on the whole feed-forward, `extra` the float32 output of the expert that every token uses.
#include "common.cuh"

#define MOE_BM 128         // rows of a tile of the list (the float32 kernel takes it as two halves of MOE_FM)
#define MOE_FM 64
#define MOE_BN 64
#define MOE_BK 16
#define MOE_MAX_EXPERTS 1024
#define MOE_MAX_TOP 64
#define MOE_ONE_BLOCK_PAIRS 512   // up to here one block groups the pairs, in ascending order inside every expert

// ------------------------------------------------------------------ route
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(pairs[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
}

// One warp: from a token's logits in shared memory to its chosen outputs and their weights (both modes; see the
// file's head).  `logits`, `choice`, `sel_p`, `sel_at` are this token's own arrays.
__device__ __forceinline__ void moe_select(float* logits, float* choice, float* sel_p, int* sel_at, size_t token,
                                           int n_outputs, int top, int* __restrict__ chosen, float* __restrict__ weights,
                                           int mode, const float* __restrict__ correction, float weight_scale,
                                           float* __restrict__ gate_logit, int lane) {
    if (gate_logit != nullptr) {
        if (lane == 0) gate_logit[token] = logits[n_outputs];
    }
    if (mode >= 1) {
        // softmax over all outputs; the choice by score + correction, the weights from the scores alone
        float peak = -INFINITY;
        for (int e = lane; e < n_outputs; e += 32) peak = fmaxf(peak, logits[e]);
        peak = warp_max(peak);
        float sum = 0.f;
        for (int e = lane; e < n_outputs; e += 32) sum += expf(logits[e] - peak);
        sum = warp_sum(sum);
        for (int e = lane; e < n_outputs; e += 32) {
            const float score = expf(logits[e] - peak) / sum;
            logits[e] = score;
            choice[e] = score + (correction != nullptr ? correction[e] : 0.f);
        }
        __syncwarp();
        float picked = 0.f;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = n_outputs;
            for (int e = lane; e < n_outputs; e += 32) {
                const float v = choice[e];
                if (v > best) { best = v; at = e; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float other = __shfl_xor_sync(0xffffffffu, best, o);
                const int other_at = __shfl_xor_sync(0xffffffffu, at, o);
                if (other > best || (other == best && other_at < at)) { best = other; at = other_at; }
            }
            if (at >= n_outputs) at = k;                               // non-finite scores: still name an output
            const float score = logits[at];
            picked += score;
            if (lane == 0) {
                sel_at[k] = at;
                sel_p[k] = score;
                choice[at] = -INFINITY;
            }
            __syncwarp();
        }
        for (int k = lane; k < top; k += 32) {
            chosen[token * top + k] = sel_at[k];
            // mode 2: the chosen scores weigh their experts as they are, not divided by their sum
            weights[token * top + k] = (mode == 2 ? sel_p[k] : sel_p[k] / (picked + 1e-20f)) * weight_scale;
        }
        return;
    }
    float best_first = 0.f, total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = n_outputs;
        for (int e = lane; e < n_outputs; e += 32) {
            const float v = logits[e];
            if (v > best) { best = v; at = e; }       // ascending e: the lower index wins a tie inside a lane
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, o);
            const int other_at = __shfl_xor_sync(0xffffffffu, at, o);
            if (other > best || (other == best && other_at < at)) { best = other; at = other_at; }
        }
        if (at >= n_outputs) { at = k; best = -INFINITY; }      // non-finite logits: still name an expert
        if (k == 0) best_first = best;
        const float p = best == -INFINITY ? 0.f : expf(best - best_first);
        total += p;
        if (lane == 0) {
            sel_at[k] = at;
            sel_p[k] = p;
            logits[at] = -INFINITY;
        }
        __syncwarp();
    }
    for (int k = lane; k < top; k += 32) {
        chosen[token * top + k] = sel_at[k];
        weights[token * top + k] = total > 0.f ? sel_p[k] / total : 0.f;
    }
}

// The same for many tokens: a block takes MOE_ROUTE_TOKENS tokens, and a warp's four router rows at a time serve all of
// them, so the router is read from L2 a quarter as often.  Every dot product is summed exactly as in the kernel below
// (the same runs per lane, the same tree): a token's logits are the same bits whichever kernel takes it.
#define MOE_ROUTE_TOKENS 4
template <typename T, typename W>
__global__ void __launch_bounds__(256)
moe_route_tile_kernel(const T* __restrict__ x, const W* __restrict__ router, const W* __restrict__ bias, int n_tokens,
                      int width, int n_outputs, int top, int* __restrict__ chosen, float* __restrict__ weights, int mode,
                      const float* __restrict__ correction, float weight_scale, float* __restrict__ gate_logit) {
    __shared__ float logits[MOE_ROUTE_TOKENS][MOE_MAX_EXPERTS];
    __shared__ float choice[MOE_ROUTE_TOKENS][MOE_MAX_EXPERTS];
    __shared__ float sel_p[MOE_ROUTE_TOKENS][MOE_MAX_TOP];
    __shared__ int sel_at[MOE_ROUTE_TOKENS][MOE_MAX_TOP];
    const int n_experts = n_outputs + (gate_logit != nullptr ? 1 : 0);
    qil_wait_for_producer();
    qil_release_consumer();
    const int token0 = blockIdx.x * MOE_ROUTE_TOKENS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int e0 = warp * 4; e0 < n_experts; e0 += warps * 4) {
        float dot[MOE_ROUTE_TOKENS][4];
#pragma unroll
        for (int t = 0; t < MOE_ROUTE_TOKENS; ++t) dot[t][0] = dot[t][1] = dot[t][2] = dot[t][3] = 0.f;
        for (int i = lane * 8; i < width; i += 256) {
            float b[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (e0 + u < n_experts) load8(router + (size_t)(e0 + u) * width + i, b[u]);
#pragma unroll
            for (int t = 0; t < MOE_ROUTE_TOKENS; ++t) {
                if (token0 + t >= n_tokens) continue;
                float a[8];
                load8(x + (size_t)(token0 + t) * width + i, a);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (e0 + u >= n_experts) continue;
#pragma unroll
                    for (int j = 0; j < 8; ++j) dot[t][u] = fmaf(a[j], b[u][j], dot[t][u]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < MOE_ROUTE_TOKENS; ++t)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float total = warp_sum(dot[t][u]);
                if (lane == 0 && e0 + u < n_experts)
                    logits[t][e0 + u] = total + (bias != nullptr ? to_f32<W>(bias[e0 + u]) : 0.f);
            }
    }
    __syncthreads();
    if (warp >= MOE_ROUTE_TOKENS || token0 + warp >= n_tokens) return;
    moe_select(logits[warp], choice[warp], sel_p[warp], sel_at[warp], (size_t)(token0 + warp), n_outputs, top, chosen, weights,
               mode, correction, weight_scale, gate_logit, lane);
}

template <typename T, typename W>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ x, const W* __restrict__ router, const W* __restrict__ bias, int width,
                 int n_outputs, int top, int* __restrict__ chosen, float* __restrict__ weights, int mode,
                 const float* __restrict__ correction, float weight_scale, float* __restrict__ gate_logit) {
    __shared__ float logits[MOE_MAX_EXPERTS];
    __shared__ float choice[MOE_MAX_EXPERTS];
    const int n_experts = n_outputs + (gate_logit != nullptr ? 1 : 0);     // rows of `router` (the gate's row is the last)
    __shared__ float sel_p[MOE_MAX_TOP];
    __shared__ int sel_at[MOE_MAX_TOP];
    qil_wait_for_producer();
    qil_release_consumer();
    const size_t token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* row = x + token * width;
    // A lane takes runs of 8 values, 16 or 32 bytes a load, four runs in flight per operand; its partial sum runs in
    // ascending order, the lanes' sums meet in a fixed tree: the same bits whatever else is in the batch.
    const bool wide = width % 8 == 0 && (((uintptr_t)x | (uintptr_t)router) & 15) == 0;
    const int warps = blockDim.x >> 5;
    if (wide) {
        // four experts at a time share every load of the token's row and keep four weight loads in flight
        for (int e0 = warp * 4; e0 < n_experts; e0 += warps * 4) {
            float dot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
            for (int i = lane * 8; i < width; i += 256) {
                float a[8];
                load8(row + i, a);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (e0 + u >= n_experts) continue;
                    float b[8];
                    load8(router + (size_t)(e0 + u) * width + i, b);
#pragma unroll
                    for (int j = 0; j < 8; ++j) dot[u] = fmaf(a[j], b[j], dot[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float total = warp_sum(dot[u]);
                if (lane == 0 && e0 + u < n_experts) logits[e0 + u] = total + (bias != nullptr ? to_f32<W>(bias[e0 + u]) : 0.f);
            }
        }
    } else {
        for (int e = warp; e < n_experts; e += warps) {
            const W* w = router + (size_t)e * width;
            float dot = 0.f;
            for (int i = lane; i < width; i += 32) dot = fmaf(to_f32<T>(row[i]), to_f32<W>(w[i]), dot);
            dot = warp_sum(dot);
            if (lane == 0) logits[e] = dot + (bias != nullptr ? to_f32<W>(bias[e]) : 0.f);
        }
    }
    __syncthreads();
    if (warp != 0) return;
    moe_select(logits, choice, sel_p, sel_at, token, n_outputs, top, chosen, weights, mode, correction, weight_scale,
               gate_logit, lane);
}

// ------------------------------------------------------------------ group
// counts, offsets and the pair list; then the tiles.  info: [0] = number of tiles; tiles: int32 [max_tiles, 3].
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int* __restrict__ sorted_pairs,
                 int* __restrict__ info, int* __restrict__ tiles, int max_tiles) {
    __shared__ int counts[MOE_MAX_EXPERTS];
    __shared__ int cursor[MOE_MAX_EXPERTS];
    qil_wait_for_producer();
    qil_release_consumer();
    for (int e = threadIdx.x; e < n_experts; e += 1024) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += 1024) {
        const int e = chosen[p];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            cursor[e] = at;
            for (int r = 0; r < counts[e] && tile < max_tiles; r += MOE_BM, ++tile) {
                tiles[3 * tile] = e;
                tiles[3 * tile + 1] = at + r;
                tiles[3 * tile + 2] = counts[e] - r < MOE_BM ? counts[e] - r : MOE_BM;
            }
            at += counts[e];
        }
        info[0] = tile;
    }
    __syncthreads();
    // pairs in ascending order inside every expert: a thread places the pairs of one expert at a time
    for (int e = threadIdx.x; e < n_experts; e += 1024) {
        if (counts[e] == 0) continue;
        int at = cursor[e];
        for (int p = 0; p < n_pairs; ++p)
            if (chosen[p] == e) sorted_pairs[at++] = p;
    }
}

// The same grouping for many pairs: placement by atomic cursor (the order inside an expert then
// varies from run to run, the results do not: every row of a product is computed by itself).
__global__ void __launch_bounds__(1024)
moe_place_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int* __restrict__ cursor_global,
                 int* __restrict__ sorted_pairs) {
    for (int p = blockIdx.x * 1024 + threadIdx.x; p < n_pairs; p += gridDim.x * 1024) {
        const int e = chosen[p];
        if (e >= 0 && e < n_experts) sorted_pairs[atomicAdd(&cursor_global[e], 1)] = p;
    }
}

__global__ void __launch_bounds__(1024)
moe_count_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int* __restrict__ cursor_global,
                 int* __restrict__ info, int* __restrict__ tiles, int max_tiles) {
    __shared__ int counts[MOE_MAX_EXPERTS];
    qil_wait_for_producer();
    qil_release_consumer();
    for (int e = threadIdx.x; e < n_experts; e += 1024) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += 1024) {
        const int e = chosen[p];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            cursor_global[e] = at;
            for (int r = 0; r < counts[e] && tile < max_tiles; r += MOE_BM, ++tile) {
                tiles[3 * tile] = e;
                tiles[3 * tile + 1] = at + r;
                tiles[3 * tile + 2] = counts[e] - r < MOE_BM ? counts[e] - r : MOE_BM;
            }
            at += counts[e];
        }
        info[0] = tile;
    }
}

// ------------------------------------------------------------------ the experts' products
__device__ __forceinline__ float expert_activation(int kind, float g, float u, float limit, float alpha) {
    if (kind == 0) return g / (1.f + expf(-g)) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

// An expert without a gate matrix: 0 silu, 1 gelu (tanh), 3 squared relu.
__device__ __forceinline__ float expert_plain_activation(int kind, float z) {
    if (kind == 0) return z / (1.f + expf(-z));
    if (kind == 1) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    const float r = fmaxf(z, 0.f);
    return r * r;
}

// MODE 1 (DUAL): two weight stacks (gate, up) [experts, n_out, k]; rows of A gathered by pair / top; activation; output
// in grouped order.  MODE 2: the same with one stack and an activation without a gate.  MODE 0: one stack; rows of A in
// grouped order; output float32 at the pair's place, scaled.
template <typename T, typename W, int MODE>
__global__ void __launch_bounds__(256)
moe_expert_gemm_kernel(const T* __restrict__ A, int lda, const W* __restrict__ w0, const W* __restrict__ w1,
                       const int* __restrict__ tiles, const int* __restrict__ info,
                       const int* __restrict__ sorted_pairs, int top, const float* __restrict__ pair_weight,
                       T* __restrict__ hidden, float* __restrict__ y, int n_out, int K, int kind, float limit,
                       float alpha) {
    constexpr bool DUAL = MODE == 1, UP = MODE != 0;
    __shared__ float As[MOE_BK][MOE_FM + 4];
    __shared__ float W0s[MOE_BK][MOE_BN + 4];
    __shared__ float W1s[DUAL ? MOE_BK : 1][MOE_BN + 4];
    __shared__ int src_row[MOE_FM];
    qil_wait_for_producer();
    qil_release_consumer();
    const int tile = blockIdx.y;
    if (tile >= info[0]) return;
    // blockIdx.z: which half of the tile's rows
    const int expert = tiles[3 * tile], row0 = tiles[3 * tile + 1] + MOE_FM * blockIdx.z;
    const int rows = min(MOE_FM, tiles[3 * tile + 2] - MOE_FM * (int)blockIdx.z);
    if (rows <= 0) return;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * MOE_BN;
    if (tid < MOE_FM) src_row[tid] = tid < rows ? (UP ? sorted_pairs[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    const W* e0 = w0 + (size_t)expert * n_out * K;
    const W* e1 = DUAL ? w1 + (size_t)expert * n_out * K : nullptr;
    float acc0[4][4], acc1[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc0[i][j] = acc1[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;
            const int r = idx >> 4, kk = idx & 15, k = k0 + kk;
            float a = 0.f, b0 = 0.f, b1 = 0.f;
            if (k < K) {
                if (src_row[r] >= 0) a = to_f32<T>(A[(size_t)src_row[r] * lda + k]);
                if (n0 + r < n_out) {
                    b0 = to_f32<W>(e0[(size_t)(n0 + r) * K + k]);
                    if (DUAL) b1 = to_f32<W>(e1[(size_t)(n0 + r) * K + k]);
                }
            }
            As[kk][r] = a;
            W0s[kk][r] = b0;
            if (DUAL) W1s[kk][r] = b1;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            float a[4], b0[4], b1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { b0[j] = W0s[kk][tx * 4 + j]; b1[j] = DUAL ? W1s[kk][tx * 4 + j] : 0.f; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc0[i][j] = fmaf(a[i], b0[j], acc0[i][j]);
                    if (DUAL) acc1[i][j] = fmaf(a[i], b1[j], acc1[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
        const int pair = UP ? 0 : sorted_pairs[row0 + r];
        const float scale = UP ? 1.f : pair_weight[pair];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= n_out) continue;
            if (DUAL) {
                // the products are rounded to the activation type first, as a projection's output is
                const float g = round_to<T>(acc0[i][j]), u = round_to<T>(acc1[i][j]);
                hidden[(size_t)(row0 + r) * n_out + n] = from_f32<T>(expert_activation(kind, g, u, limit, alpha));
            } else if (UP) {
                hidden[(size_t)(row0 + r) * n_out + n] = from_f32<T>(expert_plain_activation(kind, round_to<T>(acc0[i][j])));
            } else {
                y[(size_t)pair * n_out + n] = scale * acc0[i][j];
            }
        }
    }
}

// ------------------------------------------------------------------ the same products on the tensor cores
// bfloat16 rows and weights, float32 accumulators (mma.sync m16n8k16).  A block takes a 128-row tile of one expert
// and 64 output features (of the gate and of the up matrix at once); its eight warps own 32 x 32 corners.
// Rows and weights move through a ring of three stages of 64 k-values with cp.async; rows past the tile's end and k-values past K arrive as zeros.
#define MOE_TK 64
#define MOE_STAGES 3
#define MOE_LDS (MOE_TK + 8)       // row stride in elements: rows start 16 bytes apart mod 128

__device__ __forceinline__ void moe_cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void moe_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void moe_mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MODE>
__global__ void __launch_bounds__(256)
moe_expert_mma_kernel(const bf16* __restrict__ A, int lda, const bf16* __restrict__ w0, const bf16* __restrict__ w1,
                      const int* __restrict__ tiles, const int* __restrict__ info,
                      const int* __restrict__ sorted_pairs, int top, const float* __restrict__ pair_weight,
                      bf16* __restrict__ hidden, float* __restrict__ y, int n_out, int K, int kind, float limit,
                      float alpha) {
    constexpr bool DUAL = MODE == 1, UP = MODE != 0;
    extern __shared__ __align__(16) unsigned char moe_smem[];
    typedef bf16 (*TileA)[MOE_BM][MOE_LDS];
    typedef bf16 (*TileB)[MOE_BN][MOE_LDS];
    TileA sA = reinterpret_cast<TileA>(moe_smem);                                   // [stages][128][LDS]
    TileB sB0 = reinterpret_cast<TileB>(moe_smem + sizeof(bf16) * MOE_STAGES * MOE_BM * MOE_LDS);
    TileB sB1 = sB0 + MOE_STAGES;                                                   // only with DUAL
    __shared__ int src_row[MOE_BM];
    qil_wait_for_producer();
    qil_release_consumer();
    const int tile = blockIdx.y;
    if (tile >= info[0]) return;
    const int expert = tiles[3 * tile], row0 = tiles[3 * tile + 1], rows = tiles[3 * tile + 2];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = (warp & 3) * 32, wn = (warp >> 2) * 32;      // this warp's 32 x 32 corner of the 128 x 64 tile
    const int n0 = blockIdx.x * MOE_BN;
    if (tid < MOE_BM) src_row[tid] = tid < rows ? (UP ? sorted_pairs[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    const bf16* e0 = w0 + (size_t)expert * n_out * K;
    const bf16* e1 = DUAL ? w1 + (size_t)expert * n_out * K : nullptr;

    auto issue = [&](int stage, int k0) {
        // 16-byte pieces: 128 rows x 8 of A (four a thread), 64 rows x 8 of every weight tile (two a thread)
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;
            const int r = idx >> 3, piece = idx & 7, k = k0 + piece * 8;
            const bool a_ok = k < K && src_row[r] >= 0;
            moe_cp_async16(&sA[stage][r][piece * 8], A + (a_ok ? (size_t)src_row[r] * lda + k : 0), a_ok);
        }
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int idx = tid + it * 256;
            const int r = idx >> 3, piece = idx & 7, k = k0 + piece * 8;
            const bool b_ok = k < K && n0 + r < n_out;
            moe_cp_async16(&sB0[stage][r][piece * 8], e0 + (b_ok ? (size_t)(n0 + r) * K + k : 0), b_ok);
            if (DUAL) moe_cp_async16(&sB1[stage][r][piece * 8], e1 + (b_ok ? (size_t)(n0 + r) * K + k : 0), b_ok);
        }
    };
    float acc0[2][4][4], acc1[DUAL ? 2 : 1][4][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            acc0[m][n][0] = acc0[m][n][1] = acc0[m][n][2] = acc0[m][n][3] = 0.f;
            if (DUAL) acc1[m][n][0] = acc1[m][n][1] = acc1[m][n][2] = acc1[m][n][3] = 0.f;
        }

    // a ring of MOE_STAGES stages: the copies of the next two steps are under way while one is multiplied
    const int steps = (K + MOE_TK - 1) / MOE_TK;
#pragma unroll
    for (int ahead = 0; ahead < MOE_STAGES - 1; ++ahead) {
        if (ahead < steps) issue(ahead, ahead * MOE_TK);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    for (int step = 0; step < steps; ++step) {
        const int stage = step % MOE_STAGES;
        asm volatile("cp.async.wait_group %0;\n" ::"n"(MOE_STAGES - 2));
        __syncthreads();        // this step's stage has landed for everyone, and everyone is done with the stage refilled next
        if (step + MOE_STAGES - 1 < steps) issue((step + MOE_STAGES - 1) % MOE_STAGES, (step + MOE_STAGES - 1) * MOE_TK);
        asm volatile("cp.async.commit_group;\n" ::);
        if (wm >= rows) continue;      // a tile of few rows (single tokens): warps past them only copy
#pragma unroll
        for (int ks = 0; ks < MOE_TK / 16; ++ks) {
            unsigned a[2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m)
                moe_ldmatrix_x4(a[m][0], a[m][1], a[m][2], a[m][3],
                                &sA[stage][wm + m * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                unsigned b0, b1, b2, b3;
                moe_ldmatrix_x4(b0, b1, b2, b3,
                                &sB0[stage][wn + np * 16 + (lane >> 4) * 8 + (lane & 7)][ks * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    moe_mma_bf16(acc0[m][2 * np], a[m], b0, b1);
                    moe_mma_bf16(acc0[m][2 * np + 1], a[m], b2, b3);
                }
                if (DUAL) {
                    moe_ldmatrix_x4(b0, b1, b2, b3,
                                    &sB1[stage][wn + np * 16 + (lane >> 4) * 8 + (lane & 7)][ks * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        moe_mma_bf16(acc1[m][2 * np], a[m], b0, b1);
                        moe_mma_bf16(acc1[m][2 * np + 1], a[m], b2, b3);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm + m * 16 + (lane >> 2) + half * 8;
            if (r >= rows) continue;
            const int pair = UP ? 0 : sorted_pairs[row0 + r];
            const float scale = UP ? 1.f : pair_weight[pair];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = n0 + wn + nt * 8 + (lane & 3) * 2 + e;
                    if (n >= n_out) continue;
                    if (DUAL) {
                        const float g = round_to<bf16>(acc0[m][nt][half * 2 + e]), u = round_to<bf16>(acc1[m][nt][half * 2 + e]);
                        hidden[(size_t)(row0 + r) * n_out + n] = __float2bfloat16_rn(expert_activation(kind, g, u, limit, alpha));
                    } else if (UP) {
                        hidden[(size_t)(row0 + r) * n_out + n] =
                            __float2bfloat16_rn(expert_plain_activation(kind, round_to<bf16>(acc0[m][nt][half * 2 + e])));
                    } else {
                        y[(size_t)pair * n_out + n] = scale * acc0[m][nt][half * 2 + e];
                    }
                }
            }
        }
    }
}

static int moe_mma_smem(bool dual) {
    return (int)sizeof(bf16) * MOE_STAGES * (MOE_BM + (dual ? 2 : 1) * MOE_BN) * MOE_LDS;
}
static int moe_mma_configure() {
    static bool configured = false;
    if (configured) return 0;
    cudaError_t a = cudaFuncSetAttribute(moe_expert_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, moe_mma_smem(true));
    cudaError_t b = cudaFuncSetAttribute(moe_expert_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, moe_mma_smem(false));
    cudaError_t c = cudaFuncSetAttribute(moe_expert_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, moe_mma_smem(false));
    if (a != cudaSuccess || b != cudaSuccess || c != cudaSuccess) QIL_REFUSE("moe: cannot reserve %d bytes of shared memory", moe_mma_smem(true));
    configured = true;
    return 0;
}

static bool moe_tensor_cores_usable(int act_dtype, int weight_dtype, int lda, int K, const void* a, const void* b,
                                    const void* c) {
    return act_dtype == QIL_BF16 && weight_dtype == QIL_BF16 && K % 8 == 0 && lda % 8 == 0
        && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0;
}

// ------------------------------------------------------------------ combine
// What a combine may do beyond the sum: identity outputs of the router, an expert that every token uses, a scale.
struct CombineExtras {
    const int* chosen;         // with `x`: pairs whose choice is >= n_experts add weight * x instead of an expert's row
    const float* weights;
    const void* x;             // the experts' input rows, activation type
    int n_experts;
    const float* extra;        // float32 [N, width] or null: added times sigmoid(gate_logit[token])
    const float* gate_logit;   // float32 [N] or null (no gate: extra is added as it is)
    const float* col_scale;    // float32 [width] or null
};

template <typename R, typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const R* __restrict__ residual, R* __restrict__ out, size_t total,
                   int width, int top, CombineExtras ex) {
    qil_wait_for_producer();
    qil_release_consumer();
    const T* x = reinterpret_cast<const T*>(ex.x);
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        const size_t token = i / width;
        const int col = (int)(i % width);
        float sum = 0.f;
        for (int s = 0; s < top; ++s) {
            const size_t pair = token * top + s;
            if (x != nullptr && ex.chosen[pair] >= ex.n_experts) sum += ex.weights[pair] * to_f32<T>(x[i]);
            else sum += y[pair * width + col];
        }
        if (ex.extra != nullptr)
            sum += (ex.gate_logit != nullptr ? 1.f / (1.f + expf(-ex.gate_logit[token])) : 1.f) * ex.extra[i];
        if (ex.col_scale != nullptr) sum *= ex.col_scale[col];
        out[i] = from_f32<R>(residual != nullptr ? to_f32<R>(residual[i]) + sum : sum);
    }
}

// The same for a float32 stream whose width is a multiple of 4: a block walks rows, a thread four columns of each,
// 16 bytes a load, no division per element.  The sums are those of the kernel above, slot by slot.
__device__ __forceinline__ float4 moe_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 moe_load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_f32x4_kernel(const float* __restrict__ y, const float* __restrict__ residual, float* __restrict__ out,
                         int n_tokens, int width, int top, CombineExtras ex) {
    qil_wait_for_producer();
    qil_release_consumer();
    const T* x = reinterpret_cast<const T*>(ex.x);
    for (int token = blockIdx.x; token < n_tokens; token += gridDim.x) {
        const float gate = (ex.extra != nullptr && ex.gate_logit != nullptr) ? 1.f / (1.f + expf(-ex.gate_logit[token])) : 1.f;
        for (int col = threadIdx.x * 4; col < width; col += 1024) {
            const size_t i = (size_t)token * width + col;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < top; ++s) {
                const size_t pair = (size_t)token * top + s;
                float4 v;
                if (x != nullptr && ex.chosen[pair] >= ex.n_experts) {
                    const float w = ex.weights[pair];
                    v = moe_load4(x + i);
                    v.x *= w; v.y *= w; v.z *= w; v.w *= w;
                } else {
                    v = moe_load4(y + pair * width + col);
                }
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            if (ex.extra != nullptr) {
                const float4 v = moe_load4(ex.extra + i);
                sum.x += gate * v.x; sum.y += gate * v.y; sum.z += gate * v.z; sum.w += gate * v.w;
            }
            if (ex.col_scale != nullptr) {
                const float4 c = moe_load4(ex.col_scale + col);
                sum.x *= c.x; sum.y *= c.y; sum.z *= c.z; sum.w *= c.w;
            }
            if (residual != nullptr) {
                const float4 r = moe_load4(residual + i);
                sum.x = r.x + sum.x; sum.y = r.y + sum.y; sum.z = r.z + sum.z; sum.w = r.w + sum.w;
            }
            *reinterpret_cast<float4*>(out + i) = sum;
        }
    }
}

// ------------------------------------------------------------------ entry points
// `router` holds n_experts rows, and one more behind them when `gate_logit` is given.
extern "C" int qil_moe_route(const void* x, const void* router, const void* bias, int n_tokens, int width,
                             int n_experts, int top, int* chosen, float* weights, int mode, const float* correction,
                             float weight_scale, float* gate_logit, int act_dtype, int weight_dtype,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_experts <= 0 || n_experts + (gate_logit != nullptr ? 1 : 0) > MOE_MAX_EXPERTS || top <= 0 || top > n_experts
        || top > MOE_MAX_TOP || width <= 0)
        QIL_REFUSE("moe_route: %d experts (at most %d), %d of them per token, width %d", n_experts, MOE_MAX_EXPERTS, top, width);
    if (mode < 0 || mode > 2) QIL_REFUSE("moe_route: mode %d", mode);
    if (gate_logit != nullptr && bias != nullptr) QIL_REFUSE("moe_route: a gate row goes without router biases");
    if (n_tokens >= 64 && width % 8 == 0 && (((uintptr_t)x | (uintptr_t)router) & 15) == 0) {
        QIL_DISPATCH_2(act_dtype, weight_dtype,
            qil_launch_chained(moe_route_tile_kernel<T, W>, dim3((n_tokens + MOE_ROUTE_TOKENS - 1) / MOE_ROUTE_TOKENS), dim3(256),
                               0, stream, (const T*)x, (const W*)router, (const W*)bias, n_tokens, width, n_experts, top, chosen,
                               weights, mode, correction, weight_scale, gate_logit));
        QIL_CHECK_LAUNCH();
    }
    QIL_DISPATCH_2(act_dtype, weight_dtype,
        qil_launch_chained(moe_route_kernel<T, W>, dim3(n_tokens), dim3(256), 0, stream, (const T*)x, (const W*)router,
                           (const W*)bias, width, n_experts, top, chosen, weights, mode, correction, weight_scale,
                           gate_logit));
    QIL_CHECK_LAUNCH();
}

extern "C" int qil_moe_tile_rows() { return MOE_BM; }
extern "C" int qil_moe_one_block_pairs() { return MOE_ONE_BLOCK_PAIRS; }

// work: int32 [1 + n_experts] (tile count, then a cursor per expert); tiles: int32 [max_tiles, 3].
extern "C" int qil_moe_group(const int* chosen, int n_pairs, int n_experts, int* sorted_pairs, int* work, int* tiles,
                             int max_tiles, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (n_experts <= 0 || n_experts > MOE_MAX_EXPERTS) QIL_REFUSE("moe_group: %d experts", n_experts);
    if (n_pairs <= MOE_ONE_BLOCK_PAIRS) {
        qil_launch_chained(moe_group_kernel, dim3(1), dim3(1024), 0, stream, chosen, n_pairs, n_experts, sorted_pairs,
                           work, tiles, max_tiles);
    } else {
        qil_launch_chained(moe_count_kernel, dim3(1), dim3(1024), 0, stream, chosen, n_pairs, n_experts, work + 1, work,
                           tiles, max_tiles);
        const int blocks = (n_pairs + 1023) / 1024 < 296 ? (n_pairs + 1023) / 1024 : 296;
        moe_place_kernel<<<blocks, 1024, 0, stream>>>(chosen, n_pairs, n_experts, work + 1, sorted_pairs);
    }
    QIL_CHECK_LAUNCH();
}

extern "C" int qil_moe_gate_up(const void* x, int lda, const void* gate_w, const void* up_w, const int* tiles,
                               const int* info, int max_tiles, const int* sorted_pairs, int top, void* hidden,
                               int n_out, int K, int kind, float limit, float alpha, int act_dtype, int weight_dtype,
                               cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    if (max_tiles > 65535) QIL_REFUSE("moe_gate_up: %d row tiles are too many for one launch", max_tiles);
    dim3 grid((n_out + MOE_BN - 1) / MOE_BN, max_tiles);
    const bool gated = up_w != nullptr;        // without a second stack: h = act(A W^T), the activation has no gate
    if (!gated && kind != 0 && kind != 1 && kind != 3) QIL_REFUSE("moe_gate_up: activation %d needs a gate matrix", kind);
    if (gated && kind != 0 && kind != 2) QIL_REFUSE("moe_gate_up: activation %d takes no gate matrix", kind);
    if (moe_tensor_cores_usable(act_dtype, weight_dtype, lda, K, x, gate_w, gated ? up_w : gate_w)) {
        if (moe_mma_configure()) return -1;
        if (gated)
            qil_launch_chained(moe_expert_mma_kernel<1>, grid, dim3(256), moe_mma_smem(true), stream, (const bf16*)x, lda,
                               (const bf16*)gate_w, (const bf16*)up_w, tiles, info, sorted_pairs, top, (const float*)nullptr,
                               (bf16*)hidden, (float*)nullptr, n_out, K, kind, limit, alpha);
        else
            qil_launch_chained(moe_expert_mma_kernel<2>, grid, dim3(256), moe_mma_smem(false), stream, (const bf16*)x, lda,
                               (const bf16*)gate_w, (const bf16*)nullptr, tiles, info, sorted_pairs, top, (const float*)nullptr,
                               (bf16*)hidden, (float*)nullptr, n_out, K, kind, limit, alpha);
        QIL_CHECK_LAUNCH();
    }
    grid.z = MOE_BM / MOE_FM;
    if (gated)
        QIL_DISPATCH_2(act_dtype, weight_dtype,
            (qil_launch_chained(moe_expert_gemm_kernel<T, W, 1>, grid, dim3(256), 0, stream, (const T*)x, lda,
                                (const W*)gate_w, (const W*)up_w, tiles, info, sorted_pairs, top, (const float*)nullptr,
                                (T*)hidden, (float*)nullptr, n_out, K, kind, limit, alpha)));
    else
        QIL_DISPATCH_2(act_dtype, weight_dtype,
            (qil_launch_chained(moe_expert_gemm_kernel<T, W, 2>, grid, dim3(256), 0, stream, (const T*)x, lda,
                                (const W*)gate_w, (const W*)nullptr, tiles, info, sorted_pairs, top, (const float*)nullptr,
                                (T*)hidden, (float*)nullptr, n_out, K, kind, limit, alpha)));
    QIL_CHECK_LAUNCH();
}

extern "C" int qil_moe_down(const void* hidden, const void* down_w, const int* tiles, const int* info, int max_tiles,
                            const int* sorted_pairs, const float* pair_weight, float* y, int n_out, int K,
                            int act_dtype, int weight_dtype, cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    if (max_tiles > 65535) QIL_REFUSE("moe_down: %d row tiles are too many for one launch", max_tiles);
    dim3 grid((n_out + MOE_BN - 1) / MOE_BN, max_tiles);
    if (moe_tensor_cores_usable(act_dtype, weight_dtype, K, K, hidden, down_w, down_w)) {
        if (moe_mma_configure()) return -1;
        qil_launch_chained(moe_expert_mma_kernel<0>, grid, dim3(256), moe_mma_smem(false), stream, (const bf16*)hidden, K,
                           (const bf16*)down_w, (const bf16*)nullptr, tiles, info, sorted_pairs, 1, pair_weight,
                           (bf16*)nullptr, y, n_out, K, 0, 0.f, 0.f);
        QIL_CHECK_LAUNCH();
    }
    grid.z = MOE_BM / MOE_FM;
    QIL_DISPATCH_2(act_dtype, weight_dtype,
        (qil_launch_chained(moe_expert_gemm_kernel<T, W, 0>, grid, dim3(256), 0, stream, (const T*)hidden, K,
                            (const W*)down_w, (const W*)nullptr, tiles, info, sorted_pairs, 1, pair_weight,
                            (T*)nullptr, y, n_out, K, 0, 0.f, 0.f)));
    QIL_CHECK_LAUNCH();
}

extern "C" int qil_moe_combine(const float* y, const void* residual, void* out, int n_tokens, int width, int top,
                               int stream_dtype, const int* chosen, const float* weights, const void* x, int x_dtype,
                               int n_experts, const float* extra, const float* gate_logit, const float* col_scale,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (x != nullptr && (chosen == nullptr || weights == nullptr)) QIL_REFUSE("moe_combine: identity outputs need the choice and the weights");
    const size_t total = (size_t)n_tokens * width;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    CombineExtras ex = {chosen, weights, x, n_experts, extra, gate_logit, col_scale};
    if (stream_dtype == QIL_F32 && width % 4 == 0
        && (((uintptr_t)y | (uintptr_t)residual | (uintptr_t)out | (uintptr_t)x | (uintptr_t)extra | (uintptr_t)col_scale) & 15) == 0) {
        const int rows = n_tokens < 148 * 8 ? n_tokens : 148 * 8;
        if (x_dtype == QIL_BF16)
            qil_launch_chained(moe_combine_f32x4_kernel<bf16>, dim3(rows), dim3(256), 0, stream, y, (const float*)residual,
                               (float*)out, n_tokens, width, top, ex);
        else
            qil_launch_chained(moe_combine_f32x4_kernel<float>, dim3(rows), dim3(256), 0, stream, y, (const float*)residual,
                               (float*)out, n_tokens, width, top, ex);
        QIL_CHECK_LAUNCH();
    }
    // R: the stream's type, T: the input rows' type
    QIL_DISPATCH_2(x_dtype, stream_dtype,
        qil_launch_chained(moe_combine_kernel<W, T>, dim3(blocks), dim3(256), 0, stream, y, (const W*)residual, (W*)out,
                           total, width, top, ex));
    QIL_CHECK_LAUNCH();
}
