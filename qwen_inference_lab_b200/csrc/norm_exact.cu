// Root-mean-square norm whose arithmetic is float32 from end to end, for residual streams that are
// kept in float32 whatever the activation dtype is.
//
//   y = x / sqrt(mean(x^2) + eps) * (offset + w)
//
// Input and output types are independent (a float32 stream normed into bfloat16 rows for the
// products that follow); the statistics, the scaling and the weight multiply are float32 and the
// result is rounded once.  `offset` 1 serves weights that are stored around zero, 0 plain ones.
// With `rows` only those rows are normed, in that order.  The sum of squares is taken by a fixed
// tree over a fixed block size, so a row's result does not depend on the rest of the batch.
#include "common.cuh"

template <typename TI, typename TO, typename W>
__global__ void __launch_bounds__(256)
rmsnorm_exact_kernel(const TI* __restrict__ x, const W* __restrict__ weight, const int* __restrict__ rows,
                     TO* __restrict__ out, int width, float eps, float offset, long long ld) {
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const int r = blockIdx.x;
    const TI* src = x + (size_t)(rows ? rows[r] : r) * (size_t)ld;      // ld: the input's row stride (a column range of a wider buffer)
    TO* dst = out + (size_t)r * width;
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = to_f32<TI>(src[i]);
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, scratch);
    const float scale = 1.0f / sqrtf(sq / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += 256)
        dst[i] = from_f32<TO>(to_f32<TI>(src[i]) * scale * (offset + to_f32<W>(weight[i])));
}

extern "C" int qil_rmsnorm_exact(const void* x, int x_dtype, const void* weight, int weight_dtype, const int* rows,
                                 void* out, int out_dtype, int n_rows, int width, float eps, float offset,
                                 long long ld, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || ld < width) QIL_REFUSE("rmsnorm_exact: width %d, row stride %lld", width, ld);
#define QIL_NORM_GO(TI, TO)                                                                                  \
    do {                                                                                                     \
        if (weight_dtype == QIL_F32)                                                                         \
            qil_launch_chained(rmsnorm_exact_kernel<TI, TO, float>, dim3(n_rows), dim3(256), 0, stream,      \
                               (const TI*)x, (const float*)weight, rows, (TO*)out, width, eps, offset, ld);  \
        else                                                                                                 \
            qil_launch_chained(rmsnorm_exact_kernel<TI, TO, bf16>, dim3(n_rows), dim3(256), 0, stream,       \
                               (const TI*)x, (const bf16*)weight, rows, (TO*)out, width, eps, offset, ld);   \
    } while (0)
    if (weight_dtype != QIL_F32 && weight_dtype != QIL_BF16) QIL_REFUSE("rmsnorm_exact: weight dtype %d", weight_dtype);
    if (x_dtype == QIL_F32 && out_dtype == QIL_F32) QIL_NORM_GO(float, float);
    else if (x_dtype == QIL_F32 && out_dtype == QIL_BF16) QIL_NORM_GO(float, bf16);
    else if (x_dtype == QIL_BF16 && out_dtype == QIL_BF16) QIL_NORM_GO(bf16, bf16);
    else if (x_dtype == QIL_BF16 && out_dtype == QIL_F32) QIL_NORM_GO(bf16, float);
    else QIL_REFUSE("rmsnorm_exact: dtypes %d -> %d", x_dtype, out_dtype);
#undef QIL_NORM_GO
    QIL_CHECK_LAUNCH();
}

// Layer norm with weight and bias (null: none), float32 from end to end like the norm above:
//
//   y = (x - mean) / sqrt(var + eps) * w + b,     var = mean((x - mean)^2)
//
// Two passes over the row (the mean, then the squared deviations from it), each a fixed tree.
template <typename TI, typename TO, typename W>
__global__ void __launch_bounds__(256)
layernorm_exact_kernel(const TI* __restrict__ x, const W* __restrict__ weight, const W* __restrict__ bias,
                       const int* __restrict__ rows, TO* __restrict__ out, int width, float eps) {
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const int r = blockIdx.x;
    const TI* src = x + (size_t)(rows ? rows[r] : r) * width;
    TO* dst = out + (size_t)r * width;
    float sum = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) sum += to_f32<TI>(src[i]);
    const float mean = block_sum(sum, scratch) / (float)width;
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = to_f32<TI>(src[i]) - mean;
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, scratch);
    const float scale = 1.0f / sqrtf(sq / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += 256)
        dst[i] = from_f32<TO>((to_f32<TI>(src[i]) - mean) * scale * to_f32<W>(weight[i]) + (bias != nullptr ? to_f32<W>(bias[i]) : 0.f));
}

extern "C" int qil_layernorm_exact(const void* x, int x_dtype, const void* weight, const void* bias, int weight_dtype,
                                   const int* rows, void* out, int out_dtype, int n_rows, int width, float eps,
                                   cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) QIL_REFUSE("layernorm_exact: width %d", width);
#define QIL_NORM_GO(TI, TO)                                                                                    \
    do {                                                                                                       \
        if (weight_dtype == QIL_F32)                                                                           \
            qil_launch_chained(layernorm_exact_kernel<TI, TO, float>, dim3(n_rows), dim3(256), 0, stream,      \
                               (const TI*)x, (const float*)weight, (const float*)bias, rows, (TO*)out, width, eps); \
        else                                                                                                   \
            qil_launch_chained(layernorm_exact_kernel<TI, TO, bf16>, dim3(n_rows), dim3(256), 0, stream,       \
                               (const TI*)x, (const bf16*)weight, (const bf16*)bias, rows, (TO*)out, width, eps); \
    } while (0)
    if (weight_dtype != QIL_F32 && weight_dtype != QIL_BF16) QIL_REFUSE("layernorm_exact: weight dtype %d", weight_dtype);
    if (x_dtype == QIL_F32 && out_dtype == QIL_F32) QIL_NORM_GO(float, float);
    else if (x_dtype == QIL_F32 && out_dtype == QIL_BF16) QIL_NORM_GO(float, bf16);
    else if (x_dtype == QIL_BF16 && out_dtype == QIL_BF16) QIL_NORM_GO(bf16, bf16);
    else if (x_dtype == QIL_BF16 && out_dtype == QIL_F32) QIL_NORM_GO(bf16, float);
    else QIL_REFUSE("layernorm_exact: dtypes %d -> %d", x_dtype, out_dtype);
#undef QIL_NORM_GO
    QIL_CHECK_LAUNCH();
}

// x += y / sqrt(mean(y^2) + eps) * w: a branch that is normed by its own root mean square before it joins the
// residual stream.  float32 arithmetic; x is the stream (float32 or bfloat16), y the branch.
template <typename TX, typename TY, typename W>
__global__ void __launch_bounds__(256)
rms_scale_add_kernel(TX* __restrict__ x, const TY* __restrict__ y, const W* __restrict__ weight, int width, float eps) {
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const TY* src = y + (size_t)blockIdx.x * width;
    TX* dst = x + (size_t)blockIdx.x * width;
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = to_f32<TY>(src[i]);
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, scratch);
    const float scale = 1.0f / sqrtf(sq / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += 256)
        dst[i] = from_f32<TX>(to_f32<TX>(dst[i]) + to_f32<TY>(src[i]) * scale * to_f32<W>(weight[i]));
}

extern "C" int qil_rms_scale_add(void* x, int x_dtype, const void* y, int y_dtype, const void* weight, int weight_dtype,
                                 int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) QIL_REFUSE("rms_scale_add: width %d", width);
#define QIL_NORM_GO(TX, TY)                                                                                   \
    do {                                                                                                      \
        if (weight_dtype == QIL_F32)                                                                          \
            qil_launch_chained(rms_scale_add_kernel<TX, TY, float>, dim3(n_rows), dim3(256), 0, stream,       \
                               (TX*)x, (const TY*)y, (const float*)weight, width, eps);                       \
        else                                                                                                  \
            qil_launch_chained(rms_scale_add_kernel<TX, TY, bf16>, dim3(n_rows), dim3(256), 0, stream,        \
                               (TX*)x, (const TY*)y, (const bf16*)weight, width, eps);                        \
    } while (0)
    if (weight_dtype != QIL_F32 && weight_dtype != QIL_BF16) QIL_REFUSE("rms_scale_add: weight dtype %d", weight_dtype);
    if (x_dtype == QIL_F32 && y_dtype == QIL_F32) QIL_NORM_GO(float, float);
    else if (x_dtype == QIL_F32 && y_dtype == QIL_BF16) QIL_NORM_GO(float, bf16);
    else if (x_dtype == QIL_BF16 && y_dtype == QIL_BF16) QIL_NORM_GO(bf16, bf16);
    else if (x_dtype == QIL_BF16 && y_dtype == QIL_F32) QIL_NORM_GO(bf16, float);
    else QIL_REFUSE("rms_scale_add: dtypes %d += %d", x_dtype, y_dtype);
#undef QIL_NORM_GO
    QIL_CHECK_LAUNCH();
}

// A branch joins the stream through a norm on the branch: x += mult * rms(a; w), rms(a; w) = a / sqrt(mean(a^2) + eps) * w.
// With a second branch b the two are first normed with weights of their own and averaged:
//   y = pre * (rms(a; wa) + rms(b; wb)),   x += mult * rms(y; w).
// float32 arithmetic throughout; x is the stream (float32 or bfloat16), a and b share a type.
template <typename TX, typename TA, typename W>
__global__ void __launch_bounds__(256)
rms_join_kernel(TX* __restrict__ x, const TA* __restrict__ a, const W* __restrict__ wa, const TA* __restrict__ b,
                const W* __restrict__ wb, const W* __restrict__ w, int width, float eps, float pre, float mult,
                bf16* __restrict__ rows) {
    // rows: null, or [N, width]: the stream's new values once more, rounded to bfloat16 (what the next product reads)
    extern __shared__ float y[];             // [width] when there are two branches
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const TA* ra = a + (size_t)blockIdx.x * width;
    TX* dst = x + (size_t)blockIdx.x * width;
    bf16* copy = rows != nullptr ? rows + (size_t)blockIdx.x * width : nullptr;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = to_f32<TA>(ra[i]);
        sa = fmaf(v, v, sa);
    }
    sa = block_sum(sa, scratch);
    const float scale_a = 1.0f / sqrtf(sa / (float)width + eps);
    if (b == nullptr) {
        for (int i = threadIdx.x; i < width; i += 256) {
            const TX next = from_f32<TX>(to_f32<TX>(dst[i]) + mult * (to_f32<TA>(ra[i]) * scale_a * to_f32<W>(w[i])));
            dst[i] = next;
            if (copy != nullptr) copy[i] = from_f32<bf16>(to_f32<TX>(next));
        }
        return;
    }
    const TA* rb = b + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = to_f32<TA>(rb[i]);
        sb = fmaf(v, v, sb);
    }
    sb = block_sum(sb, scratch);
    const float scale_b = 1.0f / sqrtf(sb / (float)width + eps);
    float sy = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = pre * (to_f32<TA>(ra[i]) * scale_a * to_f32<W>(wa[i]) + to_f32<TA>(rb[i]) * scale_b * to_f32<W>(wb[i]));
        y[i] = v;
        sy = fmaf(v, v, sy);
    }
    sy = block_sum(sy, scratch);
    const float scale_y = 1.0f / sqrtf(sy / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += 256) {       // a thread reads back what it wrote itself
        const TX next = from_f32<TX>(to_f32<TX>(dst[i]) + mult * (y[i] * scale_y * to_f32<W>(w[i])));
        dst[i] = next;
        if (copy != nullptr) copy[i] = from_f32<bf16>(to_f32<TX>(next));
    }
}

extern "C" int qil_rms_join(void* x, int x_dtype, const void* a, const void* wa, const void* b, const void* wb,
                            int branch_dtype, const void* w, int weight_dtype, int n_rows, int width, float eps,
                            float pre, float mult, void* rows, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || width > 40960) QIL_REFUSE("rms_join: width %d", width);
    if (b != nullptr && (wa == nullptr || wb == nullptr)) QIL_REFUSE("rms_join: two branches need a weight each");
    const size_t smem = b != nullptr ? (size_t)width * sizeof(float) : 0;
    cudaError_t err = cudaSuccess;
#define QIL_JOIN_GO(TX, TA, WT)                                                                                   \
    do {                                                                                                          \
        if (smem > 48 * 1024)                                                                                     \
            err = cudaFuncSetAttribute(rms_join_kernel<TX, TA, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (err == cudaSuccess)                                                                                   \
            qil_launch_chained(rms_join_kernel<TX, TA, WT>, dim3(n_rows), dim3(256), smem, stream, (TX*)x,        \
                               (const TA*)a, (const WT*)wa, (const TA*)b, (const WT*)wb, (const WT*)w, width, eps, \
                               pre, mult, (bf16*)rows);                                                           \
    } while (0)
#define QIL_JOIN_W(TX, TA)                                                                                        \
    do {                                                                                                          \
        if (weight_dtype == QIL_F32) QIL_JOIN_GO(TX, TA, float); else QIL_JOIN_GO(TX, TA, bf16);                  \
    } while (0)
    if (weight_dtype != QIL_F32 && weight_dtype != QIL_BF16) QIL_REFUSE("rms_join: weight dtype %d", weight_dtype);
    if (x_dtype == QIL_F32 && branch_dtype == QIL_F32) QIL_JOIN_W(float, float);
    else if (x_dtype == QIL_F32 && branch_dtype == QIL_BF16) QIL_JOIN_W(float, bf16);
    else if (x_dtype == QIL_BF16 && branch_dtype == QIL_BF16) QIL_JOIN_W(bf16, bf16);
    else if (x_dtype == QIL_BF16 && branch_dtype == QIL_F32) QIL_JOIN_W(bf16, float);
    else QIL_REFUSE("rms_join: dtypes %d += %d", x_dtype, branch_dtype);
#undef QIL_JOIN_W
#undef QIL_JOIN_GO
    if (err != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(err)); return (int)err; }
    QIL_CHECK_LAUNCH();
}

// A branch joins the stream through a norm on the branch, and the next sublayer's norm of the new stream rides along:
//   x += norm(a; w),   rows = norm(x; next_w)          (rows and next_w are optional; rows without next_w: x rounded)
// where norm is the root-mean-square norm (center 0) or the layer norm without a bias (center 1: the mean is taken
// off first, the variance is the mean of the squared deviations).  float32 arithmetic, every reduction a fixed tree
// over one row; x is the stream (float32 or bfloat16), a the branch (float32), rows what the next product reads.
template <typename TX, typename W, typename TO>
__global__ void __launch_bounds__(256)
norm_join_kernel(TX* __restrict__ x, const float* __restrict__ a, const W* __restrict__ w, int width, float eps, int center,
                 const W* __restrict__ next_w, float next_eps, int next_center, TO* __restrict__ rows) {
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const float* ra = a + (size_t)blockIdx.x * width;
    TX* dst = x + (size_t)blockIdx.x * width;
    float mean = 0.f;
    if (center) {
        float sum = 0.f;
        for (int i = threadIdx.x; i < width; i += 256) sum += ra[i];
        mean = block_sum(sum, scratch) / (float)width;
    }
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = ra[i] - mean;
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, scratch);
    const float scale = 1.0f / sqrtf(sq / (float)width + eps);
    float sum = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {       // a thread reads back below what it wrote itself
        const TX next = from_f32<TX>(to_f32<TX>(dst[i]) + (ra[i] - mean) * scale * to_f32<W>(w[i]));
        dst[i] = next;
        sum += to_f32<TX>(next);
    }
    if (rows == nullptr) return;
    TO* out = rows + (size_t)blockIdx.x * width;
    if (next_w == nullptr) {
        for (int i = threadIdx.x; i < width; i += 256) out[i] = from_f32<TO>(to_f32<TX>(dst[i]));
        return;
    }
    mean = 0.f;
    if (next_center) mean = block_sum(sum, scratch) / (float)width;
    sq = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = to_f32<TX>(dst[i]) - mean;
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, scratch);
    const float next_scale = 1.0f / sqrtf(sq / (float)width + next_eps);
    for (int i = threadIdx.x; i < width; i += 256)
        out[i] = from_f32<TO>((to_f32<TX>(dst[i]) - mean) * next_scale * to_f32<W>(next_w[i]));
}

// The same with the row held in registers (rows of up to 256 * VPT values): the branch and the stream are read once,
// every value is summed in the order the kernel above sums it, so both give the same bits.
template <typename TX, typename W, typename TO, int VPT>
__global__ void __launch_bounds__(256)
norm_join_regs_kernel(TX* __restrict__ x, const float* __restrict__ a, const W* __restrict__ w, int width, float eps, int center,
                      const W* __restrict__ next_w, float next_eps, int next_center, TO* __restrict__ rows) {
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const float* ra = a + (size_t)blockIdx.x * width;
    TX* dst = x + (size_t)blockIdx.x * width;
    float va[VPT], vx[VPT];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * 256;
        va[k] = i < width ? ra[i] : 0.f;
        if (i < width) sum += va[k];
    }
    float mean = 0.f;
    if (center) mean = block_sum(sum, scratch) / (float)width;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
        if (threadIdx.x + k * 256 < width) { const float v = va[k] - mean; sq = fmaf(v, v, sq); }
    sq = block_sum(sq, scratch);
    const float scale = 1.0f / sqrtf(sq / (float)width + eps);
    sum = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * 256;
        vx[k] = 0.f;
        if (i < width) {
            const TX next = from_f32<TX>(to_f32<TX>(dst[i]) + (va[k] - mean) * scale * to_f32<W>(w[i]));
            dst[i] = next;
            vx[k] = to_f32<TX>(next);
            sum += vx[k];
        }
    }
    if (rows == nullptr) return;
    TO* out = rows + (size_t)blockIdx.x * width;
    if (next_w == nullptr) {
#pragma unroll
        for (int k = 0; k < VPT; ++k)
            if (threadIdx.x + k * 256 < width) out[threadIdx.x + k * 256] = from_f32<TO>(vx[k]);
        return;
    }
    mean = 0.f;
    if (next_center) mean = block_sum(sum, scratch) / (float)width;
    sq = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
        if (threadIdx.x + k * 256 < width) { const float v = vx[k] - mean; sq = fmaf(v, v, sq); }
    sq = block_sum(sq, scratch);
    const float next_scale = 1.0f / sqrtf(sq / (float)width + next_eps);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < width) out[i] = from_f32<TO>((vx[k] - mean) * next_scale * to_f32<W>(next_w[i]));
    }
}

extern "C" int qil_norm_join(void* x, int x_dtype, const float* a, const void* w, int weight_dtype, int n_rows, int width,
                             float eps, int center, const void* next_w, float next_eps, int next_center, void* rows,
                             int rows_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) QIL_REFUSE("norm_join: width %d", width);
    if (next_w != nullptr && rows == nullptr) QIL_REFUSE("norm_join: the next norm needs rows to write");
#define QIL_JOIN_ARGS(TX, WT, TO)                                                                                   \
    dim3(n_rows), dim3(256), 0, stream, (TX*)x, a, (const WT*)w, width, eps, center, (const WT*)next_w, next_eps,   \
    next_center, (TO*)rows
#define QIL_JOIN_GO(TX, WT, TO)                                                                                     \
    do {                                                                                                            \
        if (width <= 1024) qil_launch_chained(norm_join_regs_kernel<TX, WT, TO, 4>, QIL_JOIN_ARGS(TX, WT, TO));     \
        else if (width <= 2048) qil_launch_chained(norm_join_regs_kernel<TX, WT, TO, 8>, QIL_JOIN_ARGS(TX, WT, TO)); \
        else if (width <= 4096) qil_launch_chained(norm_join_regs_kernel<TX, WT, TO, 16>, QIL_JOIN_ARGS(TX, WT, TO)); \
        else qil_launch_chained(norm_join_kernel<TX, WT, TO>, QIL_JOIN_ARGS(TX, WT, TO));                           \
    } while (0)
#define QIL_JOIN_O(TX, WT)                                                                                          \
    do { if (rows_dtype == QIL_F32) QIL_JOIN_GO(TX, WT, float); else QIL_JOIN_GO(TX, WT, bf16); } while (0)
#define QIL_JOIN_W(TX)                                                                                              \
    do { if (weight_dtype == QIL_F32) QIL_JOIN_O(TX, float); else QIL_JOIN_O(TX, bf16); } while (0)
    if (weight_dtype != QIL_F32 && weight_dtype != QIL_BF16) QIL_REFUSE("norm_join: weight dtype %d", weight_dtype);
    if (rows != nullptr && rows_dtype != QIL_F32 && rows_dtype != QIL_BF16) QIL_REFUSE("norm_join: rows dtype %d", rows_dtype);
    if (x_dtype == QIL_F32) QIL_JOIN_W(float);
    else if (x_dtype == QIL_BF16) QIL_JOIN_W(bf16);
    else QIL_REFUSE("norm_join: stream dtype %d", x_dtype);
#undef QIL_JOIN_W
#undef QIL_JOIN_O
#undef QIL_JOIN_GO
#undef QIL_JOIN_ARGS
    QIL_CHECK_LAUNCH();
}
