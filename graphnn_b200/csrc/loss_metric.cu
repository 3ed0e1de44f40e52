// Loss / metric tail of the reference driver's TEST loop (targets = {loss, acc},
// examples/graph_classification/include/nn_common.h:127-146): cross entropy with softmax
// against CSR labels, argmax of a CSR row, in-top-k, int -> float cast, global mean -- each as
// the single kernel behind the corresponding factor, plus one fused launch for all of it.
#include "common.cuh"

namespace
{

// -sum_k log(p[i, col_k]) * val_k with p clamped like the reference: |p| < 1e-8 -> 1e-8
// (src/nn/cross_entropy.cpp:9-24); need_softmax: p = softmax(logits row) with max subtraction
// (src/nn/cross_entropy.cpp:44-47).
__device__ __forceinline__ float row_cross_entropy(const float* x, int C, bool need_softmax, const int32_t* ci, const float* val,
                                                   int beg, int end)
{
    float mx = 0.f, denom = 1.f;
    if (need_softmax) {
        mx = x[0];
        for (int c = 1; c < C; ++c) mx = x[c] > mx ? x[c] : mx;
        denom = 0.f;
        for (int c = 0; c < C; ++c) denom += expf(x[c] - mx);
    }
    float loss = 0.f;
    for (int k = beg; k < end; ++k) {
        float t = need_softmax ? expf(x[ci[k]] - mx) / denom : x[ci[k]];
        if (fabsf(t) < 1e-8f) t = 1e-8f;
        loss -= logf(t) * (val ? val[k] : 1.0f);
    }
    return loss;
}

// column of the largest value of a CSR row, first maximum wins (src/tensor/cpu_sparse_tensor.cpp:86-103);
// an empty row gives 0 like the reference's zero-initialised output
__device__ __forceinline__ int row_argmax_csr(const int32_t* ci, const float* val, int beg, int end)
{
    int best = 0;
    float cur = 0.f;
    for (int j = beg; j < end; ++j) {
        const float v = val ? val[j] : 1.0f;
        if (j == beg || v > cur) { cur = v; best = ci[j]; }
    }
    return best;
}

// 1 if fewer than k other classes score strictly higher than the target (src/nn/in_top_k.cpp:6-23)
__device__ __forceinline__ int row_in_top_k(const float* x, int C, int target, int k)
{
    int t = 0;
    for (int j = 0; j < C; ++j)
        if (j != target && x[j] > x[target]) ++t;
    return t < k;
}

__global__ void __launch_bounds__(256) cross_entropy_kernel(int64_t G, int C, const float* __restrict__ x, int need_softmax,
                                                            const int32_t* __restrict__ rp, const int32_t* __restrict__ ci,
                                                            const float* __restrict__ val, float* __restrict__ out)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < G; i += stride)
        out[i] = row_cross_entropy(x + i * C, C, need_softmax != 0, ci, val, rp[i], rp[i + 1]);
}

__global__ void __launch_bounds__(256) argmax_csr_kernel(int64_t G, const int32_t* __restrict__ rp, const int32_t* __restrict__ ci,
                                                         const float* __restrict__ val, int32_t* __restrict__ out)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < G; i += stride)
        out[i] = row_argmax_csr(ci, val, rp[i], rp[i + 1]);
}

__global__ void __launch_bounds__(256) in_top_k_kernel(int64_t G, int C, const float* __restrict__ x,
                                                       const int32_t* __restrict__ target, int k, int32_t* __restrict__ out)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < G; i += stride) {
        const int t = target[i];
        out[i] = (t >= 0 && t < C) ? row_in_top_k(x + i * C, C, t, k) : 0;
    }
}

__global__ void __launch_bounds__(256) cast_i32_f32_kernel(int64_t n, const int32_t* __restrict__ in, float* __restrict__ out)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = (float)in[i];
}

// One block; thread t sums elements t, t+1024, ... in order, then a fixed-shape tree combines
// the 1024 partial sums: the result does not depend on scheduling.
template <typename F>
__device__ __forceinline__ float block_sum_1024(int64_t n, F value_of)
{
    __shared__ float part[1024];
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += 1024) s += value_of(i);
    part[threadIdx.x] = s;
    __syncthreads();
    for (int w = 512; w > 0; w >>= 1) {
        if ((int)threadIdx.x < w) part[threadIdx.x] += part[threadIdx.x + w];
        __syncthreads();
    }
    const float r = part[0];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(1024) mean_kernel(int64_t n, const float* __restrict__ in, float* __restrict__ out)
{
    const float s = block_sum_1024(n, [&](int64_t i) { return in[i]; });
    if (threadIdx.x == 0) out[0] = s / (float)n;
}

__global__ void __launch_bounds__(1024) loss_acc_kernel(int64_t G, int C, const float* __restrict__ logits,
                                                        const int32_t* __restrict__ rp, const int32_t* __restrict__ ci,
                                                        const float* __restrict__ val, int topk, float* __restrict__ loss_mean,
                                                        float* __restrict__ acc_mean, float* __restrict__ per_graph_loss)
{
    const float ls = block_sum_1024(G, [&](int64_t i) {
        const float l = row_cross_entropy(logits + i * C, C, true, ci, val, rp[i], rp[i + 1]);
        if (per_graph_loss) per_graph_loss[i] = l;
        return l;
    });
    const float as = block_sum_1024(G, [&](int64_t i) {
        const int t = row_argmax_csr(ci, val, rp[i], rp[i + 1]);
        return (float)((t >= 0 && t < C) ? row_in_top_k(logits + i * C, C, t, topk) : 0);
    });
    if (threadIdx.x == 0) {
        if (loss_mean) loss_mean[0] = ls / (float)G;
        if (acc_mean) acc_mean[0] = as / (float)G;
    }
}

inline unsigned lm_grid(s2v_ctx* ctx, int64_t n)
{
    int64_t b = (n + 255) / 256;
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    if (b > cap) b = cap;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace

extern "C" {

int s2v_cross_entropy_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, int cols, const float* pred, int need_softmax,
                          const int32_t* label_row_ptr, const int32_t* label_col_idx, const float* label_val, float* out)
{
    S2V_ENTER(ctx);
    if (rows < 0 || cols <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "cross_entropy: bad shape");
    if (rows == 0) return S2V_OK;
    if (!pred || !label_row_ptr || !label_col_idx || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "cross_entropy: NULL pointer");
    cross_entropy_kernel<<<lm_grid(ctx, rows), 256, 0, s2v_pick_stream(ctx, stream)>>>(rows, cols, pred, need_softmax, label_row_ptr,
                                                                                        label_col_idx, label_val, out);
    S2V_CHECK_LAUNCH(ctx, "cross_entropy_kernel");
    return S2V_OK;
}

int s2v_argmax_csr_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, const int32_t* row_ptr, const int32_t* col_idx,
                       const float* val, int32_t* out)
{
    S2V_ENTER(ctx);
    if (rows < 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "argmax_csr: bad shape");
    if (rows == 0) return S2V_OK;
    if (!row_ptr || !col_idx || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "argmax_csr: NULL pointer");
    argmax_csr_kernel<<<lm_grid(ctx, rows), 256, 0, s2v_pick_stream(ctx, stream)>>>(rows, row_ptr, col_idx, val, out);
    S2V_CHECK_LAUNCH(ctx, "argmax_csr_kernel");
    return S2V_OK;
}

int s2v_in_top_k_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, int cols, const float* pred, const int32_t* target, int k,
                     int32_t* out)
{
    S2V_ENTER(ctx);
    if (rows < 0 || cols <= 0 || k < 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "in_top_k: bad shape");
    if (rows == 0) return S2V_OK;
    if (!pred || !target || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "in_top_k: NULL pointer");
    in_top_k_kernel<<<lm_grid(ctx, rows), 256, 0, s2v_pick_stream(ctx, stream)>>>(rows, cols, pred, target, k, out);
    S2V_CHECK_LAUNCH(ctx, "in_top_k_kernel");
    return S2V_OK;
}

int s2v_cast_i32_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, const int32_t* in, float* out)
{
    S2V_ENTER(ctx);
    if (count < 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "cast: bad size");
    if (count == 0) return S2V_OK;
    if (!in || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "cast: NULL pointer");
    cast_i32_f32_kernel<<<lm_grid(ctx, count), 256, 0, s2v_pick_stream(ctx, stream)>>>(count, in, out);
    S2V_CHECK_LAUNCH(ctx, "cast_i32_f32_kernel");
    return S2V_OK;
}

int s2v_mean_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, const float* in, float* out)
{
    S2V_ENTER(ctx);
    if (count <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "mean: needs at least one element");
    if (!in || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "mean: NULL pointer");
    mean_kernel<<<1, 1024, 0, s2v_pick_stream(ctx, stream)>>>(count, in, out);
    S2V_CHECK_LAUNCH(ctx, "mean_kernel");
    return S2V_OK;
}

int s2v_loss_acc_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int num_class, const float* logits,
                     const int32_t* label_row_ptr, const int32_t* label_col_idx, const float* label_val, int topk,
                     float* loss_mean, float* acc_mean, float* per_graph_loss)
{
    S2V_ENTER(ctx);
    if (num_graphs <= 0 || num_class <= 0 || topk < 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "loss_acc: bad shape");
    if (!logits || !label_row_ptr || !label_col_idx || (!loss_mean && !acc_mean))
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "loss_acc: NULL pointer");
    loss_acc_kernel<<<1, 1024, 0, s2v_pick_stream(ctx, stream)>>>(num_graphs, num_class, logits, label_row_ptr, label_col_idx,
                                                                   label_val, topk, loss_mean, acc_mean, per_graph_loss);
    S2V_CHECK_LAUNCH(ctx, "loss_acc_kernel");
    return S2V_OK;
}

}  // extern "C"
