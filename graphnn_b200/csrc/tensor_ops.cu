// Unfused tensor operations of the reference's DTensor<GPU,float> surface, one kernel
// each: CSR x dense, dense x dense, axpy, scale, ReLU, row softmax, row argmax.
// They back the MatMul / ElewiseAdd / ReLU / Softmax / ArgMax factors when the
// driver's original (unfused) wiring is run; the fused kernels live in level.cu and
// pool_readout.cu.
#include "common.cuh"

namespace
{

// ---------------------------------------------------------------- CSR x dense
// C[m x n] = alpha * A * B + beta * C.  One warp per row, lanes stride the n columns
// (float4 when n % 4 == 0), neighbours summed in CSR order.  Replaces CSRMMKernel
// (src/tensor/gpu_dense_tensor.cu:227-271), which used one thread per output element
// with a global read-modify-write per non-zero.
template <bool VEC4>
__global__ void __launch_bounds__(256) spmm_csr_kernel(int64_t m, int n, const int32_t* __restrict__ row_ptr,
                                                        const int32_t* __restrict__ col_idx,
                                                        const float* __restrict__ val, const float* __restrict__ B,
                                                        float alpha, float beta, float* __restrict__ C)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < m; row += warps) {
        const int beg = row_ptr[row], end = row_ptr[row + 1];
        if (VEC4) {
            const int n4 = n >> 2;
            for (int c = lane; c < n4; c += 32) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                int t = beg;
                for (; t + 4 <= end; t += 4) {
                    float4 v[4];
                    float a[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        v[u] = __ldg(reinterpret_cast<const float4*>(B) + (int64_t)col_idx[t + u] * n4 + c);
                        a[u] = val ? val[t + u] : 1.0f;
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        acc.x = fmaf(a[u], v[u].x, acc.x); acc.y = fmaf(a[u], v[u].y, acc.y);
                        acc.z = fmaf(a[u], v[u].z, acc.z); acc.w = fmaf(a[u], v[u].w, acc.w);
                    }
                }
                for (; t < end; ++t) {
                    const float4 v = __ldg(reinterpret_cast<const float4*>(B) + (int64_t)col_idx[t] * n4 + c);
                    const float a = val ? val[t] : 1.0f;
                    acc.x = fmaf(a, v.x, acc.x); acc.y = fmaf(a, v.y, acc.y);
                    acc.z = fmaf(a, v.z, acc.z); acc.w = fmaf(a, v.w, acc.w);
                }
                float4* cp = reinterpret_cast<float4*>(C) + row * n4 + c;
                float4 r = make_float4(alpha * acc.x, alpha * acc.y, alpha * acc.z, alpha * acc.w);
                if (beta != 0.f) {
                    const float4 old = *cp;
                    r.x += beta * old.x; r.y += beta * old.y; r.z += beta * old.z; r.w += beta * old.w;
                }
                *cp = r;
            }
        } else {
            for (int c = lane; c < n; c += 32) {
                float acc = 0.f;
                for (int t = beg; t < end; ++t)
                    acc = fmaf(val ? val[t] : 1.0f, __ldg(B + (int64_t)col_idx[t] * n + c), acc);
                float r = alpha * acc;
                if (beta != 0.f) r += beta * C[row * n + c];
                C[row * n + c] = r;
            }
        }
    }
}

// ---------------------------------------------------------------- dense x dense
// Row-major C = alpha*op(A)*op(B) + beta*C, 64x64 tile per CTA, 16-wide k panels in
// shared memory, 4x4 outputs per thread, k ascending.  Stands in for cublasSgemm
// (src/tensor/gpu_dense_tensor.cu:193-224) for the small products of this path
// (X*W_in, Y*W1, .*W2).
constexpr int GT = 64, GK = 16;
__global__ void __launch_bounds__(256) gemm_kernel(int ta, int tb, int64_t m, int64_t n, int64_t k, float alpha,
                                                   const float* __restrict__ A, int64_t lda,
                                                   const float* __restrict__ B, int64_t ldb, float beta,
                                                   float* __restrict__ C, int64_t ldc)
{
    __shared__ float As[GK][GT + 1];
    __shared__ float Bs[GK][GT + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t row0 = (int64_t)blockIdx.y * GT, col0 = (int64_t)blockIdx.x * GT;
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < k; k0 += GK) {
        for (int e = threadIdx.x; e < GT * GK; e += 256) {
            int r, kk;
            if (!ta) { r = e / GK; kk = e % GK; } else { kk = e / GT; r = e % GT; }  // contiguous along the stored minor axis
            const int64_t gr = row0 + r, gk = k0 + kk;
            As[kk][r] = (gr < m && gk < k) ? (ta ? A[gk * lda + gr] : A[gr * lda + gk]) : 0.f;
        }
        for (int e = threadIdx.x; e < GT * GK; e += 256) {
            int c, kk;
            if (!tb) { kk = e / GT; c = e % GT; } else { c = e / GK; kk = e % GK; }
            const int64_t gc = col0 + c, gk = k0 + kk;
            Bs[kk][c] = (gc < n && gk < k) ? (tb ? B[gc * ldb + gk] : B[gk * ldb + gc]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = row0 + ty + 16 * i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = col0 + tx + 16 * j;
            if (c >= n) continue;
            float v = alpha * acc[i][j];
            if (beta != 0.f) v += beta * C[r * ldc + c];
            C[r * ldc + c] = v;
        }
    }
}

// ---------------------------------------------------------------- element-wise
__global__ void __launch_bounds__(256) axpy_kernel(int64_t n, float a, const float* __restrict__ x, float* __restrict__ y)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = fmaf(a, x[i], y[i]);
}
__global__ void __launch_bounds__(256) scale_kernel(int64_t n, float a, float* __restrict__ x)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] = a == 0.f ? 0.f : a * x[i];
}
__global__ void __launch_bounds__(256) relu_kernel(int64_t n, const float* in, float* out)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = relu_ref(in[i]);
}

// ---------------------------------------------------------------- row softmax / argmax
// One warp per row.  Softmax: max-subtract, exp, divide by the sum of exponentials
// (src/tensor/cpu_dense_tensor.cpp:228-251).  ArgMax: first maximum wins
// (include/tensor/gpu_reduce_kernel.h:12-33).
__global__ void __launch_bounds__(256) softmax_kernel(int64_t rows, int cols, const float* in, float* out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const float* x = in + r * cols;
        float* y = out + r * cols;
        float mx = -INFINITY;
        for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, x[c]);
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float s = 0.f;
        for (int c = lane; c < cols; c += 32) {
            const float e = expf(x[c] - mx);
            y[c] = e;
            s += e;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        for (int c = lane; c < cols; c += 32) y[c] = y[c] / s;
    }
}

__global__ void __launch_bounds__(256) argmax_kernel(int64_t rows, int cols, const float* __restrict__ in,
                                                     int32_t* __restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const float* x = in + r * cols;
        float best = 0.f;
        int bi = INT_MAX;  // lanes with no element never win
        for (int c = lane; c < cols; c += 32) {
            const float v = x[c];
            if (bi == INT_MAX || v > best) { best = v; bi = c; }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != INT_MAX && (bi == INT_MAX || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
        }
        if (lane == 0) out[r] = bi;
    }
}

inline unsigned grid_for(s2v_ctx* ctx, int64_t work_items, int per_block)
{
    int64_t b = (work_items + per_block - 1) / per_block;
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    if (b > cap) b = cap;
    return (unsigned)(b < 1 ? 1 : b);
}

// Any index outside [0, limit) records S2V_ERR_INVALID_ARG (site 3) in the status word.  Run beside the level kernels,
// which only clamp the indices they use.
__global__ void __launch_bounds__(256) index_range_check_kernel(int64_t n, const int32_t* __restrict__ idx, int limit,
                                                                s2v_device_status* status)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) bad |= (unsigned)idx[i] >= (unsigned)limit;
    if (bad) {
        status->code = S2V_ERR_INVALID_ARG;
        status->where = 3;
    }
}

}  // namespace

extern "C" {

int s2v_spmm_csr_f32(s2v_ctx* ctx, s2v_stream stream, int64_t m, int64_t k, int n, const int32_t* row_ptr,
                     const int32_t* col_idx, const float* val, const float* B, float alpha, float beta, float* C)
{
    S2V_ENTER(ctx);
    if (m < 0 || k < 0 || n <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "spmm: negative size");
    if (m == 0) return S2V_OK;
    if (!row_ptr || !B || !C) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "spmm: NULL pointer");
    cudaStream_t st = s2v_pick_stream(ctx, stream);
    const bool vec = (n % 4 == 0) && s2v_aligned16(B) && s2v_aligned16(C);
    const unsigned grid = grid_for(ctx, m, 8);
    if (vec)
        spmm_csr_kernel<true><<<grid, 256, 0, st>>>(m, n, row_ptr, col_idx, val, B, alpha, beta, C);
    else
        spmm_csr_kernel<false><<<grid, 256, 0, st>>>(m, n, row_ptr, col_idx, val, B, alpha, beta, C);
    S2V_CHECK_LAUNCH(ctx, "spmm_csr_kernel");
    return S2V_OK;
}

int s2v_gemm_f32(s2v_ctx* ctx, s2v_stream stream, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k,
                 float alpha, const float* A, int64_t lda, const float* B, int64_t ldb, float beta, float* C,
                 int64_t ldc)
{
    S2V_ENTER(ctx);
    if (m < 0 || n < 0 || k < 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "gemm: negative size");
    if (m == 0 || n == 0) return S2V_OK;
    if (!C || (k > 0 && (!A || !B))) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "gemm: NULL pointer");
    const int64_t gy = (m + GT - 1) / GT, gx = (n + GT - 1) / GT;
    if (gy > 65535) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "gemm: m beyond 65535*64 rows; use the fused kernels");
    gemm_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, s2v_pick_stream(ctx, stream)>>>(
        trans_a, trans_b, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
    S2V_CHECK_LAUNCH(ctx, "gemm_kernel");
    return S2V_OK;
}

int s2v_axpy_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, float a, const float* x, float* y)
{
    S2V_ENTER(ctx);
    if (count < 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "axpy: negative size");
    if (count == 0) return S2V_OK;
    if (!x || !y) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "axpy: NULL pointer");
    axpy_kernel<<<grid_for(ctx, count, 1024), 256, 0, s2v_pick_stream(ctx, stream)>>>(count, a, x, y);
    S2V_CHECK_LAUNCH(ctx, "axpy_kernel");
    return S2V_OK;
}

int s2v_scale_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, float a, float* x)
{
    S2V_ENTER(ctx);
    if (count < 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "scale: negative size");
    if (count == 0) return S2V_OK;
    if (!x) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "scale: NULL pointer");
    scale_kernel<<<grid_for(ctx, count, 1024), 256, 0, s2v_pick_stream(ctx, stream)>>>(count, a, x);
    S2V_CHECK_LAUNCH(ctx, "scale_kernel");
    return S2V_OK;
}

int s2v_relu_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, const float* in, float* out)
{
    S2V_ENTER(ctx);
    if (count < 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "relu: negative size");
    if (count == 0) return S2V_OK;
    if (!in || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "relu: NULL pointer");
    relu_kernel<<<grid_for(ctx, count, 1024), 256, 0, s2v_pick_stream(ctx, stream)>>>(count, in, out);
    S2V_CHECK_LAUNCH(ctx, "relu_kernel");
    return S2V_OK;
}

int s2v_softmax_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, int cols, const float* in, float* out)
{
    S2V_ENTER(ctx);
    if (rows < 0 || cols <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "softmax: bad shape");
    if (rows == 0) return S2V_OK;
    if (!in || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "softmax: NULL pointer");
    softmax_kernel<<<grid_for(ctx, rows, 8), 256, 0, s2v_pick_stream(ctx, stream)>>>(rows, cols, in, out);
    S2V_CHECK_LAUNCH(ctx, "softmax_kernel");
    return S2V_OK;
}

int s2v_argmax_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, int cols, const float* in, int32_t* out)
{
    S2V_ENTER(ctx);
    if (rows < 0 || cols <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "argmax: bad shape");
    if (rows == 0) return S2V_OK;
    if (!in || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "argmax: NULL pointer");
    argmax_kernel<<<grid_for(ctx, rows, 8), 256, 0, s2v_pick_stream(ctx, stream)>>>(rows, cols, in, out);
    S2V_CHECK_LAUNCH(ctx, "argmax_kernel");
    return S2V_OK;
}

}  // extern "C"

int s2v_launch_index_check(s2v_ctx* ctx, cudaStream_t st, int64_t n, const int32_t* idx, int limit)
{
    if (n <= 0) return S2V_OK;
    int64_t blocks = (n + 2047) / 2048;
    if (blocks > (int64_t)ctx->sm_count * 4) blocks = (int64_t)ctx->sm_count * 4;
    index_range_check_kernel<<<(unsigned)blocks, 256, 0, st>>>(n, idx, limit, ctx->dstatus_dev);
    S2V_CHECK_LAUNCH(ctx, "index_range_check_kernel");
    return S2V_OK;
}
