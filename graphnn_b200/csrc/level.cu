// Fused structure2vec message-passing level for sm_100a:
//
//     out[i,:] = ReLU( (sum_{t in row i} val[t] * H[col_idx[t],:]) * W + X[i,:] )
//
// One kernel replaces the reference's CSRMMKernel + cublasSgemm + D2D copy + saxpy +
// D2D copy + ReLU kernel (src/tensor/gpu_dense_tensor.cu:209-271,
// src/nn/elewise_add.cpp:12-33, src/nn/relu.cu:8-13): every output row is written
// once and no intermediate [N x d] matrix touches HBM.
//
// Shape of the kernel (HBM-bound gather + small dense product):
//   * persistent CTAs, grid = #SMs x resident CTAs; W [d x d] is staged once per CTA
//     into shared memory with one bulk-async (TMA) copy completing on an mbarrier;
//   * each WARP owns tiles of TILE_R = 16 consecutive rows and runs on its own, with
//     only __syncwarp between phases, so warps of one SM sit in different phases and
//     the gather of one overlaps the FMAs of another:
//       1. the tile's row offsets and column indices are fetched coalesced into a
//          per-warp shared buffer (removes one dependent-load level from the gather),
//       2. gather: d/4 lanes per row, float4 loads of neighbour rows, U loads in
//          flight per lane, fp32 accumulation in CSR order,
//       3. the 16 x d tile of sums goes to shared memory and the warp multiplies it by
//          W from shared memory (4 rows x d/8 columns per lane, k ascending),
//       4. epilogue adds X (streamed, or looked up in a small table), applies ReLU and
//          stores 128 contiguous bytes per row per instruction.
#include "common.cuh"

namespace
{

constexpr int TILE_R = 16;     // rows per warp tile
constexpr int IDX_CAP = 256;   // column indices of one tile kept in shared memory
constexpr int WAIT_LIMIT = 1 << 22;

template <int D>
struct LevelCfg;
template <>
struct LevelCfg<32> {
    static constexpr int WARPS = 8, MIN_BLOCKS = 4, U = 8;
};
template <>
struct LevelCfg<64> {
    static constexpr int WARPS = 8, MIN_BLOCKS = 3, U = 8;
};
template <>
struct LevelCfg<128> {
    static constexpr int WARPS = 12, MIN_BLOCKS = 1, U = 4;
};

template <int D>
struct LevelSmem {
    static constexpr int S_STRIDE = D + 4;
    static constexpr size_t W_BYTES = sizeof(float) * D * D;
    static constexpr size_t WARP_BYTES = sizeof(float) * TILE_R * S_STRIDE + sizeof(int) * IDX_CAP + sizeof(float) * IDX_CAP;
    static constexpr size_t total(int warps) { return W_BYTES + 16 + WARP_BYTES * warps; }
};

__device__ __forceinline__ float f4_get(const float4& v, int i)
{
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// --- mbarrier + bulk-async copy (TMA, non-tensor form) ---------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int D, typename RpT, bool HAS_VAL, int XMODE /*0 none, 1 dense, 2 table lookup*/>
__global__ void __launch_bounds__(LevelCfg<D>::WARPS * 32, LevelCfg<D>::MIN_BLOCKS)
s2v_level_kernel(int64_t n_rows, int64_t num_tiles, const RpT* __restrict__ row_ptr,
                 const int32_t* __restrict__ col_idx, const float* __restrict__ val, const float* __restrict__ H,
                 const float* __restrict__ W, const float* __restrict__ X, const int32_t* __restrict__ x_index,
                 float* __restrict__ out, s2v_device_status* status)
{
    constexpr int WARPS = LevelCfg<D>::WARPS;
    constexpr int U = LevelCfg<D>::U;
    constexpr int LPR = D / 4;          // lanes that cover one row with float4
    constexpr int RPP = 32 / LPR;       // rows gathered side by side per pass
    constexpr int NPASS = TILE_R / RPP;
    constexpr int S_STRIDE = LevelSmem<D>::S_STRIDE;
    constexpr int RI = TILE_R / 4;      // rows per lane in the dense phase
    constexpr int NJ = D / 32;          // float4 column chunks per lane

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* Ws = reinterpret_cast<float*>(smem_raw);
    uint64_t* mbar = reinterpret_cast<uint64_t*>(smem_raw + LevelSmem<D>::W_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* wbase = smem_raw + LevelSmem<D>::W_BYTES + 16 + LevelSmem<D>::WARP_BYTES * warp;
    float* S = reinterpret_cast<float*>(wbase);
    int* idx_s = reinterpret_cast<int*>(wbase + sizeof(float) * TILE_R * S_STRIDE);
    float* val_s = reinterpret_cast<float*>(idx_s + IDX_CAP);

    // ---- stage W: one bulk-async copy per CTA, completion on an mbarrier
    const uint32_t bar = smem_u32(mbar);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(bar, (uint32_t)LevelSmem<D>::W_BYTES);
        bulk_copy_g2s(smem_u32(Ws), W, (uint32_t)LevelSmem<D>::W_BYTES, bar);
    }
    __syncthreads();  // barrier initialised before anyone polls it
    {
        int spins = 0;
        while (!mbar_try_wait(bar, 0)) {
            if (++spins > WAIT_LIMIT) {  // bounded: report and leave instead of hanging the GPU
                if (lane == 0) {
                    status->code = S2V_ERR_DEVICE_TIMEOUT;
                    status->where = 1;
                }
                int again = 0;
                while (!mbar_try_wait(bar, 0) && ++again < WAIT_LIMIT) {}
                return;
            }
        }
    }

    const float4* __restrict__ H4 = reinterpret_cast<const float4*>(H);
    const int sub = lane / LPR, sl = lane % LPR;
    const int rg = lane >> 3, cg = lane & 7;

    for (int64_t tile = (int64_t)blockIdx.x * WARPS + warp; tile < num_tiles; tile += (int64_t)gridDim.x * WARPS) {
        const int64_t r0 = tile * TILE_R;
        // ---- 1. row offsets (lane l holds row_ptr[r0 + l], clamped) and the tile's indices
        int64_t rpi = r0 + lane;
        if (rpi > n_rows) rpi = n_rows;
        const RpT rp_abs = lane <= TILE_R ? row_ptr[rpi] : (RpT)0;
        const RpT base = __shfl_sync(0xffffffffu, rp_abs, 0);
        const int rp_rel = (int)(rp_abs - base);
        const int tile_nnz = __shfl_sync(0xffffffffu, rp_rel, TILE_R);
        const bool fits = tile_nnz <= IDX_CAP;
        const int* ip;
        const float* vp;
        if (fits) {
            for (int t = lane; t < tile_nnz; t += 32) {
                idx_s[t] = col_idx[base + t];
                if (HAS_VAL) val_s[t] = val[base + t];
            }
            ip = idx_s;
            vp = val_s;
        } else {
            ip = col_idx + base;
            vp = HAS_VAL ? val + base : nullptr;
        }
        __syncwarp();

        // ---- 2. gather + sum in CSR order
#pragma unroll 1
        for (int p = 0; p < NPASS; ++p) {
            const int lr = p * RPP + sub;
            const int beg = __shfl_sync(0xffffffffu, rp_rel, lr);
            const int end = __shfl_sync(0xffffffffu, rp_rel, lr + 1);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            int t = beg;
            for (; t + U <= end; t += U) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) v[u] = ld_nc_f4(H4 + (int64_t)ip[t + u] * LPR + sl);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (HAS_VAL) {
                        const float a = vp[t + u];
                        acc.x = fmaf(a, v[u].x, acc.x); acc.y = fmaf(a, v[u].y, acc.y);
                        acc.z = fmaf(a, v[u].z, acc.z); acc.w = fmaf(a, v[u].w, acc.w);
                    } else {
                        acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;
                    }
                }
            }
            if (t < end) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    v[u] = (t + u < end) ? ld_nc_f4(H4 + (int64_t)ip[t + u] * LPR + sl) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (t + u < end) {
                        if (HAS_VAL) {
                            const float a = vp[t + u];
                            acc.x = fmaf(a, v[u].x, acc.x); acc.y = fmaf(a, v[u].y, acc.y);
                            acc.z = fmaf(a, v[u].z, acc.z); acc.w = fmaf(a, v[u].w, acc.w);
                        } else {
                            acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;
                        }
                    }
                }
            }
            *reinterpret_cast<float4*>(S + lr * S_STRIDE + sl * 4) = acc;
        }
        __syncwarp();

        // ---- 3. [16 x D] * W[D x D]; lane (rg, cg) owns rows rg+4i and columns cg*4+32j..+3
        float o[RI][NJ * 4];
#pragma unroll
        for (int i = 0; i < RI; ++i)
#pragma unroll
            for (int c = 0; c < NJ * 4; ++c) o[i][c] = 0.f;
#pragma unroll 2
        for (int k = 0; k < D; k += 4) {
            float4 s[RI];
#pragma unroll
            for (int i = 0; i < RI; ++i) s[i] = *reinterpret_cast<const float4*>(S + (rg + 4 * i) * S_STRIDE + k);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                float4 w[NJ];
#pragma unroll
                for (int j = 0; j < NJ; ++j) w[j] = *reinterpret_cast<const float4*>(Ws + (k + kk) * D + cg * 4 + 32 * j);
#pragma unroll
                for (int i = 0; i < RI; ++i) {
                    const float sv = f4_get(s[i], kk);
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        o[i][4 * j + 0] = fmaf(sv, w[j].x, o[i][4 * j + 0]);
                        o[i][4 * j + 1] = fmaf(sv, w[j].y, o[i][4 * j + 1]);
                        o[i][4 * j + 2] = fmaf(sv, w[j].z, o[i][4 * j + 2]);
                        o[i][4 * j + 3] = fmaf(sv, w[j].w, o[i][4 * j + 3]);
                    }
                }
            }
        }

        // ---- 4. + X, ReLU, store
#pragma unroll
        for (int i = 0; i < RI; ++i) {
            const int64_t row = r0 + rg + 4 * i;
            if (row < n_rows) {
                const float4* xrow = nullptr;
                if (XMODE == 1) xrow = reinterpret_cast<const float4*>(X) + row * LPR;
                if (XMODE == 2) xrow = reinterpret_cast<const float4*>(X) + (int64_t)__ldg(x_index + row) * LPR;
                float4* orow = reinterpret_cast<float4*>(out) + row * LPR;
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (XMODE == 1) x = ld_stream_f4(xrow + cg + 8 * j);
                    if (XMODE == 2) x = ld_nc_f4(xrow + cg + 8 * j);
                    float4 r;
                    r.x = relu_ref(o[i][4 * j + 0] + x.x);
                    r.y = relu_ref(o[i][4 * j + 1] + x.y);
                    r.z = relu_ref(o[i][4 * j + 2] + x.z);
                    r.w = relu_ref(o[i][4 * j + 3] + x.w);
                    orow[cg + 8 * j] = r;
                }
            }
        }
        __syncwarp();  // S and idx_s are rewritten by the next tile
    }
}

template <int D, typename RpT, bool HAS_VAL, int XMODE>
int launch_one(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, const RpT* row_ptr, const int32_t* col_idx,
               const float* val, const float* H, const float* W, const float* X, const int32_t* x_index, float* out)
{
    constexpr int WARPS = LevelCfg<D>::WARPS;
    auto kern = s2v_level_kernel<D, RpT, HAS_VAL, XMODE>;
    const size_t smem = LevelSmem<D>::total(WARPS);
    // Opt-in shared memory size: a per-function attribute, cheap to set on every call.
    S2V_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int resident = 0;
    S2V_CUDA_OK(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, WARPS * 32, smem));
    if (resident < 1) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "level kernel does not fit on this device");
    const int64_t num_tiles = (n_rows + TILE_R - 1) / TILE_R;
    int64_t blocks = (num_tiles + WARPS - 1) / WARPS;
    const int64_t persistent = (int64_t)ctx->sm_count * resident;
    if (blocks > persistent) blocks = persistent;
    if (blocks < 1) blocks = 1;
    kern<<<(unsigned)blocks, WARPS * 32, smem, st>>>(n_rows, num_tiles, row_ptr, col_idx, val, H, W, X, x_index, out,
                                                      ctx->dstatus_dev);
    S2V_CHECK_LAUNCH(ctx, "s2v_level_kernel");
    return S2V_OK;
}

template <int D, typename RpT>
int launch_d(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, const RpT* rp, const int32_t* ci, const float* val,
             const float* H, const float* W, const float* X, const float* table, const int32_t* x_index, float* out)
{
    const int xmode = table ? 2 : (X ? 1 : 0);
    const float* xa = table ? table : X;
#define S2V_LVL(HV, XM) return launch_one<D, RpT, HV, XM>(ctx, st, n_rows, rp, ci, val, H, W, xa, x_index, out)
    if (val) {
        if (xmode == 0) S2V_LVL(true, 0);
        if (xmode == 1) S2V_LVL(true, 1);
        S2V_LVL(true, 2);
    }
    if (xmode == 0) S2V_LVL(false, 0);
    if (xmode == 1) S2V_LVL(false, 1);
    S2V_LVL(false, 2);
#undef S2V_LVL
}

}  // namespace

int s2v_launch_level(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, int64_t n_src, int d, const void* row_ptr,
                     bool rp64, const int32_t* col_idx, const float* val, const float* H, const float* W,
                     const float* X, const float* table, const int32_t* x_index, float* out)
{
    (void)n_src;
    if (n_rows == 0) return S2V_OK;
#define S2V_D(DD)                                                                                                  \
    case DD:                                                                                                       \
        return rp64 ? launch_d<DD, int64_t>(ctx, st, n_rows, (const int64_t*)row_ptr, col_idx, val, H, W, X, table, \
                                            x_index, out)                                                          \
                    : launch_d<DD, int32_t>(ctx, st, n_rows, (const int32_t*)row_ptr, col_idx, val, H, W, X, table, \
                                            x_index, out)
    switch (d) {
        S2V_D(32);
        S2V_D(64);
        S2V_D(128);
        default:
            return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "fused level kernel supports d in {32, 64, 128}");
    }
#undef S2V_D
}
