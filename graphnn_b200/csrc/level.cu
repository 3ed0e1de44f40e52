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
//     into shared memory by bulk-async (TMA) row copies completing on one mbarrier,
//     into rows padded by 8 floats so that tensor-core B fragments load conflict-free;
//   * each WARP owns tiles of TILE_R = 16 consecutive rows and runs on its own, with
//     only __syncwarp between phases, so warps of one SM sit in different phases and
//     the gather of one overlaps the matrix product of another:
//       1. the tile's row offsets and column indices are fetched coalesced into a
//          per-warp shared buffer (removes one dependent-load level from the gather),
//       2. gather: d/4 lanes per row, float4 loads of neighbour rows; each lane group
//          walks the non-zeros of its rows as one stream so that U loads are in flight
//          per lane whatever the row lengths; fp32 accumulation in CSR order,
//       3. the 16 x d tile of sums goes to shared memory and is multiplied by W on the
//          tensor cores as 3xTF32 (m16n8k8 MMA; every operand split into a TF32 head
//          and a TF32 tail, the three significant partial products accumulated in
//          fp32), which keeps the result within fp32 rounding of an FFMA product.
//          The plain-FFMA form of this stage saturated the FMA pipe (47 % of its peak
//          at 10 % DRAM utilisation for d = 128), which is what moved it here;
//       4. the product goes back through the same shared tile so that the epilogue
//          (add X -- streamed, or looked up in a small table --, ReLU, store) touches
//          global memory in whole 128..512-byte rows.
#include "common.cuh"
#include "mma_tf32.cuh"

namespace
{

constexpr int TILE_R = 16;     // rows per warp tile
constexpr int IDX_CAP = 256;   // column indices of one tile kept in shared memory
constexpr int WAIT_LIMIT = 1 << 22;

template <int D>
struct LevelCfg;
template <>
struct LevelCfg<32> {
    static constexpr int WARPS = 8, MIN_BLOCKS = 3, U = 8;
    static constexpr bool FLAT = false;
};
template <>
struct LevelCfg<64> {
    static constexpr int WARPS = 8, MIN_BLOCKS = 3, U = 8;
    static constexpr bool FLAT = false;   // measured: per-row passes are faster at degree ~8, d = 64
};
template <>
struct LevelCfg<128> {
    static constexpr int WARPS = 12, MIN_BLOCKS = 1, U = 8;
    static constexpr bool FLAT = true;    // measured: the flat stream is faster at degree ~2, d = 128
};

template <int D>
struct LevelSmem {
    static constexpr int S_STRIDE = D + 4;   // A fragments (rows g, g+8; cols tig, tig+4) hit 32 distinct banks
    static constexpr int W_STRIDE = D + 8;   // B fragments (rows tig, tig+4; col g) hit 32 distinct banks
    static constexpr size_t W_BYTES = sizeof(float) * D * W_STRIDE;
    static constexpr size_t WARP_BYTES = sizeof(float) * TILE_R * S_STRIDE + sizeof(int) * IDX_CAP + sizeof(float) * IDX_CAP + sizeof(int) * 32;
    static constexpr size_t total(int warps) { return W_BYTES + 16 + WARP_BYTES * warps; }
};

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
                 int n_table, float* __restrict__ out, s2v_device_status* status)
{
    constexpr int WARPS = LevelCfg<D>::WARPS;
    constexpr int U = LevelCfg<D>::U;
    constexpr int LPR = D / 4;          // lanes that cover one row with float4
    constexpr int RPP = 32 / LPR;       // rows gathered side by side per pass
    constexpr int NPASS = TILE_R / RPP;
    constexpr int RPS = TILE_R / RPP;   // rows per lane group in the gather
    constexpr int S_STRIDE = LevelSmem<D>::S_STRIDE;
    constexpr int W_STRIDE = LevelSmem<D>::W_STRIDE;
    constexpr int NT = D / 8;           // 8-column MMA tiles across the output row

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* Ws = reinterpret_cast<float*>(smem_raw);
    uint64_t* mbar = reinterpret_cast<uint64_t*>(smem_raw + LevelSmem<D>::W_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* wbase = smem_raw + LevelSmem<D>::W_BYTES + 16 + LevelSmem<D>::WARP_BYTES * warp;
    float* S = reinterpret_cast<float*>(wbase);
    int* idx_s = reinterpret_cast<int*>(wbase + sizeof(float) * TILE_R * S_STRIDE);
    float* val_s = reinterpret_cast<float*>(idx_s + IDX_CAP);
    int* rp_s = reinterpret_cast<int*>(val_s + IDX_CAP);   // the tile's 17 relative row offsets

    // ---- stage W: one bulk-async copy per CTA, completion on an mbarrier
    const uint32_t bar = smem_u32(mbar);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(bar, (uint32_t)(sizeof(float) * D * D));
        for (int k = 0; k < D; ++k)  // one bulk copy per row of W, into the padded layout
            bulk_copy_g2s(smem_u32(Ws + k * W_STRIDE), W + k * D, (uint32_t)(sizeof(float) * D), bar);
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
    const int g = lane >> 2, tig = lane & 3;   // MMA fragment coordinates

    for (int64_t tile = (int64_t)blockIdx.x * WARPS + warp; tile < num_tiles; tile += (int64_t)gridDim.x * WARPS) {
        const int64_t r0 = tile * TILE_R;
        // ---- 1. row offsets (relative to the tile's first non-zero) and the tile's indices
        int64_t rpi = r0 + lane;
        if (rpi > n_rows) rpi = n_rows;
        const RpT rp_abs = lane <= TILE_R ? row_ptr[rpi] : (RpT)0;
        const RpT base = __shfl_sync(0xffffffffu, rp_abs, 0);
        const int rp_rel = (int)(rp_abs - base);
        const int tile_nnz = __shfl_sync(0xffffffffu, rp_rel, TILE_R);
        if (lane <= TILE_R) rp_s[lane] = rp_rel;
        const bool fits = tile_nnz <= IDX_CAP;   // warp-uniform; almost always true
        if (fits) {
            for (int t = lane; t < tile_nnz; t += 32) {
                idx_s[t] = col_idx[base + t];
                if (HAS_VAL) val_s[t] = val[base + t];
            }
        }
        __syncwarp();
        // index / value of the tile's t-th non-zero: shared memory when the tile fits, else global
#define S2V_IDX(t) (fits ? idx_s[(t)] : __ldg(col_idx + base + (t)))
#define S2V_VAL(t) (fits ? val_s[(t)] : __ldg(val + base + (t)))

        // ---- 2. gather + sum in CSR order.
        //   FLAT (low-degree, wide rows): each group of LPR lanes walks the non-zeros of its
        //   RPS consecutive rows as ONE stream, U loads in flight whatever the row lengths; a
        //   row's sum is flushed to the shared tile when the stream crosses its end.
        //   Otherwise: one row per lane group per pass, chunks of U neighbours.
        if constexpr (LevelCfg<D>::FLAT) {
            int row = sub * RPS;
            const int row_stop = row + RPS;
            int t = rp_s[row];
            const int ee = rp_s[row_stop];
            int row_end = rp_s[row + 1];
            float* srow = S + row * S_STRIDE + sl * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#define S2V_FLUSH_ROWS(pos)                                                  \
    while ((pos) == row_end) {                                               \
        *reinterpret_cast<float4*>(srow) = acc;                              \
        acc = make_float4(0.f, 0.f, 0.f, 0.f);                               \
        ++row;                                                               \
        srow += S_STRIDE;                                                    \
        row_end = rp_s[row + 1];                                             \
    }
#define S2V_ACCUM(u)                                                         \
    if (HAS_VAL) {                                                           \
        const float a = S2V_VAL(t + (u));                                         \
        acc.x = fmaf(a, v[u].x, acc.x); acc.y = fmaf(a, v[u].y, acc.y);      \
        acc.z = fmaf(a, v[u].z, acc.z); acc.w = fmaf(a, v[u].w, acc.w);      \
    } else {                                                                 \
        acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;  \
    }
            for (; t + U <= ee; t += U) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) v[u] = ld_nc_f4(H4 + (int64_t)S2V_IDX(t + u) * LPR + sl);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    S2V_FLUSH_ROWS(t + u)
                    S2V_ACCUM(u)
                }
            }
            if (t < ee) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (t + u < ee) v[u] = ld_nc_f4(H4 + (int64_t)S2V_IDX(t + u) * LPR + sl);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (t + u < ee) {
                        S2V_FLUSH_ROWS(t + u)
                        S2V_ACCUM(u)
                    }
                }
            }
#undef S2V_FLUSH_ROWS
#undef S2V_ACCUM
            while (row < row_stop) {  // the open row, then empty rows behind it
                *reinterpret_cast<float4*>(srow) = acc;
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
                ++row;
                srow += S_STRIDE;
            }
        } else {
#pragma unroll 1
        for (int p = 0; p < NPASS; ++p) {
            const int lr = p * RPP + sub;
            const int beg = rp_s[lr];
            const int end = rp_s[lr + 1];
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            int t = beg;
            for (; t + U <= end; t += U) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) v[u] = ld_nc_f4(H4 + (int64_t)S2V_IDX(t + u) * LPR + sl);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (HAS_VAL) {
                        const float a = S2V_VAL(t + u);
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
                    v[u] = (t + u < end) ? ld_nc_f4(H4 + (int64_t)S2V_IDX(t + u) * LPR + sl) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (t + u < end) {
                        if (HAS_VAL) {
                            const float a = S2V_VAL(t + u);
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
        }
        __syncwarp();

#undef S2V_IDX
#undef S2V_VAL
        // ---- 3. [16 x D] * W[D x D] on the tensor cores, 3xTF32
        float c[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
#pragma unroll 1
        for (int ks = 0; ks < D / 8; ++ks) {
            uint32_t ah[4], al[4];
            const float* sa = S + g * S_STRIDE + ks * 8 + tig;
            tf32_split_rn(sa[0], ah[0], al[0]);
            tf32_split_rn(sa[8 * S_STRIDE], ah[1], al[1]);
            tf32_split_rn(sa[4], ah[2], al[2]);
            tf32_split_rn(sa[8 * S_STRIDE + 4], ah[3], al[3]);
            const float* wb = Ws + (ks * 8 + tig) * W_STRIDE + g;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                uint32_t bh0, bl0, bh1, bl1;
                tf32_split_trunc(wb[nt * 8], bh0, bl0);
                tf32_split_trunc(wb[4 * W_STRIDE + nt * 8], bh1, bl1);
                mma_tf32(c[nt], al, bh0, bh1);   // small terms first
                mma_tf32(c[nt], ah, bl0, bl1);
                mma_tf32(c[nt], ah, bh0, bh1);
            }
        }
        __syncwarp();  // every lane is done reading S
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            *reinterpret_cast<float2*>(S + g * S_STRIDE + nt * 8 + 2 * tig) = make_float2(c[nt][0], c[nt][1]);
            *reinterpret_cast<float2*>(S + (g + 8) * S_STRIDE + nt * 8 + 2 * tig) = make_float2(c[nt][2], c[nt][3]);
        }
        __syncwarp();

        // ---- 4. + X, ReLU, store: whole rows, d/4 lanes per row
#pragma unroll
        for (int p = 0; p < NPASS; ++p) {
            const int lr = p * RPP + sub;
            const int64_t row = r0 + lr;
            if (row < n_rows) {
                const float4 o = *reinterpret_cast<const float4*>(S + lr * S_STRIDE + sl * 4);
                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (XMODE == 1) x = ld_stream_f4(reinterpret_cast<const float4*>(X) + row * LPR + sl);
                if (XMODE == 2) {
                    // the index is caller data (a node tag): clamped into the table here; a bad index is detected and
                    // reported by index_range_check_kernel, which the host entry point launches beside this kernel
                    const int xi = (int)min((unsigned)__ldg(x_index + row), (unsigned)(n_table - 1));
                    x = ld_nc_f4(reinterpret_cast<const float4*>(X) + (int64_t)xi * LPR + sl);
                }
                float4 r;
                r.x = relu_ref(o.x + x.x);
                r.y = relu_ref(o.y + x.y);
                r.z = relu_ref(o.z + x.z);
                r.w = relu_ref(o.w + x.w);
                reinterpret_cast<float4*>(out)[row * LPR + sl] = r;
            }
        }
        __syncwarp();  // S and idx_s are rewritten by the next tile
    }
}

template <int D, typename RpT, bool HAS_VAL, int XMODE>
int launch_one(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, const RpT* row_ptr, const int32_t* col_idx,
               const float* val, const float* H, const float* W, const float* X, const int32_t* x_index, int n_table,
               float* out)
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
    kern<<<(unsigned)blocks, WARPS * 32, smem, st>>>(n_rows, num_tiles, row_ptr, col_idx, val, H, W, X, x_index, n_table, out,
                                                      ctx->dstatus_dev);
    S2V_CHECK_LAUNCH(ctx, "s2v_level_kernel");
    return S2V_OK;
}

template <int D, typename RpT>
int launch_d(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, const RpT* rp, const int32_t* ci, const float* val,
             const float* H, const float* W, const float* X, const float* table, const int32_t* x_index, int n_table,
             float* out)
{
    const int xmode = table ? 2 : (X ? 1 : 0);
    const float* xa = table ? table : X;
#define S2V_LVL(HV, XM) return launch_one<D, RpT, HV, XM>(ctx, st, n_rows, rp, ci, val, H, W, xa, x_index, n_table, out)
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
                     const float* X, const float* table, const int32_t* x_index, int n_table, float* out)
{
    (void)n_src;
    if (n_rows == 0) return S2V_OK;
    if (!rp64 && s2v_use_tc(ctx, d, n_rows)) {
        const int rc = s2v_launch_level_tc(ctx, st, n_rows, d, (const int32_t*)row_ptr, col_idx, val, H, W, X, table,
                                           x_index, n_table, out);
        if (rc != S2V_ERR_UNSUPPORTED) return rc;
    }
#define S2V_D(DD)                                                                                                  \
    case DD:                                                                                                       \
        return rp64 ? launch_d<DD, int64_t>(ctx, st, n_rows, (const int64_t*)row_ptr, col_idx, val, H, W, X, table, \
                                            x_index, n_table, out)                                                 \
                    : launch_d<DD, int32_t>(ctx, st, n_rows, (const int32_t*)row_ptr, col_idx, val, H, W, X, table, \
                                            x_index, n_table, out)
    switch (d) {
        S2V_D(32);
        S2V_D(64);
        S2V_D(128);
        default:
            return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "fused level kernel supports d in {32, 64, 128}");
    }
#undef S2V_D
}
