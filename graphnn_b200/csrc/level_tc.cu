// Fused structure2vec level for d = 64 and d = 128 with the dense stage on the 5th-generation
// tensor cores (tcgen05.mma, accumulators and the A operand in tensor memory).
//
//     out[i,:] = ReLU( (sum_{t in row i} val[t] * H[col_idx[t],:]) * W + X[i,:] )
//
// Why a second form of the kernel: at d = 128 the product [rows x 128] * [128 x 128] in
// 3xTF32 costs 3 * 2 * 128^2 flop per row against 1.5 KB of compulsory traffic; the
// warp-level mma.sync path (level.cu) is bounded by the legacy tensor rate there, well
// above the HBM time.  tcgen05 runs the same 3xTF32 product about four times faster and
// needs no registers for the operands, so the kernel goes back to being memory-bound.
// At d = 64 the gain is the warp specialisation: dedicated gather warps keep a software-
// pipelined stream of neighbour loads in flight instead of alternating with the product.
//
// One persistent 768-thread CTA per SM, 128-row tiles, three warp roles connected by mbarriers:
//
//   gather warps (16) : the tile's CSR slice -> shared memory, neighbour rows summed in
//                       CSR order as one flat software-pipelined stream per group of d/4
//                       lanes (8 loads in flight per lane, indices prefetched a tile ahead)
//                       into a fp32 staging tile [128 x d] (two of them at d = 64);
//   operand warps (4) : read the staging tile "transposed" (thread = row), split every
//                       value into a TF32 head and tail and store both into tensor memory
//                       (tcgen05.st; double-buffered at d = 64); one elected thread then
//                       issues the 3 * d/8 MMAs (lo*hi, hi*lo, hi*hi over K = d in steps
//                       of 8) against W^T, which sits in shared memory split the same way
//                       in the K-major 128-byte-swizzle layout, and commits them to an mbarrier;
//   epilogue warps (4): tcgen05.ld the fp32 accumulator (double-buffered in tensor
//                       memory), transpose 32x32 blocks through shared memory, add X,
//                       apply ReLU and store whole 128-byte row segments.
//
// The gather of tile i+1 overlaps the operand/MMA/epilogue work of tile i.  Every wait is
// bounded: on a time-out the kernel records S2V_ERR_DEVICE_TIMEOUT, raises a CTA-wide
// abort flag, drains, frees its tensor memory and returns.
#include "common.cuh"

namespace
{

constexpr int TC_TILE = 128;           // rows per tile = MMA M
constexpr int TC_GW = 16;              // gather warps (measured: 16 x 4 loads per chunk beats 8 x 8)
constexpr int TC_AW = 4;               // operand warps (one per tensor-memory lane quarter)
constexpr int TC_EW = 4;               // epilogue warps
constexpr int TC_THREADS = (TC_GW + TC_AW + TC_EW) * 32;
constexpr int TC_ROWS_PER_GW = TC_TILE / TC_GW;   // 8
constexpr int TC_U = 4;
constexpr int TC_OUT_STRIDE = 36;                 // floats; 9 float4 per row
constexpr int TC_WAIT_LIMIT = 1 << 22;
constexpr int TC_MAX_STAGES = 2;

// Per-width configuration and shared memory map (offsets from a 1024-byte aligned base).
template <int D>
struct TcCfg {
    static constexpr int NSTAGE = (D == 64) ? 2 : 1;   // fp32 staging tiles (shared memory allows two at d = 64)
    static constexpr int NABUF = (D == 64) ? 2 : 1;    // A-operand buffers in tensor memory (512 columns allow two at d = 64)
    static constexpr int IDX_CAP = (D == 64) ? 128 : 64;   // column indices of one gather warp's 8 rows kept in shared memory
    static constexpr int STAGE_STRIDE = D + 4;         // floats; an odd number of float4 per row: thread-per-row float4 reads are conflict-free
    static constexpr size_t OFF_BHI = 0;
    static constexpr size_t OFF_BLO = OFF_BHI + sizeof(float) * D * D;
    static constexpr size_t OFF_STAGE = OFF_BLO + sizeof(float) * D * D;
    static constexpr size_t STAGE_BYTES = sizeof(float) * TC_TILE * STAGE_STRIDE;
    static constexpr size_t OFF_OUT = OFF_STAGE + STAGE_BYTES * NSTAGE;
    static constexpr size_t OFF_GW = OFF_OUT + sizeof(float) * TC_EW * 32 * TC_OUT_STRIDE;
    static constexpr size_t GW_BYTES = 2 * (sizeof(int) * IDX_CAP + sizeof(int) * 32);   // double-buffered indices + row offsets
    static constexpr size_t OFF_BAR = OFF_GW + GW_BYTES * TC_GW;
    static constexpr size_t SMEM_BYTES = OFF_BAR + 256 + 1024;   // + barriers/flags + alignment slack
    // tensor memory columns: A head/tail per buffer, then two accumulators
    static constexpr uint32_t TM_A = 0;                 // + ab*2D : head, + ab*2D + D : tail
    static constexpr uint32_t TM_ACC = 2 * D * NABUF;   // + b*D
    static_assert(2 * D * NABUF + 2 * D <= 512, "tensor memory has 512 columns");
    // instruction descriptor: D = f32, A = B = tf32, both K-major, M = 128, N = D
    static constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(TC_TILE >> 4) << 24);
};

// mbarriers.  FULL/SFREE exist per staging tile and tensor-memory lane quarter (32 rows = four gather
// warps, one operand warp).
enum {
    BAR_FULL0 = 0,                                 // +4*s+q : the quarter's 32 rows of staging tile s are written
    BAR_SFREE0 = BAR_FULL0 + 4 * TC_MAX_STAGES,    // +4*s+q : the quarter's rows have been read back and may be overwritten
    BAR_AREADY0 = BAR_SFREE0 + 4 * TC_MAX_STAGES,  // +ab : all four quarters of A-operand buffer ab are in tensor memory
    BAR_MMA0 = BAR_AREADY0 + 2, BAR_MMA1,          // the MMAs into accumulator buffer 0 / 1 are complete
    BAR_DFREE0, BAR_DFREE1,                        // accumulator buffer 0 / 1 has been read by the epilogue
    BAR_COUNT
};

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try(uint32_t bar, uint32_t parity)
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
// Bounded wait.  Returns false when the CTA is aborting (time-out here or elsewhere).
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, s2v_device_status* status,
                                        int site)
{
    int spins = 0;
    while (!tc_mbar_try(bar, parity)) {
        if (*abort_flag) return false;
        if (++spins > TC_WAIT_LIMIT) {
            *abort_flag = 1;
            status->code = S2V_ERR_DEVICE_TIMEOUT;
            status->where = site;
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ uint32_t tf32_rn(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_b_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                        // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Optional cycle accounting per warp role (compile with -DS2V_TC_TRACE): block 0 prints, per
// role, the cycles spent in each numbered section.  Compiled out by default.
#ifdef S2V_TC_TRACE
#define TC_TRACE_DECL() long long tr__[6] = {0, 0, 0, 0, 0, 0}; long long t0__ = clock64()
#define TC_TRACE(slot) do { const long long t1__ = clock64(); tr__[slot] += t1__ - t0__; t0__ = t1__; } while (0)
#define TC_TRACE_PRINT(role) do { if (blockIdx.x == 0 && lane == 0) printf("%s warp %d tiles %lld: %lld %lld %lld %lld %lld %lld\n", role, warp, (long long)my_tiles, tr__[0], tr__[1], tr__[2], tr__[3], tr__[4], tr__[5]); } while (0)
#else
#define TC_TRACE_DECL() do {} while (0)
#define TC_TRACE(slot) do {} while (0)
#define TC_TRACE_PRINT(role) do {} while (0)
#endif

template <int D, bool HAS_VAL, int XMODE, bool HSRC_TABLE>
__global__ void __launch_bounds__(TC_THREADS, 1)
s2v_level_tc_kernel(int64_t n_rows, int64_t num_tiles, const int32_t* __restrict__ row_ptr,
                    const int32_t* __restrict__ col_idx, const float* __restrict__ val, const float* __restrict__ H,
                    const float* __restrict__ W, const float* __restrict__ X, const int32_t* __restrict__ x_index,
                    float* __restrict__ out, s2v_device_status* status)
{
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    using Cfg = TcCfg<D>;
    constexpr int NSTAGE = Cfg::NSTAGE, NABUF = Cfg::NABUF, IDX_CAP = Cfg::IDX_CAP, STAGE_STRIDE = Cfg::STAGE_STRIDE;
    float* Bhi = reinterpret_cast<float*>(smem + Cfg::OFF_BHI);
    float* Blo = reinterpret_cast<float*>(smem + Cfg::OFF_BLO);
    float* stage0 = reinterpret_cast<float*>(smem + Cfg::OFF_STAGE);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 8 * BAR_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 8 * BAR_COUNT + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    // ---- set-up: barriers, tensor memory, W^T split into TF32 head/tail in the MMA layout
    if (threadIdx.x == 0) {
        for (int qq = 0; qq < 4 * NSTAGE; ++qq) {
            tc_mbar_init(bar(BAR_FULL0 + qq), TC_GW / 4);
            tc_mbar_init(bar(BAR_SFREE0 + qq), 1);
        }
        for (int ab = 0; ab < NABUF; ++ab) tc_mbar_init(bar(BAR_AREADY0 + ab), TC_AW);
        tc_mbar_init(bar(BAR_MMA0), 1);
        tc_mbar_init(bar(BAR_MMA1), 1);
        tc_mbar_init(bar(BAR_DFREE0), TC_EW);
        tc_mbar_init(bar(BAR_DFREE1), TC_EW);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // B[n][k] = W[k][n]; element (n, k) lives at  kb*(D*128) + n*128 + ((kk/4) ^ (n&7))*16 + (kk%4)*4,
    // kb = k/32, kk = k%32.  Each task converts 4 consecutive k of one n: one 16-byte store per matrix.
    for (int e = threadIdx.x; e < D * D / 4; e += TC_THREADS) {
        const int n = e % D, kq = e / D;   // k = 4*kq .. 4*kq+3
        float w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = __ldg(W + (int64_t)(4 * kq + j) * D + n);
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            hi[j] = tf32_rn(w[j]);
            lo[j] = tf32_rn(w[j] - __uint_as_float(hi[j]));
        }
        const int kb = kq >> 3, chunk = kq & 7;
        const size_t off = (size_t)kb * (D * 128) + (size_t)n * 128 + (size_t)((chunk ^ (n & 7)) * 16);
        *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(Bhi) + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(Blo) + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t TM_A = tmem_base + Cfg::TM_A, TM_ACC = tmem_base + Cfg::TM_ACC;

    const int64_t my_tiles = (num_tiles > (int64_t)blockIdx.x) ? (num_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;

    if (warp < TC_GW) {
        // =========================== gather warps ===========================
        unsigned char* gbase = smem + Cfg::OFF_GW + Cfg::GW_BYTES * warp;
        int* idx_buf[2] = {reinterpret_cast<int*>(gbase), reinterpret_cast<int*>(gbase) + IDX_CAP + 32};
        const float4* __restrict__ H4 = reinterpret_cast<const float4*>(H);
        constexpr int LPR = D / 4;                       // lanes that cover one row with float4
        constexpr int RPG = TC_ROWS_PER_GW / (32 / LPR); // consecutive rows one lane group streams through
        constexpr int IPL = IDX_CAP / 32;                // prefetched indices per lane
        const int sub = lane / LPR, sl = lane % LPR;
        const int q = warp / (TC_GW / 4);                // tensor-memory lane quarter my rows belong to
        // Row offsets are fetched two tiles ahead and column indices one tile ahead, into
        // registers while the current tile is gathered, so no tile waits on that chain.
        auto load_rp = [&](int64_t it) -> int32_t {
            int64_t rpi = (blockIdx.x + it * gridDim.x) * TC_TILE + (int64_t)warp * TC_ROWS_PER_GW + lane;
            if (rpi > n_rows) rpi = n_rows;
            return lane <= TC_ROWS_PER_GW ? row_ptr[rpi] : 0;
        };
        int32_t rp_next = load_rp(0);      // row offsets of the tile whose indices are fetched next
        int32_t rp_next2 = load_rp(1);
        int32_t base = 0;
        int nnz = 0;
        {   // tile 0: fill buffer 0 directly
            base = __shfl_sync(0xffffffffu, rp_next, 0);
            const int rel = rp_next - base;
            nnz = __shfl_sync(0xffffffffu, rel, TC_ROWS_PER_GW);
            if (lane <= TC_ROWS_PER_GW) idx_buf[0][IDX_CAP + lane] = rel;
            if (nnz <= IDX_CAP)
                for (int t = lane; t < nnz; t += 32) idx_buf[0][t] = col_idx[base + t];
            rp_next = rp_next2;
        }
        __syncwarp();
        TC_TRACE_DECL();
        for (int64_t it = 0; it < my_tiles; ++it) {
            int* idx_s = idx_buf[it & 1];
            const int* rp_s = idx_s + IDX_CAP;
            const bool fits = nnz <= IDX_CAP;   // warp-uniform; almost always true
            const int s = (int)(it % NSTAGE);
            const float* vp = HAS_VAL ? val + base : nullptr;
#define TC_IDX(t) (fits ? idx_s[(t)] : __ldg(col_idx + base + (t)))
            // prefetch (registers): offsets of tile it+2, indices of tile it+1
            rp_next2 = load_rp(it + 2);
            const int32_t base1 = __shfl_sync(0xffffffffu, rp_next, 0);
            const int rel1 = rp_next - base1;
            const int nnz1 = __shfl_sync(0xffffffffu, rel1, TC_ROWS_PER_GW);
            int idx_pref[IPL];
#pragma unroll
            for (int j = 0; j < IPL; ++j)
                idx_pref[j] = (nnz1 <= IDX_CAP && lane + 32 * j < nnz1) ? col_idx[base1 + lane + 32 * j] : 0;
            TC_TRACE(0);
            // Flat stream over the non-zeros of my lane group's RPG rows, software-pipelined: the
            // loads of chunk k+1 are in flight while chunk k is summed, and the first chunk is
            // issued before waiting for the staging tile, so the wait costs no memory latency.
            int row = sub * RPG;
            const int row_stop = row + RPG;
            int t = rp_s[row];
            const int ee = rp_s[row_stop];
            int row_end = rp_s[row + 1];
            float* srow = stage0 + (size_t)s * (TC_TILE * STAGE_STRIDE) + (size_t)(warp * TC_ROWS_PER_GW + row) * STAGE_STRIDE + sl * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float4 va[TC_U], vb[TC_U];
// HSRC_TABLE: the gather source is not a matrix but ReLU(table[x_index[col], :]) -- the first level of
// the classifier with one-hot inputs, where H0 = ReLU(W_in[tag]) need not be materialised
#define TC_LOAD(v, t0) TC_LOADN(v, t0, TC_U)
#define TC_LOADN(v, t0, NN)                                                                        \
    _Pragma("unroll") for (int u = 0; u < NN; ++u)                                                 \
        if ((t0) + u < ee) {                                                                       \
            if (HSRC_TABLE) {                                                                      \
                const int tg = __ldg(x_index + TC_IDX((t0) + u));                                      \
                const float4 w = ld_nc_f4(reinterpret_cast<const float4*>(X) + (int64_t)tg * LPR + sl); \
                v[u] = make_float4(relu_ref(w.x), relu_ref(w.y), relu_ref(w.z), relu_ref(w.w));    \
            } else {                                                                               \
                v[u] = ld_nc_f4(H4 + (int64_t)TC_IDX((t0) + u) * LPR + sl);                            \
            }                                                                                      \
        }
#define TC_CONSUME(v, t0) TC_CONSUMEN(v, t0, TC_U)
#define TC_CONSUMEN(v, t0, NN)                                                                     \
    _Pragma("unroll") for (int u = 0; u < NN; ++u) {                                               \
        if ((t0) + u < ee) {                                                                       \
            while ((t0) + u == row_end) {                                                          \
                *reinterpret_cast<float4*>(srow) = acc;                                            \
                acc = make_float4(0.f, 0.f, 0.f, 0.f);                                             \
                ++row;                                                                             \
                srow += STAGE_STRIDE;                                                              \
                row_end = rp_s[row + 1];                                                           \
            }                                                                                      \
            if (HAS_VAL) {                                                                         \
                const float a = vp[(t0) + u];                                                      \
                acc.x = fmaf(a, v[u].x, acc.x); acc.y = fmaf(a, v[u].y, acc.y);                    \
                acc.z = fmaf(a, v[u].z, acc.z); acc.w = fmaf(a, v[u].w, acc.w);                    \
            } else {                                                                               \
                acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;                \
            }                                                                                      \
        }                                                                                          \
    }
            TC_LOAD(va, t)
            // Pull the neighbour rows of the NEXT tile into L2 now, a whole tile ahead of their use:
            // a prefetch holds no register, so the rows in flight are not bounded by the register file.
            if (!HSRC_TABLE) {
#pragma unroll
                for (int j = 0; j < IPL; ++j)
                    if (nnz1 <= IDX_CAP && lane + 32 * j < nnz1) {
                        const char* rowp = reinterpret_cast<const char*>(H4 + (int64_t)idx_pref[j] * LPR);
#pragma unroll
                        for (int l = 0; l < D * 4 / 128; ++l) asm volatile("prefetch.global.L2 [%0];" ::"l"(rowp + 128 * l));
                    }
            }
            // my quarter of staging tile s is free once its operand warp has read tile it-NSTAGE
            if (it >= NSTAGE && !tc_wait(bar(BAR_SFREE0 + 4 * s + q), (uint32_t)(((it - NSTAGE) / NSTAGE) & 1), abort_flag, status, 10)) break;
            TC_TRACE(1);
            while (t < ee) {
                TC_LOAD(vb, t + TC_U)
                TC_TRACE(2);
                TC_CONSUME(va, t)
                TC_TRACE(3);
                t += TC_U;
                if (t >= ee) break;
                TC_LOAD(va, t + TC_U)
                TC_TRACE(2);
                TC_CONSUME(vb, t)
                TC_TRACE(3);
                t += TC_U;
            }
#undef TC_LOAD
#undef TC_CONSUME
#undef TC_LOADN
#undef TC_CONSUMEN
#undef TC_IDX
            while (row < row_stop) {
                *reinterpret_cast<float4*>(srow) = acc;
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
                ++row;
                srow += STAGE_STRIDE;
            }
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(bar(BAR_FULL0 + 4 * s + q));
            {   // publish the prefetched slice of tile it+1 in the other buffer
                int* nb = idx_buf[(it + 1) & 1];
                if (lane <= TC_ROWS_PER_GW) nb[IDX_CAP + lane] = rel1;
#pragma unroll
                for (int j = 0; j < IPL; ++j)
                    if (lane + 32 * j < nnz1 && nnz1 <= IDX_CAP) nb[lane + 32 * j] = idx_pref[j];
                base = base1;
                nnz = nnz1;
                rp_next = rp_next2;
            }
            __syncwarp();
            TC_TRACE(4);
        }
        TC_TRACE_PRINT("gather");
    } else if (warp < TC_GW + TC_AW) {
        // =========================== operand warps ===========================
        const int q = warp & 3;   // tensor-memory lane quarter this warp may access
        const uint32_t lane_base = (uint32_t)(32 * q) << 16;
        TC_TRACE_DECL();
        for (int64_t it = 0; it < my_tiles; ++it) {
            const int b = (int)(it & 1);
            const int s = (int)(it % NSTAGE);
            const int ab = (int)(it % NABUF);
            const float* my_row = stage0 + (size_t)s * (TC_TILE * STAGE_STRIDE) + (size_t)(32 * q + lane) * STAGE_STRIDE;
            const uint32_t TM_AHI = TM_A + (uint32_t)(2 * D * ab), TM_ALO = TM_AHI + D;
            if (!tc_wait(bar(BAR_FULL0 + 4 * s + q), (uint32_t)((it / NSTAGE) & 1), abort_flag, status, 20)) break;
            TC_TRACE(0);
            // the MMAs of the tile that used this A-operand buffer before must be done reading it
            if (it >= NABUF && !tc_wait(bar(BAR_MMA0 + (int)((it - NABUF) & 1)), (uint32_t)(((it - NABUF) >> 1) & 1), abort_flag, status, 21)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            TC_TRACE(1);
#pragma unroll 1
            for (int kc = 0; kc < D / 32; ++kc) {
                uint32_t hi[32], lo[32];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 v = *reinterpret_cast<const float4*>(my_row + 32 * kc + 4 * j);
                    hi[4 * j + 0] = tf32_rn(v.x); lo[4 * j + 0] = tf32_rn(v.x - __uint_as_float(hi[4 * j + 0]));
                    hi[4 * j + 1] = tf32_rn(v.y); lo[4 * j + 1] = tf32_rn(v.y - __uint_as_float(hi[4 * j + 1]));
                    hi[4 * j + 2] = tf32_rn(v.z); lo[4 * j + 2] = tf32_rn(v.z - __uint_as_float(hi[4 * j + 2]));
                    hi[4 * j + 3] = tf32_rn(v.w); lo[4 * j + 3] = tf32_rn(v.w - __uint_as_float(hi[4 * j + 3]));
                }
#define TC_ST32(addr, r)                                                                                             \
    asm volatile(                                                                                                    \
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"        \
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(addr),                              \
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),  \
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),    \
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),    \
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])                                                                \
        : "memory")
                TC_ST32(TM_AHI + lane_base + 32 * kc, hi);
                TC_ST32(TM_ALO + lane_base + 32 * kc, lo);
#undef TC_ST32
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(bar(BAR_SFREE0 + 4 * s + q));   // my 32 rows of the staging tile are consumed
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (lane == 0) tc_mbar_arrive(bar(BAR_AREADY0 + ab));   // my quarter of the A operand is in tensor memory
            TC_TRACE(2);
            if (q == 0) {
                // one elected thread issues the tile's MMAs
                bool ok = tc_wait(bar(BAR_AREADY0 + ab), (uint32_t)((it / NABUF) & 1), abort_flag, status, 22);
                if (ok && it >= 2) ok = tc_wait(bar(BAR_DFREE0 + b), (uint32_t)(((it - 2) >> 1) & 1), abort_flag, status, 23);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                TC_TRACE(3);
                if (lane == 0) {
                    const uint32_t d_tmem = TM_ACC + (uint32_t)(D * b);
                    const uint32_t bhi = smem_u32(Bhi), blo = smem_u32(Blo);
                    uint32_t accumulate = 0;
#pragma unroll 1
                    for (int pass = 0; pass < 3; ++pass) {   // lo*hi, hi*lo, hi*hi: small terms first
                        const uint32_t a_base = (pass == 0) ? TM_ALO : TM_AHI;
                        const uint32_t b_base = (pass == 1) ? blo : bhi;
#pragma unroll 1
                        for (int ks = 0; ks < D / 8; ++ks) {
                            const uint32_t b_addr = b_base + (uint32_t)(ks >> 2) * (uint32_t)(D * 128) + (uint32_t)(ks & 3) * 32u;
                            tc_mma(d_tmem, a_base + 8u * (uint32_t)ks, tc_b_desc(b_addr), Cfg::IDESC, accumulate);
                            accumulate = 1;
                        }
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                     bar(BAR_MMA0 + b))
                                 : "memory");
                }
                __syncwarp();
                TC_TRACE(4);
            }
        }
        TC_TRACE_PRINT("operand");
    } else {
        // =========================== epilogue warps ===========================
        const int q = warp & 3;
        const uint32_t lane_base = (uint32_t)(32 * q) << 16;
        float* ostage = reinterpret_cast<float*>(smem + Cfg::OFF_OUT) + (size_t)q * 32 * TC_OUT_STRIDE;
        const int rsub = lane >> 3, c4 = lane & 7;
        TC_TRACE_DECL();
        for (int64_t it = 0; it < my_tiles; ++it) {
            const int b = (int)(it & 1);
            const int64_t tile = blockIdx.x + it * gridDim.x;
            // X row index of "my" row (lane = row within this warp's 32 rows), fetched before the
            // wait so that its latency hides behind the MMAs
            int my_xi = 0;
            if (XMODE == 2) {
                const int64_t mr = tile * TC_TILE + 32 * q + lane;
                if (mr < n_rows) my_xi = __ldg(x_index + mr);
            }
            if (!tc_wait(bar(BAR_MMA0 + b), (uint32_t)((it >> 1) & 1), abort_flag, status, 30)) break;
            TC_TRACE(0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int cc = 0; cc < D / 32; ++cc) {
                uint32_t v[32];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                    "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(TM_ACC + (uint32_t)(D * b) + lane_base + 32u * (uint32_t)cc)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (cc == D / 32 - 1) {   // the accumulator buffer is fully read: hand it back early
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    if (lane == 0) tc_mbar_arrive(bar(BAR_DFREE0 + b));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<uint4*>(ostage + lane * TC_OUT_STRIDE + 4 * j) =
                        make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                __syncwarp();
                // 4 rows x 128 bytes per instruction; all loads of the 8 row groups are issued
                // before the first store so that their latencies overlap
                const int64_t col4 = 8 * cc + c4;
                float4 o[8], x[8];
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    const int rl = rr * 4 + rsub;
                    const int64_t row = tile * TC_TILE + 32 * q + rl;
                    o[rr] = *reinterpret_cast<const float4*>(ostage + rl * TC_OUT_STRIDE + 4 * c4);
                    x[rr] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (XMODE == 1 && row < n_rows) x[rr] = ld_stream_f4(reinterpret_cast<const float4*>(X) + row * (D / 4) + col4);
                    if (XMODE == 2) {
                        const int xi = __shfl_sync(0xffffffffu, my_xi, rl);
                        if (row < n_rows) x[rr] = ld_nc_f4(reinterpret_cast<const float4*>(X) + (int64_t)xi * (D / 4) + col4);
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    const int64_t row = tile * TC_TILE + 32 * q + rr * 4 + rsub;
                    if (row < n_rows) {
                        float4 r;
                        r.x = relu_ref(o[rr].x + x[rr].x);
                        r.y = relu_ref(o[rr].y + x[rr].y);
                        r.z = relu_ref(o[rr].z + x[rr].z);
                        r.w = relu_ref(o[rr].w + x[rr].w);
                        reinterpret_cast<float4*>(out)[row * (D / 4) + col4] = r;
                    }
                }
                __syncwarp();
            }
            TC_TRACE(1);
        }
        TC_TRACE_PRINT("epilogue");
    }

    // ---- teardown: everyone is done with tensor memory before it is released
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}

template <int D, bool HAS_VAL, int XMODE, bool HSRC_TABLE = false>
int tc_launch(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, const int32_t* rp, const int32_t* ci, const float* val,
              const float* H, const float* W, const float* X, const int32_t* x_index, float* out)
{
    auto kern = s2v_level_tc_kernel<D, HAS_VAL, XMODE, HSRC_TABLE>;
    constexpr size_t SMEM = TcCfg<D>::SMEM_BYTES;
    if (SMEM > ctx->smem_optin) return S2V_ERR_UNSUPPORTED;
    S2V_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    const int64_t num_tiles = (n_rows + TC_TILE - 1) / TC_TILE;
    int64_t blocks = num_tiles < ctx->sm_count ? num_tiles : ctx->sm_count;
    if (blocks < 1) blocks = 1;
    kern<<<(unsigned)blocks, TC_THREADS, SMEM, st>>>(n_rows, num_tiles, rp, ci, val, H, W, X, x_index, out,
                                                               ctx->dstatus_dev);
    S2V_CHECK_LAUNCH(ctx, "s2v_level_tc_kernel");
    return S2V_OK;
}

}  // namespace

// d = 64 or 128, 32-bit row offsets.  Returns S2V_ERR_UNSUPPORTED for anything else (the caller falls back).
// H == NULL with a table: the gather source is ReLU(table[x_index[col], :]) (square matrices only).
template <int D>
static int tc_dispatch(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, const int32_t* row_ptr, const int32_t* col_idx,
                       const float* val, const float* H, const float* W, const float* X, const float* table,
                       const int32_t* x_index, float* out)
{
    if (!H) {
        if (!table || !x_index) return S2V_ERR_UNSUPPORTED;
        return val ? tc_launch<D, true, 2, true>(ctx, st, n_rows, row_ptr, col_idx, val, nullptr, W, table, x_index, out)
                   : tc_launch<D, false, 2, true>(ctx, st, n_rows, row_ptr, col_idx, val, nullptr, W, table, x_index, out);
    }
    const int xmode = table ? 2 : (X ? 1 : 0);
    const float* xa = table ? table : X;
#define TC_GO(HV, XM) return tc_launch<D, HV, XM>(ctx, st, n_rows, row_ptr, col_idx, val, H, W, xa, x_index, out)
    if (val) {
        if (xmode == 0) TC_GO(true, 0);
        if (xmode == 1) TC_GO(true, 1);
        TC_GO(true, 2);
    }
    if (xmode == 0) TC_GO(false, 0);
    if (xmode == 1) TC_GO(false, 1);
    TC_GO(false, 2);
#undef TC_GO
}

int s2v_launch_level_tc(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, int d, const int32_t* row_ptr,
                        const int32_t* col_idx, const float* val, const float* H, const float* W, const float* X,
                        const float* table, const int32_t* x_index, float* out)
{
    if (d == 128) return tc_dispatch<128>(ctx, st, n_rows, row_ptr, col_idx, val, H, W, X, table, x_index, out);
    if (d == 64) return tc_dispatch<64>(ctx, st, n_rows, row_ptr, col_idx, val, H, W, X, table, x_index, out);
    return S2V_ERR_UNSUPPORTED;
}
