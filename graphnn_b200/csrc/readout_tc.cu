// Readout of the classifier on the 5th-generation tensor cores:
//
//     hidden = ReLU(Y * W1)   [G x hidden],   logits = hidden * W2   [G x C],   softmax / argmax per graph
//
// (examples/graph_classification/src/kernel_mean_field.cpp:43-47: MatMul, ReLU, MatMul; the softmax and argmax
// of the loss / prediction factors).  The first layer is a [G x d] * [d x hidden] product: 128 graphs per tile
// (MMA M), N = hidden (256 or 128), 3xTF32 like the level kernels (lo*hi, hi*lo, hi*hi into one fp32
// accumulator, small terms first).  Both operands come from shared memory in the K-major 128-byte-swizzle layout,
// split into TF32 head and tail as they are staged; K is taken 64 at a time because head + tail of W1^T for all
// 128 K values would not fit (hidden * 128 * 8 bytes).  The accumulator (hidden columns of tensor memory) is
// read back by four warps, one per lane quarter, thread = graph: ReLU, the second layer as a running dot
// product in ascending hidden order, softmax and argmax in registers.
//
// One CTA per tile (persistent over tiles when there are more tiles than SMs).  Every wait is bounded and every
// warp executes the same sequence of waits and block-wide barriers, so a time-out takes the whole CTA to the
// teardown together.
#include "common.cuh"
#include "tcgen05.cuh"

namespace
{

constexpr int RT_TILE = 128;      // graphs per tile = MMA M
constexpr int RT_KH = 64;         // K values staged at a time
constexpr int RT_THREADS = 256;
constexpr int RT_MAX_C = 8;

template <int HID>
struct RtCfg {
    static constexpr size_t A_BYTES = sizeof(float) * RT_TILE * RT_KH;   // 32 KB: one of head / tail
    static constexpr size_t B_BYTES = sizeof(float) * HID * RT_KH;       // 64 KB at hidden = 256
    static constexpr size_t OFF_AHI = 0, OFF_ALO = A_BYTES, OFF_BHI = 2 * A_BYTES, OFF_BLO = 2 * A_BYTES + B_BYTES;
    static constexpr size_t OFF_W2 = 2 * A_BYTES + 2 * B_BYTES;
    static constexpr size_t OFF_BAR = OFF_W2 + sizeof(float) * HID * RT_MAX_C;
    static constexpr size_t SMEM_BYTES = OFF_BAR + 64 + 1024;            // + barrier / flags + alignment slack
    // instruction descriptor: D = f32, A = B = tf32, both K-major, M = 128, N = HID
    static constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(HID >> 3) << 17) | ((uint32_t)(RT_TILE >> 4) << 24);
};

__device__ __forceinline__ void rt_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <int HID>
__global__ void __launch_bounds__(RT_THREADS, 1)
readout_tc_kernel(int64_t G, int d, int C, const float* __restrict__ Y, const float* __restrict__ W1, const float* __restrict__ W2,
                  float* __restrict__ logits, float* __restrict__ probs, int32_t* __restrict__ pred, s2v_device_status* status)
{
    using Cfg = RtCfg<HID>;
    extern __shared__ unsigned char rt_smem_raw[];
    unsigned char* smem = rt_smem_raw + ((1024u - (smem_u32(rt_smem_raw) & 1023u)) & 1023u);
    float* W2s = reinterpret_cast<float*>(smem + Cfg::OFF_W2);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 16);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_mma = smem_u32(bars);

    if (threadIdx.x == 0) {
        tc_mbar_init(bar_mma, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(HID) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int e = threadIdx.x; e < HID * C; e += RT_THREADS) W2s[e] = __ldg(W2 + e);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int64_t tiles = (G + RT_TILE - 1) / RT_TILE;
    const int halves = d / RT_KH;
    uint32_t commits = 0;      // MMA batches committed so far (the same count in every thread)
    bool alive = true;
    for (int64_t tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
        const int64_t g0 = tile * RT_TILE;
        const int ng = (int)((G - g0) < RT_TILE ? (G - g0) : RT_TILE);
        for (int kh = 0; kh < halves; ++kh) {
            // the operand buffers are free once the MMAs of the previous batch have completed
            if (commits > 0 && !tc_wait(bar_mma, (commits - 1) & 1u, abort_flag, status, 60)) { alive = false; break; }
            // A[m][k] = Y[g0 + m][64 kh + k]: element (m, k) at kb*(128*128) + m*128 + ((kk/4) ^ (m&7))*16 + (kk%4)*4
            // (all loads of a batch of tasks are issued before the first conversion: one memory latency per batch)
            {
                constexpr int A_TASKS = RT_TILE * (RT_KH / 4) / RT_THREADS;   // 8 per thread
                float4 av[A_TASKS];
#pragma unroll
                for (int i = 0; i < A_TASKS; ++i) {
                    const int t = threadIdx.x + i * RT_THREADS;
                    const int m = t / (RT_KH / 4), kq = t % (RT_KH / 4);
                    av[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (m < ng) av[i] = __ldg(reinterpret_cast<const float4*>(Y + (g0 + m) * d + RT_KH * kh) + kq);
                }
#pragma unroll
                for (int i = 0; i < A_TASKS; ++i) {
                    const int t = threadIdx.x + i * RT_THREADS;
                    const int m = t / (RT_KH / 4), kq = t % (RT_KH / 4);
                    uint4 hi, lo;
                    tc_split(av[i].x, hi.x, lo.x);
                    tc_split(av[i].y, hi.y, lo.y);
                    tc_split(av[i].z, hi.z, lo.z);
                    tc_split(av[i].w, hi.w, lo.w);
                    const size_t off = (size_t)(kq >> 3) * (RT_TILE * 128) + (size_t)m * 128 + (size_t)(((kq & 7) ^ (m & 7)) * 16);
                    *reinterpret_cast<uint4*>(smem + Cfg::OFF_AHI + off) = hi;
                    *reinterpret_cast<uint4*>(smem + Cfg::OFF_ALO + off) = lo;
                }
            }
            // B[n][k] = W1[64 kh + k][n]: the four k of a task are four coalesced loads across n; eight tasks per batch
            {
                constexpr int B_TASKS = HID * (RT_KH / 4) / RT_THREADS;       // 16 (hidden = 256) or 8 per thread
                constexpr int BATCH = 8;
                static_assert(B_TASKS % BATCH == 0, "batches of eight tasks");
#pragma unroll 1
                for (int b0 = 0; b0 < B_TASKS; b0 += BATCH) {
                    float wv[BATCH][4];
#pragma unroll
                    for (int i = 0; i < BATCH; ++i) {
                        const int t = threadIdx.x + (b0 + i) * RT_THREADS;
                        const int n = t % HID, kq = t / HID;
                        const float* w = W1 + (int64_t)(RT_KH * kh + 4 * kq) * HID + n;
#pragma unroll
                        for (int j = 0; j < 4; ++j) wv[i][j] = __ldg(w + (int64_t)j * HID);
                    }
#pragma unroll
                    for (int i = 0; i < BATCH; ++i) {
                        const int t = threadIdx.x + (b0 + i) * RT_THREADS;
                        const int n = t % HID, kq = t / HID;
                        uint4 hi, lo;
                        tc_split(wv[i][0], hi.x, lo.x);
                        tc_split(wv[i][1], hi.y, lo.y);
                        tc_split(wv[i][2], hi.z, lo.z);
                        tc_split(wv[i][3], hi.w, lo.w);
                        const size_t off = (size_t)(kq >> 3) * (HID * 128) + (size_t)n * 128 + (size_t)(((kq & 7) ^ (n & 7)) * 16);
                        *reinterpret_cast<uint4*>(smem + Cfg::OFF_BHI + off) = hi;
                        *reinterpret_cast<uint4*>(smem + Cfg::OFF_BLO + off) = lo;
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (threadIdx.x == 0) {
                const uint32_t ahi = smem_u32(smem + Cfg::OFF_AHI), alo = smem_u32(smem + Cfg::OFF_ALO);
                const uint32_t bhi = smem_u32(smem + Cfg::OFF_BHI), blo = smem_u32(smem + Cfg::OFF_BLO);
                uint32_t accumulate = kh > 0 ? 1u : 0u;
#pragma unroll 1
                for (int pass = 0; pass < 3; ++pass) {   // lo*hi, hi*lo, hi*hi: small terms first
                    const uint32_t a_base = (pass == 0) ? alo : ahi;
                    const uint32_t b_base = (pass == 1) ? blo : bhi;
#pragma unroll 1
                    for (int ks = 0; ks < RT_KH / 8; ++ks) {
                        const uint32_t a_addr = a_base + (uint32_t)(ks >> 2) * (uint32_t)(RT_TILE * 128) + (uint32_t)(ks & 3) * 32u;
                        const uint32_t b_addr = b_base + (uint32_t)(ks >> 2) * (uint32_t)(HID * 128) + (uint32_t)(ks & 3) * 32u;
                        rt_mma_ss(tmem_base, tc_b_desc(a_addr), tc_b_desc(b_addr), Cfg::IDESC, accumulate);
                        accumulate = 1;
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_mma) : "memory");
            }
            ++commits;
        }
        if (!alive) break;
        // the tile's accumulator is complete
        if (!tc_wait(bar_mma, (commits - 1) & 1u, abort_flag, status, 61)) { alive = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (warp < 4) {   // thread = graph (tensor-memory lane 32*warp + lane)
            float acc[RT_MAX_C];
#pragma unroll
            for (int c = 0; c < RT_MAX_C; ++c) acc[c] = 0.f;
            const uint32_t row_addr = tmem_base + ((uint32_t)(32 * warp) << 16);
#pragma unroll 1
            for (int h0 = 0; h0 < HID; h0 += 16) {
                uint32_t v[16];
                tc_ld_cols16(row_addr + (uint32_t)h0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float hv = relu_ref(__uint_as_float(v[i]));
                    const float* w2 = W2s + (h0 + i) * C;
#pragma unroll
                    for (int c = 0; c < RT_MAX_C; ++c)
                        if (c < C) acc[c] = fmaf(hv, w2[c], acc[c]);
                }
            }
            const int m = 32 * warp + lane;
            if (m < ng) {
                float mx = acc[0];
                int best = 0;
#pragma unroll
                for (int c = 1; c < RT_MAX_C; ++c)
                    if (c < C && acc[c] > mx) { mx = acc[c]; best = c; }
                float sum = 0.f;
#pragma unroll
                for (int c = 0; c < RT_MAX_C; ++c)
                    if (c < C) sum += expf(acc[c] - mx);
#pragma unroll
                for (int c = 0; c < RT_MAX_C; ++c)
                    if (c < C) {
                        logits[(g0 + m) * C + c] = acc[c];
                        if (probs) probs[(g0 + m) * C + c] = expf(acc[c] - mx) / sum;
                    }
                if (pred) pred[g0 + m] = best;
            }
        }
        // the accumulator is overwritten by the next tile's first MMA
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(HID) : "memory");
}

}  // namespace

bool s2v_readout_tc_supported(const s2v_ctx* ctx, int64_t G, int d, int hidden, int C)
{
    // A launch lasts at least the latency of one tile (about 23 us), which the mma.sync form (32-graph tiles, four CTAs
    // per SM) undercuts on small batches: 0.019 - 0.021 ms at 2,048 - 4,096 graphs, but 0.033 ms at 8,192 and 0.039 ms
    // at 16,384.
    const int64_t min_graphs = ctx->tc_mode == 2 ? 512 : 6144;
    return ctx->tc_mode != 0 && G >= min_graphs && (d == 64 || d == 128) && (hidden == 128 || hidden == 256) && C >= 1 && C <= RT_MAX_C &&
           RtCfg<256>::SMEM_BYTES <= ctx->smem_optin;
}

int s2v_launch_readout_tc(s2v_ctx* ctx, cudaStream_t st, int64_t G, int d, int hidden, int C, const float* Y, const float* W1,
                          const float* W2, float* logits, float* probs, int32_t* pred)
{
    if (!s2v_readout_tc_supported(ctx, G, d, hidden, C)) return S2V_ERR_UNSUPPORTED;
    const int64_t tiles = (G + RT_TILE - 1) / RT_TILE;
    const unsigned grid = (unsigned)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
    if (hidden == 256) {
        S2V_CUDA_OK(ctx, cudaFuncSetAttribute(readout_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RtCfg<256>::SMEM_BYTES));
        readout_tc_kernel<256><<<grid, RT_THREADS, RtCfg<256>::SMEM_BYTES, st>>>(G, d, C, Y, W1, W2, logits, probs, pred, ctx->dstatus_dev);
    } else {
        S2V_CUDA_OK(ctx, cudaFuncSetAttribute(readout_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RtCfg<128>::SMEM_BYTES));
        readout_tc_kernel<128><<<grid, RT_THREADS, RtCfg<128>::SMEM_BYTES, st>>>(G, d, C, Y, W1, W2, logits, probs, pred, ctx->dstatus_dev);
    }
    S2V_CHECK_LAUNCH(ctx, "readout_tc_kernel");
    return S2V_OK;
}
