// Fused structure2vec level for d = 64 and d = 128 with the dense stage on the 5th-generation
// tensor cores (tcgen05.mma, accumulators and the A operand in tensor memory).
//
//     out[i,:] = ReLU( (sum_{t in row i} val[t] * H[col_idx[t],:]) * W + X[i,:] )
//
// Why a second form of the kernel: at d = 128 the product [rows x 128] * [128 x 128] in
// 3xTF32 costs 3 * 2 * 128^2 flop per row against 1.5 KB of compulsory traffic; the
// warp-level mma.sync path (level.cu) is bounded by the legacy tensor rate there, well
// above the HBM time.  tcgen05 runs the same 3xTF32 product several times faster and
// needs no registers for the operands, so the kernel goes back to being memory-bound.
//
// One persistent 544-thread CTA per SM, 128-row tiles.  Sixteen symmetric worker warps and
// one MMA-issue warp, connected by mbarriers:
//
//   worker w (quarter q = w % 4 of the tensor-memory lanes, slot j = w / 4), per tile:
//     gather   : rows 32q + 8j .. +7 of the tile: the CSR slice comes through 64-entry index windows in
//                shared memory (first window prefetched a tile ahead, its rows prefetched into L2), neighbour
//                rows are summed in CSR order as one flat software-pipelined stream per group
//                of d/4 lanes (8 loads in flight per lane, no branch per non-zero: row ends come from a
//                bit mask built with warp votes) into a fp32 staging tile [128 x d];
//     operand  : once the quarter's four warps are done: thread = row, columns [d/4*j, d/4*(j+1)):
//                split every value into a TF32 head and tail and store both into tensor
//                memory (tcgen05.st);
//     epilogue : the PREVIOUS tile's accumulator, same rows and columns: tcgen05.ld, transpose
//                through the warp's own (now idle) slab of the staging tile, add X, apply ReLU
//                and store whole row segments;
//   MMA warp  : when all sixteen operand blocks are in tensor memory, one thread issues the
//                3 * d/8 MMAs (lo*hi, hi*lo, hi*hi over K = d in steps of 8) against W^T, which
//                sits in shared memory split the same way in the K-major 128-byte-swizzle
//                layout, into one of two accumulators, and commits them to an mbarrier.
//
// The MMAs of tile i overlap the epilogue of tile i-1 and the gather of tile i+1.  Every wait
// is bounded: on a time-out the kernel records S2V_ERR_DEVICE_TIMEOUT, raises a CTA-wide
// abort flag, drains, frees its tensor memory and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace
{

constexpr int TC_TILE = 128;           // rows per tile = MMA M
constexpr int TC_GW = 16;              // worker warps, four per tensor-memory lane quarter
constexpr int TC_MW = 1;               // MMA-issue warp (one elected lane)
constexpr int TC_THREADS = (TC_GW + TC_MW) * 32;
constexpr int TC_ROWS_PER_GW = TC_TILE / TC_GW;   // 8
constexpr int TC_U = 4;

// Per-width configuration and shared memory map (offsets from a 1024-byte aligned base).
template <int D>
struct TcCfg {
    static constexpr int IDX_CAP = (D == 64) ? 128 : 64;   // index-window entries per worker: 64 per lane group
    static constexpr int STAGE_STRIDE = D + 4;         // floats; an odd number of float4 per row: thread-per-row float4 reads are conflict-free
    static constexpr size_t OFF_BHI = 0;
    static constexpr size_t OFF_BLO = OFF_BHI + sizeof(float) * D * D;
    static constexpr size_t OFF_STAGE = OFF_BLO + sizeof(float) * D * D;
    static constexpr size_t STAGE_BYTES = sizeof(float) * TC_TILE * STAGE_STRIDE;
    static constexpr size_t OFF_GW = OFF_STAGE + STAGE_BYTES;
    static constexpr size_t GW_BYTES = 2 * (sizeof(int) * IDX_CAP + sizeof(int) * 32);   // double-buffered indices + row offsets
    static constexpr size_t OFF_BAR = OFF_GW + GW_BYTES * TC_GW;
    static constexpr size_t SMEM_BYTES = OFF_BAR + 256 + 1024;   // + barriers/flags + alignment slack
    // tensor memory columns: A head, A tail, two accumulators
    static constexpr uint32_t TM_AHI = 0, TM_ACC = 2 * D;   // A tail at TM_AHI + D, accumulator b at TM_ACC + b*D
    static_assert(4 * D <= 512, "tensor memory has 512 columns");
    // a worker's slab of the staging tile (8 rows) doubles as its 32 x d/4 transposition buffer
    static_assert(TC_ROWS_PER_GW * STAGE_STRIDE >= 32 * (D / 4), "transposition buffer does not fit the slab");
    // instruction descriptor: D = f32, A = B = tf32, both K-major, M = 128, N = D
    static constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(TC_TILE >> 4) << 24);
};

// mbarriers.  FULL/SFREE exist per tensor-memory lane quarter (32 rows = four workers).
enum {
    BAR_FULL0 = 0,                   // +q : the quarter's 32 rows of the staging tile are written
    BAR_SFREE0 = 4,                  // +q : the quarter's rows have been read back by all four workers
    BAR_AREADY = 8,                  // all sixteen blocks of the A operand are in tensor memory
    BAR_MMA0, BAR_MMA1,              // the MMAs into accumulator buffer 0 / 1 are complete
    BAR_DFREE0, BAR_DFREE1,          // accumulator buffer 0 / 1 has been read by all sixteen workers
    BAR_COUNT
};

template <int D, bool HAS_VAL, int XMODE, bool HSRC_TABLE>
__global__ void __launch_bounds__(TC_THREADS, 1)
s2v_level_tc_kernel(int64_t n_rows, int64_t num_tiles, const int32_t* __restrict__ row_ptr,
                    const int32_t* __restrict__ col_idx, const float* __restrict__ val, const float* __restrict__ H,
                    const float* __restrict__ W, const float* __restrict__ X, const int32_t* __restrict__ x_index,
                    int n_table, float* __restrict__ out, s2v_device_status* status)
{
    extern __shared__ unsigned char tc_smem_raw[];
    // 1024-byte alignment as an OFFSET from the shared array: a pointer rebuilt from an integer would lose
    // its address space and every access through it would become a generic load/store
    unsigned char* smem = tc_smem_raw + ((1024u - (smem_u32(tc_smem_raw) & 1023u)) & 1023u);
    using Cfg = TcCfg<D>;
    constexpr int IDX_CAP = Cfg::IDX_CAP, STAGE_STRIDE = Cfg::STAGE_STRIDE;
    float* Bhi = reinterpret_cast<float*>(smem + Cfg::OFF_BHI);
    float* Blo = reinterpret_cast<float*>(smem + Cfg::OFF_BLO);
    float* stage = reinterpret_cast<float*>(smem + Cfg::OFF_STAGE);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 8 * BAR_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 8 * BAR_COUNT + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    // ---- set-up: barriers, tensor memory, W^T split into TF32 head/tail in the MMA layout
    if (threadIdx.x == 0) {
        for (int qq = 0; qq < 4; ++qq) {
            tc_mbar_init(bar(BAR_FULL0 + qq), TC_GW / 4);
            tc_mbar_init(bar(BAR_SFREE0 + qq), TC_GW / 4);
        }
        tc_mbar_init(bar(BAR_AREADY), TC_GW);
        tc_mbar_init(bar(BAR_MMA0), 1);
        tc_mbar_init(bar(BAR_MMA1), 1);
        tc_mbar_init(bar(BAR_DFREE0), TC_GW);
        tc_mbar_init(bar(BAR_DFREE1), TC_GW);
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
    // All loads of a thread's tasks are issued before the first conversion (one memory latency, not one per task).
    {
        constexpr int NTASK = D * D / 4;
        constexpr int PER = (NTASK + TC_THREADS - 1) / TC_THREADS;
        float wv[PER][4];
#pragma unroll
        for (int t = 0; t < PER; ++t) {
            const int e = threadIdx.x + t * TC_THREADS;
            const int n = e % D, kq = e / D;   // k = 4*kq .. 4*kq+3
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) wv[t][jj] = (e < NTASK) ? __ldg(W + (int64_t)(4 * kq + jj) * D + n) : 0.f;
        }
#pragma unroll
        for (int t = 0; t < PER; ++t) {
            const int e = threadIdx.x + t * TC_THREADS;
            if (e < NTASK) {
                const int n = e % D, kq = e / D;
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    hi[jj] = tf32_rn(wv[t][jj]);
                    lo[jj] = tf32_rn(wv[t][jj] - __uint_as_float(hi[jj]));
                }
                const int kb = kq >> 3, chunk = kq & 7;
                const size_t off = (size_t)kb * (D * 128) + (size_t)n * 128 + (size_t)((chunk ^ (n & 7)) * 16);
                *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(Bhi) + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(Blo) + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t TM_AHI = tmem_base + Cfg::TM_AHI, TM_ACC = tmem_base + Cfg::TM_ACC;

    const int my_tiles = (int)((num_tiles > (int64_t)blockIdx.x) ? (num_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0);

    if (warp < TC_GW) {
        // =========================== worker warps ===========================
        constexpr int CW = D / 4;                        // operand / accumulator columns handled per worker
        constexpr int C4 = CW / 4;                       // float4 per row of my column block: 8 (d = 128) or 4 (d = 64)
        constexpr int RPI = 32 / C4;                     // rows per store instruction in the epilogue: 4 or 8
        constexpr int NRR = 32 / RPI;                    // store instructions per column block: 8 or 4
        const int q = warp & 3, j = warp >> 2;
        const int row0 = 32 * q + TC_ROWS_PER_GW * j;    // my first row within the tile
        const uint32_t lane_base = (uint32_t)(32 * q) << 16;
        unsigned char* gbase = smem + Cfg::OFF_GW + Cfg::GW_BYTES * warp;
        int* const idx_base = reinterpret_cast<int*>(gbase);   // two buffers of IDX_CAP indices + 32 row offsets
        constexpr int IDX_BUF = IDX_CAP + 32;
        const float4* __restrict__ H4 = reinterpret_cast<const float4*>(H);
        const float4* __restrict__ X4 = reinterpret_cast<const float4*>(X);
        constexpr int LPR = D / 4;                       // lanes that cover one row with float4
        constexpr int RPG = TC_ROWS_PER_GW / (32 / LPR); // consecutive rows one lane group streams through
        constexpr int IPL = IDX_CAP / 32;                // prefetched indices per lane
        const int sub = lane / LPR, sl = lane % LPR;
        float* const slab = stage + (size_t)row0 * STAGE_STRIDE;   // my 8 rows; also my transposition buffer
        const int ersub = lane / C4, ec4 = lane % C4;    // epilogue: row within a store instruction, float4 column
        // Row offsets are fetched two tiles ahead and column indices one tile ahead, into
        // registers while the current tile is gathered, so no tile waits on that chain.
        auto load_rp = [&](int it) -> int32_t {
            int64_t rpi = ((int64_t)blockIdx.x + (int64_t)it * gridDim.x) * TC_TILE + row0 + lane;
            if (rpi > n_rows) rpi = n_rows;
            return lane <= TC_ROWS_PER_GW ? tc_ld_early(row_ptr + rpi) : 0;
        };
        // X row index of "my" epilogue row (lane = row within the quarter)
        auto load_xi = [&](int it) -> int {
            const int64_t mr = ((int64_t)blockIdx.x + (int64_t)it * gridDim.x) * TC_TILE + 32 * q + lane;
            return (XMODE == 2 && it < my_tiles && mr < n_rows) ? tc_ld_early(x_index + mr) : 0;   // range-checked where it is used, a tile later
        };
        constexpr int G = 32 / LPR;        // lane groups per warp (1 at d = 128, 2 at d = 64)
        constexpr int WSZ = IDX_CAP / G;   // index window per lane group: 64 entries
        static_assert(WSZ == 64, "one 64-bit row-end mask per window");
        // Column indices of segment k (64 non-zeros per lane group) of a warp-tile whose row offsets sit in
        // lanes 0..8 as `rel` (relative to `base_abs`): entry w of the buffer belongs to group w / 64.
        // (r_mid, r_end: the offsets of rows RPG and 8, i.e. where group 0 and the last group end.)
        auto window_index = [&](int jj, int r_mid, int r_end, int32_t base_abs, int k) -> int {
            const int w = lane + 32 * jj;
            const int g = w / WSZ, p_ = w % WSZ;
            const int gs_ = (g == 0) ? 0 : r_mid, ge_ = (g == G - 1) ? r_end : r_mid;
            const int e = gs_ + WSZ * k + p_;
            return e < ge_ ? tc_ld_early(col_idx + base_abs + e) : 0;
        };
        int32_t rp_next = load_rp(0);      // row offsets of the tile whose indices are fetched next
        int32_t rp_next2 = load_rp(1);
        int32_t base = 0;
        {   // tile 0: fill buffer 0 directly
            base = __shfl_sync(0xffffffffu, rp_next, 0);
            const int rel = rp_next - base;
            if (lane <= TC_ROWS_PER_GW) idx_base[IDX_CAP + lane] = rel;
#pragma unroll
            for (int jj = 0; jj < IPL; ++jj)
            {
                const int c_ = window_index(jj, __shfl_sync(0xffffffffu, rel, RPG), __shfl_sync(0xffffffffu, rel, TC_ROWS_PER_GW), base, 0);
                idx_base[lane + 32 * jj] = HSRC_TABLE ? tc_table_row(__ldg(x_index + c_), n_table) : c_;
            }
            rp_next = rp_next2;
        }
        int xi_prev = 0;                   // X row index of my row in tile it-1 (the tile whose epilogue runs in iteration it)
        __syncwarp();
        // iteration `it`: gather + operand of tile it (it < my_tiles), epilogue of tile it-1 (it >= 1)
        for (int it = 0; it <= my_tiles; ++it) {
            const bool have_tile = it < my_tiles;
            const int xi_this = load_xi(it);   // used one iteration later: a whole tile to arrive
            if (have_tile) {
                // -------------------------------- gather --------------------------------
                int* idx_s = idx_base + (it & 1) * IDX_BUF;
                const int* rp_s = idx_s + IDX_CAP;
                // prefetch (registers): offsets of tile it+2, first index window of tile it+1
                rp_next2 = load_rp(it + 2);
                const int32_t base1 = __shfl_sync(0xffffffffu, rp_next, 0);
                const int rel1 = rp_next - base1;
                int idx_pref[IPL];
                const int r1_mid = __shfl_sync(0xffffffffu, rel1, RPG), r1_end = __shfl_sync(0xffffffffu, rel1, TC_ROWS_PER_GW);
#pragma unroll
                for (int jj = 0; jj < IPL; ++jj) idx_pref[jj] = window_index(jj, r1_mid, r1_end, base1, 0);
                // Row structure of my warp-tile, worked out by the warp together: lane r+1 speaks for row r.
                const int rel = lane <= TC_ROWS_PER_GW ? rp_s[lane] : 0;
                const int relp = __shfl_up_sync(0xffffffffu, rel, 1);
                const int rr_ = lane - 1;                                 // my row as a speaker
                const bool isrow = lane >= 1 && lane <= TC_ROWS_PER_GW;
                const int rg = isrow ? rr_ / RPG : 0;                     // my row's lane group
                const int gbeg = __shfl_sync(0xffffffffu, rel, rg * RPG); // first non-zero of that group
                const bool ne_row = isrow && rel > relp;
                const int pos = rel - 1 - gbeg;                           // my row's last non-zero, counted within its group
                const uint32_t ne_bits = __ballot_sync(0xffffffffu, ne_row) >> 1;        // bit r: row r is not empty
                const int r_lo = sub * RPG;
                const int r_mid = __shfl_sync(0xffffffffu, rel, RPG), r_end = __shfl_sync(0xffffffffu, rel, TC_ROWS_PER_GW);
                const int gs = (sub == 0) ? 0 : r_mid;                    // my group's non-zeros: [gs, gs + cnt)
                const int cnt = ((sub == G - 1) ? r_end : r_mid) - gs;
                const int cmax = (G == 1) ? r_end : max(r_mid, r_end - r_mid);
                const int nseg = (cmax + WSZ - 1) / WSZ;                  // 64-non-zero segments (warp-uniform)
                // nxtmap: 4 bits per row, the next non-empty row of the group (15: none)
                uint32_t nxtmap = 0;
                {
                    const uint32_t ne_g_sp = (ne_bits >> (rg * RPG)) & ((1u << RPG) - 1u);   // speaker view: my row's group
                    const int rin = rr_ - rg * RPG;                                        // my row within its group
                    const uint32_t above = isrow ? (ne_g_sp >> (rin + 1)) : 0u;
                    const uint32_t nxt_r = above ? (uint32_t)(rin + __ffs(above)) : 15u;
#pragma unroll
                    for (int gg = 0; gg < G; ++gg) {
                        const uint32_t nm = __reduce_or_sync(0xffffffffu, (isrow && rg == gg) ? (nxt_r << (4 * rin)) : 0u);
                        if (gg == sub) nxtmap = nm;
                    }
                }
                const uint32_t ne_g = (ne_bits >> r_lo) & ((1u << RPG) - 1u);              // worker view: my lane group
#pragma unroll
                for (int r = 0; r < RPG; ++r)   // empty rows are zero-filled up front
                    if (!((ne_g >> r) & 1u))
                        *reinterpret_cast<float4*>(slab + (size_t)(r_lo + r) * STAGE_STRIDE + sl * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                int frow = ne_g ? (__ffs(ne_g) - 1) : 15;   // the row being summed (within my group)
                const int* win = idx_s + WSZ * sub;          // my group's index window
                const float* vp = HAS_VAL ? val + base + gs : nullptr;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float4 va[TC_U], vb[TC_U];
                float wa[TC_U], wb[TC_U];
                int tag_pref[IPL];
                auto publish_next = [&]() {
                    // Pull the neighbour rows of the NEXT tile's first window into L2 now, a whole tile ahead of
                    // their use (a prefetch holds no register), and publish that window in the other buffer.
                    int* nb = idx_base + ((it + 1) & 1) * IDX_BUF;
#pragma unroll
                    for (int jj = 0; jj < IPL; ++jj) {
                        if (!HSRC_TABLE && idx_pref[jj] != 0) {   // (0 also marks an unused slot; row 0 needs no prefetch)
                            const char* rowp = reinterpret_cast<const char*>(H4 + (int64_t)idx_pref[jj] * LPR);
#pragma unroll
                            for (int l = 0; l < D * 4 / 128; ++l) asm volatile("prefetch.global.L2 [%0];" ::"l"(rowp + 128 * l));
                        }
                        // table form: the window holds the neighbour's table row, looked up here, a tile ahead
                        // (issued now, stored after the stream: see tag_pref below)
                        if (HSRC_TABLE) tag_pref[jj] = __ldg(x_index + idx_pref[jj]);   // range-checked when it is stored, after the stream
                        else nb[lane + 32 * jj] = idx_pref[jj];
                    }
                    if (lane <= TC_ROWS_PER_GW) nb[IDX_CAP + lane] = rel1;
                };
// HSRC_TABLE: the gather source is not a matrix but ReLU(table[x_index[col], :]) -- the first level of
// the classifier with one-hot inputs, where H0 = ReLU(W_in[tag]) need not be materialised.
// Slots past the segment's end load the segment's first neighbour again (a valid row, an L1 hit) and carry
// no end bit: only the last segment has such slots, after the group's last row was stored, and what they
// add to acc is never stored.
#define TC_LOADF(v, wt, p0)                                                                        \
    _Pragma("unroll") for (int u = 0; u < TC_U; ++u) {                                             \
        const bool pv = (p0) + u < seg_n;                                                          \
        const int c = pv ? win[(p0) + u] : cz;                                                     \
        if (HAS_VAL) wt[u] = pv ? __ldg(vp + WSZ * k + (p0) + u) : 0.f;                             \
        if (HSRC_TABLE) {   /* c is already the table row */                                       \
            const float4 xw = ld_nc_f4(X4 + (int64_t)c * LPR + sl);                                \
            v[u] = make_float4(relu_ref(xw.x), relu_ref(xw.y), relu_ref(xw.z), relu_ref(xw.w));    \
        } else {                                                                                   \
            v[u] = ld_nc_f4(H4 + (int64_t)c * LPR + sl);                                           \
        }                                                                                          \
    }
#define TC_CONSF(v, wt, p0)                                                                        \
    {                                                                                              \
        const uint32_t m4 = (uint32_t)em & 15u;                                                    \
        em >>= 4;                                                                                  \
        const uint32_t m4w = (G == 1) ? m4 : ((uint32_t)em_warp & 15u);   /* row ends of ANY lane group */ \
        if (G > 1) em_warp >>= 4;                                                                  \
        /* no row end among these four non-zeros in ANY lane group of the warp: sums only (the test is   \
           warp-uniform).  Measured: -3.3 % on the molecule input (d = 128, one group per warp), -2.2 % on   \
           the Erdos-Renyi d = 64 problem, -0.3 % on the protein input; testing only the lane's own group   \
           at d = 64 made the two groups diverge and cost 1.3 % there */                                   \
        if (m4w == 0u) {                                                                           \
            _Pragma("unroll") for (int u = 0; u < TC_U; ++u) {                                     \
                if (HAS_VAL) {                                                                     \
                    acc.x = fmaf(wt[u], v[u].x, acc.x); acc.y = fmaf(wt[u], v[u].y, acc.y);        \
                    acc.z = fmaf(wt[u], v[u].z, acc.z); acc.w = fmaf(wt[u], v[u].w, acc.w);        \
                } else {                                                                           \
                    acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;            \
                }                                                                                  \
            }                                                                                      \
        } else                                                                                     \
        _Pragma("unroll") for (int u = 0; u < TC_U; ++u) {                                         \
            if (HAS_VAL) {                                                                         \
                acc.x = fmaf(wt[u], v[u].x, acc.x); acc.y = fmaf(wt[u], v[u].y, acc.y);            \
                acc.z = fmaf(wt[u], v[u].z, acc.z); acc.w = fmaf(wt[u], v[u].w, acc.w);            \
            } else {                                                                               \
                acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;                \
            }                                                                                      \
            const bool last = (m4 >> u) & 1u;                                                      \
            if (last) *reinterpret_cast<float4*>(slab + (size_t)(r_lo + frow) * STAGE_STRIDE + sl * 4) = acc; \
            acc.x = last ? 0.f : acc.x; acc.y = last ? 0.f : acc.y;                                \
            acc.z = last ? 0.f : acc.z; acc.w = last ? 0.f : acc.w;                                \
            frow = last ? (int)((nxtmap >> (4 * frow)) & 15u) : frow;                              \
        }                                                                                          \
    }
                if (nseg == 0) publish_next();
#pragma unroll 1
                for (int k = 0; k < nseg; ++k) {
                    if (k > 0) {   // later windows are fetched on demand (rows this long amortise the latency)
                        __syncwarp();
#pragma unroll
                        for (int jj = 0; jj < IPL; ++jj) {
                            const int c_ = window_index(jj, r_mid, r_end, base, k);
                            idx_s[lane + 32 * jj] = HSRC_TABLE ? tc_table_row(__ldg(x_index + c_), n_table) : c_;
                        }
                        __syncwarp();
                    }
                    // "the p-th non-zero of this segment is the last of its row", per lane group
                    uint32_t em_lo = 0, em_hi = 0, any_lo = 0, any_hi = 0;
#pragma unroll
                    for (int gg = 0; gg < G; ++gg) {
                        const bool here = ne_row && rg == gg && (pos >> 6) == k;
                        const uint32_t lo = __reduce_or_sync(0xffffffffu, (here && (pos & 63) < 32) ? (1u << (pos & 31)) : 0u);
                        const uint32_t hi = __reduce_or_sync(0xffffffffu, (here && (pos & 63) >= 32) ? (1u << (pos & 31)) : 0u);
                        if (gg == sub) { em_lo = lo; em_hi = hi; }
                        any_lo |= lo;
                        any_hi |= hi;
                    }
                    unsigned long long em = ((unsigned long long)em_hi << 32) | em_lo;
                    unsigned long long em_warp = ((unsigned long long)any_hi << 32) | any_lo;   // the same for every lane of the warp
                    (void)em_warp;
                    const int seg_n = min(WSZ, cnt - WSZ * k);   // my group's non-zeros in this segment (may be <= 0)
                    if (seg_n > 0) {
                        const int cz = win[0];
                        int p = 0;
                        TC_LOADF(va, wa, 0)
                        TC_LOADF(vb, wb, TC_U)
                        if (k == 0) publish_next();
                        while (true) {
                            TC_CONSF(va, wa, p)
                            p += TC_U;
                            if (p >= seg_n) break;
                            TC_LOADF(va, wa, p + TC_U)
                            TC_CONSF(vb, wb, p)
                            p += TC_U;
                            if (p >= seg_n) break;
                            TC_LOADF(vb, wb, p + TC_U)
                        }
                    } else if (k == 0) {
                        publish_next();
                    }
                }
#undef TC_LOADF
#undef TC_CONSF
                if (HSRC_TABLE) {
                    int* nb = idx_base + ((it + 1) & 1) * IDX_BUF;
#pragma unroll
                    for (int jj = 0; jj < IPL; ++jj) nb[lane + 32 * jj] = tc_table_row(tag_pref[jj], n_table);
                }
                base = base1;
                rp_next = rp_next2;
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(bar(BAR_FULL0 + q));
            }
            // X term of tile it-1, my rows and columns: in flight across the waits below
            const int64_t prow0 = (((int64_t)blockIdx.x + (int64_t)(it - 1) * gridDim.x) * TC_TILE) + 32 * q;
            const int rows_left = it >= 1 ? (int)((n_rows - prow0) < 32 ? (n_rows - prow0) : 32) : 0;   // valid rows of my 32
            float4 x[NRR];
#pragma unroll
            for (int rr = 0; rr < NRR; ++rr) {
                const int rl = rr * RPI + ersub;
                x[rr] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (XMODE == 1 && rl < rows_left) x[rr] = ld_stream_f4(X4 + (prow0 + rl) * (D / 4) + C4 * j + ec4);
                if (XMODE == 2) {
                    const int xi = tc_table_row(__shfl_sync(0xffffffffu, xi_prev, rl), n_table);
                    if (rl < rows_left) x[rr] = ld_nc_f4(X4 + xi * (D / 4) + C4 * j + ec4);
                }
            }
            // The MMAs of tile it-1 are complete: the A operand may be overwritten, the accumulator read.
            if (it >= 1 && !tc_wait(bar(BAR_MMA0 + ((it - 1) & 1)), (uint32_t)(((it - 1) >> 1) & 1), abort_flag, status, 21)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (have_tile) {
                // -------------------------------- operand --------------------------------
                // the quarter's 32 rows are complete; thread = row, my CW columns -> TF32 head and tail
                if (!tc_wait(bar(BAR_FULL0 + q), (uint32_t)(it & 1), abort_flag, status, 20)) break;
                const float* my_row = stage + (size_t)(32 * q + lane) * STAGE_STRIDE + CW * j;
                const uint32_t tm_a = TM_AHI + lane_base + (uint32_t)(CW * j);
#pragma unroll
                for (int h = 0; h < CW / 8; ++h) {   // 8 columns at a time keeps the register count down
                    uint32_t hi[8], lo[8];
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const float4 v4 = *reinterpret_cast<const float4*>(my_row + 8 * h + 4 * c);
                        tc_split(v4.x, hi[4 * c + 0], lo[4 * c + 0]);
                        tc_split(v4.y, hi[4 * c + 1], lo[4 * c + 1]);
                        tc_split(v4.z, hi[4 * c + 2], lo[4 * c + 2]);
                        tc_split(v4.w, hi[4 * c + 3], lo[4 * c + 3]);
                    }
                    tc_st_cols8(tm_a + 8 * h, hi);
                    tc_st_cols8(tm_a + D + 8 * h, lo);
                }
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(bar(BAR_SFREE0 + q));   // my share of the staging quarter is read
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(bar(BAR_AREADY));   // my block of the A operand is in tensor memory
            }
            // my slab is free once the quarter's four workers have read it for tile `it`
            if (have_tile && !tc_wait(bar(BAR_SFREE0 + q), (uint32_t)(it & 1), abort_flag, status, 10)) break;
            if (it >= 1) {
                // -------------------------------- epilogue of tile it-1 --------------------------------
                // accumulator block -> my slab, transposed: [32 rows][C4 float4], float4 column XOR-swizzled by row
                const int b = (it - 1) & 1;
                float4* const tb = reinterpret_cast<float4*>(slab);
                const int wswz = (C4 == 8) ? (lane & 7) : ((lane >> 1) & 3);
#pragma unroll
                for (int h = 0; h < CW / 16; ++h) {   // 16 columns at a time keeps the register count down
                    uint32_t v[16];
                    tc_ld_cols16(TM_ACC + (uint32_t)(D * b) + lane_base + (uint32_t)(CW * j + 16 * h), v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        tb[lane * C4 + ((4 * h + c) ^ wswz)] = make_float4(__uint_as_float(v[4 * c]), __uint_as_float(v[4 * c + 1]),
                                                                          __uint_as_float(v[4 * c + 2]), __uint_as_float(v[4 * c + 3]));
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(bar(BAR_DFREE0 + b));   // my block of the accumulator is read
                float4* const out_t = reinterpret_cast<float4*>(out) + (prow0 + ersub) * (D / 4) + C4 * j + ec4;
#pragma unroll
                for (int rr = 0; rr < NRR; ++rr) {
                    const int rl = rr * RPI + ersub;
                    const int swz = (C4 == 8) ? (rl & 7) : ((rl >> 1) & 3);
                    const float4 o = tb[rl * C4 + (ec4 ^ swz)];
                    if (rl < rows_left) {
                        float4 r;
                        r.x = relu_ref(o.x + x[rr].x);
                        r.y = relu_ref(o.y + x[rr].y);
                        r.z = relu_ref(o.z + x[rr].z);
                        r.w = relu_ref(o.w + x[rr].w);
                        out_t[rr * RPI * (D / 4)] = r;
                    }
                }
                __syncwarp();   // the slab is rewritten by the next gather
            }
            xi_prev = xi_this;
        }
    } else {
        // =========================== MMA-issue warp ===========================
        for (int it = 0; it < my_tiles; ++it) {
            const int b = it & 1;
            // the whole A operand is in tensor memory, and the accumulator buffer has been read
            bool ok = tc_wait(bar(BAR_AREADY), (uint32_t)(it & 1), abort_flag, status, 22);
            if (ok && it >= 2) ok = tc_wait(bar(BAR_DFREE0 + b), (uint32_t)(((it - 2) >> 1) & 1), abort_flag, status, 23);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t d_tmem = TM_ACC + (uint32_t)(D * b);
                const uint32_t bhi = smem_u32(Bhi), blo = smem_u32(Blo);
                uint32_t accumulate = 0;
#pragma unroll 1
                for (int pass = 0; pass < 3; ++pass) {   // lo*hi, hi*lo, hi*hi: small terms first
                    const uint32_t a_base = (pass == 0) ? TM_AHI + D : TM_AHI;
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
        }
    }

    // ---- teardown: everyone is done with tensor memory before it is released
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}

// Self-test of the bounded wait, through tc_wait itself.  Two warps, two mbarriers that nothing ever arrives
// at.  Warp 0 waits with a small poll limit: its wait runs out, raises the abort flag and records
// S2V_ERR_DEVICE_TIMEOUT (site 98).  Warp 1 waits with a larger limit and must leave because it sees the
// flag, not because its own limit ran out.  If both happened the site is rewritten to 99.  The kernel
// returns normally: no trap, no fault, the context stays usable.
__global__ void tc_wait_selftest_kernel(s2v_device_status* status)
{
    __shared__ uint64_t never_arrives[2];
    __shared__ int abort_flag_s;
    __shared__ int saw_abort;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        tc_mbar_init(smem_u32(&never_arrives[0]), 1);
        tc_mbar_init(smem_u32(&never_arrives[1]), 1);
        abort_flag_s = 0;
        saw_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile int* abort_flag = &abort_flag_s;
    if (warp == 0) {
        tc_wait(smem_u32(&never_arrives[0]), 0, abort_flag, status, 98, 32);
    } else {
        const bool ok = tc_wait(smem_u32(&never_arrives[1]), 0, abort_flag, status, 97, 1 << 12);
        if (!ok && *abort_flag && status->where == 98 && threadIdx.x == 32) saw_abort = 1;
    }
    __syncthreads();
    if (threadIdx.x == 0 && saw_abort && status->code == S2V_ERR_DEVICE_TIMEOUT) status->where = 99;
}

template <int D, bool HAS_VAL, int XMODE, bool HSRC_TABLE = false>
int tc_launch(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, const int32_t* rp, const int32_t* ci, const float* val,
              const float* H, const float* W, const float* X, const int32_t* x_index, int n_table, float* out)
{
    auto kern = s2v_level_tc_kernel<D, HAS_VAL, XMODE, HSRC_TABLE>;
    constexpr size_t SMEM = TcCfg<D>::SMEM_BYTES;
    if (SMEM > ctx->smem_optin) return S2V_ERR_UNSUPPORTED;
    S2V_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    const int64_t num_tiles = (n_rows + TC_TILE - 1) / TC_TILE;
    int64_t blocks = num_tiles < ctx->sm_count ? num_tiles : ctx->sm_count;
    if (blocks < 1) blocks = 1;
    kern<<<(unsigned)blocks, TC_THREADS, SMEM, st>>>(n_rows, num_tiles, rp, ci, val, H, W, X, x_index, n_table, out,
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
                       const int32_t* x_index, int n_table, float* out)
{
    if (!H) {
        if (!table || !x_index) return S2V_ERR_UNSUPPORTED;
        return val ? tc_launch<D, true, 2, true>(ctx, st, n_rows, row_ptr, col_idx, val, nullptr, W, table, x_index, n_table, out)
                   : tc_launch<D, false, 2, true>(ctx, st, n_rows, row_ptr, col_idx, val, nullptr, W, table, x_index, n_table, out);
    }
    const int xmode = table ? 2 : (X ? 1 : 0);
    const float* xa = table ? table : X;
#define TC_GO(HV, XM) return tc_launch<D, HV, XM>(ctx, st, n_rows, row_ptr, col_idx, val, H, W, xa, x_index, n_table, out)
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
                        const float* table, const int32_t* x_index, int n_table, float* out)
{
    if (d == 128) return tc_dispatch<128>(ctx, st, n_rows, row_ptr, col_idx, val, H, W, X, table, x_index, n_table, out);
    if (d == 64) return tc_dispatch<64>(ctx, st, n_rows, row_ptr, col_idx, val, H, W, X, table, x_index, n_table, out);
    return S2V_ERR_UNSUPPORTED;
}

int s2v_launch_wait_selftest(s2v_ctx* ctx, cudaStream_t st)
{
    tc_wait_selftest_kernel<<<1, 64, 0, st>>>(ctx->dstatus_dev);
    S2V_CHECK_LAUNCH(ctx, "tc_wait_selftest_kernel");
    return S2V_OK;
}
