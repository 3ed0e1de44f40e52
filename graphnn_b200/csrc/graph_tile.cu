// The whole structure2vec classifier up to the pooled graph embeddings in ONE kernel, for batches of
// small graphs (every graph at most 128 nodes, one-hot node tags, latent dimension 128):
//
//     H0   = ReLU(W_in[tag])                      Hl+1 = ReLU((A * Hl) * W + W_in[tag]),  l = 0..L-1
//     Y[g] = sum of HL over the nodes of graph g  (or their mean)
//
// i.e. examples/graph_classification/src/kernel_mean_field.cpp:31-44 of the reference.  A batch of
// small graphs is block diagonal, so a tile of whole graphs never needs a row of another tile: the
// node embeddings of a tile stay in shared memory across all L levels and only the pooled [G x d]
// matrix goes to HBM (the per-level kernels write and re-read [N x d] every level).
//
// Tiles.  A planning kernel packs consecutive graphs greedily into tiles of at most 128 nodes (and at
// most 128 graphs) and writes the list of (first graph, end graph) pairs; a graph larger than a tile is
// reported in the status word and truncated.
//
// One persistent 544-thread CTA per SM: sixteen worker warps + one MMA-issue warp.
//   * The dense stage runs TRANSPOSED on the tensor cores: out^T [d x nodes] = W^T [d x d] * S^T, so the
//     constant operand W^T (TF32 head and tail) is loaded ONCE per CTA into tensor memory as the A
//     operand, and the per-tile operand S = A * H (neighbour sums, [nodes x d], row-major) is exactly the
//     K-major B operand the tensor core reads from shared memory: no transposition anywhere.
//   * Gather: eight lanes own one node row and 32 feature columns (one 128-byte line) of it; they add
//     the neighbour rows from the shared H tile in CSR order, split the sum into TF32 head and tail and
//     store both into an operand buffer in the 128-byte-swizzle layout (head rows 0..127, tail rows
//     128..255).  A level is four such chunks of 32 features through two operand buffers.
//   * MMAs per chunk and K step: W_hi * [S_hi ; S_lo] as ONE instruction with N = 256 (columns 0..127 of
//     the accumulator collect the large term, 128..255 the small term hi*lo) and W_lo * S_hi with
//     N = 128 onto columns 128..255.  32 instructions per level instead of 48, and the small terms never
//     meet the large one before the epilogue adds the two halves in fp32.
//   * Epilogue: thread = output feature (tensor-memory lane), 32 node columns per worker:
//     tcgen05.ld, large + small + W_in[tag], ReLU, back into the H tile (conflict-free 128-byte rows).
//   * After a tile's last level the worker warps sum its graphs in node order and write Y.
// A CTA keeps TWO tiles resident (two "streams", each with its own H tile and CSR slice) and splits its sixteen
// worker warps into two groups of eight, one per stream.  A group runs its tile through the levels on its own
// (gather four chunks -> wait for the MMAs -> epilogue -> group barrier -> next level; pooling; next tile); the two
// groups share the two operand buffers, the MMA-issue warp and the single accumulator (256 of the 512
// tensor-memory columns; the other 256 hold W^T), which serve the level-jobs in the fixed order
//     A.0  B.0  A.1  B.1 ...
// While one group waits -- for its MMAs, for a barrier, for the global loads of its next tile -- the other group's
// warps have work, and the tensor pipe runs one stream's MMAs during the other stream's epilogue and gathers.
// The accumulator is handed over by an "accumulator read" barrier as soon as a group has drained it into its H
// tile (raw sums); the X term and the ReLU are applied in a second, row-wise pass that is off the MMA's path.
// Every wait is an mbarrier try_wait with a poll limit; on a time-out the kernel records
// S2V_ERR_DEVICE_TIMEOUT, raises a CTA-wide flag, frees its tensor memory and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace
{

constexpr int GT_NODES = 128;                    // node rows per tile
constexpr int GT_D = 128;                        // latent dimension = MMA M
constexpr int GT_WORKERS = 16;                   // worker warps
constexpr int GT_GROUP = 8;                      // worker warps per stream (two per tensor-memory lane quarter)
constexpr int GT_THREADS = (GT_WORKERS + 1) * 32;
constexpr int GT_ROWS_PER_WARP = GT_NODES / GT_GROUP;            // rows of a worker in the gather and the row-wise passes: 16
constexpr int GT_PASSES = GT_ROWS_PER_WARP / 4;                  // gather: four rows side by side per pass
constexpr int GT_NODES_PER_SLOT = GT_NODES / (GT_GROUP / 4);     // accumulator node columns drained by a worker: 64
constexpr int GT_CHUNKS = 4;                     // K chunks of 32 features (one swizzle line per node row)
constexpr int GT_SBUF = 2;                       // operand buffers
constexpr int GT_LC_CAP = 1536;                  // non-zeros of a tile cached in shared memory
constexpr size_t GT_S_BYTES = 256 * 128;         // one operand buffer: 128 head rows + 128 tail rows, 128 bytes each
constexpr size_t GT_H_BYTES = sizeof(float) * GT_NODES * GT_D;
// per-stream arrays
constexpr size_t GT_ST_LVAL = 0;
constexpr size_t GT_ST_REC = GT_ST_LVAL + sizeof(float) * GT_LC_CAP;     // uint4 per row: shared-memory offsets of its first four neighbour rows
constexpr size_t GT_ST_LRP = GT_ST_REC + 16 * GT_NODES;
constexpr size_t GT_ST_TAGS = GT_ST_LRP + sizeof(int) * 132;
constexpr size_t GT_ST_GOFF = GT_ST_TAGS + sizeof(int) * GT_NODES;
constexpr size_t GT_ST_INFO = GT_ST_GOFF + sizeof(int) * 132;           // 8 ints describing the tile
constexpr size_t GT_ST_LCOL = GT_ST_INFO + 32;                           // local column indices are bytes
constexpr size_t GT_ST_BYTES = (GT_ST_LCOL + GT_LC_CAP + 15) / 16 * 16;
constexpr size_t GT_OFF_S = 0;
constexpr size_t GT_OFF_H = GT_OFF_S + GT_SBUF * GT_S_BYTES;
constexpr size_t GT_OFF_ST = GT_OFF_H + 2 * GT_H_BYTES;
constexpr size_t GT_OFF_ZERO = GT_OFF_ST + 2 * GT_ST_BYTES;              // one row of zeros: the "neighbour" of unused gather slots
constexpr size_t GT_OFF_BAR = GT_OFF_ZERO + sizeof(float) * GT_D;
constexpr size_t GT_SMEM_BYTES = GT_OFF_BAR + 128 + 1024;                 // + barriers/flags + alignment slack
static_assert(GT_SMEM_BYTES <= 227 * 1024, "shared memory map exceeds the 227 KB a CTA may use");
// tensor memory columns
constexpr uint32_t GT_TM_WHI = 0, GT_TM_WLO = 128, GT_TM_ACC = 256;
// instruction descriptors: D = f32, A = B = tf32, both K-major, M = 128, N = 256 / 128
constexpr uint32_t GT_IDESC_BASE = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(128 >> 4) << 24);
constexpr uint32_t GT_IDESC_N256 = GT_IDESC_BASE | ((uint32_t)(256 >> 3) << 17);
constexpr uint32_t GT_IDESC_N128 = GT_IDESC_BASE | ((uint32_t)(128 >> 3) << 17);

// mbarriers.  An mbarrier wait names a phase by its parity only, so a waiter must never be two phases away from the
// barrier; the two worker groups run independently, therefore every barrier a group WAITS on is the group's own and
// sees exactly the phases that group waits for, in order.
enum {
    GB_FULL0 = 0,               // +b      : operand buffer b holds a chunk (eight arrivals, the producing group's warps)
    GB_EMPTY0 = 2,              // +2g + b : the MMAs that read operand buffer b are complete and group g uses it next (tcgen05.commit)
    GB_ACC_FULL0 = 6,           // +g      : the MMAs of a level-job of group g are complete (tcgen05.commit)
    GB_ACC_READ = 8,            // the accumulator has been drained (eight arrivals, the draining group's warps)
    GB_GSYNC0 = 9,              // +g      : barrier of the eight worker warps of group g
    GB_COUNT = 11
};
static_assert(GT_SBUF == 2, "barrier numbering assumes two operand buffers");

// ------------------------------------------------------------------ tile planning
constexpr int PLAN_SEG = 8192;      // graphs handled per pass of the single planning CTA
constexpr int PLAN_THREADS = 1024;
constexpr size_t PLAN_SMEM = sizeof(int) * 3 * (PLAN_SEG + 1) + (PLAN_SEG + 1) + 64;

// Greedy packing of consecutive graphs into tiles, in parallel.  For every graph i the end of the tile that
// would START at i is found by binary search in the offsets (next[i]); the tile starts actually used are
// the orbit of graph 0 under `next`, marked by pointer doubling (after k rounds every start within 2^k
// tiles of the front is marked); a block-wide scan compacts them.  Passes of PLAN_SEG graphs; a tile never
// spans two passes.
__global__ void __launch_bounds__(PLAN_THREADS) gt_plan_kernel(int64_t G, const int32_t* __restrict__ graph_ptr,
                                                              int2* __restrict__ tile_range, int* __restrict__ tile_count,
                                                              s2v_device_status* status)
{
    extern __shared__ int plan_sm[];
    int* gp = plan_sm;
    int* jmp_a = gp + PLAN_SEG + 1;
    int* jmp_b = jmp_a + PLAN_SEG + 1;
    unsigned char* mark = reinterpret_cast<unsigned char*>(jmp_b + PLAN_SEG + 1);
    __shared__ int warp_sum[32];
    __shared__ int seg_total;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int tiles_done = 0;
    for (int64_t g0 = 0; g0 < G; g0 += PLAN_SEG) {
        const int n = (int)((G - g0) < PLAN_SEG ? (G - g0) : PLAN_SEG);
        for (int i = tid; i <= n; i += PLAN_THREADS) gp[i] = graph_ptr[g0 + i];
        __syncthreads();
        // end of the tile that starts at graph i: the largest j <= min(n, i + 128) with gp[j] - gp[i] <= 128
        auto next_of = [&](int i) -> int {
            if (i >= n) return n;
            int lo = i, hi = (n < i + GT_NODES) ? n : i + GT_NODES;
            const int lim = gp[i] + GT_NODES;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (gp[mid] <= lim && gp[mid] >= gp[i]) lo = mid; else hi = mid - 1;
            }
            return lo;
        };
        for (int i = tid; i <= n; i += PLAN_THREADS) {
            int nx = next_of(i);
            if (i < n && nx == i) {      // graph i alone does not fit a tile: reported, and truncated by the consumer
                nx = i + 1;
                status->code = S2V_ERR_UNSUPPORTED;
                status->where = 4;
            }
            jmp_a[i] = nx;
            mark[i] = (i == 0) ? 1 : 0;
        }
        __syncthreads();
        int* cur = jmp_a;
        int* nxt = jmp_b;
        for (int span = 1; span <= n; span <<= 1) {
            for (int i = tid; i <= n; i += PLAN_THREADS) {
                if (mark[i]) mark[cur[i]] = 1;          // only ever writes 1 to tile starts: the race is benign
                nxt[i] = cur[cur[i]];
            }
            __syncthreads();
            int* t = cur; cur = nxt; nxt = t;
        }
        // compaction: thread t owns graphs [t*per, (t+1)*per)
        const int per = (n + PLAN_THREADS - 1) / PLAN_THREADS;
        const int b = tid * per < n ? tid * per : n;
        const int e = (b + per) < n ? (b + per) : n;
        int cnt = 0;
        for (int i = b; i < e; ++i) cnt += mark[i];
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_sum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sum[lane];
            int wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += v;
            }
            warp_sum[lane] = wi - w;    // exclusive
            if (lane == 31) seg_total = wi;
        }
        __syncthreads();
        int k = tiles_done + warp_sum[warp] + incl - cnt;
        for (int i = b; i < e; ++i)
            if (mark[i]) {
                int nx = next_of(i);
                if (nx == i) nx = i + 1;
                tile_range[k++] = make_int2((int)(g0 + i), (int)(g0 + nx));
            }
        tiles_done += seg_total;
        __syncthreads();   // shared arrays are reused by the next pass
    }
    if (tid == 0) *tile_count = tiles_done;
}

// ------------------------------------------------------------------ the tile kernel
// a node tag outside [0, n) is replaced by 0 and remembered; the kernel reports it once, when it ends
__device__ __forceinline__ int gt_checked_tag(int v, int n, int& bad)
{
    const bool out = (unsigned)v >= (unsigned)n;
    bad |= out ? 1 : 0;
    return out ? 0 : v;
}

__device__ __forceinline__ float4 relu4(float4 v)
{
    return make_float4(relu_ref(v.x), relu_ref(v.y), relu_ref(v.z), relu_ref(v.w));
}

template <bool HAS_VAL>
__global__ void __launch_bounds__(GT_THREADS, 1)
s2v_graph_tile_kernel(const int2* __restrict__ tile_range, const int* __restrict__ tile_count_p,
                      const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ col_idx,
                      const float* __restrict__ val, const int32_t* __restrict__ graph_ptr,
                      const int32_t* __restrict__ tags, int num_tags, const float* __restrict__ W_in,
                      const float* __restrict__ W, const float* __restrict__ P, int levels, int pool_average, float* __restrict__ Y,
                      float* __restrict__ embed_out, s2v_device_status* status)
{
    const int num_tiles = *tile_count_p;
    if ((int)blockIdx.x >= num_tiles) return;   // the whole CTA leaves before it owns anything
    extern __shared__ unsigned char gt_smem_raw[];
    unsigned char* smem = gt_smem_raw + ((1024u - (smem_u32(gt_smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GT_OFF_BAR);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + GT_OFF_BAR + 8 * GB_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + GT_OFF_BAR + 8 * GB_COUNT + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    int bad_index = 0;   // a tag outside the table was met (reported once, at the end)
    const uint32_t s_addr0 = smem_u32(smem + GT_OFF_S);

    if (threadIdx.x == 0) {
        for (int b = 0; b < GT_SBUF; ++b) tc_mbar_init(bar(GB_FULL0 + b), GT_GROUP);
        for (int e = 0; e < 4; ++e) tc_mbar_init(bar(GB_EMPTY0 + e), 1);
        tc_mbar_init(bar(GB_ACC_FULL0), 1);
        tc_mbar_init(bar(GB_ACC_FULL0 + 1), 1);
        tc_mbar_init(bar(GB_ACC_READ), GT_GROUP);
        tc_mbar_init(bar(GB_GSYNC0), GT_GROUP);
        tc_mbar_init(bar(GB_GSYNC0 + 1), GT_GROUP);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (threadIdx.x < GT_D) reinterpret_cast<float*>(smem + GT_OFF_ZERO)[threadIdx.x] = 0.f;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int q = warp & 3;                                  // tensor-memory lane quarter of this warp
    const uint32_t lane_base = (uint32_t)(32 * q) << 16;
    if (warp < GT_WORKERS) {
        // W^T into tensor memory: lane m = output feature, column k = input feature; A[m][k] = W[k][m].
        // Warp w: features 32q..32q+31, k in [32*(w/4), 32*(w/4)+32).  Loads are coalesced across the lanes.
        const int m = 32 * q + lane;
        const int k0 = 32 * (warp >> 2);
        float wv[32];
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) wv[kk] = __ldg(W + (int64_t)(k0 + kk) * GT_D + m);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                hi[c] = tf32_rn(wv[8 * h + c]);
                lo[c] = tf32_rn(wv[8 * h + c] - __uint_as_float(hi[c]));
            }
            tc_st_cols8(tmem_base + lane_base + GT_TM_WHI + (uint32_t)(k0 + 8 * h), hi);
            tc_st_cols8(tmem_base + lane_base + GT_TM_WLO + (uint32_t)(k0 + 8 * h), lo);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // This CTA's tiles blockIdx.x + i * gridDim.x, i = 0 .. my_tiles-1, go alternately to stream 0 and stream 1.
    const int my_tiles = (num_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1;
    const int n_lj0 = ((my_tiles + 1) >> 1) * levels, n_lj1 = (my_tiles >> 1) * levels;   // level-jobs per stream
    const int n_steps = 2 * (n_lj0 > n_lj1 ? n_lj0 : n_lj1);

    if (warp < GT_WORKERS) {
        // =========================== worker warps: group s serves stream s ===========================
        const int s = warp / GT_GROUP, gw = warp % GT_GROUP;       // my stream, my place in its group
        const int j = gw >> 2;                                      // which half of the node columns I drain
        const int gtix = threadIdx.x - s * (GT_GROUP * 32);        // 0 .. 255 within the group
        const int g4 = lane >> 3, sl = lane & 7;     // gather: row within a pass of four, 16-byte piece of the 128-byte line
        const float4* __restrict__ Win4 = reinterpret_cast<const float4*>(W_in);
        unsigned char* const sb = smem + GT_OFF_ST + (size_t)s * GT_ST_BYTES;
        unsigned char* const hbase = smem + GT_OFF_H + (size_t)s * GT_H_BYTES;
        float* const lval = reinterpret_cast<float*>(sb + GT_ST_LVAL);
        uint4* const rec = reinterpret_cast<uint4*>(sb + GT_ST_REC);
        int* const lrp = reinterpret_cast<int*>(sb + GT_ST_LRP);
        int* const tag_s = reinterpret_cast<int*>(sb + GT_ST_TAGS);
        int* const goff = reinterpret_cast<int*>(sb + GT_ST_GOFF);
        int* const info = reinterpret_cast<int*>(sb + GT_ST_INFO);
        unsigned char* const lcol = sb + GT_ST_LCOL;
        float* const Hs = reinterpret_cast<float*>(hbase);
        float4* const H4s = reinterpret_cast<float4*>(hbase);
        uint32_t gs_phase = 0;                       // completed phases of my group's barrier
        bool alive = true;
        // arrive at the group barrier and wait for the other seven warps (bounded)
        auto gsync = [&](int site) -> bool {
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(bar(GB_GSYNC0 + s));
            const bool ok = tc_wait(bar(GB_GSYNC0 + s), gs_phase & 1u, abort_flag, status, site);
            ++gs_phase;
            return ok;
        };
        // level-jobs are served in the order A.0 B.0 A.1 B.1 ...: my k-th level-job is step 2k + s, and the number of
        // level-jobs served before step t is what both groups and the MMA warp derive buffer indices and parities from
        auto jobs_before = [&](int t) -> uint32_t {
            const int a0 = (t + 1) >> 1, a1 = t >> 1;
            return (uint32_t)((a0 < n_lj0 ? a0 : n_lj0) + (a1 < n_lj1 ? a1 : n_lj1));
        };
        const int my_tile_count = s == 0 ? (my_tiles + 1) >> 1 : my_tiles >> 1;
        int my_lj = 0;                               // level-jobs this group has started
        uint32_t empty_seen[2] = {0u, 0u};           // phases of my "buffer b free for me" barriers already waited for

        for (int ti = 0; ti < my_tile_count && alive; ++ti) {
            // ---- the tile enters the stream: its CSR slice, tags, graph offsets, H0, and the per-row gather records
            const int tile = (int)blockIdx.x + (2 * ti + s) * (int)gridDim.x;
            const int2 tr = tile_range[tile];
            const int node0 = __ldg(graph_ptr + tr.x);
            int nrows = __ldg(graph_ptr + tr.y) - node0;
            if (nrows > GT_NODES) nrows = GT_NODES;   // an oversized graph was reported by the planner; stay inside the tile
            if (nrows < 0) nrows = 0;
            int ngr = tr.y - tr.x;
            if (ngr > GT_NODES) ngr = GT_NODES;
            const int32_t base = __ldg(row_ptr + node0);
            int nnz = __ldg(row_ptr + node0 + nrows) - base;
            if (nnz < 0) nnz = 0;
            const bool cached = nnz <= GT_LC_CAP;      // uniform over the group
            if (gtix == 0) {
                info[0] = node0; info[1] = nrows; info[2] = ngr; info[3] = tr.x; info[4] = base; info[5] = nnz;
            }
            if (gtix <= GT_NODES) {
                int v = __ldg(row_ptr + node0 + (gtix < nrows ? gtix : nrows)) - base;
                lrp[gtix] = v < 0 ? 0 : (v > nnz ? nnz : v);
            }
            if (gtix < GT_NODES) tag_s[gtix] = gtix < nrows ? gt_checked_tag(__ldg(tags + node0 + gtix), num_tags, bad_index) : 0;
            if (gtix <= ngr) {
                int v = __ldg(graph_ptr + tr.x + gtix) - node0;
                goff[gtix] = v < 0 ? 0 : (v > nrows ? nrows : v);
            }
            if (cached) {
                for (int e = gtix; e < nnz; e += GT_GROUP * 32) {
                    int c = __ldg(col_idx + base + e) - node0;
                    if ((unsigned)c >= (unsigned)nrows) {   // an edge that leaves the tile: not a batch of separate graphs
                        status->code = S2V_ERR_BAD_CSR;
                        status->where = 5;
                        c = 0;
                    }
                    lcol[e] = (unsigned char)c;
                    if (HAS_VAL) lval[e] = __ldg(val + base + e);
                }
            }
            if (!P) {   // H0 = ReLU(W_in[tag]); `levels` MMA levels follow
#pragma unroll 4
                for (int rr = 0; rr < GT_ROWS_PER_WARP; ++rr) {
                    const int r = GT_ROWS_PER_WARP * gw + rr;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (r < nrows) v = relu4(__ldg(Win4 + (int64_t)gt_checked_tag(__ldg(tags + node0 + r), num_tags, bad_index) * 32 + lane));
                    H4s[r * 32 + lane] = v;
                }
            }
            if (!gsync(30)) { alive = false; break; }
            if (P) {
                // The first level needs no product: H0 has one distinct row per tag, so (sum_t H0[col t]) * W is a sum of
                // rows of P = ReLU(W_in) * W (row num_tags of P is zero: unused slots add it).  The tile starts at
                // H1 = ReLU(sum_t P[tag[col t]] + W_in[tag]) and `levels` counts the MMA levels that follow.
                const float4* __restrict__ P4 = reinterpret_cast<const float4*>(P);
                constexpr int GT_P1_ROWS = 2;   // rows whose table loads are in flight together (more spills registers)
#pragma unroll 1
                for (int r4 = 0; r4 < GT_ROWS_PER_WARP; r4 += GT_P1_ROWS) {
                    int pt[GT_P1_ROWS][4], dg[GT_P1_ROWS], bg[GT_P1_ROWS];
#pragma unroll
                    for (int a = 0; a < GT_P1_ROWS; ++a) {
                        const int r = GT_ROWS_PER_WARP * gw + r4 + a;
                        bg[a] = lrp[r];
                        dg[a] = r < nrows ? lrp[r + 1] - bg[a] : 0;
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            int c = 0;
                            if (u < dg[a]) {
                                if (cached) c = lcol[bg[a] + u];
                                else {
                                    c = __ldg(col_idx + base + bg[a] + u) - node0;
                                    if ((unsigned)c >= (unsigned)nrows) c = 0;   // reported when the gather records are built
                                }
                            }
                            pt[a][u] = u < dg[a] ? tag_s[c] : num_tags;
                        }
                    }
                    float4 pv[GT_P1_ROWS][4], xv[GT_P1_ROWS];
#pragma unroll
                    for (int a = 0; a < GT_P1_ROWS; ++a) {
#pragma unroll
                        for (int u = 0; u < 4; ++u) pv[a][u] = __ldg(P4 + pt[a][u] * 32 + lane);
                        xv[a] = __ldg(Win4 + tag_s[GT_ROWS_PER_WARP * gw + r4 + a] * 32 + lane);
                    }
#pragma unroll
                    for (int a = 0; a < GT_P1_ROWS; ++a) {
                        const int r = GT_ROWS_PER_WARP * gw + r4 + a;
                        float4 acc;
                        if (HAS_VAL) {
                            float w[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) w[u] = u < dg[a] ? (cached ? lval[bg[a] + u] : __ldg(val + base + bg[a] + u)) : 0.f;
                            acc = make_float4(w[0] * pv[a][0].x, w[0] * pv[a][0].y, w[0] * pv[a][0].z, w[0] * pv[a][0].w);
#pragma unroll
                            for (int u = 1; u < 4; ++u) {
                                acc.x = fmaf(w[u], pv[a][u].x, acc.x); acc.y = fmaf(w[u], pv[a][u].y, acc.y);
                                acc.z = fmaf(w[u], pv[a][u].z, acc.z); acc.w = fmaf(w[u], pv[a][u].w, acc.w);
                            }
                        } else {   // adds in CSR order; an unused slot adds the row of zeros
                            acc = make_float4((((pv[a][0].x + pv[a][1].x) + pv[a][2].x) + pv[a][3].x), (((pv[a][0].y + pv[a][1].y) + pv[a][2].y) + pv[a][3].y),
                                              (((pv[a][0].z + pv[a][1].z) + pv[a][2].z) + pv[a][3].z), (((pv[a][0].w + pv[a][1].w) + pv[a][2].w) + pv[a][3].w));
                        }
                        for (int t = 4; t < dg[a]; ++t) {   // rows with more than four neighbours
                            int c;
                            if (cached) c = lcol[bg[a] + t];
                            else {
                                c = __ldg(col_idx + base + bg[a] + t) - node0;
                                if ((unsigned)c >= (unsigned)nrows) c = 0;
                            }
                            const float4 pp = __ldg(P4 + tag_s[c] * 32 + lane);
                            if (HAS_VAL) {
                                const float w = cached ? lval[bg[a] + t] : __ldg(val + base + bg[a] + t);
                                acc.x = fmaf(w, pp.x, acc.x); acc.y = fmaf(w, pp.y, acc.y); acc.z = fmaf(w, pp.z, acc.z); acc.w = fmaf(w, pp.w, acc.w);
                            } else {
                                acc.x += pp.x; acc.y += pp.y; acc.z += pp.z; acc.w += pp.w;
                            }
                        }
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (r < nrows) v = make_float4(relu_ref(acc.x + xv[a].x), relu_ref(acc.y + xv[a].y), relu_ref(acc.z + xv[a].z), relu_ref(acc.w + xv[a].w));
                        H4s[r * 32 + lane] = v;
                    }
                }
            }
            // gather record of row r: offsets (from the shared-memory base) of the rows of its first four neighbours;
            // unused slots point at the row of zeros, so the gather needs no test per slot
            if (gtix < GT_NODES) {
                const int beg = lrp[gtix], deg = lrp[gtix + 1] - beg;
                uint32_t off[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    off[u] = (uint32_t)GT_OFF_ZERO;
                    if (u < deg) {
                        int c;
                        if (cached) c = lcol[beg + u];
                        else {
                            c = __ldg(col_idx + base + beg + u) - node0;
                            if ((unsigned)c >= (unsigned)nrows) {
                                status->code = S2V_ERR_BAD_CSR;
                                status->where = 5;
                                c = 0;
                            }
                        }
                        off[u] = (uint32_t)(GT_OFF_H + (size_t)s * GT_H_BYTES) + (uint32_t)c * 512u;
                    }
                }
                rec[gtix] = make_uint4(off[0], off[1], off[2], off[3]);
            }
            if (!gsync(35)) { alive = false; break; }

            // ---- my gather rows (GT_ROWS_PER_WARP*gw + 4p + g4): neighbour offsets and store offset, kept for the whole tile
            uint32_t na[GT_PASSES][4], da[GT_PASSES];
            bool lng = false;
#pragma unroll
            for (int p = 0; p < GT_PASSES; ++p) {
                const int r = GT_ROWS_PER_WARP * gw + 4 * p + g4;
                const uint4 rc = rec[r];
                na[p][0] = rc.x + (uint32_t)sl * 16u; na[p][1] = rc.y + (uint32_t)sl * 16u;
                na[p][2] = rc.z + (uint32_t)sl * 16u; na[p][3] = rc.w + (uint32_t)sl * 16u;
                // row r of the K-major 128-byte-swizzle layout: 16-byte piece sl sits at sl ^ (r & 7)
                da[p] = (uint32_t)GT_OFF_S + (uint32_t)r * 128u + (uint32_t)((sl ^ (r & 7)) * 16);
                lng |= (lrp[r + 1] - lrp[r]) > 4;
            }
            const bool long_rows = __any_sync(0xffffffffu, lng);   // warp-uniform: some row of mine has more than four neighbours

            for (int lv = 0; lv < levels; ++lv) {
                const uint32_t lj = jobs_before(2 * my_lj + s);      // level-jobs served before mine
                ++my_lj;
                // -------------------------------- gather: S = A * H, split, into the operand buffers --------------------------------
#pragma unroll 1
                for (int c = 0; c < GT_CHUNKS; ++c) {
                    const uint32_t job = 4u * lj + (uint32_t)c;
                    const uint32_t b = job & 1u;
                    if (job >= (uint32_t)GT_SBUF) {   // the buffer was used before (by either group): wait until its MMAs are done
                        const uint32_t par = (b == 0u ? empty_seen[0]++ : empty_seen[1]++) & 1u;
                        if (!tc_wait(bar(GB_EMPTY0 + 2 * s + (int)b), par, abort_flag, status, 36)) {
                            alive = false;
                            break;
                        }
                    }
                    const unsigned char* hb = smem + (size_t)c * 128;
                    unsigned char* sbuf = smem + (size_t)b * GT_S_BYTES;
#pragma unroll
                    for (int p = 0; p < GT_PASSES; ++p) {
                        const float4 v0 = *reinterpret_cast<const float4*>(hb + na[p][0]);
                        const float4 v1 = *reinterpret_cast<const float4*>(hb + na[p][1]);
                        const float4 v2 = *reinterpret_cast<const float4*>(hb + na[p][2]);
                        const float4 v3 = *reinterpret_cast<const float4*>(hb + na[p][3]);
                        float4 acc;
                        const int r = GT_ROWS_PER_WARP * gw + 4 * p + g4;
                        if (HAS_VAL) {
                            const int gb = lrp[r], gd = lrp[r + 1] - gb;
                            float a[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) a[u] = u < gd ? (cached ? lval[gb + u] : __ldg(val + base + gb + u)) : 0.f;
                            acc = make_float4(a[0] * v0.x, a[0] * v0.y, a[0] * v0.z, a[0] * v0.w);
                            acc.x = fmaf(a[1], v1.x, acc.x); acc.y = fmaf(a[1], v1.y, acc.y); acc.z = fmaf(a[1], v1.z, acc.z); acc.w = fmaf(a[1], v1.w, acc.w);
                            acc.x = fmaf(a[2], v2.x, acc.x); acc.y = fmaf(a[2], v2.y, acc.y); acc.z = fmaf(a[2], v2.z, acc.z); acc.w = fmaf(a[2], v2.w, acc.w);
                            acc.x = fmaf(a[3], v3.x, acc.x); acc.y = fmaf(a[3], v3.y, acc.y); acc.z = fmaf(a[3], v3.z, acc.z); acc.w = fmaf(a[3], v3.w, acc.w);
                        } else {   // adds in CSR order; an unused slot adds the row of zeros
                            acc = make_float4((((v0.x + v1.x) + v2.x) + v3.x), (((v0.y + v1.y) + v2.y) + v3.y),
                                              (((v0.z + v1.z) + v2.z) + v3.z), (((v0.w + v1.w) + v2.w) + v3.w));
                        }
                        if (long_rows) {   // rows with more than four neighbours
                            const int gb = lrp[r], gd = lrp[r + 1] - gb;
                            const unsigned char* hrow = hbase + (size_t)c * 128 + (size_t)sl * 16;
                            for (int t = 4; t < gd; ++t) {
                                int n;
                                if (cached) n = lcol[gb + t];
                                else {
                                    n = __ldg(col_idx + base + gb + t) - node0;
                                    if ((unsigned)n >= (unsigned)nrows) n = 0;
                                }
                                const float4 vv = *reinterpret_cast<const float4*>(hrow + (size_t)n * 512);
                                if (HAS_VAL) {
                                    const float a = cached ? lval[gb + t] : __ldg(val + base + gb + t);
                                    acc.x = fmaf(a, vv.x, acc.x); acc.y = fmaf(a, vv.y, acc.y);
                                    acc.z = fmaf(a, vv.z, acc.z); acc.w = fmaf(a, vv.w, acc.w);
                                } else {
                                    acc.x += vv.x; acc.y += vv.y; acc.z += vv.z; acc.w += vv.w;
                                }
                            }
                        }
                        uint4 hi, lo;
                        tc_split(acc.x, hi.x, lo.x);
                        tc_split(acc.y, hi.y, lo.y);
                        tc_split(acc.z, hi.z, lo.z);
                        tc_split(acc.w, hi.w, lo.w);
                        *reinterpret_cast<uint4*>(sbuf + da[p]) = hi;
                        *reinterpret_cast<uint4*>(sbuf + da[p] + 128 * 128) = lo;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // my stores -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) tc_mbar_arrive(bar(GB_FULL0 + b));
                }
                if (!alive) break;
                // -------------------------------- drain: accumulator -> raw sums in the H tile --------------------------------
                // X rows of my first row-wise rows are fetched now and stay in flight across the wait
                float4 xr[8];
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) xr[rr] = __ldg(Win4 + (int64_t)tag_s[GT_ROWS_PER_WARP * gw + rr] * 32 + lane);
                if (!tc_wait(bar(GB_ACC_FULL0 + s), (uint32_t)(my_lj - 1) & 1u, abort_flag, status, 31)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                {   // feature = my lane (32q + lane), node columns GT_NODES_PER_SLOT*j ..
                    const uint32_t acc_addr = tmem_base + lane_base + GT_TM_ACC + (uint32_t)(GT_NODES_PER_SLOT * j);
                    float* hcol = Hs + (GT_NODES_PER_SLOT * j) * GT_D + 32 * q + lane;
#pragma unroll
                    for (int h = 0; h < GT_NODES_PER_SLOT / 16; ++h) {
                        uint32_t big[16], sml[16];
                        tc_ld_cols16(acc_addr + (uint32_t)(16 * h), big);
                        tc_ld_cols16(acc_addr + 128u + (uint32_t)(16 * h), sml);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (h == GT_NODES_PER_SLOT / 16 - 1) {
                            // my block of the accumulator is in registers: the next level-job's MMAs may overwrite it
                            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                            __syncwarp();
                            if (lane == 0) tc_mbar_arrive(bar(GB_ACC_READ));
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i) hcol[(16 * h + i) * GT_D] = __uint_as_float(big[i]) + __uint_as_float(sml[i]);
                    }
                }
                if (!gsync(32)) { alive = false; break; }
                // -------------------------------- row-wise pass: H = ReLU(raw + X), lanes across the features --------------------------------
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) {
                        const int r = GT_ROWS_PER_WARP * gw + 8 * half + rr;
                        const float4 z = H4s[r * 32 + lane];
                        const float4 x = xr[rr];
                        H4s[r * 32 + lane] = make_float4(relu_ref(z.x + x.x), relu_ref(z.y + x.y), relu_ref(z.z + x.z), relu_ref(z.w + x.w));
                        if (half == 0) xr[rr] = __ldg(Win4 + (int64_t)tag_s[GT_ROWS_PER_WARP * gw + 8 + rr] * 32 + lane);
                    }
                }
                if (!gsync(33)) { alive = false; break; }           // H complete for the next level's gather / the pooling
            }
            if (!alive) break;
            // -------------------------------- pooling and (optionally) the node embeddings --------------------------------
            for (int k = gw; k < ngr; k += GT_GROUP) {
                const int nb = goff[k], ne = goff[k + 1];
                const float inv = pool_average ? (float)(1.0 / (double)(ne - nb)) : 1.0f;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int n = nb; n < ne; ++n) {
                    const float4 v = H4s[n * 32 + lane];
                    if (pool_average) {
                        acc.x = fmaf(inv, v.x, acc.x); acc.y = fmaf(inv, v.y, acc.y);
                        acc.z = fmaf(inv, v.z, acc.z); acc.w = fmaf(inv, v.w, acc.w);
                    } else {
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                }
                reinterpret_cast<float4*>(Y)[(int64_t)(tr.x + k) * 32 + lane] = acc;
            }
            if (embed_out) {
#pragma unroll 4
                for (int rr = 0; rr < GT_ROWS_PER_WARP; ++rr) {
                    const int r = GT_ROWS_PER_WARP * gw + rr;
                    if (r < nrows) reinterpret_cast<float4*>(embed_out)[(int64_t)(node0 + r) * 32 + lane] = H4s[r * 32 + lane];
                }
            }
            if (!gsync(34)) { alive = false; break; }       // the tile's shared arrays are rewritten by the next prologue
        }
    } else {
        // =========================== MMA-issue warp ===========================
        uint32_t jobs = 0, lj = 0;
        bool alive = true;
        auto has_job = [&](int k) { return (k >> 1) < ((k & 1) == 0 ? n_lj0 : n_lj1); };
        for (int k = 0; k < n_steps && alive; ++k) {
            if (!has_job(k)) continue;
            const int g = k & 1;                       // the group this level-job belongs to
            int k2 = k + 1;                            // the next level-job and its group (-1: none)
            while (k2 < n_steps && !has_job(k2)) ++k2;
            const int g_next = k2 < n_steps ? (k2 & 1) : -1;
#pragma unroll 1
            for (int c = 0; c < GT_CHUNKS; ++c) {
                const uint32_t b = jobs & 1u;
                if (!tc_wait(bar(GB_FULL0 + b), (jobs >> 1) & 1u, abort_flag, status, 34)) { alive = false; break; }
                // the previous level-job's accumulator must be in the workers' hands before it is overwritten
                if (c == 0 && lj > 0 && !tc_wait(bar(GB_ACC_READ), (lj - 1u) & 1u, abort_flag, status, 37)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const uint32_t sb = s_addr0 + b * (uint32_t)GT_S_BYTES;
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        const uint32_t ks = (uint32_t)(4 * c + s);
                        const uint64_t bd = tc_b_desc(sb + 32u * (uint32_t)s);
                        // W_hi * [S_hi ; S_lo]: large term -> columns 0..127, hi*lo -> columns 128..255
                        tc_mma(tmem_base + GT_TM_ACC, tmem_base + GT_TM_WHI + 8u * ks, bd, GT_IDESC_N256, ks != 0u);
                        // W_lo * S_hi onto the small-term half
                        tc_mma(tmem_base + GT_TM_ACC + 128u, tmem_base + GT_TM_WLO + 8u * ks, bd, GT_IDESC_N128, 1u);
                    }
                    // this buffer is used next by the chunk two jobs on: the same group's (c < 2) or the next level-job's
                    const int g_user = c < 2 ? g : g_next;
                    if (g_user >= 0)
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                         bar(GB_EMPTY0 + 2 * g_user + (int)b))
                                     : "memory");
                    if (c == GT_CHUNKS - 1)
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar(GB_ACC_FULL0 + g))
                                     : "memory");
                }
                __syncwarp();
                ++jobs;
            }
            ++lj;
        }
    }

    // ---- teardown: everyone is done with tensor memory before it is released
    if (bad_index) {
        status->code = S2V_ERR_INVALID_ARG;
        status->where = 3;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}

}  // namespace

size_t s2v_graph_tiles_plan_bytes(int64_t num_graphs)
{
    return sizeof(int2) * (size_t)(num_graphs > 0 ? num_graphs : 0) + 256;
}

// Plans the tiles and runs the tile kernel: Y [G x 128] = pooled last-level embeddings.  `plan` is device
// scratch of s2v_graph_tiles_plan_bytes(G) bytes, 256-byte aligned.
int s2v_launch_graph_tiles(s2v_ctx* ctx, cudaStream_t st, int64_t G, const int32_t* row_ptr, const int32_t* col_idx,
                           const float* val, const int32_t* graph_ptr, const int32_t* tags, int num_tags,
                           const float* W_in, const float* W, int levels, int pool_average, void* plan, float* P_scratch,
                           float* Y, float* embed_out)
{
    if (GT_SMEM_BYTES > ctx->smem_optin || PLAN_SMEM > ctx->smem_optin) return S2V_ERR_UNSUPPORTED;
    // With a scratch for the product table ((num_tags + 1) x 128 floats) the first level is done in the tile prologue
    // as a sum of table rows, and the kernel runs levels - 1 MMA levels.
    const float* P = nullptr;
    int mma_levels = levels;
    if (P_scratch && levels >= 1) {
        const int rc = s2v_launch_first_table_product(ctx, st, num_tags, GT_D, W_in, W, P_scratch, true);
        if (rc != S2V_OK) return rc;
        P = P_scratch;
        mma_levels = levels - 1;
    }
    int* tile_count = static_cast<int*>(plan);
    int2* tile_range = reinterpret_cast<int2*>(static_cast<unsigned char*>(plan) + 256);
    S2V_CUDA_OK(ctx, cudaFuncSetAttribute(gt_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PLAN_SMEM));
    gt_plan_kernel<<<1, PLAN_THREADS, PLAN_SMEM, st>>>(G, graph_ptr, tile_range, tile_count, ctx->dstatus_dev);
    S2V_CHECK_LAUNCH(ctx, "gt_plan_kernel");
    int64_t blocks = G < ctx->sm_count ? G : ctx->sm_count;   // at most one tile per graph; idle CTAs leave at once
    if (blocks < 1) blocks = 1;
    if (val) {
        auto kern = s2v_graph_tile_kernel<true>;
        S2V_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM_BYTES));
        kern<<<(unsigned)blocks, GT_THREADS, GT_SMEM_BYTES, st>>>(tile_range, tile_count, row_ptr, col_idx, val, graph_ptr, tags,
                                                                  num_tags, W_in, W, P, mma_levels, pool_average, Y, embed_out,
                                                                  ctx->dstatus_dev);
    } else {
        auto kern = s2v_graph_tile_kernel<false>;
        S2V_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM_BYTES));
        kern<<<(unsigned)blocks, GT_THREADS, GT_SMEM_BYTES, st>>>(tile_range, tile_count, row_ptr, col_idx, val, graph_ptr, tags,
                                                                  num_tags, W_in, W, P, mma_levels, pool_average, Y, embed_out,
                                                                  ctx->dstatus_dev);
    }
    S2V_CHECK_LAUNCH(ctx, "s2v_graph_tile_kernel");
    return S2V_OK;
}
