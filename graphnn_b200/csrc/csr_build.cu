// Node-to-node CSR from a directed edge list, on the device, bit-identical to the host builder
// (s2v_build_n2n_csr_host) and therefore to GraphStruct::AddEdge + Node2NodeMsgPass::InitCPUWeight of the
// reference (src/util/graph_struct.cpp:62-70, src/nn/msg_pass.cpp:46-67): row y lists the sources of the
// edges x -> y in the order the edges were added.
//
// A stable counting sort by destination:
//   1. count    : in-degree of every node (integer atomics: the counts do not depend on the order);
//   2. scan     : exclusive prefix sum of the counts = row_ptr (block scan, scan of the block totals, add);
//   3. place    : every edge takes the next free slot of its row (atomic cursor) and leaves its EDGE INDEX
//                 there -- the slots of a row are filled in an arbitrary order;
//   4. rank     : every edge counts the edge indices of its row that are smaller than its own; that rank
//                 is its position in insertion order, where it writes its source.  Rows are short in
//                 this domain (degree 2..30), so the count is a handful of cached loads per edge;
//   5. long rows: rows above CSR_LONG_ROW entries (listed by step 2) are left out of step 4 and sorted by
//                 edge index by one CTA each (bitonic network in global memory), so the cost never becomes quadratic.
// The result is deterministic although steps 1 and 3 use atomics.
#include "common.cuh"

namespace
{

constexpr int CSR_LONG_ROW = 512;
constexpr int SCAN_THREADS = 1024;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_BLOCK = SCAN_THREADS * SCAN_ITEMS;

__global__ void __launch_bounds__(256) csr_count_kernel(int64_t N, int64_t E, const int32_t* __restrict__ src,
                                                        const int32_t* __restrict__ dst, int32_t* __restrict__ cnt,
                                                        s2v_device_status* status)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += stride) {
        const int32_t y = dst[e], x = src[e];
        if ((uint32_t)y < (uint32_t)N && (uint32_t)x < (uint32_t)N)
            atomicAdd(cnt + y, 1);
        else {   // dropped and reported: the row offsets then no longer add up to E
            status->code = S2V_ERR_BAD_CSR;
            status->where = 6;
        }
    }
}

// block-wide exclusive scan of SCAN_BLOCK consecutive counts; the block total goes to block_sum[blockIdx.x]
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_tot, int& total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int w = warp_tot[lane];
        int wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        warp_tot[lane] = wi - w;
        if (lane == 31) warp_tot[32] = wi;
    }
    __syncthreads();
    total = warp_tot[32];
    const int r = warp_tot[warp] + incl - v;
    __syncthreads();   // warp_tot is reused by the caller's next scan
    return r;
}

__global__ void __launch_bounds__(SCAN_THREADS) csr_scan_blocks_kernel(int64_t N, const int32_t* __restrict__ cnt,
                                                                      int32_t* __restrict__ row_ptr,
                                                                      int32_t* __restrict__ block_sum)
{
    __shared__ int warp_tot[33];
    const int64_t i0 = (int64_t)blockIdx.x * SCAN_BLOCK + (int64_t)threadIdx.x * SCAN_ITEMS;
    int v[SCAN_ITEMS], s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; ++k) {
        v[k] = (i0 + k < N) ? cnt[i0 + k] : 0;
        s += v[k];
    }
    int total;
    int run = block_exclusive_scan(s, warp_tot, total);
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; ++k) {
        if (i0 + k < N) row_ptr[i0 + k] = run;   // still relative to the block; the offset is added below
        run += v[k];
    }
    if (threadIdx.x == 0) block_sum[blockIdx.x] = total;
}

// one CTA: exclusive scan of the block totals in place; block_sum[num_blocks] = grand total
__global__ void __launch_bounds__(SCAN_THREADS) csr_scan_totals_kernel(int num_blocks, int32_t* __restrict__ block_sum)
{
    __shared__ int warp_tot[33];
    int carry = 0;
    for (int b0 = 0; b0 < num_blocks; b0 += SCAN_THREADS) {
        const int i = b0 + threadIdx.x;
        const int v = i < num_blocks ? block_sum[i] : 0;
        int total;
        const int ex = block_exclusive_scan(v, warp_tot, total);
        if (i < num_blocks) block_sum[i] = carry + ex;
        carry += total;
    }
    if (threadIdx.x == 0) block_sum[num_blocks] = carry;
}

// adds the block offsets, writes row_ptr[N], clears the counters so that they can serve as the row cursors, and
// lists the rows above CSR_LONG_ROW entries (long_list[0] = how many, then the rows, in no particular order)
__global__ void __launch_bounds__(SCAN_THREADS) csr_scan_add_kernel(int64_t N, int num_blocks, const int32_t* __restrict__ block_sum,
                                                                   int32_t* __restrict__ row_ptr, int32_t* __restrict__ cnt,
                                                                   int32_t* __restrict__ long_list)
{
    const int off = block_sum[blockIdx.x];
    const int64_t i0 = (int64_t)blockIdx.x * SCAN_BLOCK + (int64_t)threadIdx.x * SCAN_ITEMS;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; ++k)
        if (i0 + k < N) {
            row_ptr[i0 + k] += off;
            if (cnt[i0 + k] > CSR_LONG_ROW) long_list[1 + atomicAdd(long_list, 1)] = (int32_t)(i0 + k);
            cnt[i0 + k] = 0;
        }
    if (blockIdx.x == 0 && threadIdx.x == 0) row_ptr[N] = block_sum[num_blocks];
}

__global__ void __launch_bounds__(256) csr_place_kernel(int64_t N, int64_t E, const int32_t* __restrict__ src,
                                                        const int32_t* __restrict__ dst, const int32_t* __restrict__ row_ptr,
                                                        int32_t* __restrict__ cursor, int32_t* __restrict__ slot_edge)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += stride) {
        const int32_t y = dst[e], x = src[e];
        if ((uint32_t)y < (uint32_t)N && (uint32_t)x < (uint32_t)N) slot_edge[row_ptr[y] + atomicAdd(cursor + y, 1)] = (int32_t)e;
    }
}

__global__ void __launch_bounds__(256) csr_rank_kernel(int64_t N, int64_t E, const int32_t* __restrict__ src,
                                                       const int32_t* __restrict__ dst, const int32_t* __restrict__ row_ptr,
                                                       const int32_t* __restrict__ slot_edge, int average,
                                                       int32_t* __restrict__ col_idx, float* __restrict__ val)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += stride) {
        const int32_t y = dst[e], x = src[e];
        if ((uint32_t)y >= (uint32_t)N || (uint32_t)x >= (uint32_t)N) continue;
        const int32_t b = row_ptr[y], en = row_ptr[y + 1];
        if (en - b > CSR_LONG_ROW) continue;   // sorted by csr_long_rows_kernel
        int rank = 0;
        for (int32_t p = b; p < en; ++p) rank += (slot_edge[p] < (int32_t)e) ? 1 : 0;
        col_idx[b + rank] = x;
        if (val) val[b + rank] = average ? (float)(1.0 / (double)(en - b)) : 1.0f;
    }
}

// Rows above CSR_LONG_ROW entries: one CTA per such row sorts the row's edge indices ascending, then writes
// the sources in that order.  The sort is a bitonic network over the next power of two in the form whose
// comparators all point the same way (stage k first compares every element with its mirror image inside the
// block of k, then runs the half-cleaners k/4, k/8, .. 1): with the positions past the row's end standing
// for +infinity no such element ever has to move, so comparators that touch them are simply skipped.
__global__ void __launch_bounds__(1024) csr_long_rows_kernel(const int32_t* __restrict__ long_list, const int32_t* __restrict__ src,
                                                             const int32_t* __restrict__ row_ptr, int32_t* __restrict__ slot_edge,
                                                             int average, int32_t* __restrict__ col_idx, float* __restrict__ val)
{
    const int n_long = long_list[0];
    for (int li = blockIdx.x; li < n_long; li += gridDim.x) {
        const int64_t row = long_list[1 + li];
        const int32_t b = row_ptr[row];
        const int n = row_ptr[row + 1] - b;
        int32_t* a = slot_edge + b;
        int m = 1;
        while (m < n) m <<= 1;
        auto compare_exchange = [&](int i, int l) {
            if (l > i && l < n) {
                const int32_t x = a[i], y = a[l];
                if (x > y) { a[i] = y; a[l] = x; }
            }
        };
        for (int k = 2; k <= m; k <<= 1) {
            for (int i = threadIdx.x; i < n; i += blockDim.x) compare_exchange(i, i ^ (k - 1));
            __syncthreads();
            for (int jj = k >> 2; jj > 0; jj >>= 1) {
                for (int i = threadIdx.x; i < n; i += blockDim.x) compare_exchange(i, i ^ jj);
                __syncthreads();
            }
        }
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            col_idx[b + i] = src[a[i]];
            if (val) val[b + i] = average ? (float)(1.0 / (double)n) : 1.0f;
        }
        __syncthreads();
    }
}

inline unsigned grid_for(s2v_ctx* ctx, int64_t items, int per_block, int per_sm)
{
    int64_t blocks = (items + per_block - 1) / per_block;
    const int64_t cap = (int64_t)ctx->sm_count * per_sm;
    if (blocks > cap) blocks = cap;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

extern "C" {

size_t s2v_build_n2n_csr_scratch_bytes(int64_t num_nodes, int64_t num_edges)
{
    if (num_nodes < 0 || num_edges < 0) return 0;
    const size_t blocks = (size_t)((num_nodes + SCAN_BLOCK - 1) / SCAN_BLOCK);
    return up256(sizeof(int32_t) * (size_t)num_nodes) + up256(sizeof(int32_t) * (size_t)num_edges) +
           up256(sizeof(int32_t) * (blocks + 1)) + up256(sizeof(int32_t) * ((size_t)num_edges / CSR_LONG_ROW + 2)) + 256;
}

int s2v_build_n2n_csr_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_nodes, int64_t num_edges, const int32_t* edge_src,
                          const int32_t* edge_dst, int average, void* scratch, size_t scratch_bytes, int32_t* row_ptr,
                          int32_t* col_idx, float* val)
{
    S2V_ENTER(ctx);
    const int64_t N = num_nodes, E = num_edges;
    if (N < 0 || E < 0 || !row_ptr) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "build_n2n_csr: bad shape or NULL row_ptr");
    if (E > 0 && (!edge_src || !edge_dst || !col_idx)) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "build_n2n_csr: NULL edge array");
    if (N >= (int64_t)INT32_MAX || E >= (int64_t)INT32_MAX) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "build_n2n_csr: int32 sizes only");
    if (!scratch || scratch_bytes < s2v_build_n2n_csr_scratch_bytes(N, E))
        return s2v_fail(ctx, S2V_ERR_WORKSPACE, "build_n2n_csr: scratch smaller than s2v_build_n2n_csr_scratch_bytes");
    cudaStream_t st = s2v_pick_stream(ctx, stream);
    if (N == 0) {
        S2V_CUDA_OK(ctx, cudaMemsetAsync(row_ptr, 0, sizeof(int32_t), st));
        return S2V_OK;
    }
    unsigned char* p = reinterpret_cast<unsigned char*>(up256(reinterpret_cast<uintptr_t>(scratch)));
    int32_t* cnt = reinterpret_cast<int32_t*>(p);
    int32_t* slot_edge = reinterpret_cast<int32_t*>(p + up256(sizeof(int32_t) * (size_t)N));
    int32_t* block_sum = reinterpret_cast<int32_t*>(p + up256(sizeof(int32_t) * (size_t)N) + up256(sizeof(int32_t) * (size_t)E));
    const int num_blocks = (int)((N + SCAN_BLOCK - 1) / SCAN_BLOCK);
    int32_t* long_list = reinterpret_cast<int32_t*>(reinterpret_cast<unsigned char*>(block_sum) + up256(sizeof(int32_t) * ((size_t)num_blocks + 1)));
    S2V_CUDA_OK(ctx, cudaMemsetAsync(cnt, 0, sizeof(int32_t) * (size_t)N, st));
    S2V_CUDA_OK(ctx, cudaMemsetAsync(long_list, 0, sizeof(int32_t), st));
    if (E > 0) {
        csr_count_kernel<<<grid_for(ctx, E, 256, 8), 256, 0, st>>>(N, E, edge_src, edge_dst, cnt, ctx->dstatus_dev);
        S2V_CHECK_LAUNCH(ctx, "csr_count_kernel");
    }
    csr_scan_blocks_kernel<<<num_blocks, SCAN_THREADS, 0, st>>>(N, cnt, row_ptr, block_sum);
    S2V_CHECK_LAUNCH(ctx, "csr_scan_blocks_kernel");
    csr_scan_totals_kernel<<<1, SCAN_THREADS, 0, st>>>(num_blocks, block_sum);
    S2V_CHECK_LAUNCH(ctx, "csr_scan_totals_kernel");
    csr_scan_add_kernel<<<num_blocks, SCAN_THREADS, 0, st>>>(N, num_blocks, block_sum, row_ptr, cnt, long_list);
    S2V_CHECK_LAUNCH(ctx, "csr_scan_add_kernel");
    if (E > 0) {
        csr_place_kernel<<<grid_for(ctx, E, 256, 8), 256, 0, st>>>(N, E, edge_src, edge_dst, row_ptr, cnt, slot_edge);
        S2V_CHECK_LAUNCH(ctx, "csr_place_kernel");
        csr_rank_kernel<<<grid_for(ctx, E, 256, 8), 256, 0, st>>>(N, E, edge_src, edge_dst, row_ptr, slot_edge, average, col_idx, val);
        S2V_CHECK_LAUNCH(ctx, "csr_rank_kernel");
        csr_long_rows_kernel<<<grid_for(ctx, E / CSR_LONG_ROW + 1, 1, 1), 1024, 0, st>>>(long_list, edge_src, row_ptr, slot_edge, average, col_idx, val);
        S2V_CHECK_LAUNCH(ctx, "csr_long_rows_kernel");
    }
    return S2V_OK;
}

}  // extern "C"
