// Shared declarations of the s2v_b200 library: context object, status plumbing,
// small device helpers.  Everything here targets sm_100a only.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdio>
#include <mutex>
#include <string>

#include "s2v_b200.h"

// Device-side status word (mapped, host-visible) written by kernels whose bounded
// waits give up.  0 = fine.
struct s2v_device_status {
    int code;
    int where;
};

struct s2v_staging {  // grow-only buffers owned by a context (host-buffer entry point)
    void* dev = nullptr;
    size_t dev_bytes = 0;
    void* pinned = nullptr;
    size_t pinned_bytes = 0;
};

// One of the two lanes of the host-buffer entry points: its own stream and staging, and what a finished batch
// still has to deliver.  Lane 0 is the context's own stream and serves the synchronous entry points.
struct s2v_lane {
    cudaStream_t stream = nullptr;
    s2v_staging staging;
    bool busy = false;
    int64_t G = 0;
    int C = 0;
    float* logits_host = nullptr;
    int32_t* pred_host = nullptr;
    int bad_edge = 0, bad_tag = 0;   // outcome of the host scan that ran beside the device work
};

struct s2v_ctx {
    int device = 0;
    int sm_count = 0;      // SMs the persistent kernels size their grids for (hardware count minus S2V_OPT_RESERVED_SMS)
    int sm_count_hw = 0;
    size_t smem_optin = 0;
    cudaStream_t stream = nullptr;       // the context's own non-blocking stream
    s2v_device_status* dstatus_host = nullptr;  // pinned + mapped
    s2v_device_status* dstatus_dev = nullptr;
    std::atomic<uint64_t> launches{0};
    std::string last_error;
    std::mutex mu;
    s2v_lane lanes[2];
    void* first_table = nullptr;     // product table of s2v_level_first_f32 (grow-only, a few hundred KB at most)
    size_t first_table_bytes = 0;
    int tc_mode = 1;  // tcgen05 level kernel: 0 never, 1 when the batch is large enough, 2 whenever the shape allows
    int graph_tiles = 2;    // whole-classifier tile kernel for batches of small graphs: 0 off, 1 whenever the batch allows, 2 automatic
    int first_table_on = 1; // first level as a gather-sum over ReLU(W_in) * W (S2V_OPT_FIRST_LEVEL_TABLE)
    int validate_host = 1;  // s2v_infer_host_f32 scans its host arrays before launching
};

inline int s2v_fail(s2v_ctx* ctx, int status, const std::string& msg)
{
    if (ctx) {
        std::lock_guard<std::mutex> g(ctx->mu);
        ctx->last_error = msg;
    }
    return status;
}

#define S2V_CUDA_OK(ctx, expr)                                                                         \
    do {                                                                                               \
        cudaError_t e__ = (expr);                                                                      \
        if (e__ != cudaSuccess)                                                                        \
            return s2v_fail((ctx), S2V_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__)); \
    } while (0)

inline bool s2v_aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline cudaStream_t s2v_pick_stream(s2v_ctx* ctx, s2v_stream s)
{
    return s ? static_cast<cudaStream_t>(s) : ctx->stream;
}

// RAII device switch: every entry point runs with the context's device current and
// restores the caller's device on return.
struct s2v_device_guard {
    int prev = -1;
    bool ok = true;
    explicit s2v_device_guard(int dev)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~s2v_device_guard()
    {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

#define S2V_ENTER(ctx)                                                                   \
    if (!(ctx)) return S2V_ERR_INVALID_ARG;                                              \
    s2v_device_guard guard__((ctx)->device);                                             \
    if (!guard__.ok) return s2v_fail((ctx), S2V_ERR_CUDA, "cannot select the context's device")

#define S2V_CHECK_LAUNCH(ctx, name)                                                                        \
    do {                                                                                                   \
        cudaError_t e__ = cudaGetLastError();                                                              \
        if (e__ != cudaSuccess)                                                                            \
            return s2v_fail((ctx), S2V_ERR_CUDA, std::string("launch of ") + name + ": " + cudaGetErrorString(e__)); \
        (ctx)->launches.fetch_add(1, std::memory_order_relaxed);                                           \
    } while (0)

// ---------------------------------------------------------------- device helpers
#ifdef __CUDACC__

__device__ __forceinline__ float4 ld_nc_f4(const float4* p)
{
    return __ldg(p);
}
// streaming (evict-first) accesses for data touched once per launch
__device__ __forceinline__ float4 ld_stream_f4(const float4* p)
{
    return __ldcs(p);
}
__device__ __forceinline__ void st_stream_f4(float4* p, float4 v)
{
    __stcs(p, v);
}
__device__ __forceinline__ float relu_ref(float v)
{
    // `if (x < 0) x = 0`: keeps -0.0 and NaN like the reference functor
    return v < 0.0f ? 0.0f : v;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

#endif  // __CUDACC__

// Rows from which the d = 64 / d = 128 level goes to the tcgen05 kernel (128-row tiles, one CTA per SM).
constexpr int64_t S2V_TC_MIN_ROWS = 16384;
inline bool s2v_use_tc(const s2v_ctx* ctx, int d, int64_t n_rows)
{
    if (d != 128 && d != 64) return false;
    return ctx->tc_mode == 2 || (ctx->tc_mode == 1 && n_rows >= S2V_TC_MIN_ROWS);
}

// launchers implemented in the .cu files (host side)
int s2v_launch_level_tc(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, int d, const int32_t* row_ptr,
                        const int32_t* col_idx, const float* val, const float* H, const float* W, const float* X,
                        const float* table, const int32_t* x_index, int n_table, float* out);
int s2v_launch_wait_selftest(s2v_ctx* ctx, cudaStream_t st);
// readout (two layers + softmax / argmax) with the first layer on tcgen05 (readout_tc.cu): d in {64, 128},
// hidden in {128, 256}, at most 8 classes, batches of at least 6,144 graphs (512 when S2V_OPT_LEVEL_TC = 2)
bool s2v_readout_tc_supported(const s2v_ctx* ctx, int64_t G, int d, int hidden, int C);
int s2v_launch_readout_tc(s2v_ctx* ctx, cudaStream_t st, int64_t G, int d, int hidden, int C, const float* Y, const float* W1,
                          const float* W2, float* logits, float* probs, int32_t* pred);
// first level from one-hot tags as a gather-sum over the product table ReLU(W_in) * W (level_first_table.cu);
// d / 4 must be a power of two <= 32; P_scratch holds s2v_first_table_scratch_bytes(n_table, d)
bool s2v_first_table_supported(int d);
size_t s2v_first_table_scratch_bytes(int n_table, int d);
int s2v_launch_first_table_product(s2v_ctx* ctx, cudaStream_t st, int n_table, int d, const float* table, const float* W,
                                   float* P, bool extra_zero_row);
int s2v_launch_level_first_table(s2v_ctx* ctx, cudaStream_t st, int64_t n, int d, const int32_t* row_ptr, const int32_t* col_idx,
                                 const float* val, const float* W, const float* table, int n_table, const int32_t* tags,
                                 float* P_scratch, float* out);
// records S2V_ERR_INVALID_ARG in the status word if any idx[i] lies outside [0, limit)
int s2v_launch_index_check(s2v_ctx* ctx, cudaStream_t st, int64_t n, const int32_t* idx, int limit);
// whole classifier up to the pooled embeddings for batches of graphs of at most S2V_TILE_NODES nodes (d = 128, tags)
constexpr int S2V_TILE_NODES = 128;
constexpr int64_t S2V_TILE_AUTO_MAX_NODES = 160000;   // automatic mode: batches up to this many nodes take the tile kernel
size_t s2v_graph_tiles_plan_bytes(int64_t num_graphs);
int s2v_launch_graph_tiles(s2v_ctx* ctx, cudaStream_t st, int64_t G, const int32_t* row_ptr, const int32_t* col_idx,
                           const float* val, const int32_t* graph_ptr, const int32_t* tags, int num_tags,
                           const float* W_in, const float* W, int levels, int pool_average, void* plan, float* P_scratch,
                           float* Y, float* embed_out);   // P_scratch: (num_tags + 1) * 128 floats, or NULL (first level through the MMAs)
int s2v_launch_level(s2v_ctx* ctx, cudaStream_t st, int64_t n_rows, int64_t n_src, int d, const void* row_ptr,
                     bool rp64, const int32_t* col_idx, const float* val, const float* H, const float* W,
                     const float* X, const float* table, const int32_t* x_index, int n_table, float* out);
