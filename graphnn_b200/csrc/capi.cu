// C ABI glue of s2v_b200: context life cycle, argument validation, the whole-model
// pipelines (device buffers and host buffers) and the host-side CSR builders.
#include <omp.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

namespace
{

const char* status_text(int s)
{
    switch (s) {
        case S2V_OK: return "ok";
        case S2V_ERR_INVALID_ARG: return "invalid argument";
        case S2V_ERR_UNSUPPORTED: return "unsupported shape";
        case S2V_ERR_CUDA: return "CUDA runtime error";
        case S2V_ERR_BAD_CSR: return "malformed CSR matrix";
        case S2V_ERR_WORKSPACE: return "workspace too small";
        case S2V_ERR_NO_DEVICE: return "no CUDA device";
        case S2V_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        case S2V_ERR_COMM: return "NCCL communication error";
        default: return "unknown status";
    }
}

inline size_t align_up(size_t v, size_t a)
{
    return (v + a - 1) / a * a;
}

int check_level_args(s2v_ctx* ctx, int64_t n_rows, int64_t n_src, int d, const void* row_ptr, const int32_t* col_idx,
                     const float* H, const float* W, const float* X, const float* out)
{
    if (n_rows < 0 || n_src < 0 || d <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level: negative size");
    if (n_rows == 0) return S2V_OK;
    if (!row_ptr || !W || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level: NULL pointer");
    // col_idx may be NULL for a matrix without non-zeros (nnz lives on the device and is not read here)
    if (n_src > 0 && !H) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level: NULL H");
    if (d != 32 && d != 64 && d != 128)
        return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "fused level kernel supports d in {32, 64, 128}");
    if (!s2v_aligned16(H) || !s2v_aligned16(W) || !s2v_aligned16(X) || !s2v_aligned16(out))
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level: H, W, X, out must be 16-byte aligned");
    if (out == H) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level: out must not alias H");
    return S2V_OK;
}

int ensure_staging(s2v_ctx* ctx, s2v_staging& s, size_t dev_bytes, size_t pinned_bytes)
{
    if (dev_bytes > s.dev_bytes) {
        if (s.dev) cudaFree(s.dev);
        s.dev = nullptr;
        s.dev_bytes = 0;
        const size_t want = align_up(dev_bytes + dev_bytes / 4, 1 << 20);
        S2V_CUDA_OK(ctx, cudaMalloc(&s.dev, want));
        s.dev_bytes = want;
    }
    if (pinned_bytes > s.pinned_bytes) {
        if (s.pinned) cudaFreeHost(s.pinned);
        s.pinned = nullptr;
        s.pinned_bytes = 0;
        const size_t want = align_up(pinned_bytes + pinned_bytes / 4, 1 << 16);
        S2V_CUDA_OK(ctx, cudaMallocHost(&s.pinned, want));
        s.pinned_bytes = want;
    }
    return S2V_OK;
}

}  // namespace

extern "C" {

const char* s2v_status_str(int status)
{
    return status_text(status);
}

int s2v_ctx_create(int device, s2v_ctx** out)
{
    if (!out) return S2V_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return S2V_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count) return S2V_ERR_INVALID_ARG;
    s2v_ctx* ctx = new (std::nothrow) s2v_ctx();
    if (!ctx) return S2V_ERR_CUDA;
    ctx->device = device;
    s2v_device_guard guard(device);
    cudaDeviceProp prop;
    if (!guard.ok || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        delete ctx;
        return S2V_ERR_CUDA;
    }
    if (prop.major != 10) {  // the kernels are built for sm_100a only
        delete ctx;
        return S2V_ERR_NO_DEVICE;
    }
    ctx->sm_count = ctx->sm_count_hw = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    bool ok = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaHostAlloc((void**)&ctx->dstatus_host, sizeof(s2v_device_status), cudaHostAllocMapped) == cudaSuccess &&
              cudaHostGetDevicePointer((void**)&ctx->dstatus_dev, ctx->dstatus_host, 0) == cudaSuccess;
    if (!ok) {
        s2v_ctx_destroy(ctx);
        return S2V_ERR_CUDA;
    }
    ctx->dstatus_host->code = 0;
    ctx->dstatus_host->where = 0;
    // S2V_LEVEL_TC = 0 | 1 | 2 : never / automatic / always use the tcgen05 level kernel (d = 128)
    if (const char* e = std::getenv("S2V_LEVEL_TC")) ctx->tc_mode = (e[0] == '0') ? 0 : (e[0] == '2' ? 2 : 1);
    if (const char* e = std::getenv("S2V_GRAPH_TILES")) ctx->graph_tiles = (e[0] == '0') ? 0 : ((e[0] == '1') ? 1 : 2);
    if (const char* e = std::getenv("S2V_VALIDATE_HOST")) ctx->validate_host = (e[0] == '0') ? 0 : 1;
    *out = ctx;
    return S2V_OK;
}

int s2v_ctx_destroy(s2v_ctx* ctx)
{
    if (!ctx) return S2V_OK;
    {
        s2v_device_guard guard(ctx->device);
        if (ctx->stream) { cudaStreamSynchronize(ctx->stream); cudaStreamDestroy(ctx->stream); }
        if (ctx->dstatus_host) cudaFreeHost(ctx->dstatus_host);
        if (ctx->first_table) cudaFree(ctx->first_table);
        for (s2v_lane& lane : ctx->lanes) {
            if (lane.stream && lane.stream != ctx->stream) { cudaStreamSynchronize(lane.stream); cudaStreamDestroy(lane.stream); }
            if (lane.staging.dev) cudaFree(lane.staging.dev);
            if (lane.staging.pinned) cudaFreeHost(lane.staging.pinned);
        }
    }
    delete ctx;
    return S2V_OK;
}

int s2v_ctx_device(const s2v_ctx* ctx)
{
    return ctx ? ctx->device : S2V_ERR_INVALID_ARG;
}

s2v_stream s2v_ctx_stream(const s2v_ctx* ctx)
{
    return ctx ? static_cast<s2v_stream>(ctx->stream) : nullptr;
}

int s2v_ctx_synchronize(s2v_ctx* ctx)
{
    return s2v_stream_status(ctx, nullptr);
}

int s2v_ctx_set_option(s2v_ctx* ctx, int option, int value)
{
    if (!ctx) return S2V_ERR_INVALID_ARG;
    switch (option) {
        case S2V_OPT_VALIDATE_HOST_INPUT: ctx->validate_host = value != 0; return S2V_OK;
        case S2V_OPT_LEVEL_TC: ctx->tc_mode = value <= 0 ? 0 : (value >= 2 ? 2 : 1); return S2V_OK;
        case S2V_OPT_GRAPH_TILES: ctx->graph_tiles = value <= 0 ? 0 : (value >= 2 ? 2 : 1); return S2V_OK;
        case S2V_OPT_FIRST_LEVEL_TABLE: ctx->first_table_on = value != 0; return S2V_OK;
        case S2V_OPT_RESERVED_SMS:
            if (value < 0 || value >= ctx->sm_count_hw) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "set_option: reserved SMs outside [0, SM count)");
            ctx->sm_count = ctx->sm_count_hw - value;
            return S2V_OK;
        default: return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "set_option: unknown option");
    }
}

int s2v_stream_status(s2v_ctx* ctx, s2v_stream stream)
{
    S2V_ENTER(ctx);
    S2V_CUDA_OK(ctx, cudaStreamSynchronize(s2v_pick_stream(ctx, stream)));
    if (ctx->dstatus_host->code != 0) {
        const int code = ctx->dstatus_host->code, where = ctx->dstatus_host->where;
        ctx->dstatus_host->code = 0;
        ctx->dstatus_host->where = 0;
        return s2v_fail(ctx, code, "a kernel reported status " + std::to_string(code) + " at site " + std::to_string(where));
    }
    return S2V_OK;
}

int s2v_selftest_wait_timeout(s2v_ctx* ctx, s2v_stream stream)
{
    S2V_ENTER(ctx);
    return s2v_launch_wait_selftest(ctx, s2v_pick_stream(ctx, stream));
}

const char* s2v_last_error(const s2v_ctx* ctx)
{
    return ctx ? ctx->last_error.c_str() : "no context";
}

uint64_t s2v_launch_count(const s2v_ctx* ctx)
{
    return ctx ? ctx->launches.load() : 0;
}

// ---------------------------------------------------------------- fused level
int s2v_level_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n_rows, int64_t n_src, int d, const int32_t* row_ptr,
                  const int32_t* col_idx, const float* val, const float* H, const float* W, const float* X,
                  float* out)
{
    S2V_ENTER(ctx);
    int rc = check_level_args(ctx, n_rows, n_src, d, row_ptr, col_idx, H, W, X, out);
    if (rc != S2V_OK || n_rows == 0) return rc;
    return s2v_launch_level(ctx, s2v_pick_stream(ctx, stream), n_rows, n_src, d, row_ptr, false, col_idx, val, H, W, X,
                            nullptr, nullptr, 0, out);
}

int s2v_level_rp64_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n_rows, int64_t n_src, int d, const int64_t* row_ptr,
                       const int32_t* col_idx, const float* val, const float* H, const float* W, const float* X,
                       float* out)
{
    S2V_ENTER(ctx);
    int rc = check_level_args(ctx, n_rows, n_src, d, row_ptr, col_idx, H, W, X, out);
    if (rc != S2V_OK || n_rows == 0) return rc;
    return s2v_launch_level(ctx, s2v_pick_stream(ctx, stream), n_rows, n_src, d, row_ptr, true, col_idx, val, H, W, X,
                            nullptr, nullptr, 0, out);
}

int s2v_level_lookup_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n_rows, int64_t n_src, int d,
                         const int32_t* row_ptr, const int32_t* col_idx, const float* val, const float* H,
                         const float* W, const float* table, int n_table, const int32_t* x_index, float* out)
{
    S2V_ENTER(ctx);
    int rc = check_level_args(ctx, n_rows, n_src, d, row_ptr, col_idx, H, W, table, out);
    if (rc != S2V_OK || n_rows == 0) return rc;
    if (!table || !x_index || n_table <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level_lookup: NULL table or index");
    // the level kernel clamps the indices it uses; this launch finds and reports the ones outside the table
    rc = s2v_launch_index_check(ctx, s2v_pick_stream(ctx, stream), n_rows, x_index, n_table);
    if (rc != S2V_OK) return rc;
    return s2v_launch_level(ctx, s2v_pick_stream(ctx, stream), n_rows, n_src, d, row_ptr, false, col_idx, val, H, W,
                            nullptr, table, x_index, n_table, out);
}

int s2v_level_first_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n, int d, const int32_t* row_ptr, const int32_t* col_idx,
                        const float* val, const float* W, const float* table, int n_table, const int32_t* tags, float* out)
{
    S2V_ENTER(ctx);
    if (n < 0 || d <= 0 || n_table <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level_first: bad shape");
    if (n == 0) return S2V_OK;
    if (!row_ptr || !W || !table || !tags || !out) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level_first: NULL pointer");
    if (!s2v_aligned16(W) || !s2v_aligned16(table) || !s2v_aligned16(out))
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "level_first: W, table, out must be 16-byte aligned");
    int rc;
    if (ctx->first_table_on && s2v_first_table_supported(d)) {   // (this kernel range-checks the tags itself)
        // gather-sum over the product table ReLU(table) * W, which lives in a small context-owned buffer
        const size_t need = s2v_first_table_scratch_bytes(n_table, d);
        if (need > ctx->first_table_bytes) {
            if (ctx->first_table) cudaFree(ctx->first_table);
            ctx->first_table = nullptr;
            ctx->first_table_bytes = 0;
            S2V_CUDA_OK(ctx, cudaMalloc(&ctx->first_table, need));
            ctx->first_table_bytes = need;
        }
        return s2v_launch_level_first_table(ctx, s2v_pick_stream(ctx, stream), n, d, row_ptr, col_idx, val, W, table, n_table, tags,
                                            static_cast<float*>(ctx->first_table), out);
    }
    if (!s2v_use_tc(ctx, d, n))
        return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "level_first: d / 4 must be a power of two up to 32; materialise H0 instead");
    rc = s2v_launch_index_check(ctx, s2v_pick_stream(ctx, stream), n, tags, n_table);
    if (rc != S2V_OK) return rc;
    rc = s2v_launch_level_tc(ctx, s2v_pick_stream(ctx, stream), n, d, row_ptr, col_idx, val, nullptr, W, nullptr, table,
                             tags, n_table, out);
    if (rc == S2V_ERR_UNSUPPORTED) return s2v_fail(ctx, rc, "level_first: shape not supported by the tcgen05 kernel");
    return rc;
}

// ---------------------------------------------------------------- tile kernel for batches of small graphs
size_t s2v_graph_tiles_workspace_bytes(int64_t num_graphs)
{
    return num_graphs < 0 ? 0 : align_up(s2v_graph_tiles_plan_bytes(num_graphs), 256) + 256;
}

int s2v_graph_tiles_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int d, int levels, const int32_t* row_ptr,
                        const int32_t* col_idx, const float* val, const int32_t* graph_ptr, const int32_t* tags, int num_tags,
                        const float* W_in, const float* W, int pool_average, void* workspace, size_t workspace_bytes, float* Y,
                        float* embed_out)
{
    S2V_ENTER(ctx);
    if (num_graphs < 0 || levels < 1 || num_tags <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "graph_tiles: bad shape");
    if (d != 128) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "graph_tiles: the tile kernel is built for d = 128");
    if (num_graphs == 0) return S2V_OK;
    if (num_graphs >= (int64_t)INT32_MAX) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "graph_tiles: int32 graph count only");
    if (!row_ptr || !graph_ptr || !tags || !W_in || !W || !Y) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "graph_tiles: NULL pointer");
    if (!s2v_aligned16(W_in) || !s2v_aligned16(W) || !s2v_aligned16(Y) || !s2v_aligned16(embed_out))
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "graph_tiles: W_in, W, Y, embed_out must be 16-byte aligned");
    if (!workspace || workspace_bytes < s2v_graph_tiles_workspace_bytes(num_graphs))
        return s2v_fail(ctx, S2V_ERR_WORKSPACE, "graph_tiles: workspace smaller than s2v_graph_tiles_workspace_bytes");
    void* plan = reinterpret_cast<void*>(align_up(reinterpret_cast<uintptr_t>(workspace), 256));
    // the product table of the first level ((num_tags + 1) x d floats) lives in a small context-owned buffer
    float* P = nullptr;
    if (ctx->first_table_on) {
        const size_t need = s2v_first_table_scratch_bytes(num_tags + 1, d);
        if (need > ctx->first_table_bytes) {
            if (ctx->first_table) cudaFree(ctx->first_table);
            ctx->first_table = nullptr;
            ctx->first_table_bytes = 0;
            S2V_CUDA_OK(ctx, cudaMalloc(&ctx->first_table, need));
            ctx->first_table_bytes = need;
        }
        P = static_cast<float*>(ctx->first_table);
    }
    const int rc = s2v_launch_graph_tiles(ctx, s2v_pick_stream(ctx, stream), num_graphs, row_ptr, col_idx, val, graph_ptr, tags,
                                          num_tags, W_in, W, levels, pool_average, plan, P, Y, embed_out);
    if (rc == S2V_ERR_UNSUPPORTED) return s2v_fail(ctx, rc, "graph_tiles: this device cannot hold the kernel's shared memory");
    return rc;
}

// ---------------------------------------------------------------- whole model, device buffers
size_t s2v_forward_workspace_bytes(int64_t num_nodes, int64_t num_graphs, int d)
{
    if (num_nodes < 0 || num_graphs < 0 || d <= 0) return 0;
    const size_t nd = align_up(sizeof(float) * (size_t)num_nodes * d, 256);
    const size_t gd = align_up(sizeof(float) * (size_t)num_graphs * d, 256);
    return 3 * nd + gd + 256 + align_up(s2v_graph_tiles_plan_bytes(num_graphs), 256);
}

int s2v_forward_f32(s2v_ctx* ctx, s2v_stream stream, const s2v_model* model, const s2v_batch* batch, void* workspace,
                    size_t workspace_bytes, float* logits, float* probs, int32_t* pred, float* embed_out)
{
    S2V_ENTER(ctx);
    if (!model || !batch) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "forward: NULL model or batch");
    const int64_t N = batch->num_nodes, G = batch->num_graphs;
    const int d = model->d, L = model->levels;
    if (N < 0 || G < 0 || L < 0 || d <= 0 || model->hidden <= 0 || model->num_class <= 0 || model->num_feat <= 0)
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "forward: bad shape");
    if (!model->w_n2l || !model->p_node_conv || !model->h1_weight || !model->h2_weight)
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "forward: NULL weight");
    if (G == 0) return S2V_OK;
    if (!logits || !batch->graph_ptr || (!batch->tags && !batch->x_dense) || (N > 0 && !batch->n2n_row_ptr))
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "forward: NULL batch array or output");
    if (workspace_bytes < s2v_forward_workspace_bytes(N, G, d) || !workspace)
        return s2v_fail(ctx, S2V_ERR_WORKSPACE, "forward: workspace smaller than s2v_forward_workspace_bytes");
    cudaStream_t st = s2v_pick_stream(ctx, stream);

    unsigned char* ws = static_cast<unsigned char*>(workspace);
    ws = reinterpret_cast<unsigned char*>(align_up(reinterpret_cast<uintptr_t>(ws), 256));
    const size_t nd = align_up(sizeof(float) * (size_t)N * d, 256);
    float* msg = reinterpret_cast<float*>(ws);
    float* ha = reinterpret_cast<float*>(ws + nd);
    float* hb = reinterpret_cast<float*>(ws + 2 * nd);
    float* y = reinterpret_cast<float*>(ws + 3 * nd);
    void* plan = ws + 3 * nd + align_up(sizeof(float) * (size_t)G * d, 256);

    int rc;
    // Batches of small graphs (the caller vouches for the largest one): the whole classifier up to the pooled
    // embeddings is one kernel that keeps the node embeddings of a tile of whole graphs in shared memory.
    // Measured on 20-40-node graphs, d = 128, 4 levels: one launch beats the per-level kernels by 1.9x at 16 k nodes,
    // 1.15x at 62 k, 1.09x at 123 k, and loses 5 % at 246 k and 11 % at 491 k (the per-level kernels stream better
    // once every SM has dozens of tiles), so the automatic mode takes it up to S2V_TILE_AUTO_MAX_NODES nodes.
    const bool want_tiles = ctx->graph_tiles == 1 || (ctx->graph_tiles == 2 && N <= S2V_TILE_AUTO_MAX_NODES);
    if (want_tiles && d == 128 && L >= 1 && batch->tags && batch->max_graph_nodes >= 1 &&
        batch->max_graph_nodes <= S2V_TILE_NODES && N > 0 && G < (int64_t)INT32_MAX) {
        if (!s2v_aligned16(model->w_n2l) || !s2v_aligned16(model->p_node_conv) || (embed_out && !s2v_aligned16(embed_out)))
            return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "forward: weights and embed_out must be 16-byte aligned");
        // the first level's product table goes into the `msg` region of the workspace, which one-hot inputs leave unused
        float* P = (ctx->first_table_on && s2v_first_table_scratch_bytes(model->num_feat + 1, d) <= nd) ? msg : nullptr;
        rc = s2v_launch_graph_tiles(ctx, st, G, batch->n2n_row_ptr, batch->n2n_col_idx, batch->n2n_val, batch->graph_ptr,
                                    batch->tags, model->num_feat, model->w_n2l, model->p_node_conv, L, model->pool_average,
                                    plan, P, y, embed_out);
        if (rc == S2V_OK)
            return s2v_readout_f32(ctx, st, G, d, model->hidden, model->num_class, y, model->h1_weight, model->h2_weight,
                                   logits, probs, pred);
        if (rc != S2V_ERR_UNSUPPORTED) return rc;
    }
    // With one-hot tags the X term of every level is a lookup in W_in, so `msg` is
    // never materialised; a dense X needs it.
    const bool onehot = batch->tags != nullptr && d % 4 == 0;
    // first level straight from the tags (no H0 in memory) when the tcgen05 kernel takes this shape
    bool first_fused = false;
    if (onehot) {
        if (!s2v_aligned16(model->w_n2l) || !s2v_aligned16(model->p_node_conv) || (embed_out && !s2v_aligned16(embed_out)))
            return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "forward: weights and embed_out must be 16-byte aligned");
    }
    bool tags_checked = false;
    if (onehot && L >= 1 && ctx->first_table_on && s2v_first_table_supported(d) &&
        s2v_first_table_scratch_bytes(model->num_feat, d) <= nd) {
        // H0 = ReLU(W_in[tag]) has one distinct row per tag, so level 1 is a gather-sum over the rows of
        // ReLU(W_in) * W (kept in the unused `msg` region of the workspace): no per-row product at all
        float* dst = (L == 1 && embed_out) ? embed_out : ha;
        rc = s2v_launch_level_first_table(ctx, st, N, d, batch->n2n_row_ptr, batch->n2n_col_idx, batch->n2n_val, model->p_node_conv,
                                          model->w_n2l, model->num_feat, batch->tags, msg, dst);
        if (rc == S2V_OK) first_fused = tags_checked = true;   // that kernel range-checks every tag itself
        else if (rc != S2V_ERR_UNSUPPORTED) return rc;
    }
    if (onehot && !tags_checked) {   // the tags are range-checked once per batch; the level kernels only clamp them
        rc = s2v_launch_index_check(ctx, st, N, batch->tags, model->num_feat);
        if (rc != S2V_OK) return rc;
    }
    if (!first_fused && onehot && L >= 1 && s2v_use_tc(ctx, d, N)) {
        float* dst = (L == 1 && embed_out) ? embed_out : ha;
        rc = s2v_launch_level_tc(ctx, st, N, d, batch->n2n_row_ptr, batch->n2n_col_idx, batch->n2n_val, nullptr, model->p_node_conv,
                                 nullptr, model->w_n2l, batch->tags, model->num_feat, dst);
        if (rc == S2V_OK) first_fused = true;
        else if (rc != S2V_ERR_UNSUPPORTED) return rc;
    }
    if (first_fused)
        rc = S2V_OK;
    else if (onehot)
        rc = s2v_input_proj_onehot_f32(ctx, st, N, model->num_feat, d, batch->tags, model->w_n2l, nullptr, ha);
    else if (batch->tags)
        return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "forward: one-hot input needs d % 4 == 0");
    else
        rc = s2v_input_proj_dense_f32(ctx, st, N, model->num_feat, d, batch->x_dense, model->w_n2l, msg, ha);
    if (rc != S2V_OK) return rc;

    float* cur = (first_fused && L == 1 && embed_out) ? embed_out : ha;
    float* nxt = hb;
    for (int lv = first_fused ? 1 : 0; lv < L; ++lv) {
        float* dst = (lv == L - 1 && embed_out) ? embed_out : nxt;
        if (onehot)
            rc = (d == 32 || d == 64 || d == 128)
                     ? s2v_launch_level(ctx, st, N, N, d, batch->n2n_row_ptr, false, batch->n2n_col_idx, batch->n2n_val, cur,
                                        model->p_node_conv, nullptr, model->w_n2l, batch->tags, model->num_feat, dst)
                     : s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "fused level kernel supports d in {32, 64, 128}");
        else
            rc = s2v_level_f32(ctx, st, N, N, d, batch->n2n_row_ptr, batch->n2n_col_idx, batch->n2n_val, cur,
                               model->p_node_conv, msg, dst);
        if (rc != S2V_OK) return rc;
        if (dst == nxt) std::swap(cur, nxt); else cur = dst;
    }
    if (L == 0 && embed_out)
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(embed_out, cur, sizeof(float) * (size_t)N * d, cudaMemcpyDeviceToDevice, st));
    rc = s2v_segment_pool_f32(ctx, st, G, d, batch->graph_ptr, cur, model->pool_average, y);
    if (rc != S2V_OK) return rc;
    return s2v_readout_f32(ctx, st, G, d, model->hidden, model->num_class, y, model->h1_weight, model->h2_weight, logits,
                           probs, pred);
}

// ---------------------------------------------------------------- host-side CSR
}  // extern "C"

namespace
{
// Row y of the result lists, for every edge x -> y in edge order, either x (payload_edge_id = false: the
// node-to-node matrix) or the edge's index (true: the edge-to-node matrix).
int build_in_edge_csr(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src, const int32_t* edge_dst, bool payload_edge_id,
                      int average, int32_t* row_ptr, int32_t* col_idx, float* val)
{
    if (num_nodes < 0 || num_edges < 0 || !row_ptr) return S2V_ERR_INVALID_ARG;
    if (num_edges > 0 && (!edge_src || !edge_dst || !col_idx)) return S2V_ERR_INVALID_ARG;
    if (num_edges >= (int64_t)INT32_MAX || num_nodes >= (int64_t)INT32_MAX) return S2V_ERR_UNSUPPORTED;
    // A stable sort of the edge list by destination: row y receives its sources in edge order,
    // which is the order GraphStruct::AddEdge appended them to in_edges[y].
    const int64_t N = num_nodes, E = num_edges;
    int T = omp_get_max_threads();
    if (T > 16) T = 16;
    if (E < (1 << 16) || T < 2) {
        // small batch: one thread, plain counting sort
        std::vector<int32_t> fill((size_t)N + 1, 0);
        for (int64_t e = 0; e < E; ++e) {
            const int32_t y = edge_dst[e], x = edge_src[e];
            if (y < 0 || y >= N || x < 0 || x >= N) return S2V_ERR_BAD_CSR;
            fill[(size_t)y + 1]++;
        }
        for (int64_t i = 0; i < N; ++i) fill[i + 1] += fill[i];
        std::memcpy(row_ptr, fill.data(), sizeof(int32_t) * ((size_t)N + 1));
        for (int64_t e = 0; e < E; ++e) col_idx[fill[edge_dst[e]]++] = payload_edge_id ? (int32_t)e : edge_src[e];
    } else {
        // large batch: the same stable sort in three parallel passes.
        //   1. every thread histograms its contiguous slice of the edge list over NB buckets of
        //      consecutive rows;  2. slices scatter their edges into bucket-partitioned scratch,
        //      slice after slice, so the edge order inside a bucket is kept;  3. buckets are
        //      finished independently (counting sort over the bucket's few hundred rows).
        int shift = 0;   // a bucket is 2^shift consecutive rows; at most 2048 buckets
        while (((N - 1) >> shift) >= 2048) ++shift;
        const int64_t rows_per_bucket = (int64_t)1 << shift;
        const int NB = (int)((N + rows_per_bucket - 1) >> shift);
        static thread_local std::vector<int32_t> scratch;   // grow-only: (src, dst) pairs by bucket
        if (scratch.size() < (size_t)(2 * E)) scratch.resize((size_t)(2 * E));
        int32_t* tmp_src = scratch.data();
        int32_t* tmp_dst = scratch.data() + E;
        std::vector<int64_t> hist((size_t)T * NB, 0), bucket_start(NB + 1, 0);
        int bad = 0;
#pragma omp parallel num_threads(T)
        {
            const int t = omp_get_thread_num();
            const int64_t e0 = E * t / T, e1 = E * (t + 1) / T;
            int64_t* h = hist.data() + (size_t)t * NB;
            int local_bad = 0;
            for (int64_t e = e0; e < e1; ++e) {
                const int32_t y = edge_dst[e], x = edge_src[e];
                if (y < 0 || y >= N || x < 0 || x >= N) { local_bad = 1; break; }
                h[y >> shift]++;
            }
            if (local_bad) {
#pragma omp atomic write
                bad = 1;
            }
#pragma omp barrier
#pragma omp single
            {
                if (!bad) {
                    int64_t run = 0;
                    for (int b = 0; b < NB; ++b) {
                        bucket_start[b] = run;
                        for (int tt = 0; tt < T; ++tt) {
                            const int64_t c = hist[(size_t)tt * NB + b];
                            hist[(size_t)tt * NB + b] = run;   // becomes this slice's write cursor in bucket b
                            run += c;
                        }
                    }
                    bucket_start[NB] = run;
                }
            }   // implicit barrier
            if (!bad) {
                for (int64_t e = e0; e < e1; ++e) {
                    const int32_t y = edge_dst[e];
                    const int64_t pos = h[y >> shift]++;
                    tmp_src[pos] = payload_edge_id ? (int32_t)e : edge_src[e];
                    tmp_dst[pos] = y;
                }
            }
#pragma omp barrier
            if (!bad) {
                std::vector<int32_t> cnt((size_t)rows_per_bucket + 1);
#pragma omp for schedule(dynamic, 8)
                for (int b = 0; b < NB; ++b) {
                    const int64_t r0 = (int64_t)b * rows_per_bucket;
                    const int64_t r1 = std::min(N, r0 + rows_per_bucket);
                    if (r0 >= r1) continue;
                    const int64_t s0 = bucket_start[b], s1 = bucket_start[b + 1];
                    std::fill(cnt.begin(), cnt.begin() + (r1 - r0) + 1, 0);
                    for (int64_t p = s0; p < s1; ++p) cnt[tmp_dst[p] - r0 + 1]++;
                    int32_t run = (int32_t)s0;
                    for (int64_t r = r0; r < r1; ++r) {
                        const int32_t c = cnt[r - r0 + 1];
                        row_ptr[r] = run;
                        cnt[r - r0 + 1] = run;   // write cursor of row r
                        run += c;
                    }
                    for (int64_t p = s0; p < s1; ++p) col_idx[cnt[tmp_dst[p] - r0 + 1]++] = tmp_src[p];
                }
            }
        }
        if (bad) return S2V_ERR_BAD_CSR;
        row_ptr[N] = (int32_t)E;
    }
    if (val) {
#pragma omp parallel for num_threads(T) schedule(static) if (E >= (1 << 16))
        for (int64_t i = 0; i < N; ++i) {
            const int32_t deg = row_ptr[i + 1] - row_ptr[i];
            const float v = average ? (float)(1.0 / deg) : 1.0f;
            for (int32_t t = row_ptr[i]; t < row_ptr[i + 1]; ++t) val[t] = v;
        }
    }
    return S2V_OK;
}
}  // namespace

extern "C" {

int s2v_build_n2n_csr_host(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src, const int32_t* edge_dst,
                           int average, int32_t* row_ptr, int32_t* col_idx, float* val)
{
    return build_in_edge_csr(num_nodes, num_edges, edge_src, edge_dst, false, average, row_ptr, col_idx, val);
}

int s2v_build_e2n_csr_host(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src, const int32_t* edge_dst,
                           int average, int32_t* row_ptr, int32_t* col_idx, float* val)
{
    return build_in_edge_csr(num_nodes, num_edges, edge_src, edge_dst, true, average, row_ptr, col_idx, val);
}

int s2v_build_n2e_csr_host(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src, int32_t* row_ptr, int32_t* col_idx,
                           float* val)
{
    if (num_nodes < 0 || num_edges < 0 || !row_ptr || (num_edges > 0 && (!edge_src || !col_idx))) return S2V_ERR_INVALID_ARG;
    if (num_edges >= (int64_t)INT32_MAX) return S2V_ERR_UNSUPPORTED;
    for (int64_t e = 0; e < num_edges; ++e) {
        if (edge_src[e] < 0 || edge_src[e] >= num_nodes) return S2V_ERR_BAD_CSR;
        row_ptr[e] = (int32_t)e;
        col_idx[e] = edge_src[e];
        if (val) val[e] = 1.0f;
    }
    row_ptr[num_edges] = (int32_t)num_edges;
    return S2V_OK;
}

int s2v_build_e2e_csr_host(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src, const int32_t* edge_dst,
                           int32_t* row_ptr, int32_t* col_idx, float* val, int64_t capacity, int64_t* nnz_out)
{
    if (num_nodes < 0 || num_edges < 0 || !row_ptr || !nnz_out) return S2V_ERR_INVALID_ARG;
    if (num_edges > 0 && (!edge_src || !edge_dst)) return S2V_ERR_INVALID_ARG;
    const int64_t N = num_nodes, E = num_edges;
    // in-edge lists of every node, in insertion order: (edge index, source) pairs
    std::vector<int32_t> in_rp((size_t)N + 1), in_edge((size_t)std::max<int64_t>(E, 1)), in_src((size_t)std::max<int64_t>(E, 1));
    int rc = build_in_edge_csr(N, E, edge_src, edge_dst, true, 0, in_rp.data(), in_edge.data(), nullptr);
    if (rc != S2V_OK) return rc;
    for (int64_t t = 0; t < E; ++t) in_src[t] = edge_src[in_edge[t]];
    // row e = (from -> to): the edges into `from`, except those that come from `to`
    int64_t nnz = 0;
    for (int64_t e = 0; e < E; ++e) {
        const int32_t from = edge_src[e], to = edge_dst[e];
        for (int32_t t = in_rp[from]; t < in_rp[from + 1]; ++t)
            if (in_src[t] != to) ++nnz;
    }
    *nnz_out = nnz;
    if (nnz >= (int64_t)INT32_MAX) return S2V_ERR_UNSUPPORTED;
    if (!col_idx || capacity < nnz) return (capacity < nnz && col_idx) ? S2V_ERR_WORKSPACE : S2V_OK;   // size query
    int64_t pos = 0;
    for (int64_t e = 0; e < E; ++e) {
        row_ptr[e] = (int32_t)pos;
        const int32_t from = edge_src[e], to = edge_dst[e];
        for (int32_t t = in_rp[from]; t < in_rp[from + 1]; ++t)
            if (in_src[t] != to) {
                col_idx[pos] = in_edge[t];
                if (val) val[pos] = 1.0f;
                ++pos;
            }
    }
    row_ptr[E] = (int32_t)pos;
    return S2V_OK;
}

int s2v_validate_csr_host(int64_t m, int64_t k, int64_t nnz, const int32_t* row_ptr, const int32_t* col_idx)
{
    if (m < 0 || k < 0 || nnz < 0 || !row_ptr || (nnz > 0 && !col_idx)) return S2V_ERR_INVALID_ARG;
    if (row_ptr[0] != 0 || row_ptr[m] != nnz) return S2V_ERR_BAD_CSR;
    for (int64_t i = 0; i < m; ++i)
        if (row_ptr[i + 1] < row_ptr[i]) return S2V_ERR_BAD_CSR;
    for (int64_t t = 0; t < nnz; ++t)
        if (col_idx[t] < 0 || col_idx[t] >= k) return S2V_ERR_BAD_CSR;
    return S2V_OK;
}

// ---------------------------------------------------------------- whole model, host buffers
int s2v_infer_host_f32(s2v_ctx* ctx, const s2v_model* model, const s2v_batch* hb, float* logits_host,
                       int32_t* pred_host)
{
    S2V_ENTER(ctx);
    if (!model || !hb) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_host: NULL model or batch");
    if (ctx->lanes[0].busy) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_host: lane 0 holds a submitted batch; wait for it first");
    const int64_t N = hb->num_nodes, G = hb->num_graphs, E = hb->num_edges;
    const int d = model->d, C = model->num_class, F = model->num_feat;
    if (N < 0 || G < 0 || E < 0 || d <= 0 || C <= 0 || F <= 0)
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_host: bad shape");
    if (G == 0) return S2V_OK;
    if (!hb->graph_ptr || !hb->n2n_row_ptr || (E > 0 && !hb->n2n_col_idx) || (!hb->tags && !hb->x_dense))
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_host: NULL batch array");
    // cheap structural check on the host (full validation is s2v_validate_csr_host)
    if (hb->n2n_row_ptr[0] != 0 || hb->n2n_row_ptr[N] != E || hb->graph_ptr[0] != 0 || hb->graph_ptr[G] != N)
        return s2v_fail(ctx, S2V_ERR_BAD_CSR, "infer_host: row_ptr / graph_ptr ends do not match the sizes");
    // The arrays are on the host here, so a malformed batch is turned away with a precise message.  What could
    // send a kernel outside its arrays -- offsets that are not monotone, a column index outside the matrix -- is
    // checked before anything is launched (N + E integers, OpenMP for large batches).  Tags are CLAMPED by the
    // kernels, so their scan runs on the host while the device already works on the batch; a bad batch is then
    // still reported, by this scan, and its results are discarded.  S2V_OPT_VALIDATE_HOST_INPUT = 0 skips both.
    int32_t max_nodes = 0;
    int T = omp_get_max_threads();
    if (T > 16) T = 16;
    {
        int bad_csr = 0;
        const int32_t* gp = hb->graph_ptr;
#pragma omp parallel for num_threads(T) schedule(static) reduction(max : max_nodes) reduction(| : bad_csr) if (G >= (1 << 15))
        for (int64_t g = 0; g < G; ++g) {
            const int32_t n = gp[g + 1] - gp[g];
            if (n < 0) bad_csr |= 1;
            if (n > max_nodes) max_nodes = n;
        }
        if (ctx->validate_host) {
            const int32_t* rp = hb->n2n_row_ptr;
#pragma omp parallel for num_threads(T) schedule(static) reduction(| : bad_csr) if (N >= (1 << 15))
            for (int64_t i = 0; i < N; ++i)
                if (rp[i + 1] < rp[i]) bad_csr |= 1;
            const int32_t* ci = hb->n2n_col_idx;
#pragma omp parallel for num_threads(T) schedule(static) reduction(| : bad_csr) if (E >= (1 << 15))
            for (int64_t t = 0; t < E; ++t)
                if (ci[t] < 0 || ci[t] >= N) bad_csr |= 1;
        }
        if (bad_csr) return s2v_fail(ctx, S2V_ERR_BAD_CSR, "infer_host: offsets not monotone or a column index outside [0, N)");
    }
    auto scan_tags = [&](int& bad_tag) {
        const int32_t* tg = hb->tags;
        int bt = 0;
        if (tg) {
#pragma omp parallel for num_threads(T) schedule(static) reduction(| : bt) if (N >= (1 << 15))
            for (int64_t i = 0; i < N; ++i)
                if (tg[i] < 0 || tg[i] >= F) bt |= 1;
        }
        bad_tag = bt;
    };

    // device layout: [row_ptr | col_idx | val? | graph_ptr | tags or X | logits | pred | workspace]
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
    const size_t o_rp = take(sizeof(int32_t) * (size_t)(N + 1));
    const size_t o_ci = take(sizeof(int32_t) * (size_t)E);
    const size_t o_val = hb->n2n_val ? take(sizeof(float) * (size_t)E) : 0;
    const size_t o_gp = take(sizeof(int32_t) * (size_t)(G + 1));
    const size_t o_in = hb->tags ? take(sizeof(int32_t) * (size_t)N) : take(sizeof(float) * (size_t)N * F);
    const size_t o_logits = take(sizeof(float) * (size_t)G * C);
    const size_t o_pred = take(sizeof(int32_t) * (size_t)G);
    const size_t ws_bytes = s2v_forward_workspace_bytes(N, G, d);
    const size_t o_ws = take(ws_bytes);
    int rc = ensure_staging(ctx, ctx->lanes[0].staging, off, sizeof(float) * (size_t)G * C + sizeof(int32_t) * (size_t)G + 512);
    if (rc != S2V_OK) return rc;
    unsigned char* dev = static_cast<unsigned char*>(ctx->lanes[0].staging.dev);
    cudaStream_t st = ctx->stream;

    S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_rp, hb->n2n_row_ptr, sizeof(int32_t) * (size_t)(N + 1), cudaMemcpyHostToDevice, st));
    if (E > 0)
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_ci, hb->n2n_col_idx, sizeof(int32_t) * (size_t)E, cudaMemcpyHostToDevice, st));
    if (hb->n2n_val && E > 0)
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_val, hb->n2n_val, sizeof(float) * (size_t)E, cudaMemcpyHostToDevice, st));
    S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_gp, hb->graph_ptr, sizeof(int32_t) * (size_t)(G + 1), cudaMemcpyHostToDevice, st));
    if (hb->tags)
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_in, hb->tags, sizeof(int32_t) * (size_t)N, cudaMemcpyHostToDevice, st));
    else
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_in, hb->x_dense, sizeof(float) * (size_t)N * F, cudaMemcpyHostToDevice, st));

    s2v_batch db = *hb;
    db.max_graph_nodes = max_nodes;
    db.n2n_row_ptr = reinterpret_cast<const int32_t*>(dev + o_rp);
    db.n2n_col_idx = reinterpret_cast<const int32_t*>(dev + o_ci);
    db.n2n_val = hb->n2n_val ? reinterpret_cast<const float*>(dev + o_val) : nullptr;
    db.graph_ptr = reinterpret_cast<const int32_t*>(dev + o_gp);
    db.tags = hb->tags ? reinterpret_cast<const int32_t*>(dev + o_in) : nullptr;
    db.x_dense = hb->tags ? nullptr : reinterpret_cast<const float*>(dev + o_in);
    float* d_logits = reinterpret_cast<float*>(dev + o_logits);
    int32_t* d_pred = reinterpret_cast<int32_t*>(dev + o_pred);
    rc = s2v_forward_f32(ctx, st, model, &db, dev + o_ws, ws_bytes, d_logits, nullptr, d_pred, nullptr);
    if (rc != S2V_OK) return rc;

    float* p_logits = static_cast<float*>(ctx->lanes[0].staging.pinned);
    int32_t* p_pred = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(ctx->lanes[0].staging.pinned) +
                                                 align_up(sizeof(float) * (size_t)G * C, 256));
    if (logits_host)
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(p_logits, d_logits, sizeof(float) * (size_t)G * C, cudaMemcpyDeviceToHost, st));
    if (pred_host)
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(p_pred, d_pred, sizeof(int32_t) * (size_t)G, cudaMemcpyDeviceToHost, st));
    int bad_tag = 0;
    if (ctx->validate_host) scan_tags(bad_tag);   // on the host, while the device works
    rc = s2v_ctx_synchronize(ctx);
    if (bad_tag) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_host: a node tag outside [0, num_feat)");
    if (rc != S2V_OK) return rc;
    if (logits_host) std::memcpy(logits_host, p_logits, sizeof(float) * (size_t)G * C);
    if (pred_host) std::memcpy(pred_host, p_pred, sizeof(int32_t) * (size_t)G);
    return S2V_OK;
}

// Same from a raw edge list: the CSR is built on the device (s2v_build_n2n_csr_f32).  Split in two halves so that
// two batches can be in flight: edges_enqueue puts everything of one batch on a lane's stream (upload, CSR build,
// forward, download into the lane's pinned buffer) and scans the host arrays while the device works; lane_finish
// waits for the lane, reports, and hands the results to the caller.
static int edges_enqueue(s2v_ctx* ctx, s2v_lane& lane, const s2v_model* model, int64_t num_graphs, int64_t num_nodes, int64_t num_edges,
                         const int32_t* edge_src_host, const int32_t* edge_dst_host, const int32_t* graph_ptr_host,
                         const int32_t* tags_host, float* logits_host, int32_t* pred_host)
{
    if (!model) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_edges: NULL model");
    const int64_t N = num_nodes, G = num_graphs, E = num_edges;
    const int d = model->d, C = model->num_class, F = model->num_feat;
    if (N < 0 || G < 0 || E < 0 || d <= 0 || C <= 0 || F <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_edges: bad shape");
    lane.G = 0;
    lane.bad_edge = lane.bad_tag = 0;
    if (G == 0) return S2V_OK;
    if (!graph_ptr_host || !tags_host || (E > 0 && (!edge_src_host || !edge_dst_host)))
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_edges: NULL batch array");
    if (N >= (int64_t)INT32_MAX || E >= (int64_t)INT32_MAX) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "infer_edges: int32 sizes only");
    if (graph_ptr_host[0] != 0 || graph_ptr_host[G] != N)
        return s2v_fail(ctx, S2V_ERR_BAD_CSR, "infer_edges: graph_ptr ends do not match the sizes");
    // graph_ptr is checked before anything is launched.  Edge endpoints and tags cannot send a kernel outside its
    // arrays (the CSR builder drops and reports an edge outside [0, N), the level kernels clamp a tag), so their scan
    // runs on the host while the device already works on the batch; a bad batch is still reported, by this scan.
    int32_t max_nodes = 0;
    {
        int bad = 0;
        for (int64_t g = 0; g < G; ++g) {
            const int32_t n = graph_ptr_host[g + 1] - graph_ptr_host[g];
            if (n < 0) bad = 1;
            if (n > max_nodes) max_nodes = n;
        }
        if (bad) return s2v_fail(ctx, S2V_ERR_BAD_CSR, "infer_edges: graph_ptr not monotone or an edge endpoint outside [0, N)");
    }
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
    const size_t o_es = take(sizeof(int32_t) * (size_t)E);
    const size_t o_ed = take(sizeof(int32_t) * (size_t)E);
    const size_t o_rp = take(sizeof(int32_t) * (size_t)(N + 1));
    const size_t o_ci = take(sizeof(int32_t) * (size_t)E);
    const size_t o_gp = take(sizeof(int32_t) * (size_t)(G + 1));
    const size_t o_tg = take(sizeof(int32_t) * (size_t)N);
    const size_t o_logits = take(sizeof(float) * (size_t)G * C);
    const size_t o_pred = take(sizeof(int32_t) * (size_t)G);
    const size_t sc_bytes = s2v_build_n2n_csr_scratch_bytes(N, E);
    const size_t o_sc = take(sc_bytes);
    const size_t ws_bytes = s2v_forward_workspace_bytes(N, G, d);
    const size_t o_ws = take(ws_bytes);
    int rc = ensure_staging(ctx, lane.staging, off, sizeof(float) * (size_t)G * C + sizeof(int32_t) * (size_t)G + 512);
    if (rc != S2V_OK) return rc;
    unsigned char* dev = static_cast<unsigned char*>(lane.staging.dev);
    cudaStream_t st = lane.stream;
    if (E > 0) {
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_es, edge_src_host, sizeof(int32_t) * (size_t)E, cudaMemcpyHostToDevice, st));
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_ed, edge_dst_host, sizeof(int32_t) * (size_t)E, cudaMemcpyHostToDevice, st));
    }
    S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_gp, graph_ptr_host, sizeof(int32_t) * (size_t)(G + 1), cudaMemcpyHostToDevice, st));
    S2V_CUDA_OK(ctx, cudaMemcpyAsync(dev + o_tg, tags_host, sizeof(int32_t) * (size_t)N, cudaMemcpyHostToDevice, st));
    lane.busy = true;   // from here on the lane's stream holds work that reads the caller's arrays
    rc = s2v_build_n2n_csr_f32(ctx, st, N, E, reinterpret_cast<const int32_t*>(dev + o_es), reinterpret_cast<const int32_t*>(dev + o_ed),
                               0, dev + o_sc, sc_bytes, reinterpret_cast<int32_t*>(dev + o_rp), reinterpret_cast<int32_t*>(dev + o_ci),
                               nullptr);
    if (rc != S2V_OK) return rc;
    s2v_batch db{};
    db.num_graphs = G;
    db.num_nodes = N;
    db.num_edges = E;
    db.n2n_row_ptr = reinterpret_cast<const int32_t*>(dev + o_rp);
    db.n2n_col_idx = reinterpret_cast<const int32_t*>(dev + o_ci);
    db.graph_ptr = reinterpret_cast<const int32_t*>(dev + o_gp);
    db.tags = reinterpret_cast<const int32_t*>(dev + o_tg);
    db.max_graph_nodes = max_nodes;
    float* d_logits = reinterpret_cast<float*>(dev + o_logits);
    int32_t* d_pred = reinterpret_cast<int32_t*>(dev + o_pred);
    rc = s2v_forward_f32(ctx, st, model, &db, dev + o_ws, ws_bytes, d_logits, nullptr, d_pred, nullptr);
    if (rc != S2V_OK) return rc;
    float* p_logits = static_cast<float*>(lane.staging.pinned);
    int32_t* p_pred = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(lane.staging.pinned) +
                                                 align_up(sizeof(float) * (size_t)G * C, 256));
    if (logits_host)
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(p_logits, d_logits, sizeof(float) * (size_t)G * C, cudaMemcpyDeviceToHost, st));
    if (pred_host)
        S2V_CUDA_OK(ctx, cudaMemcpyAsync(p_pred, d_pred, sizeof(int32_t) * (size_t)G, cudaMemcpyDeviceToHost, st));
    lane.G = G;
    lane.C = C;
    lane.logits_host = logits_host;
    lane.pred_host = pred_host;
    if (ctx->validate_host) {   // on the host, while the device works
        int T = omp_get_max_threads();
        if (T > 16) T = 16;
        int be = 0, bt = 0;
#pragma omp parallel for num_threads(T) schedule(static) reduction(| : bt) if (N >= (1 << 15))
        for (int64_t i = 0; i < N; ++i)
            if (tags_host[i] < 0 || tags_host[i] >= F) bt |= 1;
#pragma omp parallel for num_threads(T) schedule(static) reduction(| : be) if (E >= (1 << 15))
        for (int64_t e = 0; e < E; ++e)
            if (edge_src_host[e] < 0 || edge_src_host[e] >= N || edge_dst_host[e] < 0 || edge_dst_host[e] >= N) be |= 1;
        lane.bad_edge = be;
        lane.bad_tag = bt;
    }
    return S2V_OK;
}

static int lane_finish(s2v_ctx* ctx, s2v_lane& lane)
{
    if (!lane.busy) return S2V_OK;
    lane.busy = false;
    const int rc = s2v_stream_status(ctx, lane.stream);
    if (lane.bad_edge) return s2v_fail(ctx, S2V_ERR_BAD_CSR, "infer_edges: graph_ptr not monotone or an edge endpoint outside [0, N)");
    if (lane.bad_tag) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_edges: a node tag outside [0, num_feat)");
    if (rc != S2V_OK) return rc;
    const int64_t G = lane.G;
    if (G > 0) {
        const float* p_logits = static_cast<const float*>(lane.staging.pinned);
        const int32_t* p_pred = reinterpret_cast<const int32_t*>(static_cast<const unsigned char*>(lane.staging.pinned) +
                                                                 align_up(sizeof(float) * (size_t)G * lane.C, 256));
        if (lane.logits_host) std::memcpy(lane.logits_host, p_logits, sizeof(float) * (size_t)G * lane.C);
        if (lane.pred_host) std::memcpy(lane.pred_host, p_pred, sizeof(int32_t) * (size_t)G);
    }
    return S2V_OK;
}

static int lane_of(s2v_ctx* ctx, int index, s2v_lane** out)
{
    if (index < 0 || index > 1) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer: the lane is 0 or 1");
    s2v_lane& lane = ctx->lanes[index];
    if (!lane.stream) {
        if (index == 0) lane.stream = ctx->stream;
        else S2V_CUDA_OK(ctx, cudaStreamCreateWithFlags(&lane.stream, cudaStreamNonBlocking));
    }
    *out = &lane;
    return S2V_OK;
}

int s2v_infer_edges_host_f32(s2v_ctx* ctx, const s2v_model* model, int64_t num_graphs, int64_t num_nodes, int64_t num_edges,
                             const int32_t* edge_src_host, const int32_t* edge_dst_host, const int32_t* graph_ptr_host,
                             const int32_t* tags_host, float* logits_host, int32_t* pred_host)
{
    S2V_ENTER(ctx);
    s2v_lane* lane = nullptr;
    int rc = lane_of(ctx, 0, &lane);
    if (rc != S2V_OK) return rc;
    if (lane->busy) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_edges: lane 0 holds a submitted batch; wait for it first");
    rc = edges_enqueue(ctx, *lane, model, num_graphs, num_nodes, num_edges, edge_src_host, edge_dst_host, graph_ptr_host, tags_host,
                       logits_host, pred_host);
    const int rc2 = lane_finish(ctx, *lane);   // also drains the stream after a failed enqueue
    return rc != S2V_OK ? rc : rc2;
}

int s2v_infer_edges_host_submit(s2v_ctx* ctx, int lane_index, const s2v_model* model, int64_t num_graphs, int64_t num_nodes,
                                int64_t num_edges, const int32_t* edge_src_host, const int32_t* edge_dst_host,
                                const int32_t* graph_ptr_host, const int32_t* tags_host, float* logits_host, int32_t* pred_host)
{
    S2V_ENTER(ctx);
    s2v_lane* lane = nullptr;
    int rc = lane_of(ctx, lane_index, &lane);
    if (rc != S2V_OK) return rc;
    if (lane->busy) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "infer_edges_submit: the lane holds a submitted batch; wait for it first");
    rc = edges_enqueue(ctx, *lane, model, num_graphs, num_nodes, num_edges, edge_src_host, edge_dst_host, graph_ptr_host, tags_host,
                       logits_host, pred_host);
    if (rc != S2V_OK) lane_finish(ctx, *lane);   // drain what was enqueued; the enqueue error is the one reported
    return rc;
}

int s2v_infer_host_wait(s2v_ctx* ctx, int lane_index)
{
    S2V_ENTER(ctx);
    s2v_lane* lane = nullptr;
    const int rc = lane_of(ctx, lane_index, &lane);
    if (rc != S2V_OK) return rc;
    return lane_finish(ctx, *lane);
}

}  // extern "C"
