/*
 * s2v_b200 -- C ABI of the B200 (sm_100a) implementation of graphnn's structure2vec
 * mean-field inference path.
 *
 * Conventions
 *   - Every function returns S2V_OK (0) or a negative s2v_status; nothing throws,
 *     aborts or prints across this boundary.  s2v_last_error(ctx) gives the detail.
 *   - Unless a name ends in `_host`, every data pointer is a DEVICE pointer owned by
 *     the caller, matrices are dense row-major fp32 with leading dimension = columns
 *     (the layout of the reference's DenseData, include/tensor/t_data.h:79-113), and
 *     CSR matrices are the reference's 3-array, zero-based, int32 form
 *     (val / col_idx / row_ptr, include/tensor/t_data.h:122-165).
 *   - `stream` is a cudaStream_t passed as void*; NULL selects the context's own
 *     non-blocking stream (the reference launches on cudaStreamPerThread).  Calls are
 *     asynchronous with respect to the host; results are visible after the stream is
 *     synchronised, like the reference's kernels before its blocking cudaMemcpy.
 *   - Shapes are validated on the host before any launch.  CSR *contents* are not
 *     read back by the device entry points; use s2v_validate_csr_host on host copies.
 *   - Device entry points allocate nothing.  Only s2v_ctx_create
 *     and s2v_infer_host_f32 (grow-only staging owned by the context) allocate.
 *
 * Each entry cites the reference interface it stands in for (paths inside the
 * Hanjun-Dai/graphnn tree).
 */
#ifndef S2V_B200_H
#define S2V_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct s2v_ctx s2v_ctx;
typedef void* s2v_stream; /* cudaStream_t */

typedef enum s2v_status {
    S2V_OK = 0,
    S2V_ERR_INVALID_ARG = -1,   /* NULL pointer, negative size, misaligned pointer */
    S2V_ERR_UNSUPPORTED = -2,   /* shape outside what the kernels implement */
    S2V_ERR_CUDA = -3,          /* a CUDA runtime call failed; see s2v_last_error */
    S2V_ERR_BAD_CSR = -4,       /* row_ptr not monotone, col_idx out of range */
    S2V_ERR_WORKSPACE = -5,     /* caller's workspace too small */
    S2V_ERR_NO_DEVICE = -6,     /* no CUDA device / driver */
    S2V_ERR_DEVICE_TIMEOUT = -7, /* a bounded device-side wait gave up */
    S2V_ERR_COMM = -8            /* the NCCL library is missing or one of its calls failed; see s2v_comm_last_error */
} s2v_status;

/* ---- context: GpuHandle::Init / Destroy (include/tensor/gpu_handle.h:38-59,
 *      src/tensor/gpu_handle.cu:17-44).  Unlike the reference it does not reset the
 *      device and holds no cuBLAS/cuSPARSE/cuRAND state. */
int s2v_ctx_create(int device, s2v_ctx** out);
int s2v_ctx_destroy(s2v_ctx* ctx);
int s2v_ctx_device(const s2v_ctx* ctx);
s2v_stream s2v_ctx_stream(const s2v_ctx* ctx);
/* Synchronises the context's own stream, then reports and clears the device status word (below). */
int s2v_ctx_synchronize(s2v_ctx* ctx);
/* Device status word.  Kernels never trap: a bounded wait that gives up, a node tag outside the table, an
 * edge that leaves its tile or a graph too large for the tile kernel is recorded in ONE status word per
 * context (not per stream; the last writer wins) and the kernel carries on with a harmless substitute.
 * s2v_stream_status synchronises `stream` (NULL = the context's stream), returns the recorded status
 * (S2V_OK if none) and clears the word.  Callers that launch on their own stream use this instead of
 * s2v_ctx_synchronize; reading the word while kernels of another stream of the same context still run
 * may miss or clear their report, so collect the status after the last stream has been synchronised. */
int s2v_stream_status(s2v_ctx* ctx, s2v_stream stream);
const char* s2v_status_str(int status);
const char* s2v_last_error(const s2v_ctx* ctx);
/* Per-context switches (no counterpart in the reference).  Returns S2V_ERR_INVALID_ARG for an unknown option. */
typedef enum s2v_option {
    S2V_OPT_VALIDATE_HOST_INPUT = 1, /* s2v_infer_host_f32 scans its host arrays before any launch (default 1;
                                        the environment variable S2V_VALIDATE_HOST=0 sets the default to 0) */
    S2V_OPT_LEVEL_TC = 2,            /* tcgen05 level kernel: 0 never, 1 automatic (default), 2 whenever the shape allows
                                        (default from S2V_LEVEL_TC) */
    S2V_OPT_GRAPH_TILES = 3,         /* whole-classifier tile kernel (s2v_graph_tiles_f32) inside s2v_forward_f32 for batches of
                                        small graphs: 0 never, 1 whenever the batch allows, 2 automatic (default: batches of at
                                        most 160,000 nodes, where one launch beats the per-level kernels by 1.1x - 1.9x; larger
                                        batches stream better through the per-level kernels).  Default from S2V_GRAPH_TILES */
    S2V_OPT_RESERVED_SMS = 4,        /* the persistent kernels size their grids for (SM count - value) SMs, leaving the rest to
                                        kernels of another stream -- a communication library's, which cannot start while
                                        one-CTA-per-SM kernels hold every SM (default 0; 0 <= value < SM count) */
    S2V_OPT_FIRST_LEVEL_TABLE = 5    /* first level from one-hot tags as a gather-sum over the product table ReLU(W_in) * W
                                        (see s2v_level_first_f32): 1 (default) whenever d allows, 0 never (the level kernels'
                                        own table-lookup form is used instead) */
} s2v_option;
int s2v_ctx_set_option(s2v_ctx* ctx, int option, int value);
/* Diagnostic, no counterpart in the reference: launches a two-warp kernel whose bounded barrier waits (the
 * very routine every wait of the tensor-core kernels goes through) can never be satisfied.  Warp 0 runs out
 * of polls, raises the block's abort flag and records the time-out; warp 1 must notice the flag and leave
 * too.  The kernel returns normally; the next status read reports S2V_ERR_DEVICE_TIMEOUT at site 99 (98 if
 * warp 1 did not see the flag) and clears it, and the context stays usable. */
int s2v_selftest_wait_timeout(s2v_ctx* ctx, s2v_stream stream);

/* Number of kernels this library has launched through `ctx` since creation. */
uint64_t s2v_launch_count(const s2v_ctx* ctx);

/* ---- fused message-passing level: out = ReLU((A*H)*W + X).
 * Replaces the factor chain MatMul(sparse A, H) -> MatMul(., W) -> ElewiseAdd(., X)
 * -> ReLU of examples/graph_classification/src/kernel_mean_field.cpp:38-41, i.e.
 * CSRMMKernel + cublasSgemm + memcpy/saxpy + memcpy/UnaryReLU
 * (src/tensor/gpu_dense_tensor.cu:209-271, src/nn/elewise_add.cpp:12-33,
 * src/nn/relu.cu:8-13).
 *   A   : CSR [n_rows x n_src]; val may be NULL (all ones, the sum-pooling form of
 *         Node2NodeMsgPass, src/nn/msg_pass.cpp:60)
 *   H   : [n_src x d]   W : [d x d]   X : [n_rows x d] or NULL   out : [n_rows x d]
 * out must not alias H.  Fused kernels exist for d in {32, 64, 128}; other d return
 * S2V_ERR_UNSUPPORTED (compose s2v_spmm_csr_f32 + s2v_gemm_f32 + s2v_axpy_f32 +
 * s2v_relu_f32 instead).  H, W, X, out must be 16-byte aligned. */
int s2v_level_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n_rows, int64_t n_src, int d, const int32_t* row_ptr,
                  const int32_t* col_idx, const float* val, const float* H, const float* W, const float* X,
                  float* out);
/* Same with 64-bit row offsets, for shards whose nnz reaches 2^31 (the reference is
 * int32 throughout and cannot represent them). */
int s2v_level_rp64_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n_rows, int64_t n_src, int d,
                       const int64_t* row_ptr, const int32_t* col_idx, const float* val, const float* H,
                       const float* W, const float* X, float* out);
/* Level whose X term is a table lookup: X[i,:] = table[x_index[i],:]; this is
 * X = onehot(tags) * W_in without materialising the product (the reference's
 * node_input * w_n2l, kernel_mean_field.cpp:31, with the one-hot X GetBatch builds,
 * nn_common.h:57-70).  table : [n_table x d], x_index : int32 [n_rows].  An index outside [0, n_table) never
 * leaves the table (the kernel clamps it) and is reported through the status word by a small checking launch
 * that accompanies the level (S2V_ERR_INVALID_ARG); the level's result is then meaningless. */
int s2v_level_lookup_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n_rows, int64_t n_src, int d,
                         const int32_t* row_ptr, const int32_t* col_idx, const float* val, const float* H,
                         const float* W, const float* table, int n_table, const int32_t* x_index, float* out);

/* First level of the classifier with one-hot inputs, without materialising H0:
 * out = ReLU((A * ReLU(table[tags,:])) * W + table[tags,:]), A square [n x n]; i.e. MatMul(data, w_n2l),
 * ReLU and the first level (kernel_mean_field.cpp:31-41) in one call.  H0 has one distinct row per tag and the
 * product is linear in the gathered sum, so for d in {4, 8, 16, 32, 64, 128} the level runs as a gather-sum over
 * the rows of P = ReLU(table) * W (n_table x d, computed by a tiny launch into a context-owned buffer that is
 * allocated on first use): no per-row matrix product at all; sums in CSR order in fp32, which differs from "sum
 * first, multiply after" by fp32 rounding only.  Other d: the tcgen05 kernel when it takes the shape, else
 * S2V_ERR_UNSUPPORTED (run s2v_input_proj_onehot_f32 + s2v_level_lookup_f32 instead). */
int s2v_level_first_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n, int d, const int32_t* row_ptr,
                        const int32_t* col_idx, const float* val, const float* W, const float* table, int n_table,
                        const int32_t* tags, float* out);

/* ---- unfused tensor operations, one kernel each (the reference's DTensor<GPU,float>
 *      surface used by MatMul / ElewiseAdd / ReLU / Softmax / ArgMax factors) ---- */

/* C[m x n] = alpha * A_csr[m x k] * B[k x n] + beta * C.
 * DTensor<GPU>::MM(SpTensor, DTensor, Trans::N, Trans::N) (src/tensor/gpu_dense_tensor.cu:257-271). */
int s2v_spmm_csr_f32(s2v_ctx* ctx, s2v_stream stream, int64_t m, int64_t k, int n, const int32_t* row_ptr,
                     const int32_t* col_idx, const float* val, const float* B, float alpha, float beta, float* C);
/* C[m x n] = alpha * op(A) * op(B) + beta * C, row-major, trans flags 0 = N, 1 = T.
 * DTensor<GPU>::MM(DTensor, DTensor) (src/tensor/gpu_dense_tensor.cu:193-224). */
int s2v_gemm_f32(s2v_ctx* ctx, s2v_stream stream, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k,
                 float alpha, const float* A, int64_t lda, const float* B, int64_t ldb, float beta, float* C,
                 int64_t ldc);
/* y += a * x : DTensor<GPU>::Axpy (src/tensor/gpu_dense_tensor.cu:489-496). */
int s2v_axpy_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, float a, const float* x, float* y);
/* x *= a (a == 0 stores zeros) : DTensor<GPU>::Scale / Zeros. */
int s2v_scale_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, float a, float* x);
/* out = in < 0 ? 0 : in (in-place allowed) : ReLU factor (src/nn/relu.cu:8-13,
 * include/tensor/gpu_unary_functor.h:178-190). */
int s2v_relu_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, const float* in, float* out);
/* Row softmax with max subtraction (in-place allowed): DTensor<GPU>::Softmax
 * (src/tensor/gpu_dense_tensor.cu:298-370; CPU form cpu_dense_tensor.cpp:228-251). */
int s2v_softmax_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, int cols, const float* in, float* out);
/* Per-row index of the maximum, first index wins ties: DTensor<GPU>::ArgMax
 * (src/tensor/gpu_dense_tensor.cu:184-190, include/tensor/gpu_reduce_kernel.h:12-33). */
int s2v_argmax_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, int cols, const float* in, int32_t* out);

/* ---- loss / metric tail of the driver's TEST loop (targets = {loss, acc}, nn_common.h:127-146) ----
 * Labels are a CSR matrix [rows x cols] as GetBatch builds them (one entry per graph, nn_common.h:92-99). */
/* out[i] = -sum_k log(p[i, col_k]) * val_k, p = softmax(pred row) when need_softmax, |p| < 1e-8 clamped
 * to 1e-8: CrossEntropy factor (src/nn/cross_entropy.cpp:9-50).  label_val may be NULL (ones). */
int s2v_cross_entropy_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, int cols, const float* pred, int need_softmax,
                          const int32_t* label_row_ptr, const int32_t* label_col_idx, const float* label_val, float* out);
/* Column of the largest value of every CSR row, first maximum wins: SpTensor::ArgMax
 * (src/tensor/gpu_sparse_tensor.cu:82-122, CPU form cpu_sparse_tensor.cpp:86-103). */
int s2v_argmax_csr_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, const int32_t* row_ptr, const int32_t* col_idx,
                       const float* val, int32_t* out);
/* out[i] = 1 if fewer than k classes score strictly higher than target[i]: InTopK (src/nn/in_top_k.cpp:6-23). */
int s2v_in_top_k_f32(s2v_ctx* ctx, s2v_stream stream, int64_t rows, int cols, const float* pred, const int32_t* target,
                     int k, int32_t* out);
/* int32 -> float: TypeCast factor (src/nn/type_cast.cpp:14-30). */
int s2v_cast_i32_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, const int32_t* in, float* out);
/* out[0] = sum(in) / count, deterministic: DTensor::Mean / ReduceMean (src/nn/reduce_mean.cpp:14-42). */
int s2v_mean_f32(s2v_ctx* ctx, s2v_stream stream, int64_t count, const float* in, float* out);
/* All of the above in one launch: mean cross entropy (with softmax) and mean top-k accuracy of
 * logits [G x C] against CSR labels; per_graph_loss [G] may be NULL; loss_mean or acc_mean may be NULL. */
int s2v_loss_acc_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int num_class, const float* logits,
                     const int32_t* label_row_ptr, const int32_t* label_col_idx, const float* label_val, int topk,
                     float* loss_mean, float* acc_mean, float* per_graph_loss);

/* ---- graph pooling: Y[g,:] = sum of H[n,:] over n in [seg_ptr[g], seg_ptr[g+1]).
 * Replaces MatMul(SubgraphMsgPass CSR, H) (kernel_mean_field.cpp:44,
 * src/nn/msg_pass.cpp:156-177) for the batcher's layout, where graph g owns a
 * contiguous node range (nn_common.h:63-73).  Non-contiguous pooling matrices go
 * through s2v_spmm_csr_f32. */
int s2v_segment_sum_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int d, const int32_t* seg_ptr,
                        const float* H, float* Y);
/* Same with the mean-pooling form: average != 0 weights every node row by 1 / |graph| as it is added
 * (SubgraphMsgPass with average = true, src/nn/msg_pass.cpp:170). */
int s2v_segment_pool_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int d, const int32_t* seg_ptr,
                         const float* H, int average, float* Y);

/* ---- readout: logits = ReLU(Y*W1)*W2, probs = softmax(logits), pred = argmax(logits).
 * Replaces MatMul, ReLU, MatMul (kernel_mean_field.cpp:45-47) + Softmax + ArgMax.
 * Y [G x d], W1 [d x hidden], W2 [hidden x C]; probs and pred may be NULL. */
int s2v_readout_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int d, int hidden, int num_class,
                    const float* Y, const float* W1, const float* W2, float* logits, float* probs, int32_t* pred);

/* ---- input projection: msg = X*W_in, h0 = ReLU(msg) (kernel_mean_field.cpp:31-32).
 * One-hot form: tags int32 [N] in [0, F); msg[i,:] = W_in[tags[i],:].  msg or h0 may be NULL. */
int s2v_input_proj_onehot_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n, int num_tags, int d,
                              const int32_t* tags, const float* W_in, float* msg, float* h0);
/* Dense form: X [N x F] arbitrary. */
int s2v_input_proj_dense_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n, int num_feat, int d, const float* X,
                             const float* W_in, float* msg, float* h0);

/* ---- batches of small graphs: input projection, all L levels and the pooling in ONE kernel.
 * Y[g,:] = sum (or mean) over the nodes of graph g of H_L, with H_0 = ReLU(W_in[tags]),
 * H_{l+1} = ReLU((A*H_l)*W + W_in[tags]) -- kernel_mean_field.cpp:31-44 for one-hot inputs.
 * Requires d = 128, every graph at most 128 nodes with a contiguous node range (graph_ptr, nn_common.h:63-73)
 * and no edge between graphs.  Consecutive graphs are packed into tiles of at most 128 nodes; a tile's node
 * embeddings stay in shared memory across the levels, the dense stage runs on the tcgen05 tensor cores in
 * 3xTF32, and only Y [G x d] (plus embed_out [N x d] if given) is written.  A larger graph, an edge that
 * leaves its graph's tile or a tag outside [0, num_tags) is reported through the status word, not faulted.
 * val may be NULL (all ones).  workspace: s2v_graph_tiles_workspace_bytes(G) bytes of device memory. */
size_t s2v_graph_tiles_workspace_bytes(int64_t num_graphs);
int s2v_graph_tiles_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int d, int levels, const int32_t* row_ptr,
                        const int32_t* col_idx, const float* val, const int32_t* graph_ptr, const int32_t* tags, int num_tags,
                        const float* W_in, const float* W, int pool_average, void* workspace, size_t workspace_bytes, float* Y,
                        float* embed_out);

/* ---- the whole classifier on device buffers (FactorGraph::FeedForward of the model
 *      in kernel_mean_field.cpp:28-47 with targets = output). ---- */
typedef struct s2v_model {
    int num_feat;   /* F */
    int d;          /* latent dimension (cfg::conv_size) */
    int levels;     /* cfg::max_lv */
    int hidden;     /* cfg::n_hidden */
    int num_class;
    const float* w_n2l;       /* [F x d]       "input-node-to-latent" */
    const float* p_node_conv; /* [d x d]       "linear-node-conv"     */
    const float* h1_weight;   /* [d x hidden]  */
    const float* h2_weight;   /* [hidden x C]  */
    int pool_average;         /* 0: sum pooling (the shipped model, kernel_mean_field.cpp:12); 1: mean pooling */
} s2v_model;

typedef struct s2v_batch {
    int64_t num_graphs;
    int64_t num_nodes;
    int64_t num_edges;          /* nnz of the node-to-node matrix */
    const int32_t* n2n_row_ptr; /* [N+1] */
    const int32_t* n2n_col_idx; /* [E]   */
    const float* n2n_val;       /* [E] or NULL (all ones) */
    const int32_t* graph_ptr;   /* [G+1] node range of each graph */
    const int32_t* tags;        /* [N] one-hot node types, or NULL when x_dense is given */
    const float* x_dense;       /* [N x F] or NULL */
    int32_t max_graph_nodes;    /* node count of the largest graph of the batch, or 0 if unknown.  Device entry
                                   points cannot read graph_ptr on the host; with 1..128 here (and d = 128, tags,
                                   S2V_OPT_GRAPH_TILES on) s2v_forward_f32 runs the whole classifier as one tile kernel
                                   that keeps the embeddings in shared memory.  A value that understates the truth is reported
                                   through the status word (S2V_ERR_UNSUPPORTED) and the oversized graphs are
                                   truncated.  s2v_infer_host_f32 computes it itself. */
} s2v_batch;

/* Bytes of device workspace s2v_forward_f32 needs (three [N x d] buffers + [G x d] + the tile plan). */
size_t s2v_forward_workspace_bytes(int64_t num_nodes, int64_t num_graphs, int d);
/* logits [G x C]; probs, pred, embed_out ([N x d], the last level) may be NULL.
 * model weights and batch arrays are device pointers. */
int s2v_forward_f32(s2v_ctx* ctx, s2v_stream stream, const s2v_model* model, const s2v_batch* batch,
                    void* workspace, size_t workspace_bytes, float* logits, float* probs, int32_t* pred,
                    float* embed_out);

/* ---- the whole classifier for callers that cannot allocate device memory.
 * No counterpart in the reference (its tensors call cudaMalloc through MemHolder).
 * Same arguments and results as s2v_forward_f32 minus the workspace: the scratch lives
 * in a fixed S2V_STATIC_SCRATCH_BYTES array inside the loaded module, so no cudaMalloc /
 * cudaFree happens on this path.  Meant for hosts whose device memory is owned
 * entirely by another pool, or that may not call the allocator because it
 * synchronises the whole device.  Batches whose s2v_forward_workspace_bytes exceeds
 * the array are rejected with S2V_ERR_WORKSPACE.  The first call on a device resolves
 * the array's address (do it at set-up, before any stream capture begins).  All calls
 * on a GPU share the array and keep its last contents; nothing needs zeroing, but
 * calls that overlap on the same GPU race and must be serialised by the caller.
 * With d = 128 the array bounds the batch to fewer than 10,900 nodes, below the 16,384 rows from which the
 * per-level tcgen05 kernel is chosen: this entry runs the warp-level (mma.sync) level kernel, or the tile
 * kernel when max_graph_nodes allows it. */
#define S2V_STATIC_SCRATCH_BYTES (16u << 20)
int s2v_forward_static_f32(s2v_ctx* ctx, s2v_stream stream, const s2v_model* model, const s2v_batch* batch,
                           float* logits, float* probs, int32_t* pred, float* embed_out);

/* ---- host-side batch construction, bit-identical to the reference ----
 * Node-to-node CSR from a directed edge list in AddEdge order: row y lists the sources
 * of edges x->y in insertion order (GraphStruct::AddEdge, src/util/graph_struct.cpp:62-70
 * + Node2NodeMsgPass::InitCPUWeight, src/nn/msg_pass.cpp:46-67).  val may be NULL;
 * `average` != 0 writes 1/in-degree.  All pointers are HOST pointers. */
int s2v_build_n2n_csr_host(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src,
                           const int32_t* edge_dst, int average, int32_t* row_ptr, int32_t* col_idx, float* val);
/* The other message-passing matrices of the reference (edge-level embeddings, e.g. loopy belief propagation),
 * built from the same edge list (edge e = edge_src[e] -> edge_dst[e], in AddEdge order); HOST pointers.
 *   edge-to-node [N x E]: row y lists the INDICES of the edges into y in insertion order, val 1 or 1/in-degree
 *                         (Edge2NodeMsgPass::InitCPUWeight, src/nn/msg_pass.cpp:72-94);
 *   node-to-edge [E x N]: row e has the single entry edge_src[e], val 1 (Node2EdgeMsgPass, msg_pass.cpp:98-116);
 *   edge-to-edge [E x E]: row e = (from -> to) lists the indices of the edges into `from` except those coming
 *                         from `to`, in insertion order, val 1 (Edge2EdgeMsgPass, msg_pass.cpp:120-152).
 * The number of entries of the edge-to-edge matrix is not known in advance: call once with col_idx = NULL to get
 * *nnz_out, then with arrays of that capacity (S2V_ERR_WORKSPACE if capacity is too small; *nnz_out is always set). */
int s2v_build_e2n_csr_host(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src, const int32_t* edge_dst,
                           int average, int32_t* row_ptr, int32_t* col_idx, float* val);
int s2v_build_n2e_csr_host(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src, int32_t* row_ptr, int32_t* col_idx,
                           float* val);
int s2v_build_e2e_csr_host(int64_t num_nodes, int64_t num_edges, const int32_t* edge_src, const int32_t* edge_dst,
                           int32_t* row_ptr, int32_t* col_idx, float* val, int64_t capacity, int64_t* nnz_out);
/* Checks a host CSR: row_ptr[0]==0, monotone, row_ptr[m]==nnz, 0 <= col_idx < k. */
int s2v_validate_csr_host(int64_t m, int64_t k, int64_t nnz, const int32_t* row_ptr, const int32_t* col_idx);

/* The same sort on the DEVICE (device pointers, int32 arrays): a stable counting sort of the edge list by
 * destination with this library's own kernels, output bit-identical to s2v_build_n2n_csr_host.
 * `scratch` needs s2v_build_n2n_csr_scratch_bytes(num_nodes, num_edges) bytes.  Edges with an endpoint
 * outside [0, num_nodes) are dropped from the count and reported through the status word (S2V_ERR_BAD_CSR). */
size_t s2v_build_n2n_csr_scratch_bytes(int64_t num_nodes, int64_t num_edges);
int s2v_build_n2n_csr_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_nodes, int64_t num_edges, const int32_t* edge_src,
                          const int32_t* edge_dst, int average, void* scratch, size_t scratch_bytes, int32_t* row_ptr,
                          int32_t* col_idx, float* val);

/* ---- the whole classifier from HOST buffers: what one FeedForward call of the
 * reference driver does per batch, uploads included (SpTensor<GPU>::CopyFrom(CPU),
 * src/tensor/gpu_sparse_tensor.cu:55-63; input.CopyFrom(x_cpu), nn_common.h:101).
 * `batch` arrays are host pointers (pinned memory makes the copies asynchronous);
 * `model` weights are DEVICE pointers (parameters live on the device in the
 * reference too).  Writes logits_host [G x C] and pred_host [G] (either may be NULL)
 * and returns after they are valid.  Staging buffers are owned by ctx and only grow.
 * The host arrays are scanned (unless S2V_OPT_VALIDATE_HOST_INPUT is 0): row_ptr and graph_ptr monotone with the
 * right ends, 0 <= col_idx < N, 0 <= tags < F; a violation returns S2V_ERR_BAD_CSR (or S2V_ERR_INVALID_ARG for a
 * tag) and no result is written.  Offsets and column indices are scanned before anything is copied or launched;
 * tags, which the kernels clamp into the table themselves, are scanned while the device already works. */
int s2v_infer_host_f32(s2v_ctx* ctx, const s2v_model* model, const s2v_batch* batch_host, float* logits_host,
                       int32_t* pred_host);

/* The same from a raw directed edge list in AddEdge order (what GraphStruct::edge_list holds after GetBatch,
 * src/util/graph_struct.cpp:62-70, nn_common.h:76-90): the edge list is uploaded and the node-to-node CSR is
 * built on the device by s2v_build_n2n_csr_f32, so the host does no sorting at all.  All array arguments are HOST
 * pointers (pinned memory makes the copies asynchronous).  graph_ptr is checked before anything is launched; edge
 * endpoints and tags are scanned on the host while the device already works (the device-side builder drops and
 * reports an edge outside [0, N), the kernels clamp a tag), with the same return codes as s2v_infer_host_f32. */
int s2v_infer_edges_host_f32(s2v_ctx* ctx, const s2v_model* model, int64_t num_graphs, int64_t num_nodes, int64_t num_edges,
                             const int32_t* edge_src_host, const int32_t* edge_dst_host, const int32_t* graph_ptr_host,
                             const int32_t* tags_host, float* logits_host, int32_t* pred_host);

/* Two batches in flight (no counterpart in the reference, whose FeedForward is synchronous).  A context has two
 * lanes, 0 and 1, each with its own stream and staging memory.  s2v_infer_edges_host_submit puts one batch on a
 * lane -- upload, CSR build, forward, download, all asynchronous -- and returns after scanning the host arrays
 * (which it does while the device already works); s2v_infer_host_wait blocks until that lane's batch is done,
 * reports what the scan or a kernel found, and only then writes logits_host / pred_host.  A serving loop that
 * submits batch i+1 on the other lane before it waits for batch i overlaps the PCIe transfers of one batch with
 * the kernels of the other.  The caller's arrays (inputs and outputs) must stay valid and untouched from submit to
 * wait; pinned input arrays keep the submit asynchronous.  Submitting to a lane that still holds a batch, or
 * calling a synchronous host entry point (they use lane 0) while lane 0 holds one, returns S2V_ERR_INVALID_ARG;
 * waiting on an idle lane returns S2V_OK. */
int s2v_infer_edges_host_submit(s2v_ctx* ctx, int lane, const s2v_model* model, int64_t num_graphs, int64_t num_nodes,
                                int64_t num_edges, const int32_t* edge_src_host, const int32_t* edge_dst_host,
                                const int32_t* graph_ptr_host, const int32_t* tags_host, float* logits_host, int32_t* pred_host);
int s2v_infer_host_wait(s2v_ctx* ctx, int lane);

/* ---- several GPUs (no counterpart in the reference, which drives one GPU: src/tensor/gpu_handle.cu:17-44).
 * The path needs two exchanges and no reduction: the final gather of the logits when a batch is sharded by
 * graph, and one exchange of embedding rows per level when a single giant graph is partitioned by rows (all
 * slabs to everyone, or to every rank only the rows it references).  All go straight to NCCL, which is opened at run time (libnccl.so.2, or the library named by the environment
 * variable S2V_NCCL_LIBRARY); a process that already has an NCCL loaded shares it.  Any NCCL failure is returned
 * as S2V_ERR_COMM with NCCL's message in s2v_comm_last_error (pass NULL for failures before a communicator
 * exists).  Calls are asynchronous on `stream`, which belongs to the communicator's device. */
typedef struct s2v_comm s2v_comm;
#define S2V_COMM_ID_BYTES 128
/* One process, several GPUs: out[0..ngpu) receive one communicator per device of devs (ncclCommInitAll);
 * each is then used by the host thread that drives that GPU. */
int s2v_comm_create(int ngpu, const int* devs, s2v_comm** out);
/* One process per GPU: rank 0 obtains an id and hands its S2V_COMM_ID_BYTES bytes to the other ranks by any
 * means (a file, MPI, a key-value store); every rank then calls s2v_comm_create_rank with its own device.
 * device = -1 leaves the device selection to the caller. */
int s2v_comm_unique_id(void* id_out);
int s2v_comm_create_rank(int device, const void* id, int world, int rank, s2v_comm** out);
int s2v_comm_destroy(s2v_comm* comm);
int s2v_comm_rank(const s2v_comm* comm);
int s2v_comm_world(const s2v_comm* comm);
const char* s2v_comm_last_error(const s2v_comm* comm);
/* full[r*rows*d ..] = slab of rank r, for equal slabs of rows x d floats (in place if slab already sits at
 * full + rank*rows*d): the per-level exchange of a row-partitioned graph. */
int s2v_allgather_rows_f32(s2v_comm* comm, s2v_stream stream, int64_t rows, int d, const float* slab, float* full);
/* Pairwise exchange of rows of d floats with per-peer counts (an all-to-all-v): this rank sends rows
 * [send_offsets[p], send_offsets[p+1]) of `send` to rank p and receives recv_rows[p] rows from rank p at
 * recv + recv_offsets[p]*d.  send_offsets (world+1 entries), recv_offsets and recv_rows (world entries) are
 * HOST arrays; a count of zero skips the peer; rows addressed to the calling rank itself are exchanged like any
 * other.  One group of ncclSend / ncclRecv.  This is the per-level exchange of a row-partitioned graph when
 * every rank fetches only the rows of H its own rows reference instead of all of H. */
int s2v_exchange_rows_f32(s2v_comm* comm, s2v_stream stream, int d, const float* send, const int64_t* send_offsets,
                          float* recv, const int64_t* recv_offsets, const int64_t* recv_rows);
/* Gather of the results of a batch sharded by graph: rank r holds graphs_per_rank[r] rows (a HOST array of
 * `world` counts, the same on every rank); logits_all [sum x C] and pred_all [sum] receive all ranks' rows in
 * rank order on EVERY rank.  Either pair (logits / pred) may be NULL. */
int s2v_gather_logits(s2v_comm* comm, s2v_stream stream, const int64_t* graphs_per_rank, int num_class, const float* logits_local,
                      const int32_t* pred_local, float* logits_all, int32_t* pred_all);

#ifdef __cplusplus
}
#endif
#endif /* S2V_B200_H */
