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
    S2V_ERR_DEVICE_TIMEOUT = -7 /* a bounded device-side wait gave up */
} s2v_status;

/* ---- context: GpuHandle::Init / Destroy (include/tensor/gpu_handle.h:38-59,
 *      src/tensor/gpu_handle.cu:17-44).  Unlike the reference it does not reset the
 *      device and holds no cuBLAS/cuSPARSE/cuRAND state. */
int s2v_ctx_create(int device, s2v_ctx** out);
int s2v_ctx_destroy(s2v_ctx* ctx);
int s2v_ctx_device(const s2v_ctx* ctx);
s2v_stream s2v_ctx_stream(const s2v_ctx* ctx);
int s2v_ctx_synchronize(s2v_ctx* ctx);
const char* s2v_status_str(int status);
const char* s2v_last_error(const s2v_ctx* ctx);
/* Diagnostic, no counterpart in the reference: launches a one-warp kernel whose bounded barrier wait runs
 * out on purpose (nothing ever arrives).  The kernel returns normally; the next s2v_ctx_synchronize reports
 * S2V_ERR_DEVICE_TIMEOUT (site 99) and clears it, and the context stays usable.  This is the path every
 * wait in the level kernels takes instead of hanging the GPU. */
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
 * nn_common.h:57-70).  table : [n_table x d], x_index : int32 [n_rows]. */
int s2v_level_lookup_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n_rows, int64_t n_src, int d,
                         const int32_t* row_ptr, const int32_t* col_idx, const float* val, const float* H,
                         const float* W, const float* table, int n_table, const int32_t* x_index, float* out);

/* First level of the classifier with one-hot inputs, without materialising H0:
 * out = ReLU((A * ReLU(table[tags,:])) * W + table[tags,:]), A square [n x n]; i.e. MatMul(data, w_n2l),
 * ReLU and the first level (kernel_mean_field.cpp:31-41) in one kernel.  Only the tcgen05 kernel
 * (d = 64 or 128) has this form (n >= 16,384 unless forced); otherwise S2V_ERR_UNSUPPORTED: run
 * s2v_input_proj_onehot_f32 + s2v_level_lookup_f32 instead. */
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
} s2v_batch;

/* Bytes of device workspace s2v_forward_f32 needs (three [N x d] buffers + [G x d]). */
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
 * calls that overlap on the same GPU race and must be serialised by the caller. */
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
/* Checks a host CSR: row_ptr[0]==0, monotone, row_ptr[m]==nnz, 0 <= col_idx < k. */
int s2v_validate_csr_host(int64_t m, int64_t k, int64_t nnz, const int32_t* row_ptr, const int32_t* col_idx);

/* ---- the whole classifier from HOST buffers: what one FeedForward call of the
 * reference driver does per batch, uploads included (SpTensor<GPU>::CopyFrom(CPU),
 * src/tensor/gpu_sparse_tensor.cu:55-63; input.CopyFrom(x_cpu), nn_common.h:101).
 * `batch` arrays are host pointers (pinned memory makes the copies asynchronous);
 * `model` weights are DEVICE pointers (parameters live on the device in the
 * reference too).  Writes logits_host [G x C] and pred_host [G] (either may be NULL)
 * and returns after they are valid.  Staging buffers are owned by ctx and only grow. */
int s2v_infer_host_f32(s2v_ctx* ctx, const s2v_model* model, const s2v_batch* batch_host, float* logits_host,
                       int32_t* pred_host);

#ifdef __cplusplus
}
#endif
#endif /* S2V_B200_H */
