/*
 * CPU restatement of the structure2vec mean-field inference path of
 * Hanjun-Dai/graphnn.  TEST INFRASTRUCTURE ONLY: this file is the parity checker
 * for the CUDA library (and, where the reference itself was not compiled, the
 * timed CPU baseline).  The product never links, loads or calls it.
 *
 * Pinning: the reference holds no golden vectors for this path.  This file is
 * pinned against the reference's own C++ (built with MKL replaced by plain loops,
 * see build.py / ref_harness.cpp): integer outputs bit-exact, floats within
 * 1e-5 relative / 1e-5 absolute; the outputs of that build on a seeded batch are
 * committed as fixtures under tests/golden/.
 *
 * Each function cites the reference code it follows (paths inside the reference
 * checkout).  Sums run in single precision, one output at a time, in stored order
 * (CSR order for sparse rows, ascending k for dense products), which is what the
 * reference's CPU path does up to MKL's unknown internal order.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 1;

void oracle_set_threads(int n)
{
    g_threads = n < 1 ? 1 : n;
}

/*
 * CSR A [N x N] of in-neighbour sums.
 * GraphStruct::AddEdge (src/util/graph_struct.cpp:62-70) appends (edge id, x) to
 * in_edges[y] for edge x->y; Node2NodeMsgPass::InitCPUWeight
 * (src/nn/msg_pass.cpp:46-67) then writes, for each node i in order, the sources of
 * in_edges[i] in insertion order with value 1 (or 1/in-degree when `average`).
 * A stable counting sort of the edge list by destination gives the same arrays.
 * Returns nnz (== E), or -1 on a node id out of range.
 */
int64_t oracle_build_n2n_csr(int64_t N, int64_t E, const int32_t* edge_src, const int32_t* edge_dst, int average,
                             int32_t* row_ptr, int32_t* col_idx, float* val)
{
    int64_t* fill = (int64_t*)calloc((size_t)N + 1, sizeof(int64_t));
    for (int64_t e = 0; e < E; ++e) {
        if (edge_dst[e] < 0 || edge_dst[e] >= N || edge_src[e] < 0 || edge_src[e] >= N) {
            free(fill);
            return -1;
        }
        fill[edge_dst[e] + 1]++;
    }
    for (int64_t i = 0; i < N; ++i) fill[i + 1] += fill[i];
    for (int64_t i = 0; i <= N; ++i) row_ptr[i] = (int32_t)fill[i];
    for (int64_t e = 0; e < E; ++e) {
        int64_t pos = fill[edge_dst[e]]++;
        col_idx[pos] = edge_src[e];
    }
    for (int64_t i = 0; i < N; ++i) {
        int32_t deg = row_ptr[i + 1] - row_ptr[i];
        for (int32_t t = row_ptr[i]; t < row_ptr[i + 1]; ++t) val[t] = average ? (float)(1.0 / deg) : 1.0f;
    }
    free(fill);
    return E;
}

/*
 * The edge-level message-passing matrices (src/nn/msg_pass.cpp:72-152), restated with per-node lists
 * of (edge index, source) pairs kept in insertion order exactly like GraphStruct::in_edges
 * (src/util/graph_struct.cpp:62-70).  which: 1 edge-to-node [N x E], 2 node-to-edge [E x N],
 * 3 edge-to-edge [E x E].  Returns nnz; col_idx / val receive at most `capacity` entries.
 */
int64_t oracle_build_edge_csr(int which, int64_t N, int64_t E, const int32_t* edge_src, const int32_t* edge_dst, int average,
                              int32_t* row_ptr, int32_t* col_idx, float* val, int64_t capacity)
{
    /* in_edges as linked lists: head/tail per node, next per edge */
    int32_t* first = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N > 0 ? N : 1));
    int32_t* last = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N > 0 ? N : 1));
    int32_t* next = (int32_t*)malloc(sizeof(int32_t) * (size_t)(E > 0 ? E : 1));
    int32_t* count = (int32_t*)calloc((size_t)(N > 0 ? N : 1), sizeof(int32_t));
    for (int64_t i = 0; i < N; ++i) first[i] = last[i] = -1;
    for (int64_t e = 0; e < E; ++e) {   /* AddEdge(e, x, y): in_edges[y].push_back({e, x}) */
        const int32_t y = edge_dst[e];
        next[e] = -1;
        if (first[y] < 0) first[y] = (int32_t)e; else next[last[y]] = (int32_t)e;
        last[y] = (int32_t)e;
        count[y]++;
    }
    int64_t nnz = 0;
    if (which == 1) {          /* Edge2NodeMsgPass: row i = indices of the edges into i */
        for (int64_t i = 0; i < N; ++i) {
            row_ptr[i] = (int32_t)nnz;
            for (int32_t e = first[i]; e >= 0; e = next[e]) {
                if (nnz < capacity) {
                    val[nnz] = average ? (float)(1.0 / count[i]) : 1.0f;
                    col_idx[nnz] = e;
                }
                nnz++;
            }
        }
        row_ptr[N] = (int32_t)nnz;
    } else if (which == 2) {   /* Node2EdgeMsgPass: row e = { source of edge e } */
        for (int64_t e = 0; e < E; ++e) {
            row_ptr[e] = (int32_t)nnz;
            if (nnz < capacity) {
                val[nnz] = 1.0f;
                col_idx[nnz] = edge_src[e];
            }
            nnz++;
        }
        row_ptr[E] = (int32_t)nnz;
    } else {                   /* Edge2EdgeMsgPass: row e = (from -> to): edges into `from` that do not come from `to` */
        for (int64_t e = 0; e < E; ++e) {
            row_ptr[e] = (int32_t)nnz;
            const int32_t from = edge_src[e], to = edge_dst[e];
            for (int32_t f = first[from]; f >= 0; f = next[f]) {
                if (edge_src[f] == to) continue;
                if (nnz < capacity) {
                    val[nnz] = 1.0f;
                    col_idx[nnz] = f;
                }
                nnz++;
            }
        }
        row_ptr[E] = (int32_t)nnz;
    }
    free(first); free(last); free(next); free(count);
    return nnz;
}

/*
 * CSR S [G x N] for graph pooling.
 * GetBatch (examples/graph_classification/include/nn_common.h:63-73) adds node
 * prefix[g]+j to subgraph g for j ascending; SubgraphMsgPass::InitCPUWeight
 * (src/nn/msg_pass.cpp:156-177) lists them in that order with value 1 (or 1/|g|).
 */
int64_t oracle_build_subgraph_csr(int64_t G, const int32_t* nodes_per_graph, int average, int32_t* row_ptr,
                                  int32_t* col_idx, float* val)
{
    int64_t nnz = 0;
    for (int64_t g = 0; g < G; ++g) {
        row_ptr[g] = (int32_t)nnz;
        for (int32_t j = 0; j < nodes_per_graph[g]; ++j) {
            val[nnz] = average ? (float)(1.0 / nodes_per_graph[g]) : 1.0f;
            col_idx[nnz] = (int32_t)nnz;
            nnz++;
        }
    }
    row_ptr[G] = (int32_t)nnz;
    return nnz;
}

/*
 * C[m x n] = A[m x k] * B[k x n], row-major, alpha 1, beta 0:
 * DTensor<CPU>::MM(dense, dense) -> cblas_sgemm (src/tensor/cpu_dense_tensor.cpp:199-211).
 */
void oracle_gemm(int64_t m, int64_t n, int64_t k, const float* A, const float* B, float* C)
{
#pragma omp parallel for num_threads(g_threads) if (g_threads > 1) schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        float* c = C + i * n;
        for (int64_t j = 0; j < n; ++j) c[j] = 0.0f;
        for (int64_t p = 0; p < k; ++p) {
            const float a = A[i * k + p];
            const float* b = B + p * n;
            for (int64_t j = 0; j < n; ++j) c[j] += a * b[j];
        }
    }
}

/*
 * C[m x n] = A_csr[m x k] * B[k x n], row-major, alpha 1, beta 0:
 * DTensor<CPU>::MM(sparse, dense) -> mkl_scsrmm "GLNC" (src/tensor/cpu_dense_tensor.cpp:214-225).
 * val may be NULL (all ones).
 */
void oracle_csrmm(int64_t m, int64_t n, const int32_t* row_ptr, const int32_t* col_idx, const float* val,
                  const float* B, float* C)
{
#pragma omp parallel for num_threads(g_threads) if (g_threads > 1) schedule(dynamic, 256)
    for (int64_t i = 0; i < m; ++i) {
        float* c = C + i * n;
        for (int64_t j = 0; j < n; ++j) c[j] = 0.0f;
        for (int32_t t = row_ptr[i]; t < row_ptr[i + 1]; ++t) {
            const float v = val ? val[t] : 1.0f;
            const float* b = B + (int64_t)col_idx[t] * n;
            for (int64_t j = 0; j < n; ++j) c[j] += v * b[j];
        }
    }
}

/* out = a + b: ElewiseAdd::Forward = CopyFrom + Axpy(1.0) (src/nn/elewise_add.cpp:12-33). */
void oracle_add(int64_t cnt, const float* a, const float* b, float* out)
{
#pragma omp parallel for num_threads(g_threads) if (g_threads > 1) schedule(static)
    for (int64_t i = 0; i < cnt; ++i) out[i] = a[i] + b[i];
}

/* ReLU: `if (x < 0) x = 0` keeps -0.0 and NaN (src/nn/relu.cpp:6-14). */
void oracle_relu(int64_t cnt, const float* in, float* out)
{
#pragma omp parallel for num_threads(g_threads) if (g_threads > 1) schedule(static)
    for (int64_t i = 0; i < cnt; ++i) {
        float v = in[i];
        out[i] = v < 0.0f ? 0.0f : v;
    }
}

/*
 * Row softmax with max subtraction, exponentials divided by their absolute sum
 * (src/tensor/cpu_dense_tensor.cpp:228-251).
 */
void oracle_softmax(int64_t rows, int64_t cols, const float* in, float* out)
{
    for (int64_t i = 0; i < rows; ++i) {
        const float* x = in + i * cols;
        float* y = out + i * cols;
        float mx = x[0];
        for (int64_t j = 1; j < cols; ++j)
            if (x[j] > mx) mx = x[j];
        float s = 0.0f;
        for (int64_t j = 0; j < cols; ++j) {
            y[j] = expf(x[j] - mx);
            s += fabsf(y[j]);
        }
        for (int64_t j = 0; j < cols; ++j) y[j] /= s;
    }
}

/* Per-row index of the maximum, first index wins ties (src/tensor/cpu_dense_tensor.cpp:177-196). */
void oracle_argmax(int64_t rows, int64_t cols, const float* in, int32_t* out)
{
    for (int64_t i = 0; i < rows; ++i) {
        const float* x = in + i * cols;
        int32_t best = 0;
        float mx = x[0];
        for (int64_t j = 1; j < cols; ++j)
            if (x[j] > mx) {
                mx = x[j];
                best = (int32_t)j;
            }
        out[i] = best;
    }
}

/*
 * One level: out = ReLU((A*H)*W + X); X may be NULL.  Factor chain of
 * examples/graph_classification/src/kernel_mean_field.cpp:38-41.
 * scratch: 2 * n_rows * d floats.
 */
void oracle_level(int64_t n_rows, int64_t d, const int32_t* row_ptr, const int32_t* col_idx, const float* val,
                  const float* H, const float* W, const float* X, float* out, float* scratch)
{
    float* pool = scratch;
    float* lin = scratch + n_rows * d;
    oracle_csrmm(n_rows, d, row_ptr, col_idx, val, H, pool);
    oracle_gemm(n_rows, d, d, pool, W, lin);
    if (X) oracle_add(n_rows * d, lin, X, lin);
    oracle_relu(n_rows * d, lin, out);
}

/*
 * The same level with every sum carried in double (row sums and the product with W), rounded to float once at
 * the end.  Not a restatement of the reference (which accumulates in float in an order its BLAS chooses): it is
 * the order-independent yardstick for rows so long that two float summation orders differ by more than the
 * parity bar (a row of a million entries summed sequentially in float carries ~1e-4 relative error itself).
 * No scratch needed.
 */
void oracle_level_f64(int64_t n_rows, int64_t d, const int32_t* row_ptr, const int32_t* col_idx, const float* val,
                      const float* H, const float* W, const float* X, float* out)
{
#pragma omp parallel for num_threads(g_threads) if (g_threads > 1) schedule(dynamic, 16)
    for (int64_t i = 0; i < n_rows; ++i) {
        double* s = (double*)calloc((size_t)(2 * d), sizeof(double));
        double* y = s + d;
        for (int32_t t = row_ptr[i]; t < row_ptr[i + 1]; ++t) {
            const double v = val ? (double)val[t] : 1.0;
            const float* b = H + (int64_t)col_idx[t] * d;
            for (int64_t j = 0; j < d; ++j) s[j] += v * (double)b[j];
        }
        for (int64_t p = 0; p < d; ++p) {
            const float* w = W + p * d;
            for (int64_t j = 0; j < d; ++j) y[j] += s[p] * (double)w[j];
        }
        for (int64_t j = 0; j < d; ++j) {
            double r = y[j] + (X ? (double)X[i * d + j] : 0.0);
            out[i * d + j] = (float)(r < 0.0 ? 0.0 : r);
        }
        free(s);
    }
}

/*
 * The whole classifier, same argument list as the harness around the reference
 * (ref_s2v_forward): model wiring of kernel_mean_field.cpp:28-47.
 */
int oracle_s2v_forward(int G, const int32_t* nodes_per_graph, int E, const int32_t* edge_src,
                       const int32_t* edge_dst, int F, const float* X, int d, int L, int hidden, int C,
                       const float* w_n2l, const float* p_node_conv, const float* h1_weight, const float* h2_weight,
                       int32_t* n2n_row_ptr, int32_t* n2n_col_idx, float* n2n_val, int32_t* sub_row_ptr,
                       int32_t* sub_col_idx, float* sub_val, float* msg_out, float* levels, float* pooled_out,
                       float* logits_out, float* probs_out, int32_t* argmax_out)
{
    if (G <= 0 || F <= 0 || d <= 0 || L < 0 || hidden <= 0 || C <= 0) return -1;
    int64_t N = 0;
    for (int g = 0; g < G; ++g) N += nodes_per_graph[g];
    int rc = 0;

    int32_t* rp = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N + 1));
    int32_t* ci = (int32_t*)malloc(sizeof(int32_t) * (size_t)(E > 0 ? E : 1));
    float* av = (float*)malloc(sizeof(float) * (size_t)(E > 0 ? E : 1));
    int32_t* srp = (int32_t*)malloc(sizeof(int32_t) * (size_t)(G + 1));
    int32_t* sci = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N > 0 ? N : 1));
    float* sv = (float*)malloc(sizeof(float) * (size_t)(N > 0 ? N : 1));
    float* msg = (float*)malloc(sizeof(float) * (size_t)N * d);
    float* cur = (float*)malloc(sizeof(float) * (size_t)N * d);
    float* nxt = (float*)malloc(sizeof(float) * (size_t)N * d);
    float* scratch = (float*)malloc(sizeof(float) * (size_t)N * d * 2);
    float* y = (float*)malloc(sizeof(float) * (size_t)G * d);
    float* hid = (float*)malloc(sizeof(float) * (size_t)G * hidden);
    float* logits = (float*)malloc(sizeof(float) * (size_t)G * C);
    float* probs = (float*)malloc(sizeof(float) * (size_t)G * C);

    if (oracle_build_n2n_csr(N, E, edge_src, edge_dst, 0, rp, ci, av) != E) rc = -2;
    if (rc == 0 && oracle_build_subgraph_csr(G, nodes_per_graph, 0, srp, sci, sv) != N) rc = -2;
    if (rc == 0) {
        oracle_gemm(N, d, F, X, w_n2l, msg);   /* input_message = X * W_in */
        oracle_relu(N * d, msg, cur);         /* input_potential_layer     */
        if (levels) memcpy(levels, cur, sizeof(float) * (size_t)N * d);
        for (int lv = 0; lv < L; ++lv) {
            oracle_level(N, d, rp, ci, av, cur, p_node_conv, msg, nxt, scratch);
            float* t = cur; cur = nxt; nxt = t;
            if (levels) memcpy(levels + (size_t)(lv + 1) * N * d, cur, sizeof(float) * (size_t)N * d);
        }
        oracle_csrmm(G, d, srp, sci, sv, cur, y);          /* y_potential */
        oracle_gemm(G, hidden, d, y, h1_weight, hid);
        oracle_relu((int64_t)G * hidden, hid, hid);
        oracle_gemm(G, C, hidden, hid, h2_weight, logits);
        oracle_softmax(G, C, logits, probs);
        if (argmax_out) oracle_argmax(G, C, logits, argmax_out);

        if (n2n_row_ptr) memcpy(n2n_row_ptr, rp, sizeof(int32_t) * (size_t)(N + 1));
        if (n2n_col_idx) memcpy(n2n_col_idx, ci, sizeof(int32_t) * (size_t)E);
        if (n2n_val) memcpy(n2n_val, av, sizeof(float) * (size_t)E);
        if (sub_row_ptr) memcpy(sub_row_ptr, srp, sizeof(int32_t) * (size_t)(G + 1));
        if (sub_col_idx) memcpy(sub_col_idx, sci, sizeof(int32_t) * (size_t)N);
        if (sub_val) memcpy(sub_val, sv, sizeof(float) * (size_t)N);
        if (msg_out) memcpy(msg_out, msg, sizeof(float) * (size_t)N * d);
        if (pooled_out) memcpy(pooled_out, y, sizeof(float) * (size_t)G * d);
        if (logits_out) memcpy(logits_out, logits, sizeof(float) * (size_t)G * C);
        if (probs_out) memcpy(probs_out, probs, sizeof(float) * (size_t)G * C);
    }
    free(rp); free(ci); free(av); free(srp); free(sci); free(sv); free(msg); free(cur); free(nxt);
    free(scratch); free(y); free(hid); free(logits); free(probs);
    return rc;
}

/*
 * Loss / metric tail of the driver's TEST loop: loss = mean cross entropy with softmax against CSR
 * labels (src/nn/cross_entropy.cpp:9-50: probabilities with |p| < 1e-8 are clamped to 1e-8), acc =
 * mean of "fewer than topk classes score strictly higher than the label's argmax"
 * (ArgMax of the CSR label row, src/tensor/cpu_sparse_tensor.cpp:86-103; InTopK,
 * src/nn/in_top_k.cpp:6-23; TypeCast; ReduceMean = sequential sum / count,
 * src/tensor/cpu_dense_tensor.cpp:283-293).  per_graph_loss may be NULL.
 */
void oracle_loss_acc(int64_t G, int64_t C, const float* logits, const int32_t* label_rp, const int32_t* label_ci,
                     const float* label_val, int topk, float* loss_mean, float* acc_mean, float* per_graph_loss)
{
    float* probs = (float*)malloc(sizeof(float) * (size_t)G * (size_t)C);
    oracle_softmax(G, C, logits, probs);
    float loss_sum = 0.0f, acc_sum = 0.0f;
    for (int64_t i = 0; i < G; ++i) {
        float loss = 0.0f;
        for (int32_t k = label_rp[i]; k < label_rp[i + 1]; ++k) {
            float t = probs[C * i + label_ci[k]];
            if (fabs(t) < 1e-8) t = 1e-8f;
            loss -= logf(t) * (label_val ? label_val[k] : 1.0f);
        }
        if (per_graph_loss) per_graph_loss[i] = loss;
        loss_sum += loss;
        int32_t target = 0;
        float cur = 0.0f;
        for (int32_t j = label_rp[i]; j < label_rp[i + 1]; ++j) {
            float v = label_val ? label_val[j] : 1.0f;
            if (j == label_rp[i] || v > cur) { cur = v; target = label_ci[j]; }
        }
        int t = 0;
        for (int64_t j = 0; j < C; ++j)
            if (j != target && logits[C * i + j] > logits[C * i + target]) t++;
        acc_sum += (float)(t < topk);
    }
    *loss_mean = loss_sum / (float)G;
    *acc_mean = acc_sum / (float)G;
    free(probs);
}
