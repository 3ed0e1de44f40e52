/*
 * Harness around the UNMODIFIED reference (Hanjun-Dai/graphnn) CPU code, TEST INFRASTRUCTURE ONLY.
 *
 * This file is compiled together with the reference's own src/ ** / *.cpp (taken
 * where they lie in a checkout of the reference, nothing copied) and the MKL/TBB
 * stand-ins in shim/.  It exposes, with C linkage, two calls that drive the
 * reference's classes in `mode = CPU`:
 *
 *   ref_s2v_forward : the structure2vec mean-field classifier wired exactly like
 *                     examples/graph_classification/src/kernel_mean_field.cpp:28-47
 *                     (MatMul/ReLU/ElewiseAdd over Node2NodeMsgPass and
 *                     SubgraphMsgPass), fed the way nn_common.h:36-105 feeds it
 *                     (GraphStruct::Resize/AddNode/AddEdge, dense X), run through
 *                     FactorGraph::FeedForward(..., Phase::TEST)
 *                     (src/nn/factor_graph.cpp:146-180).
 *   ref_level_forward : one message-passing level, the factor chain
 *                     MatMul(sparse A, H) -> MatMul(., W) -> ElewiseAdd(., X) -> ReLU
 *                     (kernel_mean_field.cpp:38-41) on caller-supplied CSR.
 *
 *   ref_msgpass_matrix : any of the five message-passing matrices as the reference's own factor builds it.
 *
 * Both return the per-iteration wall time of FeedForward so the same binary is
 * the timed CPU baseline.  The built library lives in oracle/_ref/ and is never
 * linked into, or loaded by, the product.
 */
#include <chrono>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "tensor/tensor_all.h"
#include "nn/nn_all.h"
#include "util/graph_struct.h"
#include "mkl.h"

using namespace gnn;

namespace
{

typedef CPU mode;
typedef float Dtype;
typedef std::shared_ptr<DTensorVar<mode, Dtype>> DVar;

void fill_param(DVar& p, const float* src)
{
    std::memcpy(p->value.data->ptr, src, sizeof(float) * p->value.shape.Count());
}

void copy_out(float* dst, DTensor<mode, Dtype>& t)
{
    if (dst) std::memcpy(dst, t.data->ptr, sizeof(float) * t.shape.Count());
}

double now_s()
{
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace

extern "C" {

void ref_set_threads(int n)
{
    s2v_shim_set_threads(n);
}

/*
 * nodes_per_graph[G]; directed edges (edge_src[e] -> edge_dst[e]) in global node
 * ids, in the order the caller wants GraphStruct::AddEdge to see them; X is the
 * dense [N x F] node-feature matrix.  Every output pointer may be NULL.
 *   levels : [(L+1) x N x d]  H0 .. HL         msg : [N x d] pre-activation X*W_in
 * Returns 0, or a negative value when the arguments are inconsistent.
 */
int ref_s2v_forward(int G, const int* nodes_per_graph, int E, const int* edge_src, const int* edge_dst, int F,
                    const float* X, int d, int L, int hidden, int C, const float* w_n2l, const float* p_node_conv,
                    const float* h1_weight, const float* h2_weight, int* n2n_row_ptr, int* n2n_col_idx,
                    float* n2n_val, int* sub_row_ptr, int* sub_col_idx, float* sub_val, float* msg, float* levels,
                    float* pooled, float* logits, float* probs, int* argmax, int iters, double* seconds)
{
    if (G <= 0 || F <= 0 || d <= 0 || L < 0 || hidden <= 0 || C <= 0) return -1;
    size_t N = 0;
    for (int g = 0; g < G; ++g) N += nodes_per_graph[g];

    /* --- batch construction, following GetBatch (nn_common.h:36-105) --- */
    GraphStruct graph;
    graph.Resize(G, N);
    {
        int node = 0;
        for (int g = 0; g < G; ++g)
            for (int j = 0; j < nodes_per_graph[g]; ++j) graph.AddNode(g, node++);
        for (int e = 0; e < E; ++e) graph.AddEdge(e, edge_src[e], edge_dst[e]);
    }
    DTensor<mode, Dtype> input;
    input.Reshape({N, (size_t)F});
    std::memcpy(input.data->ptr, X, sizeof(float) * N * F);

    /* --- model, following InitModel (kernel_mean_field.cpp:6-47) --- */
    FactorGraph fg;
    ParamSet<mode, Dtype> model;
    auto gvar = add_const<GraphVar>(fg, "graph", true);
    auto n2nsum_param = af<Node2NodeMsgPass<mode, Dtype>>(fg, {gvar});
    auto subgsum_param = af<SubgraphMsgPass<mode, Dtype>>(fg, {gvar});

    auto p_w_n2l = add_diff<DTensorVar>(model, "input-node-to-latent", {(uint)F, (uint)d});
    auto p_conv = add_diff<DTensorVar>(model, "linear-node-conv", {(uint)d, (uint)d});
    auto p_h1 = add_diff<DTensorVar>(model, "h1_weight", {(uint)d, (uint)hidden});
    auto p_h2 = add_diff<DTensorVar>(model, "h2_weight", {(uint)hidden, (uint)C});
    fill_param(p_w_n2l, w_n2l);
    fill_param(p_conv, p_node_conv);
    fill_param(p_h1, h1_weight);
    fill_param(p_h2, h2_weight);
    fg.AddParam(p_w_n2l);
    fg.AddParam(p_conv);
    fg.AddParam(p_h1);
    fg.AddParam(p_h2);

    auto node_input = add_const<DTensorVar<mode, Dtype>>(fg, "data", true);
    auto input_message = af<MatMul>(fg, {node_input, p_w_n2l});
    auto input_potential = af<ReLU>(fg, {input_message});
    std::vector<DVar> level_vars;
    level_vars.push_back(input_potential);
    auto cur = input_potential;
    for (int lv = 0; lv < L; ++lv) {
        auto n2npool = af<MatMul>(fg, {n2nsum_param, cur});
        auto node_linear = af<MatMul>(fg, {n2npool, p_conv});
        auto merged = af<ElewiseAdd>(fg, {node_linear, input_message});
        cur = af<ReLU>(fg, {merged});
        level_vars.push_back(cur);
    }
    auto y_potential = af<MatMul>(fg, {subgsum_param, cur});
    auto hid = af<MatMul>(fg, {y_potential, p_h1});
    auto hid_act = af<ReLU>(fg, {hid});
    auto output = af<MatMul>(fg, {hid_act, p_h2});
    auto prob = af<Softmax>(fg, {output});
    auto pred = af<ArgMax>(fg, {output});

    std::map<std::string, void*> feed;
    feed["data"] = &input;
    feed["graph"] = &graph;
    std::vector<std::shared_ptr<Variable>> targets;
    targets.push_back(output);
    targets.push_back(prob);
    targets.push_back(pred);

    if (iters < 1) iters = 1;
    for (int it = 0; it < iters; ++it) {
        double t0 = now_s();
        fg.FeedForward(targets, feed, Phase::TEST);
        double t1 = now_s();
        if (seconds) seconds[it] = t1 - t0;
    }

    auto& A = n2nsum_param->value;
    if (n2n_row_ptr) std::memcpy(n2n_row_ptr, A.data->row_ptr, sizeof(int) * (N + 1));
    if (n2n_col_idx) std::memcpy(n2n_col_idx, A.data->col_idx, sizeof(int) * A.data->nnz);
    if (n2n_val) std::memcpy(n2n_val, A.data->val, sizeof(float) * A.data->nnz);
    auto& S = subgsum_param->value;
    if (sub_row_ptr) std::memcpy(sub_row_ptr, S.data->row_ptr, sizeof(int) * (G + 1));
    if (sub_col_idx) std::memcpy(sub_col_idx, S.data->col_idx, sizeof(int) * S.data->nnz);
    if (sub_val) std::memcpy(sub_val, S.data->val, sizeof(float) * S.data->nnz);
    copy_out(msg, input_message->value);
    if (levels)
        for (size_t l = 0; l < level_vars.size(); ++l) copy_out(levels + l * N * d, level_vars[l]->value);
    copy_out(pooled, y_potential->value);
    copy_out(logits, output->value);
    copy_out(probs, prob->value);
    if (argmax) std::memcpy(argmax, pred->value.data->ptr, sizeof(int) * G);
    if ((int)A.data->nnz != E || (int)S.data->nnz != (int)N) return -2;
    return 0;
}

/*
 * Writes a checkpoint with the reference's own ParamSet::Save (src/nn/param_set.cpp:28-41) holding the four
 * parameters of the classifier under the names the driver gives them (kernel_mean_field.cpp:14-17).
 */
int ref_save_model(const char* path, int F, int d, int hidden, int C, const float* w_n2l, const float* p_node_conv,
                   const float* h1_weight, const float* h2_weight)
{
    ParamSet<mode, Dtype> model;
    auto a = add_diff<DTensorVar>(model, "input-node-to-latent", {(uint)F, (uint)d});
    auto b = add_diff<DTensorVar>(model, "linear-node-conv", {(uint)d, (uint)d});
    auto c = add_diff<DTensorVar>(model, "h1_weight", {(uint)d, (uint)hidden});
    auto e = add_diff<DTensorVar>(model, "h2_weight", {(uint)hidden, (uint)C});
    fill_param(a, w_n2l);
    fill_param(b, p_node_conv);
    fill_param(c, h1_weight);
    fill_param(e, h2_weight);
    model.Save(path);
    return 0;
}

/*
 * Loss / metric tail exactly as the driver wires it (kernel_mean_field.cpp:49-56): CrossEntropy(output,
 * label, need_softmax) -> ReduceMean; ArgMax(label) -> InTopK(output, truth) -> TypeCast -> ReduceMean.
 * logits [G x C]; labels as the CSR tensor GetBatch builds (nn_common.h:92-99).
 */
int ref_loss_acc(int G, int C, const float* logits, const int* label_rp, const int* label_ci, const float* label_val,
                 float* loss_mean, float* acc_mean, float* per_graph_loss)
{
    if (G <= 0 || C <= 0) return -1;
    DTensor<mode, Dtype> out_t;
    out_t.Reshape({(size_t)G, (size_t)C});
    std::memcpy(out_t.data->ptr, logits, sizeof(float) * (size_t)G * C);
    SpTensor<mode, Dtype> y;
    y.Reshape({(size_t)G, (size_t)C});
    y.ResizeSp(label_rp[G], G + 1);
    std::memcpy(y.data->row_ptr, label_rp, sizeof(int) * (G + 1));
    std::memcpy(y.data->col_idx, label_ci, sizeof(int) * label_rp[G]);
    for (int i = 0; i < label_rp[G]; ++i) y.data->val[i] = label_val ? label_val[i] : 1.0f;

    FactorGraph fg;
    auto output = add_const<DTensorVar<mode, Dtype>>(fg, "output", true);
    auto label = add_const<SpTensorVar<mode, Dtype>>(fg, "label", true);
    auto ce = af<CrossEntropy>(fg, {output, label}, true);
    auto loss = af<ReduceMean>(fg, {ce});
    auto truth = af<ArgMax>(fg, {label});
    auto cmp = af<InTopK<mode, Dtype>>(fg, std::make_pair(output, truth));
    auto real_cmp = af<TypeCast<mode, Dtype>>(fg, {cmp});
    auto acc = af<ReduceMean>(fg, {real_cmp});
    std::map<std::string, void*> feed;
    feed["output"] = &out_t;
    feed["label"] = &y;
    std::vector<std::shared_ptr<Variable>> targets;
    targets.push_back(loss);
    targets.push_back(acc);
    fg.FeedForward(targets, feed, Phase::TEST);
    *loss_mean = loss->AsScalar();
    *acc_mean = acc->AsScalar();
    copy_out(per_graph_loss, ce->value);
    return 0;
}

/*
 * One level on caller-supplied CSR A [n_rows x n_src] (int32, 3-array), H [n_src x d],
 * W [d x d], X [n_rows x d] (may be NULL: then the ElewiseAdd factor is left out).
 * out [n_rows x d] = ReLU((A*H)*W + X), through the reference's factors.
 */
int ref_level_forward(int n_rows, int n_src, int nnz, const int* row_ptr, const int* col_idx, const float* val,
                      int d, const float* H, const float* W, const float* X, float* out, int iters,
                      double* seconds)
{
    if (n_rows <= 0 || n_src <= 0 || d <= 0 || nnz < 0) return -1;
    SpTensor<mode, Dtype> A;
    A.Reshape({(size_t)n_rows, (size_t)n_src});
    A.ResizeSp(nnz, n_rows + 1);
    std::memcpy(A.data->row_ptr, row_ptr, sizeof(int) * (n_rows + 1));
    std::memcpy(A.data->col_idx, col_idx, sizeof(int) * nnz);
    if (val)
        std::memcpy(A.data->val, val, sizeof(float) * nnz);
    else
        for (int i = 0; i < nnz; ++i) A.data->val[i] = 1.0f;

    DTensor<mode, Dtype> h, x;
    h.Reshape({(size_t)n_src, (size_t)d});
    std::memcpy(h.data->ptr, H, sizeof(float) * (size_t)n_src * d);
    if (X) {
        x.Reshape({(size_t)n_rows, (size_t)d});
        std::memcpy(x.data->ptr, X, sizeof(float) * (size_t)n_rows * d);
    }

    FactorGraph fg;
    ParamSet<mode, Dtype> model;
    auto a_var = add_const<SpTensorVar<mode, Dtype>>(fg, "n2n", true);
    auto h_var = add_const<DTensorVar<mode, Dtype>>(fg, "h", true);
    auto p_conv = add_diff<DTensorVar>(model, "linear-node-conv", {(uint)d, (uint)d});
    fill_param(p_conv, W);
    fg.AddParam(p_conv);
    auto n2npool = af<MatMul>(fg, {a_var, h_var});
    auto node_linear = af<MatMul>(fg, {n2npool, p_conv});
    DVar result;
    std::map<std::string, void*> feed;
    feed["n2n"] = &A;
    feed["h"] = &h;
    if (X) {
        auto x_var = add_const<DTensorVar<mode, Dtype>>(fg, "x", true);
        auto merged = af<ElewiseAdd>(fg, {node_linear, x_var});
        result = af<ReLU>(fg, {merged});
        feed["x"] = &x;
    } else {
        result = af<ReLU>(fg, {node_linear});
    }
    std::vector<std::shared_ptr<Variable>> targets;
    targets.push_back(result);
    if (iters < 1) iters = 1;
    for (int it = 0; it < iters; ++it) {
        double t0 = now_s();
        fg.FeedForward(targets, feed, Phase::TEST);
        double t1 = now_s();
        if (seconds) seconds[it] = t1 - t0;
    }
    copy_out(out, result->value);
    return 0;
}

/*
 * The message-passing matrices of a graph as the reference's own factors build them
 * (Node2Node / Edge2Node / Node2Edge / Edge2Edge / SubgraphMsgPass::InitCPUWeight, src/nn/msg_pass.cpp:46-177),
 * with the factors' `average` flag.  which: 0 n2n, 1 e2n, 2 n2e, 3 e2e, 4 subgraph.  Returns nnz (or a negative
 * value); row_ptr needs rows+1 entries, col_idx / val `capacity` entries (nothing beyond capacity is written).
 */
int ref_msgpass_matrix(int which, int average, int G, const int* nodes_per_graph, int E, const int* edge_src, const int* edge_dst,
                       int* row_ptr, int* col_idx, float* val, int capacity)
{
    if (G <= 0) return -1;
    size_t N = 0;
    for (int g = 0; g < G; ++g) N += nodes_per_graph[g];
    GraphStruct graph;
    graph.Resize(G, N);
    int node = 0;
    for (int g = 0; g < G; ++g)
        for (int j = 0; j < nodes_per_graph[g]; ++j) graph.AddNode(g, node++);
    for (int e = 0; e < E; ++e) graph.AddEdge(e, edge_src[e], edge_dst[e]);

    FactorGraph fg;
    auto gvar = add_const<GraphVar>(fg, "graph", true);
    std::shared_ptr<SpTensorVar<mode, Dtype>> out;
    switch (which) {
        case 0: out = af<Node2NodeMsgPass<mode, Dtype>>(fg, {gvar}, average != 0); break;
        case 1: out = af<Edge2NodeMsgPass<mode, Dtype>>(fg, {gvar}, average != 0); break;
        case 2: out = af<Node2EdgeMsgPass<mode, Dtype>>(fg, {gvar}, average != 0); break;
        case 3: out = af<Edge2EdgeMsgPass<mode, Dtype>>(fg, {gvar}, average != 0); break;
        case 4: out = af<SubgraphMsgPass<mode, Dtype>>(fg, {gvar}, average != 0); break;
        default: return -1;
    }
    std::map<std::string, void*> feed;
    feed["graph"] = &graph;
    std::vector<std::shared_ptr<Variable>> targets;
    targets.push_back(out);
    fg.FeedForward(targets, feed, Phase::TEST);
    auto& M = out->value;
    const int nnz = (int)M.data->nnz;
    const size_t rows = M.rows();
    if (row_ptr) std::memcpy(row_ptr, M.data->row_ptr, sizeof(int) * (rows + 1));
    const int n = nnz < capacity ? nnz : capacity;
    if (col_idx) std::memcpy(col_idx, M.data->col_idx, sizeof(int) * n);
    if (val) std::memcpy(val, M.data->val, sizeof(float) * n);
    return nnz;
}

}  // extern "C"
