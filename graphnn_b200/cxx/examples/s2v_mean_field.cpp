// structure2vec mean-field classifier, inference only, written against the graphnn
// operator interface as this library provides it (the same calls a driver written for the
// reference makes: GpuHandle::Init, GraphStruct::AddNode/AddEdge, add_const / add_diff / af<>,
// FactorGraph::FeedForward).  The model is the one of the reference's
// examples/graph_classification/src/kernel_mean_field.cpp:28-47 and the batch is assembled the
// way its GetBatch does (include/nn_common.h:36-105).
//
//   s2v_mean_field <batch.bin> <out.bin> [--fused 0|1] [--iters K] [--labels labels.bin]
//
// --labels  : int32 class of every graph; the driver then also evaluates the reference's targets
//             {loss, acc} (CrossEntropy -> ReduceMean, ArgMax -> InTopK -> TypeCast -> ReduceMean,
//             kernel_mean_field.cpp:49-56) and prints them on stdout as "loss <v> acc <v>".
//
// --fused 0 : the reference's wiring, one factor per tensor operation
//             (MatMul, ReLU, MatMul(sparse), MatMul, ElewiseAdd, ReLU, ...)
// --fused 1 : S2VLevel / GraphPool / S2VReadout, one kernel per level
//
// batch.bin : int32 header {G, N, E, F, d, L, hidden, C}, then nodes_per_graph[G],
//             edge_src[E], edge_dst[E], tags[N] (int32) and the four weight matrices (fp32).
// out.bin   : logits[G*C], probs[G*C] (fp32), pred[G] (int32), embedding[N*d] (fp32),
//             then the n2n CSR: row_ptr[N+1], col_idx[E] (int32).
#include <chrono>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "nn/nn_all.h"
#include "tensor/tensor_all.h"
#include "util/graph_struct.h"

using namespace gnn;

typedef GPU mode;
typedef float Dtype;

namespace cfg
{
int node_dim, conv_size, max_lv, n_hidden, num_class;
}

struct Batch {
    int G, N, E;
    std::vector<int> nodes_per_graph, edge_src, edge_dst, tags;
    std::vector<float> w_n2l, p_node_conv, h1_weight, h2_weight;
};

template <typename T>
static void read_vec(FILE* f, std::vector<T>& v, size_t n)
{
    v.resize(n);
    ASSERT(n == 0 || fread(v.data(), sizeof(T), n, f) == n, "batch file is truncated");
}

static Batch load_batch(const char* path)
{
    FILE* f = fopen(path, "rb");
    ASSERT(f, "cannot open " << path);
    int h[8];
    ASSERT(fread(h, sizeof(int), 8, f) == 8, "batch file has no header");
    Batch b;
    b.G = h[0]; b.N = h[1]; b.E = h[2];
    cfg::node_dim = h[3]; cfg::conv_size = h[4]; cfg::max_lv = h[5]; cfg::n_hidden = h[6]; cfg::num_class = h[7];
    read_vec(f, b.nodes_per_graph, b.G);
    read_vec(f, b.edge_src, b.E);
    read_vec(f, b.edge_dst, b.E);
    read_vec(f, b.tags, b.N);
    read_vec(f, b.w_n2l, (size_t)cfg::node_dim * cfg::conv_size);
    read_vec(f, b.p_node_conv, (size_t)cfg::conv_size * cfg::conv_size);
    read_vec(f, b.h1_weight, (size_t)cfg::conv_size * cfg::n_hidden);
    read_vec(f, b.h2_weight, (size_t)cfg::n_hidden * cfg::num_class);
    fclose(f);
    return b;
}

static void set_param(std::shared_ptr<DTensorVar<mode, Dtype>>& p, std::vector<float>& host)
{
    DTensor<CPU, Dtype> view(p->value.shape, host.data());
    p->value.CopyFrom(view);
}

int main(int argc, const char** argv)
{
    if (argc < 3) {
        fprintf(stderr, "usage: %s <batch.bin> <out.bin> [--fused 0|1] [--iters K]\n", argv[0]);
        return 2;
    }
    int fused = 1, iters = 1;
    const char* labels_path = nullptr;
    for (int i = 3; i + 1 < argc; i += 2) {
        if (!strcmp(argv[i], "--fused")) fused = atoi(argv[i + 1]);
        if (!strcmp(argv[i], "--iters")) iters = atoi(argv[i + 1]);
        if (!strcmp(argv[i], "--labels")) labels_path = argv[i + 1];
    }
    Batch b = load_batch(argv[1]);
    GpuHandle::Init(0, 1);

    // ---- the batch: block-diagonal GraphStruct + one-hot node features
    GraphStruct graph;
    DTensor<CPU, Dtype> x_cpu;
    DTensor<mode, Dtype> input;
    graph.Resize(b.G, b.N);
    x_cpu.Reshape({(size_t)b.N, (size_t)cfg::node_dim});
    x_cpu.Zeros();
    {
        int node = 0;
        for (int g = 0; g < b.G; ++g)
            for (int j = 0; j < b.nodes_per_graph[g]; ++j, ++node) {
                x_cpu.data->ptr[(size_t)node * cfg::node_dim + b.tags[node]] = 1.0;
                graph.AddNode(g, node);
            }
        for (int e = 0; e < b.E; ++e) graph.AddEdge(e, b.edge_src[e], b.edge_dst[e]);
    }
    input.CopyFrom(x_cpu);

    // ---- the model
    FactorGraph fg;
    ParamSet<mode, Dtype> model;
    auto gvar = add_const<GraphVar>(fg, "graph", true);
    auto n2nsum_param = af<Node2NodeMsgPass<mode, Dtype>>(fg, {gvar});
    auto subgsum_param = af<SubgraphMsgPass<mode, Dtype>>(fg, {gvar});
    auto w_n2l = add_diff<DTensorVar>(model, "input-node-to-latent", {(uint)cfg::node_dim, (uint)cfg::conv_size});
    auto p_node_conv = add_diff<DTensorVar>(model, "linear-node-conv", {(uint)cfg::conv_size, (uint)cfg::conv_size});
    auto h1_weight = add_diff<DTensorVar>(model, "h1_weight", {(uint)cfg::conv_size, (uint)cfg::n_hidden});
    auto h2_weight = add_diff<DTensorVar>(model, "h2_weight", {(uint)cfg::n_hidden, (uint)cfg::num_class});
    set_param(w_n2l, b.w_n2l);
    set_param(p_node_conv, b.p_node_conv);
    set_param(h1_weight, b.h1_weight);
    set_param(h2_weight, b.h2_weight);
    fg.AddParam(w_n2l);
    fg.AddParam(p_node_conv);
    fg.AddParam(h1_weight);
    fg.AddParam(h2_weight);

    auto node_input = add_const<DTensorVar<mode, Dtype>>(fg, "data", true);
    auto input_message = af<MatMul>(fg, {node_input, w_n2l});
    auto cur_message_layer = af<ReLU>(fg, {input_message});
    for (int lv = 0; lv < cfg::max_lv; ++lv) {
        if (fused) {
            cur_message_layer = af<S2VLevel>(fg, {n2nsum_param, cur_message_layer, p_node_conv, input_message});
        } else {
            auto n2npool = af<MatMul>(fg, {n2nsum_param, cur_message_layer});
            auto node_linear = af<MatMul>(fg, {n2npool, p_node_conv});
            auto merged_linear = af<ElewiseAdd>(fg, {node_linear, input_message});
            cur_message_layer = af<ReLU>(fg, {merged_linear});
        }
    }
    std::shared_ptr<DTensorVar<mode, Dtype>> output, prob;
    std::shared_ptr<DTensorVar<mode, int>> pred;
    std::shared_ptr<S2VReadout<mode, Dtype>> readout;
    if (fused) {
        auto y_potential = af<GraphPool>(fg, {subgsum_param, cur_message_layer});
        output = af<S2VReadout>(fg, {y_potential, h1_weight, h2_weight});
    } else {
        auto y_potential = af<MatMul>(fg, {subgsum_param, cur_message_layer});
        auto hidden = af<MatMul>(fg, {y_potential, h1_weight});
        auto reluact_out_nn = af<ReLU>(fg, {hidden});
        output = af<MatMul>(fg, {reluact_out_nn, h2_weight});
    }
    prob = af<Softmax>(fg, {output});
    pred = af<ArgMax>(fg, {output});

    std::map<std::string, void*> inputs;
    inputs["data"] = &input;
    inputs["graph"] = &graph;
    std::vector<std::shared_ptr<Variable>> targets;
    targets.push_back(output);
    targets.push_back(prob);
    targets.push_back(pred);
    targets.push_back(cur_message_layer);

    // ---- optional loss / accuracy targets, labels as the CSR tensor GetBatch builds (nn_common.h:92-99)
    SpTensor<CPU, Dtype> y_cpu;
    SpTensor<mode, Dtype> label;
    std::shared_ptr<DTensorVar<mode, Dtype>> loss, acc;
    if (labels_path) {
        std::vector<int> lab;
        FILE* lf = fopen(labels_path, "rb");
        ASSERT(lf, "cannot open " << labels_path);
        read_vec(lf, lab, b.G);
        fclose(lf);
        y_cpu.Reshape({(size_t)b.G, (size_t)cfg::num_class});
        y_cpu.ResizeSp(b.G, b.G + 1);
        for (int i = 0; i < b.G; ++i) {
            y_cpu.data->row_ptr[i] = i;
            y_cpu.data->val[i] = 1.0;
            y_cpu.data->col_idx[i] = lab[i];
        }
        y_cpu.data->row_ptr[b.G] = b.G;
        label.CopyFrom(y_cpu);
        auto label_var = add_const<SpTensorVar<mode, Dtype>>(fg, "label", true);
        auto ce = af<CrossEntropy>(fg, {output, label_var}, true);
        loss = af<ReduceMean>(fg, {ce});
        auto truth = af<ArgMax>(fg, {label_var});
        auto cmp = af<InTopK<mode, Dtype>>(fg, std::make_pair(output, truth));
        auto real_cmp = af<TypeCast<mode, Dtype>>(fg, {cmp});
        acc = af<ReduceMean>(fg, {real_cmp});
        inputs["label"] = &label;
        targets.push_back(loss);
        targets.push_back(acc);
    }

    double best = 1e30;
    for (int it = 0; it < iters; ++it) {
        auto t0 = std::chrono::steady_clock::now();
        fg.FeedForward(targets, inputs, Phase::TEST);
        GpuHandle::Synchronize();
        double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (s < best) best = s;
    }
    fprintf(stderr, "s2v_mean_field: %d graphs, %d nodes, %d edges, fused=%d, %zu factors, %llu kernel launches, best FeedForward %.3f ms\n",
            b.G, b.N, b.E, fused, fg.NumFactors(), (unsigned long long)s2v_launch_count(GpuHandle::ctx()), best * 1e3);

    if (labels_path) printf("loss %.9g acc %.9g\n", (double)loss->AsScalar(), (double)acc->AsScalar());

    // ---- results back to the host
    DTensor<CPU, Dtype> logits_cpu, probs_cpu, embed_cpu;
    DTensor<CPU, int> pred_cpu;
    SpTensor<CPU, Dtype> n2n_cpu;
    logits_cpu.CopyFrom(output->value);
    probs_cpu.CopyFrom(prob->value);
    pred_cpu.CopyFrom(pred->value);
    embed_cpu.CopyFrom(cur_message_layer->value);
    n2n_cpu.CopyFrom(n2nsum_param->value);
    FILE* f = fopen(argv[2], "wb");
    ASSERT(f, "cannot open " << argv[2]);
    fwrite(logits_cpu.data->ptr, sizeof(float), logits_cpu.shape.Count(), f);
    fwrite(probs_cpu.data->ptr, sizeof(float), probs_cpu.shape.Count(), f);
    fwrite(pred_cpu.data->ptr, sizeof(int), pred_cpu.shape.Count(), f);
    fwrite(embed_cpu.data->ptr, sizeof(float), embed_cpu.shape.Count(), f);
    fwrite(n2n_cpu.data->row_ptr, sizeof(int), n2n_cpu.data->len_ptr, f);
    fwrite(n2n_cpu.data->col_idx, sizeof(int), n2n_cpu.data->nnz, f);
    fclose(f);
    GpuHandle::Destroy();
    return 0;
}
