// Serves a trained structure2vec classifier on a text data set: the TEST loop of the
// reference driver (examples/graph_classification/include/nn_common.h:36-105,127-146) for a
// checkpoint written by ParamSet::Save.
//
//   s2v_classify -graph data.txt -model weights.model -test_idx idx.txt -conv 64 -hidden 64 -lv 3 -b 50 -out pred.txt
//
// Flags follow the reference's (include/config.h:26-82).  Differences: the node feature width
// is (largest tag + 1) -- the reference uses the largest tag itself, which makes the highest
// tag spill into the next row (kernel_mean_field.cpp:75-84); pass -node_dim to reproduce a
// checkpoint trained that way.  Writes "index prediction label" per test graph to -out and prints
// "test loss <v> acc <v>" (averages weighted by batch size, as the reference accumulates them).
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "dataset.h"
#include "nn/nn_all.h"
#include "tensor/tensor_all.h"

using namespace gnn;
typedef GPU mode;
typedef float Dtype;

int main(int argc, const char** argv)
{
    std::map<std::string, std::string> arg;
    for (int i = 1; i + 1 < argc; i += 2) arg[argv[i]] = argv[i + 1];
    auto geti = [&](const char* k, int dflt) { return arg.count(k) ? atoi(arg[k].c_str()) : dflt; };
    ASSERT(arg.count("-graph") && arg.count("-model"), "usage: s2v_classify -graph data.txt -model weights.model [-test_idx idx.txt] "
                                                       "[-conv 64] [-hidden 64] [-lv 3] [-b 50] [-out pred.txt] [-node_dim F] [-device 0]");
    const int conv = geti("-conv", 64), hidden = geti("-hidden", 64), lv = geti("-lv", 3), bsize = geti("-b", 50);

    std::vector<Graph> graph_data;
    std::vector<int> labels, test_idx;
    int max_tag = 0;
    const int num_class = LoadRawData(arg["-graph"].c_str(), graph_data, labels, max_tag);
    const int node_dim = geti("-node_dim", max_tag + 1);
    if (arg.count("-test_idx"))
        LoadIndexes(arg["-test_idx"].c_str(), test_idx);
    else
        for (size_t i = 0; i < graph_data.size(); ++i) test_idx.push_back((int)i);

    GpuHandle::Init(geti("-device", 0), 1);
    FactorGraph fg;
    ParamSet<mode, Dtype> model;
    auto gvar = add_const<GraphVar>(fg, "graph", true);
    auto n2n = af<Node2NodeMsgPass<mode, Dtype>>(fg, {gvar});
    auto subg = af<SubgraphMsgPass<mode, Dtype>>(fg, {gvar});
    auto w_n2l = add_diff<DTensorVar>(model, "input-node-to-latent", {(uint)node_dim, (uint)conv});
    auto p_conv = add_diff<DTensorVar>(model, "linear-node-conv", {(uint)conv, (uint)conv});
    auto h1 = add_diff<DTensorVar>(model, "h1_weight", {(uint)conv, (uint)hidden});
    auto h2 = add_diff<DTensorVar>(model, "h2_weight", {(uint)hidden, (uint)num_class});
    model.Load(arg["-model"]);
    ASSERT(w_n2l->value.rows() == (size_t)node_dim && w_n2l->value.cols() == (size_t)conv && h2->value.cols() == (size_t)num_class,
           "checkpoint shapes do not match -conv/-hidden/-node_dim and the data set");
    fg.AddParam(w_n2l);
    fg.AddParam(p_conv);
    fg.AddParam(h1);
    fg.AddParam(h2);
    auto node_input = add_const<DTensorVar<mode, Dtype>>(fg, "data", true);
    auto label_var = add_const<SpTensorVar<mode, Dtype>>(fg, "label", true);
    auto msg = af<MatMul>(fg, {node_input, w_n2l});
    auto cur = af<ReLU>(fg, {msg});
    for (int l = 0; l < lv; ++l) cur = af<S2VLevel>(fg, {n2n, cur, p_conv, msg});
    auto y = af<GraphPool>(fg, {subg, cur});
    auto output = af<S2VReadout>(fg, {y, h1, h2});
    auto pred = af<ArgMax>(fg, {output});
    auto ce = af<CrossEntropy>(fg, {output, label_var}, true);
    auto loss = af<ReduceMean>(fg, {ce});
    auto truth = af<ArgMax>(fg, {label_var});
    auto cmp = af<InTopK<mode, Dtype>>(fg, std::make_pair(output, truth));
    auto real_cmp = af<TypeCast<mode, Dtype>>(fg, {cmp});
    auto acc = af<ReduceMean>(fg, {real_cmp});

    GraphStruct graph;
    DTensor<CPU, Dtype> x_cpu;
    SpTensor<CPU, Dtype> y_cpu;
    DTensor<mode, Dtype> input;
    SpTensor<mode, Dtype> label;
    DTensor<CPU, int> pred_cpu;
    std::map<std::string, void*> inputs;
    inputs["data"] = &input;
    inputs["label"] = &label;
    inputs["graph"] = &graph;
    std::vector<std::shared_ptr<Variable>> targets = {loss, acc, pred};

    FILE* out = arg.count("-out") ? fopen(arg["-out"].c_str(), "w") : nullptr;
    double loss_total = 0, acc_total = 0;
    for (size_t st = 0; st < test_idx.size(); st += bsize) {
        const size_t ed = std::min(test_idx.size(), st + (size_t)bsize), num = ed - st;
        // ---- GetBatch: block-diagonal graph, one-hot features, CSR labels
        std::vector<unsigned> prefix(num + 1, 0);
        for (size_t i = 0; i < num; ++i) prefix[i + 1] = prefix[i] + graph_data[test_idx[st + i]].num_nodes;
        const unsigned node_cnt = prefix[num];
        graph.Resize(num, node_cnt);
        x_cpu.Reshape({node_cnt, (size_t)node_dim});
        x_cpu.Zeros();
        y_cpu.Reshape({num, (size_t)num_class});
        y_cpu.ResizeSp(num, num + 1);
        int cur_edge = 0;
        for (size_t i = 0; i < num; ++i) {
            auto& g = graph_data[test_idx[st + i]];
            for (int j = 0; j < g.num_nodes; ++j) {
                ASSERT(g.node_label[j] < node_dim, "node tag beyond -node_dim");
                x_cpu.data->ptr[(size_t)(prefix[i] + j) * node_dim + g.node_label[j]] = 1.0;
                graph.AddNode(i, prefix[i] + j);
            }
        }
        for (size_t i = 0; i < num; ++i) {
            auto& g = graph_data[test_idx[st + i]];
            for (int j = 0; j < g.num_nodes; ++j)
                for (int nb : g.adj[j]) graph.AddEdge(cur_edge++, prefix[i] + j, prefix[i] + nb);
            y_cpu.data->row_ptr[i] = i;
            y_cpu.data->val[i] = 1.0;
            y_cpu.data->col_idx[i] = labels[test_idx[st + i]];
        }
        y_cpu.data->row_ptr[num] = num;
        input.CopyFrom(x_cpu);
        label.CopyFrom(y_cpu);

        fg.FeedForward(targets, inputs, Phase::TEST);
        loss_total += num * (double)loss->AsScalar();
        acc_total += num * (double)acc->AsScalar();
        pred_cpu.CopyFrom(pred->value);
        if (out)
            for (size_t i = 0; i < num; ++i) fprintf(out, "%d %d %d\n", test_idx[st + i], pred_cpu.data->ptr[i], labels[test_idx[st + i]]);
    }
    if (out) fclose(out);
    printf("test loss %.9g acc %.9g\n", loss_total / test_idx.size(), acc_total / test_idx.size());
    GpuHandle::Destroy();
    return 0;
}
