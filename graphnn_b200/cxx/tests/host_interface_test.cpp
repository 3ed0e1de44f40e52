// Host-only checks of the operator interface (no GPU needed): scheduling semantics of
// FactorGraph::FeedForward and the CSR matrices the message-passing factors build from a
// GraphStruct, in CPU mode.  Prints "ok <name>" per case; any failure aborts.
//
// The reference has no test for these (its gtest suite covers tensor arithmetic only); the
// expectations below restate src/nn/factor_graph.cpp:44-180 and src/nn/msg_pass.cpp:46-67,156-177.
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "nn/nn_all.h"

using namespace gnn;

static std::vector<std::string> g_trace;

// a factor that only records that it ran
class Probe : public Factor
{
public:
    static std::string StrType() { return "Probe"; }
    using OutType = std::shared_ptr<GraphVar>;
    OutType CreateOutVar() { return std::make_shared<GraphVar>(this->name + ":out_0"); }
    Probe(std::string _name, std::string _tag) : Factor(_name), tag(_tag) {}
    void Forward(std::vector<std::shared_ptr<Variable>>&, std::vector<std::shared_ptr<Variable>>&, Phase) override
    {
        g_trace.push_back(tag);
    }
    std::string tag;
};

#define CHECK(cond)                                                          \
    do {                                                                     \
        if (!(cond)) {                                                       \
            fprintf(stderr, "CHECK failed: %s (line %d)\n", #cond, __LINE__); \
            return 1;                                                        \
        }                                                                    \
    } while (0)

static int test_schedule()
{
    FactorGraph fg;
    GraphStruct dummy;
    auto in = add_const<GraphVar>(fg, "in", true);
    auto konst = add_const<GraphVar>(fg, "konst", false);
    auto a = af<Probe>(fg, {in}, "a");
    auto b = af<Probe>(fg, {a, konst}, "b");
    auto c = af<Probe>(fg, {a}, "c");          // not needed for target d
    auto d = af<Probe>(fg, {b, a}, "d");
    auto e = af<Probe>(fg, {c, d}, "e");
    CHECK(fg.NumFactors() == 5 && a->name == "Probe_0:out_0" && e->name == "Probe_4:out_0");
    std::map<std::string, void*> feed;
    feed["in"] = &dummy;
    g_trace.clear();
    fg.FeedForward({d}, feed, Phase::TEST);
    CHECK((g_trace == std::vector<std::string>{"a", "b", "d"}));   // c and e are pruned
    g_trace.clear();
    fg.FeedForward({e}, feed, Phase::TEST);
    CHECK(g_trace.size() == 5 && g_trace[0] == "a" && g_trace[4] == "e");
    g_trace.clear();
    fg.FeedForward({a, c}, feed, Phase::TEST);                     // second call: state is rebuilt per call
    CHECK((g_trace == std::vector<std::string>{"a", "c"}));
    CHECK(in->graph == &dummy);                                     // placeholder bound by pointer
    bool threw = false;
    try {
        fg.FeedForward({a}, feed, Phase::TEST, 2);
    } catch (const std::runtime_error&) {
        threw = true;
    }
    CHECK(threw);                                                   // n_thread != 1 is not implemented, as in the reference
    puts("ok schedule");
    return 0;
}

static int test_msg_pass_matrices()
{
    // two graphs: a path 0-1-2 and a single edge 3-4, symmetric, added source-ascending
    GraphStruct g;
    g.Resize(2, 5);
    for (int i = 0; i < 3; ++i) g.AddNode(0, i);
    for (int i = 3; i < 5; ++i) g.AddNode(1, i);
    const int edges[][2] = {{0, 1}, {1, 0}, {1, 2}, {2, 1}, {3, 4}, {4, 3}, {2, 0}};   // last one is directed only
    for (int e = 0; e < 7; ++e) g.AddEdge(e, edges[e][0], edges[e][1]);
    CHECK(g.num_edges == 7 && g.in_edges->head[0].size() == 2 && g.in_edges->head[0][1].second == 2);

    FactorGraph fg;
    auto gv = add_const<GraphVar>(fg, "graph", true);
    auto n2n = af<Node2NodeMsgPass<CPU, float>>(fg, {gv});
    auto n2n_avg = af<Node2NodeMsgPass<CPU, float>>(fg, {gv}, true);
    auto sub = af<SubgraphMsgPass<CPU, float>>(fg, {gv});
    std::map<std::string, void*> feed;
    feed["graph"] = &g;
    fg.FeedForward({n2n, n2n_avg, sub}, feed, Phase::TEST);
    auto& A = n2n->value;
    const int want_rp[] = {0, 2, 4, 5, 6, 7};
    const int want_ci[] = {1, 2, 0, 2, 1, 4, 3};    // row 0 lists sources 1 then 2: insertion order
    CHECK(A.rows() == 5 && A.cols() == 5 && A.data->nnz == 7 && A.data->len_ptr == 6);
    CHECK(!memcmp(A.data->row_ptr, want_rp, sizeof(want_rp)) && !memcmp(A.data->col_idx, want_ci, sizeof(want_ci)));
    for (int t = 0; t < 7; ++t) CHECK(A.data->val[t] == 1.0f);
    CHECK(n2n_avg->value.data->val[0] == 0.5f && n2n_avg->value.data->val[4] == 1.0f);
    auto& S = sub->value;
    const int want_srp[] = {0, 3, 5}, want_sci[] = {0, 1, 2, 3, 4};
    CHECK(S.rows() == 2 && S.cols() == 5 && S.data->nnz == 5);
    CHECK(!memcmp(S.data->row_ptr, want_srp, sizeof(want_srp)) && !memcmp(S.data->col_idx, want_sci, sizeof(want_sci)));
    // the edge-level matrices of the same graph (worked out by hand from the in-edge lists above)
    auto e2n = af<Edge2NodeMsgPass<CPU, float>>(fg, {gv});
    auto e2n_avg = af<Edge2NodeMsgPass<CPU, float>>(fg, {gv}, true);
    auto n2e = af<Node2EdgeMsgPass<CPU, float>>(fg, {gv});
    auto e2e = af<Edge2EdgeMsgPass<CPU, float>>(fg, {gv});
    fg.FeedForward({e2n, e2n_avg, n2e, e2e}, feed, Phase::TEST);
    const int want_e2n_ci[] = {1, 6, 0, 3, 2, 5, 4};
    CHECK(e2n->value.rows() == 5 && e2n->value.cols() == 7 && e2n->value.data->nnz == 7);
    CHECK(!memcmp(e2n->value.data->row_ptr, want_rp, sizeof(want_rp)) && !memcmp(e2n->value.data->col_idx, want_e2n_ci, sizeof(want_e2n_ci)));
    CHECK(e2n_avg->value.data->val[1] == 0.5f && e2n_avg->value.data->val[6] == 1.0f);
    const int want_n2e_ci[] = {0, 1, 1, 2, 3, 4, 2};
    CHECK(n2e->value.rows() == 7 && n2e->value.cols() == 5 && !memcmp(n2e->value.data->col_idx, want_n2e_ci, sizeof(want_n2e_ci)));
    CHECK(n2e->value.data->row_ptr[7] == 7 && n2e->value.data->row_ptr[3] == 3);
    const int want_e2e_rp[] = {0, 1, 2, 3, 3, 3, 3, 4}, want_e2e_ci[] = {6, 3, 0, 2};
    CHECK(e2e->value.rows() == 7 && e2e->value.cols() == 7 && e2e->value.data->nnz == 4);
    CHECK(!memcmp(e2e->value.data->row_ptr, want_e2e_rp, sizeof(want_e2e_rp)) && !memcmp(e2e->value.data->col_idx, want_e2e_ci, sizeof(want_e2e_ci)));
    // a smaller batch through the same factors: the tensors shrink logically, capacity is kept
    g.Resize(1, 2);
    g.AddNode(0, 0);
    g.AddNode(0, 1);
    g.AddEdge(0, 0, 1);
    fg.FeedForward({n2n, sub}, feed, Phase::TEST);
    CHECK(A.data->nnz == 1 && A.data->len_ptr == 3 && A.data->row_ptr[2] == 1 && A.data->col_idx[0] == 0 && A.data->nzCap >= 7);
    puts("ok msg_pass");
    return 0;
}

static int test_cpu_tensors()
{
    DTensor<CPU, float> t({3, 4});
    CHECK(t.rows() == 3 && t.cols() == 4 && t.shape.Count() == 12 && t.data->mem_size == 12);
    t.Fill(2.5f);
    auto v = t.GetRowRef(1, 2);
    CHECK(v.rows() == 2 && v.data->is_referring && v.data->ptr == t.data->ptr + 4 && v.data->ptr[7] == 2.5f);
    t.Reshape({2, 2});                 // grow-only storage
    CHECK(t.data->mem_size == 12);
    DTensor<CPU, float> u;
    u.CopyFrom(t);
    CHECK(u.shape == t.shape && u.data->ptr != t.data->ptr && u.data->ptr[3] == 2.5f);
    DTensor<CPU, float> w;
    w.ShallowCopy(t);
    CHECK(w.data->ptr == t.data->ptr);
    DTensor<CPU, float> one({1});
    one.data->ptr[0] = 7.f;
    CHECK(one.AsScalar() == 7.f);
    CHECK(fmt::sprintf("%s_%d", std::string("MatMul"), 3) == "MatMul_3");
    puts("ok cpu_tensors");
    return 0;
}

// argv[1]: a checkpoint written by the reference's ParamSet::Save (F=3, d=4, hidden=5, C=2);
// argv[2]: where to write it back with this library's Save.  The caller compares the bytes.
static int test_checkpoint(const char* in_path, const char* out_path)
{
    ParamSet<CPU, float> model;
    auto a = add_diff<DTensorVar>(model, "input-node-to-latent", {3u, 4u});
    auto b = add_diff<DTensorVar>(model, "linear-node-conv", {4u, 4u});
    auto c = add_diff<DTensorVar>(model, "h1_weight", {4u, 5u});
    auto e = add_diff<DTensorVar>(model, "h2_weight", {5u, 2u});
    model.Load(in_path);
    CHECK(a->value.rows() == 3 && a->value.cols() == 4 && c->value.cols() == 5 && e->value.shape.Count() == 10);
    printf("first %.9g %.9g %.9g %.9g\n", a->value.data->ptr[0], b->value.data->ptr[0], c->value.data->ptr[0], e->value.data->ptr[9]);
    model.Save(out_path);
    puts("ok checkpoint");
    return 0;
}

int main(int argc, const char** argv)
{
    if (argc == 3) return test_checkpoint(argv[1], argv[2]);
    return test_schedule() || test_msg_pass_matrices() || test_cpu_tensors();
}
