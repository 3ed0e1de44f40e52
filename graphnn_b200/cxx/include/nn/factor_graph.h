// Computation graph with the reference's interface (include/nn/factor_graph.h:95-175,
// 310-351): AddConst / AddParam / AddFactor, FeedForward(targets, feed_dict, phase), and
// the af<> / add_const<> helpers.  Behaviour of FeedForward follows
// src/nn/factor_graph.cpp:44-180: variables the targets depend on are marked, placeholders
// are bound by pointer, factors run in dependency order and only if one of their outputs is
// needed; a target that cannot be produced is an error.  The bookkeeping here is by integer
// index built once at registration (the reference walks std::map<std::string, ...> per call).
// Back-propagation is not part of this library.
#ifndef S2V_FACTOR_GRAPH_H
#define S2V_FACTOR_GRAPH_H

#include <map>
#include <memory>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

#include "nn/factor.h"
#include "nn/variable.h"

namespace gnn
{

class FactorGraph
{
public:
    typedef std::shared_ptr<Variable> VarPtr;
    typedef std::vector<VarPtr> VarList;
    typedef std::shared_ptr<Factor> FactorPtr;

    FactorGraph() {}

    void AddConst(VarPtr var, bool isPlaceholder)
    {
        const size_t i = Register(var);
        nodes_[i].is_const = true;
        nodes_[i].always_ready = !isPlaceholder;
    }
    void AddParam(VarPtr var)
    {
        const size_t i = Register(var);
        nodes_[i].always_ready = true;
    }

    template <typename FactorPtrT, typename VarPtrList, typename VarOutList>
    void AddFactor(FactorPtrT factor, VarPtrList vars_in, VarOutList vars_out)
    {
        ASSERT(factor_index_.count(factor->name) == 0, "factor " << factor->name << " is already inserted");
        FactorNode fn;
        fn.factor = factor;
        const size_t f = factors_.size();
        for (size_t i = 0; i < vars_in.size(); ++i) {
            auto it = var_index_.find(vars_in[i]->name);
            ASSERT(it != var_index_.end(), "the operand " << vars_in[i]->name << " must be registered beforehand");
            fn.in.push_back(it->second);
            fn.operands.push_back(vars_in[i]);
            nodes_[it->second].consumers.push_back(f);
        }
        for (size_t i = 0; i < vars_out.size(); ++i) {
            const size_t v = Register(vars_out[i]);
            if (factor->properr == PropErr::N) nodes_[v].is_const = true;
            fn.out.push_back(v);
            fn.outputs.push_back(vars_out[i]);
            nodes_[v].producers.push_back(f);
        }
        factor_index_[factor->name] = f;
        factors_.push_back(fn);
    }

    VarList FeedForward(std::vector<VarPtr> targets, std::map<std::string, void*> feed_dict, Phase phase,
                        uint n_thread = 1)
    {
        if (n_thread != 1) throw std::runtime_error("not implemented");
        const size_t nv = nodes_.size(), nf = factors_.size();
        // 1. what do the targets need?  reverse breadth-first walk over producers
        required_.assign(nv, 0);
        std::queue<size_t> q;
        for (auto& t : targets) {
            const size_t v = VarIdx(t);
            if (!required_[v]) { required_[v] = 1; q.push(v); }
        }
        while (!q.empty()) {
            const size_t v = q.front();
            q.pop();
            for (size_t f : nodes_[v].producers)
                for (size_t u : factors_[f].in)
                    if (!required_[u]) { required_[u] = 1; q.push(u); }
        }
        // 2. what is available?  constants, parameters, and the placeholders fed now
        ready_.assign(nv, 0);
        for (size_t v = 0; v < nv; ++v) ready_[v] = nodes_[v].always_ready;
        for (auto& kv : feed_dict) {
            const size_t v = VarIdx(kv.first);
            nodes_[v].var->SetRef(kv.second);
            ready_[v] = 1;
        }
        // 3. run factors whose operands are all available, in dependency order
        pending_.resize(nf);
        std::queue<size_t> runnable;
        for (size_t f = 0; f < nf; ++f) pending_[f] = factors_[f].in.size();
        for (size_t v = 0; v < nv; ++v)
            if (ready_[v])
                for (size_t f : nodes_[v].consumers)
                    if (--pending_[f] == 0) runnable.push(f);
        while (!runnable.empty()) {
            const size_t f = runnable.front();
            runnable.pop();
            FactorNode& fn = factors_[f];
            bool needed = false;
            for (size_t v : fn.out) needed = needed || required_[v];
            if (!needed) continue;   // its outputs stay unavailable, so nothing downstream runs either
            fn.factor->Forward(fn.operands, fn.outputs, phase);
            for (size_t v : fn.out) {
                ready_[v] = 1;
                for (size_t g : nodes_[v].consumers)
                    if (--pending_[g] == 0) runnable.push(g);
            }
        }
        for (auto& t : targets) ASSERT(ready_[VarIdx(t)], "required variable " << t->name << " is not ready");
        return VarList(targets.begin(), targets.end());
    }

    void BackPropagate(std::vector<VarPtr>, uint = 1) { throw std::logic_error("BackPropagate: training is outside this library"); }

    size_t VarIdx(const std::string& var_name)
    {
        auto it = var_index_.find(var_name);
        ASSERT(it != var_index_.end(), "variable " << var_name << " is not registered");
        return it->second;
    }
    size_t VarIdx(VarPtr var) { return VarIdx(var->name); }
    size_t NumFactors() const { return factors_.size(); }
    size_t NumVars() const { return nodes_.size(); }

private:
    struct VarNode {
        VarPtr var;
        std::vector<size_t> producers, consumers;
        char always_ready = 0;
        bool is_const = false;
    };
    struct FactorNode {
        FactorPtr factor;
        std::vector<size_t> in, out;
        VarList operands, outputs;
    };
    size_t Register(VarPtr var)
    {
        ASSERT(var_index_.count(var->name) == 0, "variable " << var->name << " is already inserted");
        VarNode n;
        n.var = var;
        var_index_[var->name] = nodes_.size();
        nodes_.push_back(n);
        return nodes_.size() - 1;
    }
    std::vector<VarNode> nodes_;
    std::vector<FactorNode> factors_;
    std::unordered_map<std::string, size_t> var_index_, factor_index_;
    std::vector<char> required_, ready_;
    std::vector<size_t> pending_;
};

// ---- helpers with the reference's spelling -------------------------------------------------
template <typename VarType, typename... Args>
std::shared_ptr<VarType> add_const(FactorGraph& g, std::string var_name, bool isPlaceholder, Args&&... args)
{
    auto v = std::make_shared<VarType>(var_name, std::forward<Args>(args)...);
    g.AddConst(v, isPlaceholder);
    return v;
}

// af<FactorType>(graph, operands, ctor args...): create the factor "<StrType>_<k>", its output
// variable, register both, return the output variable.
template <typename FacType, typename VarPtrT, typename... Args>
typename FacType::OutType af(FactorGraph& g, std::vector<VarPtrT> operands, Args&&... args)
{
    auto f = std::make_shared<FacType>(FacType::StrType() + "_" + std::to_string(g.NumFactors()), std::forward<Args>(args)...);
    auto out = f->CreateOutVar();
    std::vector<std::shared_ptr<Variable>> outs(1, out);
    g.AddFactor(f, operands, outs);
    return out;
}
template <typename FacType, typename VarPtrT, typename... Args>
typename FacType::OutType af(FactorGraph& g, std::initializer_list<VarPtrT> op, Args&&... args)
{
    return af<FacType>(g, std::vector<VarPtrT>(op), std::forward<Args>(args)...);
}
// af<InTopK<mode, Dtype>>(graph, std::make_pair(pred, labels)): operands of two different types
template <typename FacType, typename VarPtr1, typename VarPtr2, typename... Args>
typename FacType::OutType af(FactorGraph& g, std::pair<VarPtr1, VarPtr2> op, Args&&... args)
{
    std::vector<std::shared_ptr<Variable>> ops(2);
    ops[0] = op.first;
    ops[1] = op.second;
    return af<FacType>(g, ops, std::forward<Args>(args)...);
}
// af<MatMul>(graph, {a, b}): mode and element type deduced from the operands
template <template <typename, typename> class FacType, typename... Args>
typename FacType<GPU, float>::OutType af(FactorGraph& g, std::vector<std::shared_ptr<TensorVar<GPU, float>>> op, Args&&... args)
{
    return af<FacType<GPU, float>>(g, op, std::forward<Args>(args)...);
}

}  // namespace gnn
#endif
