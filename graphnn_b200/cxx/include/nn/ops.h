// The operators of the structure2vec inference path with the reference's names and
// constructor arguments: MatMul, ElewiseAdd, ReLU, Softmax, ArgMax (one library kernel per
// tensor method, exactly the calls the reference's Forward bodies make), the two
// message-passing matrix builders, and the fused forms this library adds (S2VLevel,
// GraphPool, S2VReadout).
#ifndef S2V_OPS_H
#define S2V_OPS_H

#include <memory>
#include <string>
#include <vector>

#include "nn/factor.h"
#include "nn/variable.h"

namespace gnn
{

namespace detail
{
template <typename mode, typename Dtype>
inline DTensor<mode, Dtype>& dense(std::shared_ptr<Variable>& v)
{
    auto* p = dynamic_cast<DTensorVar<mode, Dtype>*>(v.get());
    ASSERT(p, "operand " << v->name << " is not a dense tensor of the expected mode/type");
    return p->value;
}
template <typename mode, typename Dtype>
inline SpTensor<mode, Dtype>& sparse(std::shared_ptr<Variable>& v)
{
    auto* p = dynamic_cast<SpTensorVar<mode, Dtype>*>(v.get());
    ASSERT(p, "operand " << v->name << " is not a CSR tensor of the expected mode/type");
    return p->value;
}
}  // namespace detail

#define S2V_DENSE_OUT(StrName)                                                                         \
    static std::string StrType() { return StrName; }                                                   \
    using OutType = std::shared_ptr<DTensorVar<mode, Dtype>>;                                          \
    OutType CreateOutVar() { return std::make_shared<DTensorVar<mode, Dtype>>(this->name + ":out_0"); }

// out = op(lhs) * op(rhs), lhs dense or CSR (src/nn/matmul.cpp:13-33)
template <typename mode, typename Dtype>
class MatMul : public Factor
{
public:
    S2V_DENSE_OUT("MatMul")
    MatMul(std::string _name, Trans _transA = Trans::N, Trans _transB = Trans::N, PropErr _properr = PropErr::T)
        : Factor(_name, _properr), transA(_transA), transB(_transB) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 2, StrType() << ": wrong number of operands");
        ASSERT(outputs.size() == 1, StrType() << ": wrong number of outputs");
        auto& output = detail::dense<mode, Dtype>(outputs[0]);
        auto* lhs = dynamic_cast<TensorVar<mode, Dtype>*>(operands[0].get());
        auto* rhs = dynamic_cast<TensorVar<mode, Dtype>*>(operands[1].get());
        ASSERT(lhs && rhs, "operands of the wrong mode/type for " << StrType());
        ASSERT(rhs->GetMatType() == MatType::dense, StrType() << ": the right-hand operand must be a dense matrix");
        auto& right = rhs->template Derived<DENSE>().value;
        if (lhs->GetMatType() == MatType::dense)
            output.MM(lhs->template Derived<DENSE>().value, right, transA, transB, 1.0, 0.0);
        else
            output.MM(lhs->template Derived<CSR_SPARSE>().value, right, transA, transB, 1.0, 0.0);
    }
    Trans transA, transB;
};

// out = sum_i coeff_i * op_i (src/nn/elewise_add.cpp:12-33): copy, optional scale, axpy per operand
template <typename mode, typename Dtype>
class ElewiseAdd : public Factor
{
public:
    S2V_DENSE_OUT("ElewiseAdd")
    ElewiseAdd(std::string _name, std::vector<Dtype> _coeff = std::vector<Dtype>(), PropErr _properr = PropErr::T)
        : Factor(_name, _properr), coeff(_coeff) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() >= 2, StrType() << ": wrong number of operands");
        ASSERT(outputs.size() == 1, StrType() << ": wrong number of outputs");
        ASSERT(coeff.size() == 0 || operands.size() == coeff.size(), "wrong number of coefficients");
        auto& output = detail::dense<mode, Dtype>(outputs[0]);
        output.CopyFrom(detail::dense<mode, Dtype>(operands[0]));
        if (coeff.size()) output.Scale(coeff[0]);
        for (size_t i = 1; i < operands.size(); ++i) {
            auto& op_i = detail::dense<mode, Dtype>(operands[i]);
            ASSERT(op_i.shape == output.shape, StrType() << ": every operand must have the shape of the output");
            output.Axpy(coeff.size() ? coeff[i] : 1.0, op_i);
        }
    }
    std::vector<Dtype> coeff;
};

// out = in < 0 ? 0 : in (src/nn/relu.cpp:31-43; one kernel instead of copy + in-place clamp)
template <typename mode, typename Dtype>
class ReLU : public Factor
{
public:
    S2V_DENSE_OUT("ReLU")
    ReLU(std::string _name, PropErr _properr = PropErr::T) : Factor(_name, _properr) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 1, StrType() << ": wrong number of operands");
        ASSERT(outputs.size() == 1, StrType() << ": wrong number of outputs");
        auto& in = detail::dense<mode, Dtype>(operands[0]);
        auto& out = detail::dense<mode, Dtype>(outputs[0]);
        out.Reshape(in.shape.dims);
        S2V_ASSERT_OK(s2v_relu_f32(GpuHandle::ctx(), nullptr, (int64_t)in.shape.Count(), in.data->ptr, out.data->ptr));
    }
};

// row softmax (src/nn/softmax.cpp:37-50)
template <typename mode, typename Dtype>
class Softmax : public Factor
{
public:
    S2V_DENSE_OUT("Softmax")
    Softmax(std::string _name, PropErr _properr = PropErr::T) : Factor(_name, _properr) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 1, StrType() << ": wrong number of operands");
        ASSERT(outputs.size() == 1, StrType() << ": wrong number of outputs");
        auto& out = detail::dense<mode, Dtype>(outputs[0]);
        out.CopyFrom(detail::dense<mode, Dtype>(operands[0]));
        out.Softmax();
    }
};

// per-row index of the maximum (src/nn/arg_max.cpp:14-29)
template <typename mode, typename Dtype>
class ArgMax : public Factor
{
public:
    static std::string StrType() { return "ArgMax"; }
    using OutType = std::shared_ptr<DTensorVar<mode, int>>;
    OutType CreateOutVar() { return std::make_shared<DTensorVar<mode, int>>(this->name + ":out_0"); }
    ArgMax(std::string _name, uint _axis = 0) : Factor(_name, PropErr::N), axis(_axis)
    {
        ASSERT(axis == 0, StrType() << ": only axis 0 (per-row) is built");
    }
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 1, StrType() << ": wrong number of operands");
        ASSERT(outputs.size() == 1, StrType() << ": wrong number of outputs");
        auto* out = dynamic_cast<DTensorVar<mode, int>*>(outputs[0].get());
        ASSERT(out, "wrong output type for " << StrType());
        auto* in = dynamic_cast<TensorVar<mode, Dtype>*>(operands[0].get());
        ASSERT(in, "wrong operand type for " << StrType());
        if (in->GetMatType() == MatType::dense) {
            in->template Derived<DENSE>().value.ArgMax(out->value);
        } else {   // label matrices are CSR: column of the largest value per row
            auto& sp = in->template Derived<CSR_SPARSE>().value;
            out->value.Reshape({sp.rows()});
            S2V_ASSERT_OK(s2v_argmax_csr_f32(GpuHandle::ctx(), nullptr, (int64_t)sp.rows(), sp.data->row_ptr, sp.data->col_idx,
                                             sp.data->val, out->value.data->ptr));
        }
    }
    uint axis;
};

// ---- loss / metric tail of the driver (kernel_mean_field.cpp:49-56) ---------------------------
// per-row cross entropy of dense predictions against CSR labels (src/nn/cross_entropy.cpp:33-50)
template <typename mode, typename Dtype>
class CrossEntropy : public Factor
{
public:
    S2V_DENSE_OUT("CrossEntropy")
    CrossEntropy(std::string _name, bool _need_softmax, PropErr _properr = PropErr::T)
        : Factor(_name, _properr), need_softmax(_need_softmax) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 2, StrType() << ": wrong number of operands");
        auto& pred = detail::dense<mode, Dtype>(operands[0]);
        auto& label = detail::sparse<mode, Dtype>(operands[1]);
        ASSERT(pred.cols() == label.cols() && pred.rows() == label.rows(), StrType() << ": prediction and label matrices differ in shape");
        auto& out = detail::dense<mode, Dtype>(outputs[0]);
        out.Reshape({pred.rows(), 1});
        S2V_ASSERT_OK(s2v_cross_entropy_f32(GpuHandle::ctx(), nullptr, (int64_t)pred.rows(), (int)pred.cols(), pred.data->ptr,
                                            need_softmax ? 1 : 0, label.data->row_ptr, label.data->col_idx, label.data->val,
                                            out.data->ptr));
    }
    bool need_softmax;
};

// global mean -> tensor of one element (src/nn/reduce_mean.cpp:14-42)
template <typename mode, typename Dtype>
class ReduceMean : public Factor
{
public:
    S2V_DENSE_OUT("ReduceMean")
    ReduceMean(std::string _name, int _axis = -1, bool _keep_dim = false, PropErr _properr = PropErr::T)
        : Factor(_name, _properr), axis(_axis), keep_dim(_keep_dim) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 1, StrType() << ": wrong number of operands");
        ASSERT(axis == -1 && keep_dim == false, StrType() << ": only the mean over all elements (axis = -1, keep_dim = false) is built");
        auto& in = detail::dense<mode, Dtype>(operands[0]);
        auto& out = detail::dense<mode, Dtype>(outputs[0]);
        out.Reshape({1});
        S2V_ASSERT_OK(s2v_mean_f32(GpuHandle::ctx(), nullptr, (int64_t)in.shape.Count(), in.data->ptr, out.data->ptr));
    }
    int axis;
    bool keep_dim;
};

// operands {predictions (dense), labels (int)}: 1 where the label is among the top k (src/nn/in_top_k.cpp:6-49)
template <typename mode, typename Dtype>
class InTopK : public Factor
{
public:
    static std::string StrType() { return "InTopK"; }
    using OutType = std::shared_ptr<DTensorVar<mode, int>>;
    OutType CreateOutVar() { return std::make_shared<DTensorVar<mode, int>>(this->name + ":out_0"); }
    InTopK(std::string _name, int _topK = 1) : Factor(_name, PropErr::N), topK(_topK) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 2, StrType() << ": wrong number of operands");
        auto& pred = detail::dense<mode, Dtype>(operands[0]);
        auto* lab = dynamic_cast<DTensorVar<mode, int>*>(operands[1].get());
        auto* out = dynamic_cast<DTensorVar<mode, int>*>(outputs[0].get());
        ASSERT(lab && out, "wrong operand types for " << StrType());
        ASSERT(pred.rows() == lab->value.shape.Count(), StrType() << ": one label per prediction row is required");
        out->value.Reshape(lab->value.shape.dims);
        S2V_ASSERT_OK(s2v_in_top_k_f32(GpuHandle::ctx(), nullptr, (int64_t)pred.rows(), (int)pred.cols(), pred.data->ptr,
                                       lab->value.data->ptr, topK, out->value.data->ptr));
    }
    int topK;
};

// int tensor -> Dtype tensor (src/nn/type_cast.cpp:14-30)
template <typename mode, typename Dtype>
class TypeCast : public Factor
{
public:
    S2V_DENSE_OUT("TypeCast")
    TypeCast(std::string _name, PropErr _properr = PropErr::T) : Factor(_name, _properr) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 1, StrType() << ": wrong number of operands");
        auto* in = dynamic_cast<DTensorVar<mode, int>*>(operands[0].get());
        ASSERT(in, StrType() << " is implemented for int -> float");
        auto& out = detail::dense<mode, Dtype>(outputs[0]);
        out.Reshape(in->value.shape.dims);
        S2V_ASSERT_OK(s2v_cast_i32_f32(GpuHandle::ctx(), nullptr, (int64_t)in->value.shape.Count(), in->value.data->ptr, out.data->ptr));
    }
};

// ---- message-passing matrices (src/nn/msg_pass.cpp:25-67,156-177): built on the host from the
//      GraphStruct on every Forward, then uploaded
template <typename mode, typename Dtype>
class IMsgPass : public Factor
{
public:
    IMsgPass(std::string _name, bool _average) : Factor(_name, PropErr::N), average(_average) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 1 && outputs.size() == 1, "unexpected operand count for a message-passing factor");
        auto* gv = dynamic_cast<GraphVar*>(operands[0].get());
        ASSERT(gv && gv->graph, "the operand must be a bound GraphVar");
        InitCPUWeight(gv->graph);
        detail::sparse<mode, Dtype>(outputs[0]).CopyFrom(cpu_weight);
    }

protected:
    virtual void InitCPUWeight(GraphStruct* graph) = 0;
    SpTensor<CPU, Dtype> cpu_weight;
    bool average;
};

#define S2V_SPARSE_OUT(StrName)                                                                         \
    static std::string StrType() { return StrName; }                                                    \
    using OutType = std::shared_ptr<SpTensorVar<mode, Dtype>>;                                          \
    OutType CreateOutVar() { return std::make_shared<SpTensorVar<mode, Dtype>>(this->name + ":out_0"); }

// [N x N]: row i = sources of the edges into i, in the order they were added
template <typename mode, typename Dtype>
class Node2NodeMsgPass : public IMsgPass<mode, Dtype>
{
public:
    S2V_SPARSE_OUT("Node2NodeMsgPass")
    Node2NodeMsgPass(std::string _name, bool _average = false) : IMsgPass<mode, Dtype>(_name, _average) {}

protected:
    void InitCPUWeight(GraphStruct* graph) override
    {
        auto& w = this->cpu_weight;
        w.Reshape({graph->num_nodes, graph->num_nodes});
        w.ResizeSp(graph->num_edges, graph->num_nodes + 1);
        // the library's builder reproduces the in_edges insertion order from the edge list
        src_.resize(graph->num_edges);
        dst_.resize(graph->num_edges);
        for (size_t e = 0; e < graph->edge_list.size(); ++e) {
            src_[e] = graph->edge_list[e].first;
            dst_[e] = graph->edge_list[e].second;
        }
        const int rc = s2v_build_n2n_csr_host(graph->num_nodes, graph->num_edges, src_.data(), dst_.data(), this->average,
                                              w.data->row_ptr, w.data->col_idx, w.data->val);
        ASSERT(rc == 0, "s2v_build_n2n_csr_host: " << s2v_status_str(rc));
    }
    std::vector<int32_t> src_, dst_;
};

// [G x N]: row g = the nodes of graph g
template <typename mode, typename Dtype>
class SubgraphMsgPass : public IMsgPass<mode, Dtype>
{
public:
    S2V_SPARSE_OUT("SubgraphMsgPass")
    SubgraphMsgPass(std::string _name, bool _average = false) : IMsgPass<mode, Dtype>(_name, _average) {}

protected:
    void InitCPUWeight(GraphStruct* graph) override
    {
        auto& w = this->cpu_weight;
        w.Reshape({graph->num_subgraph, graph->num_nodes});
        w.ResizeSp(graph->num_nodes, graph->num_subgraph + 1);
        int nnz = 0;
        for (unsigned g = 0; g < graph->num_subgraph; ++g) {
            w.data->row_ptr[g] = nnz;
            const auto& nodes = graph->subgraph->head[g];
            for (int node : nodes) {
                w.data->val[nnz] = this->average ? (Dtype)(1.0 / nodes.size()) : (Dtype)1.0;
                w.data->col_idx[nnz++] = node;
            }
        }
        ASSERT(nnz == (int)graph->num_nodes, "every node must belong to exactly one subgraph");
        w.data->row_ptr[graph->num_subgraph] = nnz;
    }
};

// ---- edge-level matrices (src/nn/msg_pass.cpp:72-152): embeddings that live on edges (loopy BP style models)
namespace detail
{
inline void edge_arrays(GraphStruct* graph, std::vector<int32_t>& src, std::vector<int32_t>& dst)
{
    src.resize(graph->num_edges);
    dst.resize(graph->num_edges);
    for (size_t e = 0; e < graph->edge_list.size(); ++e) {
        src[e] = graph->edge_list[e].first;
        dst[e] = graph->edge_list[e].second;
    }
}
}  // namespace detail

// [N x E]: row i = indices of the edges into node i, in the order they were added
template <typename mode, typename Dtype>
class Edge2NodeMsgPass : public IMsgPass<mode, Dtype>
{
public:
    S2V_SPARSE_OUT("Edge2NodeMsgPass")
    Edge2NodeMsgPass(std::string _name, bool _average = false) : IMsgPass<mode, Dtype>(_name, _average) {}

protected:
    void InitCPUWeight(GraphStruct* graph) override
    {
        auto& w = this->cpu_weight;
        w.Reshape({graph->num_nodes, graph->num_edges});
        w.ResizeSp(graph->num_edges, graph->num_nodes + 1);
        detail::edge_arrays(graph, src_, dst_);
        const int rc = s2v_build_e2n_csr_host(graph->num_nodes, graph->num_edges, src_.data(), dst_.data(), this->average,
                                              w.data->row_ptr, w.data->col_idx, w.data->val);
        ASSERT(rc == 0, "s2v_build_e2n_csr_host: " << s2v_status_str(rc));
    }
    std::vector<int32_t> src_, dst_;
};

// [E x N]: row e = the source node of edge e
template <typename mode, typename Dtype>
class Node2EdgeMsgPass : public IMsgPass<mode, Dtype>
{
public:
    S2V_SPARSE_OUT("Node2EdgeMsgPass")
    Node2EdgeMsgPass(std::string _name, bool _average = false) : IMsgPass<mode, Dtype>(_name, _average) {}

protected:
    void InitCPUWeight(GraphStruct* graph) override
    {
        auto& w = this->cpu_weight;
        w.Reshape({graph->num_edges, graph->num_nodes});
        w.ResizeSp(graph->num_edges, graph->num_edges + 1);
        detail::edge_arrays(graph, src_, dst_);
        const int rc = s2v_build_n2e_csr_host(graph->num_nodes, graph->num_edges, src_.data(), w.data->row_ptr, w.data->col_idx,
                                              w.data->val);
        ASSERT(rc == 0, "s2v_build_n2e_csr_host: " << s2v_status_str(rc));
    }
    std::vector<int32_t> src_, dst_;
};

// [E x E]: row e = (from -> to): the edges into `from` other than the ones coming back from `to`
template <typename mode, typename Dtype>
class Edge2EdgeMsgPass : public IMsgPass<mode, Dtype>
{
public:
    S2V_SPARSE_OUT("Edge2EdgeMsgPass")
    Edge2EdgeMsgPass(std::string _name, bool _average = false) : IMsgPass<mode, Dtype>(_name, _average) {}

protected:
    void InitCPUWeight(GraphStruct* graph) override
    {
        auto& w = this->cpu_weight;
        detail::edge_arrays(graph, src_, dst_);
        int64_t nnz = 0;
        rp_.resize(graph->num_edges + 1);
        int rc = s2v_build_e2e_csr_host(graph->num_nodes, graph->num_edges, src_.data(), dst_.data(), rp_.data(), nullptr, nullptr, 0, &nnz);
        ASSERT(rc == 0, "s2v_build_e2e_csr_host (size query): " << s2v_status_str(rc));
        w.Reshape({graph->num_edges, graph->num_edges});
        w.ResizeSp((size_t)nnz, graph->num_edges + 1);
        rc = s2v_build_e2e_csr_host(graph->num_nodes, graph->num_edges, src_.data(), dst_.data(), w.data->row_ptr, w.data->col_idx,
                                    w.data->val, nnz, &nnz);
        ASSERT(rc == 0, "s2v_build_e2e_csr_host: " << s2v_status_str(rc));
    }
    std::vector<int32_t> src_, dst_, rp_;
};

// ---- fused forms (no counterpart in the reference; registered through the same af<>) --------
// operands {A (CSR), H, W, X}: out = ReLU((A*H)*W + X) in one kernel
template <typename mode, typename Dtype>
class S2VLevel : public Factor
{
public:
    S2V_DENSE_OUT("S2VLevel")
    S2VLevel(std::string _name, PropErr _properr = PropErr::T) : Factor(_name, _properr) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 3 || operands.size() == 4, "S2VLevel takes {A, H, W} or {A, H, W, X}");
        auto& A = detail::sparse<mode, Dtype>(operands[0]);
        auto& H = detail::dense<mode, Dtype>(operands[1]);
        auto& W = detail::dense<mode, Dtype>(operands[2]);
        const Dtype* X = operands.size() == 4 ? detail::dense<mode, Dtype>(operands[3]).data->ptr : nullptr;
        ASSERT(A.cols() == H.rows() && H.cols() == W.rows() && W.rows() == W.cols(), "shape mismatch in S2VLevel");
        auto& out = detail::dense<mode, Dtype>(outputs[0]);
        out.Reshape({A.rows(), W.cols()});
        S2V_ASSERT_OK(s2v_level_f32(GpuHandle::ctx(), nullptr, (int64_t)A.rows(), (int64_t)A.cols(), (int)W.cols(), A.data->row_ptr,
                                    A.data->col_idx, A.data->val, H.data->ptr, W.data->ptr, X, out.data->ptr));
    }
};

// operands {S (CSR [G x N] whose row g is a contiguous node range), H}: Y = S*H as a segmented sum
template <typename mode, typename Dtype>
class GraphPool : public Factor
{
public:
    S2V_DENSE_OUT("GraphPool")
    GraphPool(std::string _name, PropErr _properr = PropErr::T) : Factor(_name, _properr) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 2, "GraphPool takes {S, H}");
        auto& S = detail::sparse<mode, Dtype>(operands[0]);
        auto& H = detail::dense<mode, Dtype>(operands[1]);
        ASSERT(S.cols() == H.rows() && (size_t)S.data->nnz == H.rows(), "GraphPool needs one pooling entry per node");
        auto& out = detail::dense<mode, Dtype>(outputs[0]);
        out.Reshape({S.rows(), H.cols()});
        // row_ptr of S is the node range of every graph when nodes are numbered graph by graph
        S2V_ASSERT_OK(s2v_segment_sum_f32(GpuHandle::ctx(), nullptr, (int64_t)S.rows(), (int)H.cols(), S.data->row_ptr, H.data->ptr,
                                          out.data->ptr));
    }
};

// operands {Y, W1, W2}: logits = ReLU(Y*W1)*W2; probs and predictions are kept as members
template <typename mode, typename Dtype>
class S2VReadout : public Factor
{
public:
    S2V_DENSE_OUT("S2VReadout")
    S2VReadout(std::string _name, PropErr _properr = PropErr::T) : Factor(_name, _properr) {}
    void Forward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<std::shared_ptr<Variable>>& outputs, Phase) override
    {
        ASSERT(operands.size() == 3, "S2VReadout takes {Y, W1, W2}");
        auto& Y = detail::dense<mode, Dtype>(operands[0]);
        auto& W1 = detail::dense<mode, Dtype>(operands[1]);
        auto& W2 = detail::dense<mode, Dtype>(operands[2]);
        ASSERT(Y.cols() == W1.rows() && W1.cols() == W2.rows(), "shape mismatch in S2VReadout");
        auto& out = detail::dense<mode, Dtype>(outputs[0]);
        out.Reshape({Y.rows(), W2.cols()});
        probs.Reshape({Y.rows(), W2.cols()});
        pred.Reshape({Y.rows()});
        S2V_ASSERT_OK(s2v_readout_f32(GpuHandle::ctx(), nullptr, (int64_t)Y.rows(), (int)Y.cols(), (int)W1.cols(), (int)W2.cols(),
                                      Y.data->ptr, W1.data->ptr, W2.data->ptr, out.data->ptr, probs.data->ptr, pred.data->ptr));
    }
    DTensor<mode, Dtype> probs;
    DTensor<mode, int> pred;
};

}  // namespace gnn
#endif
