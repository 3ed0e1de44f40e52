// Variables of the factor graph (interface of include/nn/variable.h in the reference):
// named nodes holding a graph, a dense tensor or a CSR tensor; placeholders are bound to
// caller-owned objects by pointer (SetRef -> ShallowCopy, src/nn/variable.cpp:29-32,51-56).
#ifndef S2V_VARIABLE_H
#define S2V_VARIABLE_H

#include <memory>
#include <string>
#include <vector>

#include "tensor/tensor_all.h"
#include "util/graph_struct.h"

namespace gnn
{

class Variable
{
public:
    explicit Variable(std::string _name) : name(_name) {}
    virtual ~Variable() {}
    virtual void SetRef(void*) NOT_IMPLEMENTED
    virtual EleType GetEleType() = 0;
    virtual MatMode GetMode() = 0;
    std::string name;
};

class GraphVar : public Variable
{
public:
    explicit GraphVar(std::string _name) : Variable(_name), graph(nullptr) {}
    EleType GetEleType() override { return EleType::UNKNOWN; }
    MatMode GetMode() override { return MatMode::cpu; }
    void SetRef(void* p) override { graph = static_cast<GraphStruct*>(p); }
    GraphStruct* graph;
};

template <typename mode, typename matType, typename Dtype> class TensorVarTemplate;
template <typename mode, typename Dtype> using DTensorVar = TensorVarTemplate<mode, DENSE, Dtype>;
template <typename mode, typename Dtype> using SpTensorVar = TensorVarTemplate<mode, CSR_SPARSE, Dtype>;

template <typename mode, typename Dtype>
class TensorVar : public Variable
{
public:
    explicit TensorVar(std::string _name) : Variable(_name) {}
    template <typename matType>
    TensorVarTemplate<mode, matType, Dtype>& Derived()
    {
        auto* ret = dynamic_cast<TensorVarTemplate<mode, matType, Dtype>*>(this);
        ASSERT(ret, "wrong derived type of TensorVar");
        return *ret;
    }
    EleType GetEleType() override { return Dtype2Enum<Dtype>(); }
    MatMode GetMode() override { return mode::type; }
    virtual Dtype AsScalar() = 0;
    virtual MatType GetMatType() = 0;
};

template <typename mode, typename Dtype>
class TensorVarTemplate<mode, DENSE, Dtype> : public TensorVar<mode, Dtype>
{
public:
    explicit TensorVarTemplate(std::string _name) : TensorVar<mode, Dtype>(_name) {}
    TensorVarTemplate(std::string _name, std::vector<size_t> l) : TensorVar<mode, Dtype>(_name) { value.Reshape(l); }
    TensorVarTemplate(std::string _name, std::vector<int> l) : TensorVarTemplate(_name, std::vector<size_t>(l.begin(), l.end())) {}
    TensorVarTemplate(std::string _name, std::vector<uint> l) : TensorVarTemplate(_name, std::vector<size_t>(l.begin(), l.end())) {}
    void SetRef(void* p) override { value.ShallowCopy(*static_cast<DTensor<mode, Dtype>*>(p)); }
    Dtype AsScalar() override { return value.AsScalar(); }
    MatType GetMatType() override { return MatType::dense; }
    DTensor<mode, Dtype> value;
    RowSpTensor<mode, Dtype> grad;   // unused on the inference path
};

template <typename mode, typename Dtype>
class TensorVarTemplate<mode, CSR_SPARSE, Dtype> : public TensorVar<mode, Dtype>
{
public:
    explicit TensorVarTemplate(std::string _name) : TensorVar<mode, Dtype>(_name) {}
    void SetRef(void* p) override { value.ShallowCopy(*static_cast<SpTensor<mode, Dtype>*>(p)); }
    Dtype AsScalar() override { return 0; }
    MatType GetMatType() override { return MatType::sparse; }
    SpTensor<mode, Dtype> value;
};

}  // namespace gnn
#endif
