// Named set of model parameters (interface of include/nn/param_set.h:17-84 in the reference).
#ifndef S2V_PARAM_SET_H
#define S2V_PARAM_SET_H

#include <map>
#include <memory>
#include <string>

#include "nn/variable.h"

namespace gnn
{

template <typename mode, typename Dtype>
class ParamSet
{
public:
    void AddParam(std::shared_ptr<DTensorVar<mode, Dtype>> param)
    {
        ASSERT(params.count(param->name) == 0, "duplicated parameter " << param->name);
        params[param->name] = param;
    }
    std::map<std::string, std::shared_ptr<DTensorVar<mode, Dtype>>> params;
};

template <template <typename, typename> class ParamType, typename mode, typename Dtype, typename IdxType, typename... Args>
std::shared_ptr<ParamType<mode, Dtype>> add_diff(ParamSet<mode, Dtype>& pset, std::string param_name,
                                                 std::initializer_list<IdxType> l, Args&&... args)
{
    auto p = std::make_shared<ParamType<mode, Dtype>>(param_name, std::vector<IdxType>(l), std::forward<Args>(args)...);
    pset.AddParam(p);
    return p;
}

}  // namespace gnn
#endif
