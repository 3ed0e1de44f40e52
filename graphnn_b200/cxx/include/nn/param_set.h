// Named set of model parameters (interface of include/nn/param_set.h:17-84 in the reference).
#ifndef S2V_PARAM_SET_H
#define S2V_PARAM_SET_H

#include <cstdio>
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
    // Checkpoint = the tensors' records one after another in name order, as the reference writes
    // them (src/nn/param_set.cpp:28-54); a file saved by the reference loads here and vice versa.
    void Save(std::string filename)
    {
        FILE* fid = fopen(filename.c_str(), "wb");
        ASSERT(fid, "file " + filename + " cannot be written");
        for (auto& p : params) p.second->value.Serialize(fid);
        fclose(fid);
    }
    void Load(std::string filename)
    {
        FILE* fid = fopen(filename.c_str(), "rb");
        ASSERT(fid, "file " + filename + " is not found");
        for (auto& p : params) p.second->value.Deserialize(fid);
        fclose(fid);
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
