// Operator base class (interface of include/nn/factor.h:15-56 in the reference).
#ifndef S2V_FACTOR_H
#define S2V_FACTOR_H

#include <memory>
#include <string>
#include <vector>

#include "nn/variable.h"
#include "util/fmt.h"

namespace gnn
{

class Factor
{
public:
    Factor(std::string _name, PropErr _properr = PropErr::T) : name(_name), properr(_properr) {}
    virtual ~Factor() {}
    virtual void Forward(std::vector<std::shared_ptr<Variable>>& operands,
                         std::vector<std::shared_ptr<Variable>>& outputs, Phase phase) NOT_IMPLEMENTED
    // training is outside this library
    virtual void Backward(std::vector<std::shared_ptr<Variable>>& operands, std::vector<bool>& isConst,
                          std::vector<std::shared_ptr<Variable>>& outputs) NOT_IMPLEMENTED
    std::string name;
    PropErr properr;
};

}  // namespace gnn
#endif
