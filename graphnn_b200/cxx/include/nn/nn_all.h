#ifndef S2V_NN_ALL_H
#define S2V_NN_ALL_H
#include "nn/factor.h"
#include "nn/factor_graph.h"
#include "nn/ops.h"
#include "nn/param_set.h"
#include "nn/variable.h"
#endif
