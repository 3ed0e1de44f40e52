#ifndef S2V_NN_RELU_H
#define S2V_NN_RELU_H
#include "nn/ops.h"
#endif
