#ifndef S2V_NN_SOFTMAX_H
#define S2V_NN_SOFTMAX_H
#include "nn/ops.h"
#endif
