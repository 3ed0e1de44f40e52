#ifndef S2V_NN_MATMUL_H
#define S2V_NN_MATMUL_H
#include "nn/ops.h"
#endif
