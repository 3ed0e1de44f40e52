#ifndef S2V_NN_ARG_MAX_H
#define S2V_NN_ARG_MAX_H
#include "nn/ops.h"
#endif
