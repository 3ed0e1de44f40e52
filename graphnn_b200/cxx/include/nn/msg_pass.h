#ifndef S2V_NN_MSG_PASS_H
#define S2V_NN_MSG_PASS_H
#include "nn/ops.h"
#endif
