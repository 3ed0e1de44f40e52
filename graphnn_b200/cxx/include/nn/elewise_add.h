#ifndef S2V_NN_ELEWISE_ADD_H
#define S2V_NN_ELEWISE_ADD_H
#include "nn/ops.h"
#endif
