#ifndef S2V_TENSOR_ALL_H
#define S2V_TENSOR_ALL_H
#include "tensor/gpu_handle.h"
#include "tensor/tensor.h"
#endif
