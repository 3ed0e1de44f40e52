// Warp-level 3xTF32 building blocks (mma.sync.m16n8k8): the TF32 head/tail split of an fp32 value and the MMA wrapper.
#pragma once

#include "common.cuh"

namespace
{

// TF32 split helpers.  head = value rounded to TF32, tail = (value - head) cut to TF32.
__device__ __forceinline__ uint32_t tf32_round(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ void tf32_split_rn(float v, uint32_t& head, uint32_t& tail)
{
    head = tf32_round(v);
    tail = tf32_round(v - __uint_as_float(head));
}
// cheaper form for W, applied on every use: head by truncation (the subtraction is exact)
__device__ __forceinline__ void tf32_split_trunc(float v, uint32_t& head, uint32_t& tail)
{
    head = __float_as_uint(v) & 0xffffe000u;
    tail = __float_as_uint(v - __uint_as_float(head)) & 0xffffe000u;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

}  // namespace
