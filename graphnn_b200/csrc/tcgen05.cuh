// Building blocks shared by the kernels that use the 5th-generation tensor cores (tcgen05, tensor memory):
// mbarrier primitives with a bounded, warp-uniform wait, the TF32 head/tail split, the shared-memory
// matrix descriptor of the K-major 128-byte-swizzle layout, and thin wrappers around tcgen05.mma / .st / .ld.
#pragma once

#include "common.cuh"

namespace
{

constexpr int TC_WAIT_LIMIT = 1 << 17;        // polls before a wait gives up (each may sleep up to TC_SUSPEND_NS)
constexpr uint32_t TC_SUSPEND_NS = 10000;    // a waiting thread sleeps in the barrier unit instead of spinning through the issue port

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(TC_SUSPEND_NS)
        : "memory");
    return ok != 0;
}
// Bounded wait, called by all 32 lanes of a warp together.  Every lane polls; the verdict is the warp's:
// true only if every lane saw the phase complete, false for all lanes as soon as one of them saw the CTA-wide
// abort flag or ran out of polls (it then raises the flag and records the time-out).  A warp therefore never
// splits into lanes that go on and lanes that leave, and the warp-wide instructions after a wait
// (shuffles, votes, tcgen05.ld/st) always run with all lanes present.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, s2v_device_status* status,
                                        int site, int limit = TC_WAIT_LIMIT)
{
    int spins = 0;
    bool ok = true;
    while (!tc_mbar_try(bar, parity)) {
        if (*abort_flag) { ok = false; break; }
        if (++spins > limit) {
            *abort_flag = 1;
            status->code = S2V_ERR_DEVICE_TIMEOUT;
            status->where = site;
            ok = false;
            break;
        }
    }
    return __all_sync(0xffffffffu, ok);
}
// A table row index that came from the caller's data (a node tag) is clamped into [0, n_table) where it is used:
// one instruction, so no lookup can leave the table whatever the data holds.  DETECTING a bad index is not done in
// the level kernels (a compare-and-record there cost 6 % of the level's time): the host entry points launch
// index_range_check_kernel over the index array beside the level, which records S2V_ERR_INVALID_ARG.
__device__ __forceinline__ int tc_table_row(int v, int n_table)
{
    return (int)min((unsigned)v, (unsigned)(n_table - 1));
}
// TF32 head rounded to nearest (add half an ulp of TF32 to the bit pattern, then cut: integer pipe only,
// no conversion-unit instruction), tail = v - head (exact) cut to TF32.  head + tail differs from v by
// less than 2^-23 |v|.
__device__ __forceinline__ void tc_split(float v, uint32_t& head, uint32_t& tail)
{
    head = (__float_as_uint(v) + 0x1000u) & 0xffffe000u;
    tail = __float_as_uint(v - __uint_as_float(head)) & 0xffffe000u;
}
// A 32-bit load that stays where it is written: the values fetched a tile ahead (row offsets, X row
// indices) must be issued early, and a plain load may be moved down to its first use.
__device__ __forceinline__ int32_t tc_ld_early(const int32_t* p)
{
    int32_t v;
    asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t tf32_rn(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_b_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                        // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// tcgen05.st / tcgen05.ld of this thread's tensor-memory lane, 8 or 16 consecutive 32-bit columns
__device__ __forceinline__ void tc_st_cols8(uint32_t addr, const uint32_t* r)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(addr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tc_ld_cols16(uint32_t addr, uint32_t* v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(addr)
        : "memory");
}

}  // namespace
