// First level of the classifier when the node features are one-hot tags, without any per-row matrix product.
//
//     H1[i,:] = ReLU( (sum_{t in row i} val[t] * H0[col[t],:]) * W + W_in[tag[i],:] ),   H0[j,:] = ReLU(W_in[tag[j],:])
//
// (examples/graph_classification/src/kernel_mean_field.cpp:31-41, first pass of the level loop, with the one-hot X
// of nn_common.h:57-70).  H0 has only as many distinct rows as there are tags, and the product is linear in the
// gathered sum, so
//
//     (sum_t val[t] * H0[col[t],:]) * W  =  sum_t val[t] * P[tag[col[t]],:],      P = ReLU(W_in) * W    [num_tags x d]
//
// P is a few dozen rows, computed once per call by a tiny launch; the level itself becomes a gather-sum from a table
// that sits in L1, plus the X lookup and the ReLU: no split, no tensor-memory round trip, no MMA.  The launch is
// then bounded by writing H1 (N*d*4 bytes); the dependent chain row offset -> column -> tag -> table row is cut to
// three latencies per 32 rows by staging the neighbours' tags in shared memory a warp-load at a time.  Sums run over
// the non-zeros in CSR order in fp32, so the result is deterministic; it differs from the "sum first, multiply
// after" order of the other kernels by fp32 rounding only.
#include "common.cuh"

namespace
{

// P[t, j] = sum_k ReLU(table[t, k]) * W[k, j], k ascending, one CTA per table row, one thread per column (strided).
__global__ void __launch_bounds__(256) first_table_product_kernel(int n_table, int d, const float* __restrict__ table,
                                                                  const float* __restrict__ W, float* __restrict__ P)
{
    extern __shared__ float h0[];
    const int t = blockIdx.x;
    if (t >= n_table) {   // the extra row some callers ask for: zeros (what an unused gather slot adds)
        for (int j = threadIdx.x; j < d; j += blockDim.x) P[(int64_t)t * d + j] = 0.f;
        return;
    }
    for (int k = threadIdx.x; k < d; k += blockDim.x) h0[k] = relu_ref(__ldg(table + (int64_t)t * d + k));
    __syncthreads();
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float acc = 0.f;
#pragma unroll 16
        for (int k = 0; k < d; ++k) acc = fmaf(h0[k], __ldg(W + (int64_t)k * d + j), acc);   // the loads of 16 steps go out together
        P[(int64_t)t * d + j] = acc;
    }
}

// A warp takes 32 consecutive rows at a time.  Their row offsets and own tags are fetched with one coalesced load
// each; then, for as many whole rows as fit FT_CAP non-zeros, the column indices (coalesced) and the neighbours'
// tags (a gather) are staged in shared memory -- three dependent memory latencies per 32 rows instead of four per
// row.  After that each group of LPR = d/4 lanes sums one row at a time from the staged tags: table rows come from
// L1, sums run in CSR order.  A row with more than FT_CAP non-zeros is summed straight from global memory.
constexpr int FT_CAP = 256;
constexpr int FT_WARPS = 8;

template <bool HAS_VAL, int LPR_T>   // LPR_T: d/4 fixed at compile time (32, 16, 8), or 0 = read it from the argument
__global__ void __launch_bounds__(FT_WARPS * 32) first_level_table_kernel(int64_t n, int lpr_arg, const int32_t* __restrict__ row_ptr,
                                                                         const int32_t* __restrict__ col_idx, const float* __restrict__ val,
                                                                         const int32_t* __restrict__ tags, int n_table,
                                                                         const float4* __restrict__ P, const float4* __restrict__ table,
                                                                         float4* __restrict__ out, s2v_device_status* status)
{
    __shared__ int s_tag[FT_WARPS][FT_CAP];
    __shared__ float s_val[HAS_VAL ? FT_WARPS : 1][HAS_VAL ? FT_CAP : 1];
    const int lpr = LPR_T ? LPR_T : lpr_arg;
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int rows_per_warp = 32 / lpr;
    const int sub = lane / lpr, sl = lane - sub * lpr;
    const int64_t warp = (int64_t)blockIdx.x * FT_WARPS + wib;
    const int64_t warps = (int64_t)gridDim.x * FT_WARPS;
    const unsigned top = (unsigned)(n_table - 1);
    int* const my_tags = s_tag[wib];
    float* const my_vals = s_val[HAS_VAL ? wib : 0];
    const unsigned FULL = 0xffffffffu;
    bool bad_tag = false;

    for (int64_t base = warp * 32; base < n; base += warps * 32) {
        const int nrows = (int)((n - base) < 32 ? (n - base) : 32);
        // lane i: [rp_lo, rp_hi) = row base + i (empty beyond the last row); its own tag, clamped (a separate launch reports bad tags)
        const int64_t ri = base + (lane < nrows ? lane : nrows);
        const int32_t rp_lo = __ldg(row_ptr + ri);
        const int32_t rp_hi = lane < nrows ? __ldg(row_ptr + ri + 1) : rp_lo;
        // every node is a row here, so checking the rows' own tags checks all of them: a tag outside the table is
        // clamped where it is used and reported once, at the end of the kernel (S2V_ERR_INVALID_ARG)
        const unsigned raw_tag = lane < nrows ? (unsigned)__ldg(tags + base + lane) : 0u;
        bad_tag |= raw_tag > top;
        const unsigned row_tag = min(raw_tag, top);
        int r0 = 0;
        while (r0 < nrows) {
            const int32_t start = __shfl_sync(FULL, rp_lo, r0);
            // whole rows from r0 on that fit the staging buffer (their ends are monotone, so the set is a run from r0)
            const unsigned fit = __ballot_sync(FULL, lane >= r0 && lane < nrows && rp_hi - start <= FT_CAP) >> r0;
            const int nfit = (fit == FULL) ? 32 : (__ffs(~fit) - 1);
            if (nfit == 0) {
                // row r0 alone is longer than the buffer: summed straight from global memory by the first lane group
                const int32_t e = __shfl_sync(FULL, rp_hi, r0);
                const unsigned tg_row = __shfl_sync(FULL, row_tag, r0);
                if (sub == 0) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int32_t t = start; t < e; ++t) {
                        const unsigned g = min((unsigned)__ldg(tags + __ldg(col_idx + t)), top);
                        const float4 p = __ldg(P + (int64_t)g * lpr + sl);
                        if (HAS_VAL) {
                            const float w = __ldg(val + t);
                            acc.x = fmaf(w, p.x, acc.x); acc.y = fmaf(w, p.y, acc.y); acc.z = fmaf(w, p.z, acc.z); acc.w = fmaf(w, p.w, acc.w);
                        } else {
                            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
                        }
                    }
                    const float4 x = __ldg(table + (int64_t)tg_row * lpr + sl);
                    float4 r;
                    r.x = relu_ref(acc.x + x.x); r.y = relu_ref(acc.y + x.y); r.z = relu_ref(acc.z + x.z); r.w = relu_ref(acc.w + x.w);
                    st_stream_f4(out + (base + r0) * lpr + sl, r);
                }
                r0 += 1;
                continue;
            }
            const int r1 = r0 + nfit;
            const int total = __shfl_sync(FULL, rp_hi, r1 - 1) - start;   // <= FT_CAP
            // stage: all column indices first, then all tags (two latencies for the whole run of rows)
            int32_t c[FT_CAP / 32];
#pragma unroll
            for (int k = 0; k < FT_CAP / 32; ++k) {
                const int i = lane + 32 * k;
                c[k] = i < total ? __ldg(col_idx + start + i) : -1;
                if (HAS_VAL && i < total) my_vals[i] = __ldg(val + start + i);
            }
#pragma unroll
            for (int k = 0; k < FT_CAP / 32; ++k) {
                const int i = lane + 32 * k;
                if (c[k] >= 0) my_tags[i] = (int)min((unsigned)__ldg(tags + c[k]), top);
            }
            __syncwarp();
            for (int rr = r0; rr < r1; rr += rows_per_warp) {
                const int r = rr + sub;
                const bool have = r < r1;
                const int rs = have ? r : r0;
                const int b = __shfl_sync(FULL, rp_lo, rs) - start, e = __shfl_sync(FULL, rp_hi, rs) - start;
                const unsigned tg_row = __shfl_sync(FULL, row_tag, rs);
                if (have) {
                    const float4 x = __ldg(table + ((int)tg_row * lpr + sl));
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    int t = b;
                    for (; t + 4 <= e; t += 4) {
                        float4 p[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) p[u] = __ldg(P + (my_tags[t + u] * lpr + sl));
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            if (HAS_VAL) {
                                const float w = my_vals[t + u];
                                acc.x = fmaf(w, p[u].x, acc.x); acc.y = fmaf(w, p[u].y, acc.y);
                                acc.z = fmaf(w, p[u].z, acc.z); acc.w = fmaf(w, p[u].w, acc.w);
                            } else {
                                acc.x += p[u].x; acc.y += p[u].y; acc.z += p[u].z; acc.w += p[u].w;
                            }
                        }
                    }
                    for (; t < e; ++t) {
                        const float4 p = __ldg(P + (my_tags[t] * lpr + sl));
                        if (HAS_VAL) {
                            const float w = my_vals[t];
                            acc.x = fmaf(w, p.x, acc.x); acc.y = fmaf(w, p.y, acc.y); acc.z = fmaf(w, p.z, acc.z); acc.w = fmaf(w, p.w, acc.w);
                        } else {
                            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
                        }
                    }
                    float4 o;
                    o.x = relu_ref(acc.x + x.x); o.y = relu_ref(acc.y + x.y); o.z = relu_ref(acc.z + x.z); o.w = relu_ref(acc.w + x.w);
                    st_stream_f4(out + (base + r) * lpr + sl, o);
                }
            }
            __syncwarp();   // the buffer is refilled by the next run of rows
            r0 = r1;
        }
    }
    if (bad_tag) {   // record, do not fault
        status->code = S2V_ERR_INVALID_ARG;
        status->where = 2;
    }
}

}  // namespace

bool s2v_first_table_supported(int d)
{
    const int lpr = d / 4;
    return d >= 4 && d % 4 == 0 && lpr <= 32 && (lpr & (lpr - 1)) == 0;   // d in {4, 8, 16, 32, 64, 128}
}

size_t s2v_first_table_scratch_bytes(int n_table, int d)
{
    return sizeof(float) * (size_t)n_table * (size_t)d;
}

// P[t,:] = ReLU(table[t,:]) * W for the n_table rows of the table; with extra_zero_row one more row of zeros follows.
int s2v_launch_first_table_product(s2v_ctx* ctx, cudaStream_t st, int n_table, int d, const float* table, const float* W,
                                   float* P, bool extra_zero_row)
{
    first_table_product_kernel<<<n_table + (extra_zero_row ? 1 : 0), d < 256 ? ((d + 31) / 32) * 32 : 256, sizeof(float) * (size_t)d, st>>>(
        n_table, d, table, W, P);
    S2V_CHECK_LAUNCH(ctx, "first_table_product_kernel");
    return S2V_OK;
}

// out = the first level for all n rows; P_scratch holds n_table * d floats (overwritten).  The kernel also range-checks
// all n tags (it reads each of them as a row's own tag), so no separate checking launch is needed beside it.
int s2v_launch_level_first_table(s2v_ctx* ctx, cudaStream_t st, int64_t n, int d, const int32_t* row_ptr, const int32_t* col_idx,
                                 const float* val, const float* W, const float* table, int n_table, const int32_t* tags,
                                 float* P_scratch, float* out)
{
    if (!s2v_first_table_supported(d)) return S2V_ERR_UNSUPPORTED;
    const int rc = s2v_launch_first_table_product(ctx, st, n_table, d, table, W, P_scratch, false);
    if (rc != S2V_OK) return rc;
    const int lpr = d / 4;
    const int64_t rows_per_block = (int64_t)FT_WARPS * 32;   // a warp takes 32 rows at a time
    int64_t blocks = (n + rows_per_block - 1) / rows_per_block;
    const int64_t cap = (int64_t)ctx->sm_count * 8;   // eight 256-thread CTAs fill an SM's 64 warps
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const float4* P4 = reinterpret_cast<const float4*>(P_scratch);
    const float4* T4 = reinterpret_cast<const float4*>(table);
    float4* O4 = reinterpret_cast<float4*>(out);
#define FT_LAUNCH(HV, L) first_level_table_kernel<HV, L><<<(unsigned)blocks, FT_WARPS * 32, 0, st>>>(n, lpr, row_ptr, col_idx, val, tags, n_table, P4, T4, O4, ctx->dstatus_dev)
    if (val) {
        if (lpr == 32) FT_LAUNCH(true, 32); else if (lpr == 16) FT_LAUNCH(true, 16); else if (lpr == 8) FT_LAUNCH(true, 8); else FT_LAUNCH(true, 0);
    } else {
        if (lpr == 32) FT_LAUNCH(false, 32); else if (lpr == 16) FT_LAUNCH(false, 16); else if (lpr == 8) FT_LAUNCH(false, 8); else FT_LAUNCH(false, 0);
    }
#undef FT_LAUNCH
    S2V_CHECK_LAUNCH(ctx, "first_level_table_kernel");
    return S2V_OK;
}
