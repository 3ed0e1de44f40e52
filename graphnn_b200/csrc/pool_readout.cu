// Graph pooling (segmented sum), fused readout MLP + softmax + argmax, and the
// input projection of the structure2vec classifier, for sm_100a.
#include "common.cuh"
#include "mma_tf32.cuh"

namespace
{

// ---------------------------------------------------------------- input projection
// One-hot node features make X * W_in a row lookup: msg[i,:] = W_in[tag[i],:],
// h0 = ReLU(msg) (examples/graph_classification/src/kernel_mean_field.cpp:31-32 with
// the X of nn_common.h:57-70).  d/4 lanes per node, float4 copies; W_in stays in L1/L2.
__global__ void __launch_bounds__(256) input_proj_onehot_kernel(int64_t n, int num_tags, int d4,
                                                                 const int32_t* __restrict__ tags,
                                                                 const float4* __restrict__ W_in,
                                                                 float4* __restrict__ msg, float4* __restrict__ h0,
                                                                 s2v_device_status* status)
{
    const int64_t total = n * d4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int64_t i = e / d4;
        const int c = (int)(e - i * d4);
        const int tag = tags[i];
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tag >= 0 && tag < num_tags)
            v = __ldg(W_in + (int64_t)tag * d4 + c);
        else if (c == 0) {  // record, do not fault: a tag outside [0, F) contributes a zero row
            status->code = S2V_ERR_INVALID_ARG;
            status->where = 2;
        }
        if (msg) msg[e] = v;
        if (h0) h0[e] = make_float4(relu_ref(v.x), relu_ref(v.y), relu_ref(v.z), relu_ref(v.w));
    }
}

// Dense form: msg = X[N x F] * W_in[F x d].  F is small (3..82) and W_in fits in
// shared memory; one warp per node row, lanes stride the d columns, k ascending.
__global__ void __launch_bounds__(256) input_proj_dense_kernel(int64_t n, int F, int d, const float* __restrict__ X,
                                                                const float* __restrict__ W_in, float* __restrict__ msg,
                                                                float* __restrict__ h0)
{
    extern __shared__ float Wsm[];
    for (int e = threadIdx.x; e < F * d; e += blockDim.x) Wsm[e] = W_in[e];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
        const float* x = X + i * F;
        for (int c = lane; c < d; c += 32) {
            float acc = 0.f;
            for (int k = 0; k < F; ++k) acc = fmaf(__ldg(x + k), Wsm[k * d + c], acc);
            if (msg) msg[i * d + c] = acc;
            if (h0) h0[i * d + c] = relu_ref(acc);
        }
    }
}

// ---------------------------------------------------------------- segmented sum
// Y[g,:] = sum_{n in [seg[g], seg[g+1])} H[n,:].  One warp per graph; d/4 lanes cover a
// node row with float4, 32/(d/4) node rows are summed side by side and combined with
// warp shuffles at the end.  Replaces the [G x N] CSR x dense product of
// SubgraphMsgPass (src/nn/msg_pass.cpp:156-177) when every graph owns a contiguous
// node range.  `average` gives the mean-pooling form (SubgraphMsgPass with average = true,
// src/nn/msg_pass.cpp:170): every node row is weighted by 1 / |graph| as it is added.
template <int LPR>
__global__ void __launch_bounds__(256) segment_sum_kernel(int64_t G, const int32_t* __restrict__ seg,
                                                           const float4* __restrict__ H4, float4* __restrict__ Y4,
                                                           int average)
{
    constexpr int RPP = 32 / LPR;
    const int lane = threadIdx.x & 31, sub = lane / LPR, sl = lane % LPR;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; g < G; g += warps) {
        const int beg = seg[g], end = seg[g + 1];
        const float wgt = average ? (float)(1.0 / (double)(end - beg)) : 1.0f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int t = beg + sub;
        for (; t + 3 * RPP < end; t += 4 * RPP) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldcs(H4 + (int64_t)(t + u * RPP) * LPR + sl);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (average) {
                    acc.x = fmaf(wgt, v[u].x, acc.x); acc.y = fmaf(wgt, v[u].y, acc.y);
                    acc.z = fmaf(wgt, v[u].z, acc.z); acc.w = fmaf(wgt, v[u].w, acc.w);
                } else {
                    acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;
                }
            }
        }
        for (; t < end; t += RPP) {
            const float4 v = __ldcs(H4 + (int64_t)t * LPR + sl);
            if (average) {
                acc.x = fmaf(wgt, v.x, acc.x); acc.y = fmaf(wgt, v.y, acc.y);
                acc.z = fmaf(wgt, v.z, acc.z); acc.w = fmaf(wgt, v.w, acc.w);
            } else {
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
#pragma unroll
        for (int o = 16; o >= LPR; o >>= 1) {
            acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
            acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
            acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
            acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
        }
        if (sub == 0) Y4[g * LPR + sl] = acc;
    }
}

// generic d: one warp per graph, lanes stride columns, nodes in order
__global__ void __launch_bounds__(256) segment_sum_generic_kernel(int64_t G, int d, const int32_t* __restrict__ seg,
                                                                   const float* __restrict__ H, float* __restrict__ Y,
                                                                   int average)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; g < G; g += warps) {
        const int beg = seg[g], end = seg[g + 1];
        const float wgt = average ? (float)(1.0 / (double)(end - beg)) : 1.0f;
        for (int c = lane; c < d; c += 32) {
            float acc = 0.f;
            for (int t = beg; t < end; ++t) acc = average ? fmaf(wgt, H[(int64_t)t * d + c], acc) : acc + H[(int64_t)t * d + c];
            Y[g * d + c] = acc;
        }
    }
}

// ---------------------------------------------------------------- readout
// logits = ReLU(Y*W1)*W2, probs = softmax(logits), pred = argmax(logits), one CTA per
// tile of TG graphs:
//   phase 1: Y tile -> shared memory; thread h of 256 computes hidden unit h (+256...)
//            for all TG graphs (W1 column read once per CTA, coalesced across threads;
//            Y values broadcast from shared memory), k ascending;
//   phase 2: one warp per graph reduces hidden x W2 with shuffles, lane 0 finishes the
//            row softmax / first-max argmax (C is small).
constexpr int TG = 16;
__global__ void __launch_bounds__(256) readout_kernel(int64_t G, int d, int hidden, int C, const float* __restrict__ Y,
                                                      const float* __restrict__ W1, const float* __restrict__ W2,
                                                      float* __restrict__ logits, float* __restrict__ probs,
                                                      int32_t* __restrict__ pred)
{
    extern __shared__ float sm[];
    float* Ys = sm;                 // [TG][d]
    float* Hs = sm + TG * d;        // [TG][hidden]
    float* Ls = Hs + TG * hidden;   // [TG][C]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t g0 = (int64_t)blockIdx.x * TG; g0 < G; g0 += (int64_t)gridDim.x * TG) {
        const int ng = (int)((G - g0) < TG ? (G - g0) : TG);
        for (int e = threadIdx.x; e < TG * d; e += blockDim.x) Ys[e] = (e / d) < ng ? Y[g0 * d + e] : 0.f;
        __syncthreads();
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
            float acc[TG];
#pragma unroll
            for (int g = 0; g < TG; ++g) acc[g] = 0.f;
            for (int k = 0; k < d; ++k) {
                const float w = __ldg(W1 + (int64_t)k * hidden + h);
#pragma unroll
                for (int g = 0; g < TG; ++g) acc[g] = fmaf(Ys[g * d + k], w, acc[g]);
            }
#pragma unroll
            for (int g = 0; g < TG; ++g) Hs[g * hidden + h] = relu_ref(acc[g]);
        }
        __syncthreads();
        for (int g = warp; g < ng; g += (blockDim.x >> 5)) {
            for (int c = 0; c < C; ++c) {
                float acc = 0.f;
                for (int h = lane; h < hidden; h += 32) acc = fmaf(Hs[g * hidden + h], __ldg(W2 + (int64_t)h * C + c), acc);
#pragma unroll
                for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (lane == 0) Ls[g * C + c] = acc;
            }
            __syncwarp();
            if (lane == 0) {
                const float* l = Ls + g * C;
                float mx = l[0];
                int best = 0;
                for (int c = 1; c < C; ++c)
                    if (l[c] > mx) { mx = l[c]; best = c; }
                float s = 0.f;
                for (int c = 0; c < C; ++c) s += expf(l[c] - mx);
                for (int c = 0; c < C; ++c) {
                    logits[(g0 + g) * C + c] = l[c];
                    if (probs) probs[(g0 + g) * C + c] = expf(l[c] - mx) / s;
                }
                if (pred) pred[g0 + g] = best;
            }
        }
        __syncthreads();
    }
}

// Register-tiled form for d % 4 == 0 and hidden % 4 == 0 (the configurations of the path):
// a CTA takes 32 graphs; a thread owns 4 consecutive hidden units x 8 graphs, walks k in steps of
// 4 with one 16-byte load of W1 per k (L1-resident after the first tile: W1 is at most 128 KB)
// and one 16-byte shared load of Y per graph, 128 FMAs per 12 loads; k ascending per output.
constexpr int TG4 = 32;
__global__ void __launch_bounds__(256) readout_v4_kernel(int64_t G, int d, int hidden, int C, const float* __restrict__ Y,
                                                         const float* __restrict__ W1, const float* __restrict__ W2,
                                                         float* __restrict__ logits, float* __restrict__ probs,
                                                         int32_t* __restrict__ pred)
{
    extern __shared__ __align__(16) float sm4[];
    const int ys = d + 4, hs = hidden + 4;
    float* Ys = sm4;                  // [TG4][d + 4]
    float* Hs = Ys + TG4 * ys;        // [TG4][hidden + 4]
    float* Ls = Hs + TG4 * hs;        // [TG4][C]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int d4 = d >> 2, hq = hidden >> 2;
    for (int64_t g0 = (int64_t)blockIdx.x * TG4; g0 < G; g0 += (int64_t)gridDim.x * TG4) {
        const int ng = (int)((G - g0) < TG4 ? (G - g0) : TG4);
        for (int e = threadIdx.x; e < TG4 * d4; e += blockDim.x) {
            const int g = e / d4, c = e - g * d4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g < ng) v = __ldcs(reinterpret_cast<const float4*>(Y + (g0 + g) * d) + c);
            *reinterpret_cast<float4*>(Ys + g * ys + 4 * c) = v;
        }
        __syncthreads();
        for (int item = threadIdx.x; item < hq * 4; item += blockDim.x) {
            const int h4 = (item % hq) * 4, gb = (item / hq) * 8;
            float acc[8][4];
#pragma unroll
            for (int g = 0; g < 8; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
            for (int k = 0; k < d; k += 4) {
                float4 w[4];
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) w[kk] = __ldg(reinterpret_cast<const float4*>(W1 + (int64_t)(k + kk) * hidden + h4));
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 y = *reinterpret_cast<const float4*>(Ys + (gb + g) * ys + k);
                    const float yy[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        acc[g][0] = fmaf(yy[kk], w[kk].x, acc[g][0]);
                        acc[g][1] = fmaf(yy[kk], w[kk].y, acc[g][1]);
                        acc[g][2] = fmaf(yy[kk], w[kk].z, acc[g][2]);
                        acc[g][3] = fmaf(yy[kk], w[kk].w, acc[g][3]);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < 8; ++g)
                *reinterpret_cast<float4*>(Hs + (gb + g) * hs + h4) =
                    make_float4(relu_ref(acc[g][0]), relu_ref(acc[g][1]), relu_ref(acc[g][2]), relu_ref(acc[g][3]));
        }
        __syncthreads();
        for (int g = warp; g < ng; g += (blockDim.x >> 5)) {
            for (int c = 0; c < C; ++c) {
                float acc = 0.f;
                for (int h = lane; h < hidden; h += 32) acc = fmaf(Hs[g * hs + h], __ldg(W2 + (int64_t)h * C + c), acc);
#pragma unroll
                for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (lane == 0) Ls[g * C + c] = acc;
            }
            __syncwarp();
            if (lane == 0) {
                const float* l = Ls + g * C;
                float mx = l[0];
                int best = 0;
                for (int c = 1; c < C; ++c)
                    if (l[c] > mx) { mx = l[c]; best = c; }
                float s = 0.f;
                for (int c = 0; c < C; ++c) s += expf(l[c] - mx);
                for (int c = 0; c < C; ++c) {
                    logits[(g0 + g) * C + c] = l[c];
                    if (probs) probs[(g0 + g) * C + c] = expf(l[c] - mx) / s;
                }
                if (pred) pred[g0 + g] = best;
            }
        }
        __syncthreads();
    }
}

// Tensor-core form of the first readout layer for d % 8 == 0 and hidden % 32 == 0: a CTA of eight warps takes 32
// graphs; warp (gh, hq) computes graphs 16*gh .. +15 x hidden units hq*hidden/4 .. as 3xTF32 mma.sync.m16n8k8 tiles
// (Y fragments from shared memory split head/tail with rounding, W1 fragments straight from L1/L2 split by
// truncation, small terms first, fp32 accumulate), then ReLU into the shared hidden tile.  The second layer
// (hidden x C, C small) and softmax / argmax follow as in the register-tiled form: one warp per graph.
template <int NT /* 8-column MMA tiles per warp = hidden / 32 */>
__global__ void __launch_bounds__(256, 4) readout_mma_kernel(int64_t G, int d, int C, const float* __restrict__ Y,
                                                          const float* __restrict__ W1, const float* __restrict__ W2,
                                                          float* __restrict__ logits, float* __restrict__ probs,
                                                          int32_t* __restrict__ pred)
{
    extern __shared__ __align__(16) float smm[];
    constexpr int hidden = NT * 32;
    const int ys = d + 4, hs = hidden + 4;   // A fragments (rows g, g+8; cols tig, tig+4) hit 32 distinct banks
    float* Ys = smm;                  // [32][d + 4]
    float* Hs = Ys + TG4 * ys;        // [32][hidden + 4]
    float* Ls = Hs + TG4 * hs;        // [32][C]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tig = lane & 3;        // MMA fragment coordinates
    const int gh = warp & 1, hq = warp >> 1;
    const int d4 = d >> 2;
    for (int64_t g0 = (int64_t)blockIdx.x * TG4; g0 < G; g0 += (int64_t)gridDim.x * TG4) {
        const int ng = (int)((G - g0) < TG4 ? (G - g0) : TG4);
        for (int e = threadIdx.x; e < TG4 * d4; e += blockDim.x) {
            const int gg = e / d4, c = e - gg * d4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gg < ng) v = __ldcs(reinterpret_cast<const float4*>(Y + (g0 + gg) * d) + c);
            *reinterpret_cast<float4*>(Ys + gg * ys + 4 * c) = v;
        }
        __syncthreads();
        float c[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
        const float* ya = Ys + (16 * gh + g) * ys + tig;
        const float* wb = W1 + (int64_t)tig * hidden + hq * (NT * 8) + g;
#pragma unroll 2
        for (int ks = 0; ks < d / 8; ++ks) {
            uint32_t ah[4], al[4];
            tf32_split_rn(ya[ks * 8], ah[0], al[0]);
            tf32_split_rn(ya[8 * ys + ks * 8], ah[1], al[1]);
            tf32_split_rn(ya[ks * 8 + 4], ah[2], al[2]);
            tf32_split_rn(ya[8 * ys + ks * 8 + 4], ah[3], al[3]);
            const float* w = wb + (int64_t)(ks * 8) * hidden;
            float w0[NT], w1[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                w0[nt] = __ldg(w + nt * 8);
                w1[nt] = __ldg(w + (int64_t)4 * hidden + nt * 8);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                uint32_t bh0, bl0, bh1, bl1;
                tf32_split_trunc(w0[nt], bh0, bl0);
                tf32_split_trunc(w1[nt], bh1, bl1);
                mma_tf32(c[nt], al, bh0, bh1);   // small terms first
                mma_tf32(c[nt], ah, bl0, bl1);
                mma_tf32(c[nt], ah, bh0, bh1);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float* h0 = Hs + (16 * gh + g) * hs + hq * (NT * 8) + nt * 8 + 2 * tig;
            *reinterpret_cast<float2*>(h0) = make_float2(relu_ref(c[nt][0]), relu_ref(c[nt][1]));
            *reinterpret_cast<float2*>(h0 + 8 * hs) = make_float2(relu_ref(c[nt][2]), relu_ref(c[nt][3]));
        }
        __syncthreads();
        for (int gg = warp; gg < ng; gg += (blockDim.x >> 5)) {
            for (int cc = 0; cc < C; ++cc) {
                float acc = 0.f;
                for (int h = lane; h < hidden; h += 32) acc = fmaf(Hs[gg * hs + h], __ldg(W2 + (int64_t)h * C + cc), acc);
#pragma unroll
                for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (lane == 0) Ls[gg * C + cc] = acc;
            }
            __syncwarp();
            if (lane == 0) {
                const float* l = Ls + gg * C;
                float mx = l[0];
                int best = 0;
                for (int cc = 1; cc < C; ++cc)
                    if (l[cc] > mx) { mx = l[cc]; best = cc; }
                float sum = 0.f;
                for (int cc = 0; cc < C; ++cc) sum += expf(l[cc] - mx);
                for (int cc = 0; cc < C; ++cc) {
                    logits[(g0 + gg) * C + cc] = l[cc];
                    if (probs) probs[(g0 + gg) * C + cc] = expf(l[cc] - mx) / sum;
                }
                if (pred) pred[g0 + gg] = best;
            }
        }
        __syncthreads();
    }
}

inline unsigned grid_cap(s2v_ctx* ctx, int64_t blocks, int per_sm)
{
    const int64_t cap = (int64_t)ctx->sm_count * per_sm;
    if (blocks > cap) blocks = cap;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace

extern "C" {

int s2v_input_proj_onehot_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n, int num_tags, int d, const int32_t* tags,
                              const float* W_in, float* msg, float* h0)
{
    S2V_ENTER(ctx);
    if (n < 0 || num_tags <= 0 || d <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "input_proj: bad shape");
    if (n == 0) return S2V_OK;
    if (!tags || !W_in || (!msg && !h0)) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "input_proj: NULL pointer");
    if (d % 4 != 0 || !s2v_aligned16(W_in) || (msg && !s2v_aligned16(msg)) || (h0 && !s2v_aligned16(h0)))
        return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "input_proj_onehot: d must be a multiple of 4 and pointers 16-byte aligned");
    const int d4 = d / 4;
    input_proj_onehot_kernel<<<grid_cap(ctx, (n * d4 + 255) / 256, 8), 256, 0, s2v_pick_stream(ctx, stream)>>>(
        n, num_tags, d4, tags, reinterpret_cast<const float4*>(W_in), reinterpret_cast<float4*>(msg),
        reinterpret_cast<float4*>(h0), ctx->dstatus_dev);
    S2V_CHECK_LAUNCH(ctx, "input_proj_onehot_kernel");
    return S2V_OK;
}

int s2v_input_proj_dense_f32(s2v_ctx* ctx, s2v_stream stream, int64_t n, int num_feat, int d, const float* X,
                             const float* W_in, float* msg, float* h0)
{
    S2V_ENTER(ctx);
    if (n < 0 || num_feat <= 0 || d <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "input_proj: bad shape");
    if (n == 0) return S2V_OK;
    if (!X || !W_in || (!msg && !h0)) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "input_proj: NULL pointer");
    const size_t smem = sizeof(float) * (size_t)num_feat * d;
    if (smem > 200 * 1024) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "input_proj_dense: W_in beyond 200 KB; use s2v_gemm_f32");
    S2V_CUDA_OK(ctx, cudaFuncSetAttribute(input_proj_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    input_proj_dense_kernel<<<grid_cap(ctx, (n + 7) / 8, 4), 256, smem, s2v_pick_stream(ctx, stream)>>>(n, num_feat, d, X,
                                                                                                          W_in, msg, h0);
    S2V_CHECK_LAUNCH(ctx, "input_proj_dense_kernel");
    return S2V_OK;
}

int s2v_segment_sum_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int d, const int32_t* seg_ptr,
                        const float* H, float* Y)
{
    return s2v_segment_pool_f32(ctx, stream, num_graphs, d, seg_ptr, H, 0, Y);
}

int s2v_segment_pool_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int d, const int32_t* seg_ptr,
                         const float* H, int average, float* Y)
{
    S2V_ENTER(ctx);
    if (num_graphs < 0 || d <= 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "segment_sum: bad shape");
    if (num_graphs == 0) return S2V_OK;
    if (!seg_ptr || !H || !Y) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "segment_sum: NULL pointer");
    cudaStream_t st = s2v_pick_stream(ctx, stream);
    const unsigned grid = grid_cap(ctx, (num_graphs + 7) / 8, 8);
    const bool vec = s2v_aligned16(H) && s2v_aligned16(Y);
    const float4* H4 = reinterpret_cast<const float4*>(H);
    float4* Y4 = reinterpret_cast<float4*>(Y);
    if (vec && d == 32)
        segment_sum_kernel<8><<<grid, 256, 0, st>>>(num_graphs, seg_ptr, H4, Y4, average);
    else if (vec && d == 64)
        segment_sum_kernel<16><<<grid, 256, 0, st>>>(num_graphs, seg_ptr, H4, Y4, average);
    else if (vec && d == 128)
        segment_sum_kernel<32><<<grid, 256, 0, st>>>(num_graphs, seg_ptr, H4, Y4, average);
    else
        segment_sum_generic_kernel<<<grid, 256, 0, st>>>(num_graphs, d, seg_ptr, H, Y, average);
    S2V_CHECK_LAUNCH(ctx, "segment_sum_kernel");
    return S2V_OK;
}

int s2v_readout_f32(s2v_ctx* ctx, s2v_stream stream, int64_t num_graphs, int d, int hidden, int num_class,
                    const float* Y, const float* W1, const float* W2, float* logits, float* probs, int32_t* pred)
{
    S2V_ENTER(ctx);
    if (num_graphs < 0 || d <= 0 || hidden <= 0 || num_class <= 0)
        return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "readout: bad shape");
    if (num_graphs == 0) return S2V_OK;
    if (!Y || !W1 || !W2 || !logits) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "readout: NULL pointer");
    if (s2v_readout_tc_supported(ctx, num_graphs, d, hidden, num_class) && s2v_aligned16(Y)) {
        // batches of hundreds of graphs and the widths of the path: first layer on the 5th-generation tensor cores
        const int rc = s2v_launch_readout_tc(ctx, s2v_pick_stream(ctx, stream), num_graphs, d, hidden, num_class, Y, W1, W2, logits, probs, pred);
        if (rc != S2V_ERR_UNSUPPORTED) return rc;
    }
    const size_t smem4 = sizeof(float) * (size_t)TG4 * ((size_t)d + 4 + hidden + 4 + num_class);
    if (d % 8 == 0 && (hidden == 256 || hidden == 128) && smem4 <= 96 * 1024 && s2v_aligned16(Y) && num_graphs >= 256) {
        // batches of hundreds of graphs and the two hidden sizes of the path: first layer on the tensor cores
        // four CTAs per SM (64 registers, 50 KB of shared memory each): the 512 tiles of a 16,384-graph batch run as one wave
        const unsigned grid = grid_cap(ctx, (num_graphs + TG4 - 1) / TG4, 4);
        if (hidden == 256) {
            S2V_CUDA_OK(ctx, cudaFuncSetAttribute(readout_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4));
            readout_mma_kernel<8><<<grid, 256, smem4, s2v_pick_stream(ctx, stream)>>>(num_graphs, d, num_class, Y, W1, W2, logits, probs, pred);
        } else {
            S2V_CUDA_OK(ctx, cudaFuncSetAttribute(readout_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4));
            readout_mma_kernel<4><<<grid, 256, smem4, s2v_pick_stream(ctx, stream)>>>(num_graphs, d, num_class, Y, W1, W2, logits, probs, pred);
        }
        S2V_CHECK_LAUNCH(ctx, "readout_mma_kernel");
        return S2V_OK;
    }
    if (d % 4 == 0 && hidden % 4 == 0 && smem4 <= 96 * 1024 && s2v_aligned16(Y) && s2v_aligned16(W1)) {
        S2V_CUDA_OK(ctx, cudaFuncSetAttribute(readout_v4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4));
        readout_v4_kernel<<<grid_cap(ctx, (num_graphs + TG4 - 1) / TG4, 2), 256, smem4, s2v_pick_stream(ctx, stream)>>>(
            num_graphs, d, hidden, num_class, Y, W1, W2, logits, probs, pred);
        S2V_CHECK_LAUNCH(ctx, "readout_v4_kernel");
        return S2V_OK;
    }
    const size_t smem = sizeof(float) * (size_t)TG * ((size_t)d + hidden + num_class);
    if (smem > 200 * 1024) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "readout: d + hidden + classes too large for shared memory");
    S2V_CUDA_OK(ctx, cudaFuncSetAttribute(readout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    readout_kernel<<<grid_cap(ctx, (num_graphs + TG - 1) / TG, 4), 256, smem, s2v_pick_stream(ctx, stream)>>>(
        num_graphs, d, hidden, num_class, Y, W1, W2, logits, probs, pred);
    S2V_CHECK_LAUNCH(ctx, "readout_kernel");
    return S2V_OK;
}

}  // extern "C"
