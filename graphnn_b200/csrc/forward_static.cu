// s2v_forward_static_f32: the whole-classifier entry point for callers that must not
// allocate device memory.
//
// s2v_forward_f32 needs scratch space (three [N x d] buffers and one [G x d] buffer)
// and asks its caller to provide it, which normally means a cudaMalloc somewhere in
// the caller.  Some hosts of this library cannot do that: a serving process whose
// device memory was handed in full to another component's pool at start-up, a plug-in
// that is forbidden to call the allocator because cudaMalloc/cudaFree synchronise the
// whole device and stall every other stream of the process, or a small embedded
// caller that links no allocator wrapper at all.  For them this entry point keeps its
// scratch in a fixed array that is part of the loaded module itself, so the call path
// contains no cudaMalloc, cudaFree or other allocating routine.
//
// Properties a user must know:
//   * The array is S2V_STATIC_SCRATCH_BYTES (16 MiB) and every GPU that loads this
//     library holds it until the process exits.  A batch whose scratch need
//     (s2v_forward_workspace_bytes) is larger is rejected with S2V_ERR_WORKSPACE.
//   * The first call on each device looks up the device address of the array
//     (cudaGetSymbolAddress, with that device current).  Make that first call during
//     set-up, before any stream capture is begun.
//   * Every call on a device uses the same array and leaves its last contents there.
//     Nothing in it has to start at zero: each buffer is fully written by the
//     pipeline before it is read.  Two calls that overlap on the same GPU (different
//     streams, or different contexts of this library) race on the array; serialise
//     them.
#include <mutex>

#include "common.cuh"

namespace
{

// File-scope device array.  In host code this name is only a handle for the runtime
// (never a device address); device code may name it directly.
static __device__ __align__(256) unsigned char s2v_static_scratch[S2V_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
void* g_scratch_dev_ptr[kMaxDevices] = {};  // device address of the array, per device ordinal

// Once per device, with that device current: resolve the array's device address.
int scratch_address(s2v_ctx* ctx, void** out)
{
    const int dev = ctx->device;
    if (dev < 0 || dev >= kMaxDevices) return s2v_fail(ctx, S2V_ERR_UNSUPPORTED, "forward_static: device ordinal beyond 63");
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (!g_scratch_dev_ptr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, s2v_static_scratch);
        if (e != cudaSuccess || !p)
            return s2v_fail(ctx, S2V_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
        g_scratch_dev_ptr[dev] = p;
    }
    *out = g_scratch_dev_ptr[dev];
    return S2V_OK;
}

}  // namespace

extern "C" int s2v_forward_static_f32(s2v_ctx* ctx, s2v_stream stream, const s2v_model* model, const s2v_batch* batch,
                                      float* logits, float* probs, int32_t* pred, float* embed_out)
{
    S2V_ENTER(ctx);  // makes the context's device current for the set-up below
    if (!model || !batch) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "forward_static: NULL model or batch");
    const size_t need = s2v_forward_workspace_bytes(batch->num_nodes, batch->num_graphs, model->d);
    if (need == 0) return s2v_fail(ctx, S2V_ERR_INVALID_ARG, "forward_static: bad shape");
    if (need > (size_t)S2V_STATIC_SCRATCH_BYTES)
        return s2v_fail(ctx, S2V_ERR_WORKSPACE,
                        "forward_static: this batch needs " + std::to_string(need) + " bytes of scratch, the built-in array holds " +
                            std::to_string((size_t)S2V_STATIC_SCRATCH_BYTES) + "; use s2v_forward_f32 with your own workspace");
    void* scratch = nullptr;
    const int rc = scratch_address(ctx, &scratch);
    if (rc != S2V_OK) return rc;
    return s2v_forward_f32(ctx, stream, model, batch, scratch, (size_t)S2V_STATIC_SCRATCH_BYTES, logits, probs, pred, embed_out);
}
