// GPU context of the host-side mirror: GpuHandle::Init / Destroy with the reference's
// signature (include/tensor/gpu_handle.h:38-59).  Where the reference created cuBLAS,
// cuSPARSE and cuRAND handles (src/tensor/gpu_handle.cu:17-44), this owns one s2v_ctx
// and exposes its stream; every tensor operation and copy of the mirror runs on it.
#ifndef S2V_GPU_HANDLE_H
#define S2V_GPU_HANDLE_H

#include <cuda_runtime_api.h>

#include "s2v_b200.h"
#include "util/gnn_macros.h"

namespace gnn
{

struct GpuHandle {
    static void Init(int dev_id, unsigned int /*streamcnt*/ = 1)
    {
        ASSERT(instance() == nullptr, "GpuHandle::Init called twice");
        ASSERT(cudaSetDevice(dev_id) == cudaSuccess, "cannot select device " << dev_id);
        s2v_ctx* c = nullptr;
        const int rc = s2v_ctx_create(dev_id, &c);
        ASSERT(rc == 0, "s2v_ctx_create: " << s2v_status_str(rc));
        instance() = c;
    }
    static void Destroy()
    {
        if (instance()) s2v_ctx_destroy(instance());
        instance() = nullptr;
    }
    static s2v_ctx* ctx()
    {
        ASSERT(instance() != nullptr, "GpuHandle::Init has not been called");
        return instance();
    }
    static cudaStream_t stream() { return static_cast<cudaStream_t>(s2v_ctx_stream(ctx())); }
    static void Synchronize()
    {
        const int rc = s2v_ctx_synchronize(ctx());
        ASSERT(rc == 0, "s2v_ctx_synchronize: " << s2v_status_str(rc) << ": " << s2v_last_error(ctx()));
    }

private:
    static s2v_ctx*& instance()
    {
        static s2v_ctx* p = nullptr;
        return p;
    }
};

}  // namespace gnn
#endif
