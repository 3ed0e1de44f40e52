// Multi-GPU entry points of the C ABI, directly on NCCL.
//
// The inference path needs exactly two exchanges and no reduction:
//   * shard-by-graph batches: one final gather of the per-rank logits / predictions (ragged: ranks own
//     different numbers of graphs), done as a group of broadcasts, one rooted at every rank;
//   * a row-partitioned giant graph: per level either one all-gather of the [rows x d] embedding slabs, or --
//     when a rank references only a fraction of the remote rows -- a pairwise exchange of exactly those rows
//     (a group of sends and receives with per-peer counts).
// NCCL is opened at run time (dlopen of libnccl.so.2, or of the library named by S2V_NCCL_LIBRARY), so the
// single-GPU product does not depend on it and a process that already has an NCCL loaded -- a torch process
// -- shares that copy.  Every NCCL status other than success becomes S2V_ERR_COMM with NCCL's own message
// kept for s2v_comm_last_error; nothing aborts.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace
{

// The subset of NCCL's C interface used here, declared locally (the types below follow nccl.h: a 128-byte
// unique id, opaque communicator handles, ncclFloat32 = 7, ncclInt32 = 2, ncclSuccess = 0).
struct nccl_unique_id { char internal[128]; };
typedef void* nccl_comm_t;
typedef int nccl_result_t;
constexpr int NCCL_INT32 = 2, NCCL_FLOAT32 = 7;

struct nccl_api {
    void* handle = nullptr;
    nccl_result_t (*GetUniqueId)(nccl_unique_id*) = nullptr;
    nccl_result_t (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int) = nullptr;
    nccl_result_t (*CommInitAll)(nccl_comm_t*, int, const int*) = nullptr;
    nccl_result_t (*CommDestroy)(nccl_comm_t) = nullptr;
    nccl_result_t (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
    nccl_result_t (*Broadcast)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    nccl_result_t (*Send)(const void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    nccl_result_t (*Recv)(void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    nccl_result_t (*GroupStart)() = nullptr;
    nccl_result_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(nccl_result_t) = nullptr;
    std::string load_error;
};

std::mutex g_api_mu;
nccl_api g_api;
bool g_api_tried = false;

const nccl_api* api()
{
    std::lock_guard<std::mutex> lock(g_api_mu);
    if (g_api_tried) return g_api.handle ? &g_api : nullptr;
    g_api_tried = true;
    const char* name = std::getenv("S2V_NCCL_LIBRARY");
    if (!name || !*name) name = "libnccl.so.2";
    void* h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        g_api.load_error = std::string("cannot open ") + name + ": " + dlerror();
        return nullptr;
    }
    bool ok = true;
    auto sym = [&](const char* s) -> void* {
        void* p = dlsym(h, s);
        if (!p) {
            ok = false;
            g_api.load_error = std::string(name) + " lacks " + s;
        }
        return p;
    };
    g_api.GetUniqueId = reinterpret_cast<decltype(g_api.GetUniqueId)>(sym("ncclGetUniqueId"));
    g_api.CommInitRank = reinterpret_cast<decltype(g_api.CommInitRank)>(sym("ncclCommInitRank"));
    g_api.CommInitAll = reinterpret_cast<decltype(g_api.CommInitAll)>(sym("ncclCommInitAll"));
    g_api.CommDestroy = reinterpret_cast<decltype(g_api.CommDestroy)>(sym("ncclCommDestroy"));
    g_api.AllGather = reinterpret_cast<decltype(g_api.AllGather)>(sym("ncclAllGather"));
    g_api.Broadcast = reinterpret_cast<decltype(g_api.Broadcast)>(sym("ncclBroadcast"));
    g_api.Send = reinterpret_cast<decltype(g_api.Send)>(sym("ncclSend"));
    g_api.Recv = reinterpret_cast<decltype(g_api.Recv)>(sym("ncclRecv"));
    g_api.GroupStart = reinterpret_cast<decltype(g_api.GroupStart)>(sym("ncclGroupStart"));
    g_api.GroupEnd = reinterpret_cast<decltype(g_api.GroupEnd)>(sym("ncclGroupEnd"));
    g_api.GetErrorString = reinterpret_cast<decltype(g_api.GetErrorString)>(sym("ncclGetErrorString"));
    if (!ok) {
        dlclose(h);
        return nullptr;
    }
    g_api.handle = h;
    return &g_api;
}

std::string g_global_error;   // failures before a communicator exists

}  // namespace

struct s2v_comm {
    nccl_comm_t nccl = nullptr;
    int device = -1;    // CUDA device the communicator was created on; -1: the caller keeps the right device current
    int rank = 0;
    int world = 1;
    std::string last_error;
    std::mutex mu;
};

namespace
{

int comm_fail(s2v_comm* c, const std::string& msg)
{
    if (c) {
        std::lock_guard<std::mutex> g(c->mu);
        c->last_error = msg;
    } else {
        std::lock_guard<std::mutex> g(g_api_mu);
        g_global_error = msg;
    }
    return S2V_ERR_COMM;
}

std::string nccl_text(const nccl_api* a, const char* call, nccl_result_t r)
{
    return std::string(call) + " failed: " + (a->GetErrorString ? a->GetErrorString(r) : "unknown") + " (NCCL status " +
           std::to_string(r) + ")";
}

// the communicator's device is made current for the call (NCCL requires it) and the caller's restored
struct comm_device_guard {
    int prev = -1;
    bool ok = true;
    explicit comm_device_guard(int dev)
    {
        if (dev < 0) return;
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~comm_device_guard()
    {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

}  // namespace

extern "C" {

int s2v_comm_unique_id(void* id_out)
{
    if (!id_out) return S2V_ERR_INVALID_ARG;
    const nccl_api* a = api();
    if (!a) return comm_fail(nullptr, g_api.load_error);
    nccl_unique_id id;
    std::memset(&id, 0, sizeof(id));
    const nccl_result_t r = a->GetUniqueId(&id);
    if (r != 0) return comm_fail(nullptr, nccl_text(a, "ncclGetUniqueId", r));
    std::memcpy(id_out, &id, S2V_COMM_ID_BYTES);
    return S2V_OK;
}

int s2v_comm_create_rank(int device, const void* id, int world, int rank, s2v_comm** out)
{
    if (!out) return S2V_ERR_INVALID_ARG;
    *out = nullptr;
    if (!id || world < 1 || rank < 0 || rank >= world) return S2V_ERR_INVALID_ARG;
    const nccl_api* a = api();
    if (!a) return comm_fail(nullptr, g_api.load_error);
    comm_device_guard guard(device);
    if (!guard.ok) return S2V_ERR_CUDA;
    s2v_comm* c = new (std::nothrow) s2v_comm();
    if (!c) return S2V_ERR_CUDA;
    c->device = device;
    c->rank = rank;
    c->world = world;
    nccl_unique_id uid;
    std::memcpy(&uid, id, sizeof(uid));
    const nccl_result_t r = a->CommInitRank(&c->nccl, world, uid, rank);
    if (r != 0) {
        const int rc = comm_fail(nullptr, nccl_text(a, "ncclCommInitRank", r));
        delete c;
        return rc;
    }
    *out = c;
    return S2V_OK;
}

int s2v_comm_create(int ngpu, const int* devs, s2v_comm** out)
{
    if (!out || !devs || ngpu < 1) return S2V_ERR_INVALID_ARG;
    for (int i = 0; i < ngpu; ++i) out[i] = nullptr;
    const nccl_api* a = api();
    if (!a) return comm_fail(nullptr, g_api.load_error);
    std::vector<nccl_comm_t> comms((size_t)ngpu, nullptr);
    const nccl_result_t r = a->CommInitAll(comms.data(), ngpu, devs);
    if (r != 0) return comm_fail(nullptr, nccl_text(a, "ncclCommInitAll", r));
    for (int i = 0; i < ngpu; ++i) {
        s2v_comm* c = new (std::nothrow) s2v_comm();
        if (!c) {
            for (int k = 0; k < ngpu; ++k) {
                if (out[k]) { delete out[k]; out[k] = nullptr; }
                if (comms[k]) a->CommDestroy(comms[k]);
            }
            return S2V_ERR_CUDA;
        }
        c->nccl = comms[i];
        c->device = devs[i];
        c->rank = i;
        c->world = ngpu;
        out[i] = c;
    }
    return S2V_OK;
}

int s2v_comm_destroy(s2v_comm* comm)
{
    if (!comm) return S2V_OK;
    int rc = S2V_OK;
    const nccl_api* a = api();
    if (a && comm->nccl) {
        comm_device_guard guard(comm->device);
        const nccl_result_t r = a->CommDestroy(comm->nccl);
        if (r != 0) rc = comm_fail(nullptr, nccl_text(a, "ncclCommDestroy", r));
    }
    delete comm;
    return rc;
}

int s2v_comm_rank(const s2v_comm* comm) { return comm ? comm->rank : S2V_ERR_INVALID_ARG; }
int s2v_comm_world(const s2v_comm* comm) { return comm ? comm->world : S2V_ERR_INVALID_ARG; }

const char* s2v_comm_last_error(const s2v_comm* comm)
{
    if (comm) return comm->last_error.c_str();
    return g_global_error.c_str();
}

int s2v_allgather_rows_f32(s2v_comm* comm, s2v_stream stream, int64_t rows, int d, const float* slab, float* full)
{
    if (!comm) return S2V_ERR_INVALID_ARG;
    if (rows < 0 || d <= 0 || (rows > 0 && (!slab || !full))) {
        comm_fail(comm, "allgather_rows: bad shape or NULL pointer");
        return S2V_ERR_INVALID_ARG;
    }
    if (rows == 0) return S2V_OK;
    const nccl_api* a = api();
    if (!a) return comm_fail(comm, g_api.load_error);
    comm_device_guard guard(comm->device);
    if (!guard.ok) return S2V_ERR_CUDA;
    const nccl_result_t r = a->AllGather(slab, full, (size_t)rows * (size_t)d, NCCL_FLOAT32, comm->nccl, static_cast<cudaStream_t>(stream));
    if (r != 0) return comm_fail(comm, nccl_text(a, "ncclAllGather", r));
    return S2V_OK;
}

int s2v_exchange_rows_f32(s2v_comm* comm, s2v_stream stream, int d, const float* send, const int64_t* send_offsets,
                          float* recv, const int64_t* recv_offsets, const int64_t* recv_rows)
{
    if (!comm) return S2V_ERR_INVALID_ARG;
    if (d <= 0 || !send_offsets || !recv_offsets || !recv_rows) {
        comm_fail(comm, "exchange_rows: bad width or NULL count array");
        return S2V_ERR_INVALID_ARG;
    }
    int64_t n_send = 0, n_recv = 0;
    for (int p = 0; p < comm->world; ++p) {
        if (send_offsets[p + 1] < send_offsets[p] || send_offsets[p] < 0 || recv_rows[p] < 0 || recv_offsets[p] < 0) {
            comm_fail(comm, "exchange_rows: offsets not monotone or a negative count");
            return S2V_ERR_INVALID_ARG;
        }
        n_send += send_offsets[p + 1] - send_offsets[p];
        n_recv += recv_rows[p];
    }
    if ((n_send > 0 && !send) || (n_recv > 0 && !recv)) {
        comm_fail(comm, "exchange_rows: NULL buffer");
        return S2V_ERR_INVALID_ARG;
    }
    if (n_send == 0 && n_recv == 0) return S2V_OK;
    const nccl_api* a = api();
    if (!a) return comm_fail(comm, g_api.load_error);
    comm_device_guard guard(comm->device);
    if (!guard.ok) return S2V_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    nccl_result_t r = a->GroupStart();
    if (r != 0) return comm_fail(comm, nccl_text(a, "ncclGroupStart", r));
    nccl_result_t first_bad = 0;
    const char* bad_call = nullptr;
    for (int p = 0; p < comm->world; ++p) {
        const int64_t ns = send_offsets[p + 1] - send_offsets[p];
        if (ns > 0) {
            r = a->Send(send + send_offsets[p] * d, (size_t)ns * (size_t)d, NCCL_FLOAT32, p, comm->nccl, st);
            if (r != 0 && !first_bad) { first_bad = r; bad_call = "ncclSend"; }
        }
        if (recv_rows[p] > 0) {
            r = a->Recv(recv + recv_offsets[p] * d, (size_t)recv_rows[p] * (size_t)d, NCCL_FLOAT32, p, comm->nccl, st);
            if (r != 0 && !first_bad) { first_bad = r; bad_call = "ncclRecv"; }
        }
    }
    r = a->GroupEnd();   // always closed, so that the communicator is not left inside an open group
    if (first_bad) return comm_fail(comm, nccl_text(a, bad_call, first_bad));
    if (r != 0) return comm_fail(comm, nccl_text(a, "ncclGroupEnd", r));
    return S2V_OK;
}

int s2v_gather_logits(s2v_comm* comm, s2v_stream stream, const int64_t* graphs_per_rank, int num_class, const float* logits_local,
                      const int32_t* pred_local, float* logits_all, int32_t* pred_all)
{
    if (!comm) return S2V_ERR_INVALID_ARG;
    if (!graphs_per_rank || num_class <= 0) {
        comm_fail(comm, "gather_logits: NULL counts or bad class count");
        return S2V_ERR_INVALID_ARG;
    }
    int64_t total = 0;
    for (int r = 0; r < comm->world; ++r) {
        if (graphs_per_rank[r] < 0) {
            comm_fail(comm, "gather_logits: negative graph count");
            return S2V_ERR_INVALID_ARG;
        }
        total += graphs_per_rank[r];
    }
    if (total == 0) return S2V_OK;
    if ((logits_all && graphs_per_rank[comm->rank] > 0 && !logits_local) || (pred_all && graphs_per_rank[comm->rank] > 0 && !pred_local) ||
        (!logits_all && !pred_all)) {
        comm_fail(comm, "gather_logits: NULL buffer");
        return S2V_ERR_INVALID_ARG;
    }
    const nccl_api* a = api();
    if (!a) return comm_fail(comm, g_api.load_error);
    comm_device_guard guard(comm->device);
    if (!guard.ok) return S2V_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // ragged all-gather: one broadcast rooted at every rank, all in one group (one fused NCCL launch)
    nccl_result_t r = a->GroupStart();
    if (r != 0) return comm_fail(comm, nccl_text(a, "ncclGroupStart", r));
    nccl_result_t first_bad = 0;
    const char* bad_call = nullptr;
    int64_t off = 0;
    for (int root = 0; root < comm->world; ++root) {
        const int64_t g = graphs_per_rank[root];
        if (g > 0) {
            if (logits_all) {
                // (ranks other than the root pass the receive address as the unused send address: a valid pointer)
                r = a->Broadcast(root == comm->rank ? logits_local : logits_all + off * num_class, logits_all + off * num_class, (size_t)g * (size_t)num_class,
                                 NCCL_FLOAT32, root, comm->nccl, st);
                if (r != 0 && !first_bad) { first_bad = r; bad_call = "ncclBroadcast(logits)"; }
            }
            if (pred_all) {
                r = a->Broadcast(root == comm->rank ? pred_local : pred_all + off, pred_all + off, (size_t)g, NCCL_INT32, root, comm->nccl, st);
                if (r != 0 && !first_bad) { first_bad = r; bad_call = "ncclBroadcast(pred)"; }
            }
        }
        off += g;
    }
    r = a->GroupEnd();   // always closed, so that the communicator is not left inside an open group
    if (first_bad) return comm_fail(comm, nccl_text(a, bad_call, first_bad));
    if (r != 0) return comm_fail(comm, nccl_text(a, "ncclGroupEnd", r));
    return S2V_OK;
}

}  // extern "C"
