/* A stand-in for libnccl used ONLY by the CPU tests of the s2v_comm_* entry points (test infrastructure).
 * World size 1, host pointers: collectives are memcpy.  The environment variable FAKE_NCCL_FAIL names one
 * entry point and the status it must return ("ncclAllGather:5"), which is how the tests inject a failing
 * NCCL call on the host without any GPU. */
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;
typedef int ncclResult_t;

static int fail_code(const char* fn)
{
    const char* e = getenv("FAKE_NCCL_FAIL");
    if (!e) return 0;
    size_t n = strlen(fn);
    if (strncmp(e, fn, n) == 0 && e[n] == ':') return atoi(e + n + 1);
    return 0;
}

static size_t type_size(int t) { return (t == 0 || t == 1) ? 1 : ((t == 6 || t == 9) ? 2 : ((t == 4 || t == 5 || t == 8) ? 8 : 4)); }

static int group_depth = 0;
int fake_nccl_group_depth(void) { return group_depth; }

ncclResult_t ncclGetUniqueId(ncclUniqueId* id)
{
    int f = fail_code("ncclGetUniqueId");
    if (f) return f;
    for (int i = 0; i < 128; ++i) id->internal[i] = (char)(i * 7 + 1);
    return 0;
}
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int n, ncclUniqueId id, int rank)
{
    int f = fail_code("ncclCommInitRank");
    if (f) return f;
    if (id.internal[1] != (char)8 || rank >= n) return 4; /* invalid argument */
    *comm = malloc(16);
    return 0;
}
ncclResult_t ncclCommInitAll(ncclComm_t* comms, int n, const int* devs)
{
    int f = fail_code("ncclCommInitAll");
    if (f) return f;
    (void)devs;
    for (int i = 0; i < n; ++i) comms[i] = malloc(16);
    return 0;
}
ncclResult_t ncclCommDestroy(ncclComm_t comm)
{
    free(comm);
    return fail_code("ncclCommDestroy");
}
ncclResult_t ncclAllGather(const void* send, void* recv, size_t count, int type, ncclComm_t comm, void* stream)
{
    int f = fail_code("ncclAllGather");
    (void)comm; (void)stream;
    if (f) return f;
    if (send != recv) memmove(recv, send, count * type_size(type));
    return 0;
}
ncclResult_t ncclBroadcast(const void* send, void* recv, size_t count, int type, int root, ncclComm_t comm, void* stream)
{
    int f = fail_code("ncclBroadcast");
    (void)comm; (void)stream; (void)root;
    if (f) return f;
    if (send != recv) memmove(recv, send, count * type_size(type));
    return 0;
}
/* send / receive with the only peer there is (rank 0 itself): whichever of the pair comes second does the copy */
static const void* pending_send = NULL;
static void* pending_recv = NULL;
static size_t pending_bytes = 0;
ncclResult_t ncclSend(const void* send, size_t count, int type, int peer, ncclComm_t comm, void* stream)
{
    int f = fail_code("ncclSend");
    (void)comm; (void)stream;
    if (f) return f;
    if (peer != 0) return 4;
    if (pending_recv) { memmove(pending_recv, send, count * type_size(type)); pending_recv = NULL; }
    else { pending_send = send; pending_bytes = count * type_size(type); }
    return 0;
}
ncclResult_t ncclRecv(void* recv, size_t count, int type, int peer, ncclComm_t comm, void* stream)
{
    int f = fail_code("ncclRecv");
    (void)comm; (void)stream;
    if (f) return f;
    if (peer != 0) return 4;
    if (pending_send) { memmove(recv, pending_send, count * type_size(type) < pending_bytes ? count * type_size(type) : pending_bytes); pending_send = NULL; }
    else pending_recv = recv;
    return 0;
}
ncclResult_t ncclGroupStart(void)
{
    int f = fail_code("ncclGroupStart");
    if (f) return f;
    ++group_depth;
    return 0;
}
ncclResult_t ncclGroupEnd(void)
{
    --group_depth;
    return fail_code("ncclGroupEnd");
}
const char* ncclGetErrorString(ncclResult_t r)
{
    switch (r) {
        case 0: return "no error";
        case 1: return "unhandled cuda error";
        case 2: return "unhandled system error";
        case 3: return "internal error";
        case 4: return "invalid argument";
        case 5: return "invalid usage";
        case 6: return "remote process exited or there was a network error";
        default: return "unknown result code";
    }
}
