// psk_comm_*: the one exchange step of the sharded path, for a caller that is not Python.
//
// The forward pass shards by the batch axis with no data-path collective; what the ranks exchange is
// a few words at the end of a call: the loss (a sum of per-rank means) and, under `presk calibrate`,
// each site's magnitudes (a maximum and a minimum). The reference has no collective of its own (its
// executors are single-process); these entry points are what its `Backend` for several GPUs would call
// where a single-GPU one reads a scalar back (presk-kernel/src/host.rs:1584, 1844).
//
// NCCL is found at run time (dlopen of libnccl.so.2), so that a process that already holds a copy of it
// (PyTorch's) shares that copy, and the library builds where NCCL is absent. Only five functions of
// NCCL's public API are used; their signatures are restated below.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <cstring>
#include <string>

#include "../../include/presk_cuda.h"

namespace {

struct NcclId { char bytes[128]; }; // ncclUniqueId: 128 opaque bytes
typedef int (*GetUniqueIdFn)(NcclId *);
typedef int (*CommInitRankFn)(void **comm, int nranks, NcclId id, int rank);
typedef int (*AllReduceFn)(const void *send, void *recv, size_t count, int dtype, int op, void *comm, cudaStream_t stream);
typedef int (*CommDestroyFn)(void *comm);
typedef const char *(*GetErrorStringFn)(int);

struct Nccl {
    void *lib = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    AllReduceFn all_reduce = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GetErrorStringFn get_error_string = nullptr;
    std::string error;
};

Nccl &nccl()
{
    static Nccl n;
    if (n.lib || !n.error.empty()) return n;
    n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) { n.error = std::string("NCCL is not available: ") + dlerror(); return n; }
    n.get_unique_id = (GetUniqueIdFn)dlsym(n.lib, "ncclGetUniqueId");
    n.comm_init_rank = (CommInitRankFn)dlsym(n.lib, "ncclCommInitRank");
    n.all_reduce = (AllReduceFn)dlsym(n.lib, "ncclAllReduce");
    n.comm_destroy = (CommDestroyFn)dlsym(n.lib, "ncclCommDestroy");
    n.get_error_string = (GetErrorStringFn)dlsym(n.lib, "ncclGetErrorString");
    if (!n.get_unique_id || !n.comm_init_rank || !n.all_reduce || !n.comm_destroy || !n.get_error_string) {
        n.error = "libnccl.so.2 lacks a function this library calls";
        n.lib = nullptr;
    }
    return n;
}

thread_local std::string g_comm_error;

} // namespace

struct psk_comm {
    void *comm = nullptr;
    psk_exec *exec = nullptr;
    int nranks = 1, rank = 0;
    std::string error;
};

extern "C" {

int psk_comm_unique_id(uint8_t id[PSK_COMM_ID_BYTES])
{
    Nccl &n = nccl();
    if (!n.lib) { g_comm_error = n.error; return PSK_E10001; }
    NcclId u;
    int r = n.get_unique_id(&u);
    if (r != 0) { g_comm_error = std::string("ncclGetUniqueId: ") + n.get_error_string(r); return PSK_E10001; }
    memcpy(id, u.bytes, PSK_COMM_ID_BYTES);
    return PSK_OK;
}

psk_comm *psk_comm_create(psk_exec *e, int32_t nranks, int32_t rank, const uint8_t id[PSK_COMM_ID_BYTES])
{
    Nccl &n = nccl();
    if (!n.lib) { g_comm_error = n.error; return nullptr; }
    if (!e || nranks < 1 || rank < 0 || rank >= nranks) { g_comm_error = "psk_comm_create: an executor, and a rank below the number of ranks"; return nullptr; }
    psk_exec_sync(e); // also selects the executor's device for this thread
    NcclId u;
    memcpy(u.bytes, id, PSK_COMM_ID_BYTES);
    psk_comm *c = new psk_comm;
    c->exec = e; c->nranks = nranks; c->rank = rank;
    int r = n.comm_init_rank(&c->comm, nranks, u, rank);
    if (r != 0) {
        g_comm_error = std::string("ncclCommInitRank: ") + n.get_error_string(r);
        delete c;
        return nullptr;
    }
    return c;
}

void psk_comm_destroy(psk_comm *c)
{
    if (!c) return;
    if (c->comm) {
        psk_exec_sync(c->exec);
        nccl().comm_destroy(c->comm);
    }
    delete c;
}

const char *psk_comm_error(const psk_comm *c) { return c ? c->error.c_str() : g_comm_error.c_str(); }

int psk_comm_allreduce(psk_comm *c, void *device_buf, int64_t count, int32_t dtype, int32_t op)
{
    if (!c || !c->comm) return PSK_E10001;
    // NCCL's ncclDataType_t and ncclRedOp_t: uint32 3, int64 4, float16 6, float32 7, float64 8, bfloat16 9; sum 0, max 2, min 3
    int nd;
    switch (dtype) {
    case PSK_F32: nd = 7; break;
    case PSK_F64: nd = 8; break;
    case PSK_F16: nd = 6; break;
    case PSK_BF16: nd = 9; break;
    case PSK_I64: nd = 4; break;
    case PSK_COMM_U32: nd = 3; break;
    default: c->error = "psk_comm_allreduce: f32, f64, bf16, f16, i64 or raw 32-bit words"; return PSK_E7001;
    }
    int no;
    switch (op) {
    case PSK_COMM_SUM: no = 0; break;
    case PSK_COMM_MAX: no = 2; break;
    case PSK_COMM_MIN: no = 3; break;
    default: c->error = "psk_comm_allreduce: sum, max or min"; return PSK_E7001;
    }
    if (count < 0) { c->error = "psk_comm_allreduce: a negative count"; return PSK_E7001; }
    if (count == 0) return PSK_OK;
    int r = nccl().all_reduce(device_buf, device_buf, (size_t)count, nd, no, c->comm, (cudaStream_t)psk_exec_stream(c->exec));
    if (r != 0) { c->error = std::string("ncclAllReduce: ") + nccl().get_error_string(r); return PSK_E10001; }
    return PSK_OK;
}

int32_t psk_comm_rank(const psk_comm *c) { return c ? c->rank : 0; }
int32_t psk_comm_size(const psk_comm *c) { return c ? c->nranks : 1; }

} // extern "C"
