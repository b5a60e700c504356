// NCCL through dlopen: the library has no link-time dependency on NCCL, and a process that already carries
// one (a PyTorch host) shares that copy instead of loading a second one.  Only the handful of calls the
// tensor-parallel decode step needs are bound.
#include <dlfcn.h>
#include <string.h>

#include "vb_internal.cuh"
#include "vb_nccl.h"

namespace vb {

namespace {
struct NcclApi {
    void* so = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
} g_nccl;

bool load_api() {
    if (g_nccl.ok) return true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        g_nccl.so = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.so) break;
    }
    if (!g_nccl.so) { set_error("NCCL not found (dlopen libnccl.so.2: %s)", dlerror()); return false; }
#define VB_SYM(field, name) *(void**)(&g_nccl.field) = dlsym(g_nccl.so, name); if (!g_nccl.field) { set_error("NCCL symbol %s missing", name); return false; }
    VB_SYM(GetUniqueId, "ncclGetUniqueId");
    VB_SYM(CommInitRank, "ncclCommInitRank");
    VB_SYM(CommDestroy, "ncclCommDestroy");
    VB_SYM(AllReduce, "ncclAllReduce");
    VB_SYM(AllGather, "ncclAllGather");
    VB_SYM(GetErrorString, "ncclGetErrorString");
#undef VB_SYM
    g_nccl.ok = true;
    return true;
}

int32_t nccl_fail(int rc, const char* what) {
    set_error("NCCL error %d (%s) in %s", rc, g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?", what);
    return VB_ERR_COMM;
}
}  // namespace

int32_t nccl_unique_id(NcclUniqueId* id) {
    if (!load_api()) return VB_ERR_COMM;
    const int rc = g_nccl.GetUniqueId(id);
    return rc == 0 ? VB_OK : nccl_fail(rc, "ncclGetUniqueId");
}

int32_t nccl_comm_init(void** comm, int n_ranks, const NcclUniqueId* id, int rank) {
    if (!load_api()) return VB_ERR_COMM;
    const int rc = g_nccl.CommInitRank(comm, n_ranks, *id, rank);
    return rc == 0 ? VB_OK : nccl_fail(rc, "ncclCommInitRank");
}

void nccl_comm_destroy(void* comm) {
    if (comm && g_nccl.ok) g_nccl.CommDestroy(comm);
}

// ncclFloat32 = 7, ncclUint8 = 1, ncclSum = 0 (nccl.h; stable across NCCL 2.x)
int32_t nccl_allreduce_sum_f32(void* comm, float* buf, size_t count, cudaStream_t stream) {
    const int rc = g_nccl.AllReduce(buf, buf, count, 7, 0, comm, stream);
    return rc == 0 ? VB_OK : nccl_fail(rc, "ncclAllReduce");
}

int32_t nccl_allgather_bytes(void* comm, const void* send, void* recv, size_t bytes_per_rank, cudaStream_t stream) {
    const int rc = g_nccl.AllGather(send, recv, bytes_per_rank, 1, comm, stream);
    return rc == 0 ? VB_OK : nccl_fail(rc, "ncclAllGather");
}

}  // namespace vb
