// NCCL communicator behind the C ABI: the one collective of the attention path, the all-gather of
// the per-GPU partials of the KV-sharded decode, followed by the log-sum-exp merge.
//
// The reference has no communication backend at all; these entry points exist so that the sharded
// decode needs no framework around it -- one process per GPU, each with a grl_device and a
// grl_group.  libnccl is opened at run time (dlopen of "libnccl.so.2"): the library stays loadable on
// a machine without NCCL, and inside a process that has already loaded an NCCL (under the same
// soname) that copy is the one used.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <thread>

#include "common.cuh"

struct grl_group {
    ncclComm_t comm = nullptr;
    grl_device* dev = nullptr;
    int rank = 0, world = 1;
    bool aborted = false;
};

namespace grl {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
    bool ok = false;
    char why[256] = "";
};

static NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            snprintf(api.why, sizeof(api.why), "libnccl.so.2 could not be opened: %s", dlerror());
            return;
        }
        bool all = true;
        auto sym = [&](const char* name) {
            void* p = dlsym(h, name);
            if (!p) { all = false; snprintf(api.why, sizeof(api.why), "libnccl lacks %s", name); }
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
        api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(sym("ncclGetVersion"));
        api.ok = all;
    });
    return api;
}

#define GRL_NCCL(call)                                                                                      \
    do {                                                                                                    \
        ncclResult_t _r = (call);                                                                           \
        if (_r != ncclSuccess)                                                                              \
            return set_error(GRL_ERR_CUDA, "%s failed: %s", #call, nccl().GetErrorString(_r));             \
    } while (0)

static int need_nccl() {
    if (!nccl().ok) return set_error(GRL_ERR_UNSUPPORTED, "NCCL is not available: %s", nccl().why);
    return GRL_OK;
}

}  // namespace grl

using namespace grl;

extern "C" {

int grl_group_unique_id(void* id_out_128_bytes) {
    GRL_REQUIRE(id_out_128_bytes, "NULL argument");
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    int rc = need_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    GRL_NCCL(nccl().GetUniqueId(&id));
    memcpy(id_out_128_bytes, &id, sizeof(id));
    return GRL_OK;
}

int grl_group_init_rank(grl_device* dev, const void* id_128_bytes, int rank, int world, grl_group** out) {
    GRL_REQUIRE(dev && id_128_bytes && out, "NULL argument");
    GRL_REQUIRE(world >= 1 && rank >= 0 && rank < world, "bad rank %d / world %d", rank, world);
    int rc = need_nccl();
    if (rc) return rc;
    DeviceGuard g(dev->ordinal);
    ncclUniqueId id;
    memcpy(&id, id_128_bytes, sizeof(id));
    grl_group* grp = new grl_group();
    grp->dev = dev; grp->rank = rank; grp->world = world;
    ncclResult_t r = nccl().CommInitRank(&grp->comm, world, id, rank);
    if (r != ncclSuccess) {
        delete grp;
        return set_error(GRL_ERR_CUDA, "ncclCommInitRank failed: %s", nccl().GetErrorString(r));
    }
    *out = grp;
    return GRL_OK;
}

int grl_group_info(grl_group* g, int* rank, int* world, int* nccl_version) {
    GRL_REQUIRE(g, "group is NULL");
    if (rank) *rank = g->rank;
    if (world) *world = g->world;
    if (nccl_version) {
        *nccl_version = 0;
        if (nccl().ok) nccl().GetVersion(nccl_version);
    }
    return GRL_OK;
}

int grl_group_allgather(grl_group* g, const void* send, void* recv, size_t bytes_per_rank) {
    GRL_REQUIRE(g && g->comm && !g->aborted, "group is not usable");
    GRL_REQUIRE(send && recv, "NULL buffer");
    DeviceGuard dg(g->dev->ordinal);
    GRL_NCCL(nccl().AllGather(send, recv, bytes_per_rank, ncclInt8, g->comm, g->dev->stream));
    return GRL_OK;
}

int grl_group_allreduce_max_f64(grl_group* g, double* inout_device, size_t n) {
    GRL_REQUIRE(g && g->comm && !g->aborted, "group is not usable");
    GRL_REQUIRE(inout_device, "NULL buffer");
    DeviceGuard dg(g->dev->ordinal);
    GRL_NCCL(nccl().AllReduce(inout_device, inout_device, n, ncclFloat64, ncclMax, g->comm, g->dev->stream));
    return GRL_OK;
}

// Waits for the group's stream like grl_sync, looking at the communicator's asynchronous state while it
// waits: a remote failure or the time limit aborts the communicator (ncclCommAbort) so that the kernel
// that waits for a peer which will never come is torn down instead of blocking the stream.
int grl_group_sync(grl_group* g, uint64_t timeout_ns) {
    GRL_REQUIRE(g && g->comm, "group is NULL");
    DeviceGuard dg(g->dev->ordinal);
    if (g->aborted) return set_error(GRL_ERR_CUDA, "the communicator was aborted after an earlier failure");
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        ncclResult_t async = ncclSuccess;
        ncclResult_t r = nccl().CommGetAsyncError(g->comm, &async);
        if (r != ncclSuccess || (async != ncclSuccess && async != ncclInProgress)) {
            nccl().CommAbort(g->comm);
            g->aborted = true;
            return set_error(GRL_ERR_CUDA, "NCCL reported %s; the communicator was aborted",
                             nccl().GetErrorString(r != ncclSuccess ? r : async));
        }
        cudaError_t e = cudaStreamQuery(g->dev->stream);
        if (e == cudaSuccess) return grl_sync(g->dev, 0);     // done: collect the kernels' status word too
        if (e != cudaErrorNotReady) return set_error(GRL_ERR_CUDA, "stream failed: %s", cudaGetErrorString(e));
        const uint64_t ns = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
                                std::chrono::steady_clock::now() - t0).count();
        if (timeout_ns && ns > timeout_ns) {
            nccl().CommAbort(g->comm);
            g->aborted = true;
            return set_error(GRL_ERR_TIMEOUT, "collective did not finish within %llu ns; the communicator was aborted",
                             (unsigned long long)timeout_ns);
        }
        if (ns > 500000) std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
}

int grl_group_allgather_merge(grl_group* g, const float* partial, int rows, int head_dim, float* gather_buf,
                              float* out, uint64_t timeout_ns) {
    GRL_REQUIRE(g && g->comm && !g->aborted, "group is not usable");
    GRL_REQUIRE(partial && gather_buf && out, "NULL buffer");
    GRL_REQUIRE(rows > 0 && head_dim > 0, "bad shape");
    const size_t n = (size_t)rows * (head_dim + 2);
    DeviceGuard dg(g->dev->ordinal);
    if (g->world == 1) {
        int rc = grl_lse_merge(g->dev, partial, 1, n, rows, head_dim, 1, out);
        if (rc || !timeout_ns) return rc;
        return grl_sync(g->dev, timeout_ns);
    }
    GRL_NCCL(nccl().AllGather(partial, gather_buf, n, ncclFloat32, g->comm, g->dev->stream));
    int rc = grl_lse_merge(g->dev, gather_buf, g->world, n, rows, head_dim, 1, out);
    if (rc || !timeout_ns) return rc;
    return grl_group_sync(g, timeout_ns);
}

int grl_group_destroy(grl_group* g) {
    if (!g) return GRL_OK;
    if (g->comm && nccl().ok) {
        DeviceGuard dg(g->dev->ordinal);
        if (g->aborted) { /* already torn down by ncclCommAbort */ }
        else {
            cudaStreamSynchronize(g->dev->stream);
            nccl().CommDestroy(g->comm);
        }
    }
    delete g;
    return GRL_OK;
}

}  // extern "C"
