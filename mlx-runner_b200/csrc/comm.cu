// Output-row sharding across GPUs: an NCCL communicator (one process per GPU) and the shard forward
// that all-gathers the fp32 output slices.  NCCL is bound at first use with dlopen so that libmlxq
// loads on hosts without it and shares the copy a host process (e.g. PyTorch) has already loaded.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <new>

#include "../../include/mlxq.h"
#include "api_internal.h"

namespace {

// The slice of nccl.h this file needs (stable across NCCL 2.x).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclSuccess = 0 };
enum { ncclFloat32 = 7 };

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    const char* (*GetErrorString)(ncclResult_t);
    bool ok = false;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

const NcclApi& nccl() {
    std::call_once(g_nccl_once, [] {
        void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) return;
        g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
        g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
        g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
        g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(dlsym(lib, "ncclAllGather"));
        g_nccl.GroupStart = reinterpret_cast<decltype(g_nccl.GroupStart)>(dlsym(lib, "ncclGroupStart"));
        g_nccl.GroupEnd = reinterpret_cast<decltype(g_nccl.GroupEnd)>(dlsym(lib, "ncclGroupEnd"));
        g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
        g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.AllGather &&
                    g_nccl.GroupStart && g_nccl.GroupEnd && g_nccl.GetErrorString;
    });
    return g_nccl;
}

int nccl_fail(ncclResult_t r, const char* what) {
    return mlxq::fail(MLXQ_NCCL_FAILURE, "%s: %s", what, nccl().GetErrorString(r));
}

}  // namespace

struct mlxq_comm {
    ncclComm_t comm;
    int rank, size, device;
};

static_assert(sizeof(ncclUniqueId) == MLXQ_COMM_ID_BYTES, "rendezvous token size");

extern "C" {

int mlxq_comm_unique_id(uint8_t id[MLXQ_COMM_ID_BYTES]) {
    if (!id) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "null id");
    if (!nccl().ok) return mlxq::fail(MLXQ_NCCL_FAILURE, "libnccl.so.2 could not be loaded");
    ncclUniqueId u;
    ncclResult_t r = nccl().GetUniqueId(&u);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(id, &u, sizeof u);
    return MLXQ_OK;
}

int mlxq_comm_create(const uint8_t id[MLXQ_COMM_ID_BYTES], int rank, int nranks, int device, mlxq_comm_t* out) {
    if (!out) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (nranks < 1 || rank < 0 || rank >= nranks) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "rank %d of %d", rank, nranks);
    auto* c = new (std::nothrow) mlxq_comm{nullptr, rank, nranks, device};
    if (!c) return mlxq::fail(MLXQ_OUT_OF_MEMORY, "communicator allocation");
    if (nranks > 1) {
        if (!id) { delete c; return mlxq::fail(MLXQ_INVALID_ARGUMENT, "null id"); }
        if (!nccl().ok) { delete c; return mlxq::fail(MLXQ_NCCL_FAILURE, "libnccl.so.2 could not be loaded"); }
        cudaError_t ce = cudaSetDevice(device);
        if (ce != cudaSuccess) { delete c; return mlxq::cuda_fail(ce, "cudaSetDevice"); }
        ncclUniqueId u;
        memcpy(&u, id, sizeof u);
        ncclResult_t r = nccl().CommInitRank(&c->comm, nranks, u, rank);
        if (r != ncclSuccess) { delete c; return nccl_fail(r, "ncclCommInitRank"); }
    }
    *out = c;
    return MLXQ_OK;
}

void mlxq_comm_destroy(mlxq_comm_t c) {
    if (!c) return;
    if (c->comm) nccl().CommDestroy(c->comm);
    delete c;
}

int mlxq_comm_rank(mlxq_comm_t c) { return c ? c->rank : -1; }
int mlxq_comm_size(mlxq_comm_t c) { return c ? c->size : 0; }

int mlxq_linear_forward_gather(mlxq_linear_t h, mlxq_comm_t c, mlxq_stream_t stream, const void* x, int x_dtype,
                               int64_t x_stride, float* y, int64_t y_stride, int64_t T) {
    if (!h || !c) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (h->shard_count != c->size || h->shard_rank != c->rank)
        return mlxq::fail(MLXQ_INVALID_ARGUMENT, "layer is shard %d of %d but the communicator is rank %d of %d",
                          h->shard_rank, h->shard_count, c->rank, c->size);
    if (!y) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "y is null");
    if (T > 1 && y_stride < h->total_out) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "y stride %lld < %lld rows", (long long)y_stride, (long long)h->total_out);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // This rank's rows land at their place in the full output, then the slices are gathered in place.
    int rc = mlxq::forward_impl(h, st, x, x_dtype, x_stride, y + h->row_offset, MLXQ_F32, y_stride, T);
    if (rc != MLXQ_OK || c->size == 1) return rc;
    const NcclApi& n = nccl();
    ncclResult_t r = n.GroupStart();
    if (r != ncclSuccess) return nccl_fail(r, "ncclGroupStart");
    for (int64_t t = 0; t < T; t++) {
        float* row = y + static_cast<size_t>(t) * y_stride;
        r = n.AllGather(row + h->row_offset, row, static_cast<size_t>(h->out_dim), ncclFloat32, c->comm, st);
        if (r != ncclSuccess) { n.GroupEnd(); return nccl_fail(r, "ncclAllGather"); }
    }
    r = n.GroupEnd();
    if (r != ncclSuccess) return nccl_fail(r, "ncclGroupEnd");
    return MLXQ_OK;
}

}  // extern "C"
