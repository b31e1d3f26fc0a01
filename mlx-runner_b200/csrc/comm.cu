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
#include "aux_kernels.cuh"

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

// The gather window: two buffers of `bytes` each (calls alternate between them, so a rank that runs ahead
// never overwrites rows a slower rank's next kernels still read), mapped into every peer through CUDA IPC,
// plus one flag word per rank (its calls whose rows are complete), a CTA counter and the count of completed calls.
struct GatherWindow {
    char* local = nullptr;
    char* peer[mlxq::MAX_PEERS + 1] = {};        // by rank; [rank] == local
    unsigned* flags = nullptr;                   // this rank's flag array
    unsigned* peer_flags[mlxq::MAX_PEERS + 1] = {};
    unsigned* counter = nullptr;
    unsigned* epoch_ctr = nullptr;               // completed fused calls, kept on the device (see PeerGather::epoch_ctr)
    size_t bytes = 0;
    unsigned epoch = 0;
};

struct mlxq_comm {
    ncclComm_t comm;
    int rank, size, device;
    GatherWindow win;
};

namespace {

// The flag words of the other ranks' arrays (this rank's word in each), by rank.
struct PeerFlags {
    unsigned* flag[mlxq::MAX_PEERS + 1];
};

// One warp.  First lane p publishes this rank's completed fused calls in rank p's flag array (the calls' kernels do
// not publish themselves: the next kernel of the communicator on the rank does, and after the last call that is this
// one -- the grids that stored the rows are complete here, so one release store covers them).  Then lane p waits
// (bounded, two seconds) until peer p's word in this rank's array has reached the same number.  The number is read
// from the device, so that the launch can be replayed from a graph.
__global__ void gather_wait_kernel(const unsigned* my_flags, PeerFlags peers, int rank, int nranks, const unsigned* epoch_ctr, unsigned* err) {
    const int p = threadIdx.x;
    if (p >= nranks || p == rank) return;
    const unsigned epoch = *reinterpret_cast<const volatile unsigned*>(epoch_ctr);
    if (epoch == 0u) return;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flag[p] + rank), "r"(epoch) : "memory");
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        unsigned seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(my_flags + p) : "memory");
        if (static_cast<int>(seen - epoch) >= 0) return;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > 2000000000ull) { atomicOr(err, 2u | 8u); return; }     // ERR_WAIT_TIMEOUT | ERR_PEER_FLAG
    }
}

struct IpcPair {
    cudaIpcMemHandle_t window, flags;
};

void close_window(mlxq_comm* c) {
    GatherWindow& w = c->win;
    for (int r = 0; r < c->size && r <= mlxq::MAX_PEERS; r++) {
        if (r == c->rank) continue;
        if (w.peer[r]) cudaIpcCloseMemHandle(w.peer[r]);
        if (w.peer_flags[r]) cudaIpcCloseMemHandle(w.peer_flags[r]);
    }
    if (w.local) cudaFree(w.local);
    if (w.flags) cudaFree(w.flags);
    w = GatherWindow();
}

}  // namespace

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
    auto* c = new (std::nothrow) mlxq_comm{nullptr, rank, nranks, device, GatherWindow()};
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
    close_window(c);
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

int mlxq_linear_forward_blockmax_gather(mlxq_linear_t h, mlxq_comm_t c, mlxq_stream_t stream, const void* x, int x_dtype,
                                        int64_t x_stride, int64_t T, float* y_local, uint32_t* pairs) {
    if (!h || !c || !y_local || !pairs) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (h->shard_count != c->size || h->shard_rank != c->rank)
        return mlxq::fail(MLXQ_INVALID_ARGUMENT, "layer is shard %d of %d but the communicator is rank %d of %d",
                          h->shard_rank, h->shard_count, c->rank, c->size);
    if (h->out_dim * c->size != h->total_out)
        return mlxq::fail(MLXQ_UNSUPPORTED, "shards of unequal size (%lld rows of %lld on %d ranks)", (long long)h->out_dim, (long long)h->total_out, c->size);
    if (T < 1 || h->total_out > 0x7fffff00ll) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "T %lld, %lld rows", (long long)T, (long long)h->total_out);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = mlxq::forward_impl(h, st, x, x_dtype, x_stride, y_local, MLXQ_F32, h->out_dim, T);
    if (rc != MLXQ_OK) return rc;
    const int64_t nb = (h->out_dim + mlxq::SELECT_BLOCK - 1) / mlxq::SELECT_BLOCK;
    const size_t seg = static_cast<size_t>(2) * T * nb;
    uint32_t* mine = pairs + seg * c->rank;
    cudaError_t e = mlxq::launch_block_max(y_local, h->out_dim, h->out_dim, T, static_cast<int>(h->row_offset), mine, st);
    if (e != cudaSuccess) return mlxq::cuda_fail(e, "block maxima launch");
    if (c->size == 1) return MLXQ_OK;
    ncclResult_t r = nccl().AllGather(mine, pairs, seg, ncclFloat32, c->comm, st);      // (raw 4-byte words)
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllGather (block maxima)");
    return MLXQ_OK;
}

int mlxq_comm_window(mlxq_comm_t c, size_t bytes) {
    if (!c) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "null communicator");
    if (bytes == 0 || bytes % 256 != 0) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "window size %zu is not a positive multiple of 256", bytes);
    if (c->size > mlxq::MAX_PEERS + 1) return mlxq::fail(MLXQ_UNSUPPORTED, "%d ranks: the fused gather serves up to %d", c->size, mlxq::MAX_PEERS + 1);
    if (c->win.local) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "the communicator already has a window");
    cudaError_t e = cudaSetDevice(c->device);
    if (e != cudaSuccess) return mlxq::cuda_fail(e, "cudaSetDevice");
    GatherWindow& w = c->win;
    // flags: a word per rank (0-7), the CTA counter (32), completed calls (40)
    if ((e = cudaMalloc(&w.local, 2 * bytes)) != cudaSuccess) return mlxq::cuda_fail(e, "window allocation");
    if ((e = cudaMalloc(&w.flags, 256)) != cudaSuccess) { close_window(c); return mlxq::cuda_fail(e, "flag allocation"); }
    cudaMemset(w.local, 0, 2 * bytes);
    cudaMemset(w.flags, 0, 256);
    w.counter = w.flags + 32;
    w.epoch_ctr = w.flags + 40;
    w.bytes = bytes;
    w.peer[c->rank] = w.local;
    w.peer_flags[c->rank] = w.flags;
    if (c->size == 1) return cudaDeviceSynchronize() == cudaSuccess ? MLXQ_OK : mlxq::fail(MLXQ_GPU_FAILURE, "window set-up");
    // exchange the IPC handles with an all-gather on the communicator itself
    IpcPair mine;
    if ((e = cudaIpcGetMemHandle(&mine.window, w.local)) != cudaSuccess || (e = cudaIpcGetMemHandle(&mine.flags, w.flags)) != cudaSuccess) {
        close_window(c);
        return mlxq::cuda_fail(e, "cudaIpcGetMemHandle");
    }
    IpcPair* dev = nullptr;
    IpcPair all[mlxq::MAX_PEERS + 1];
    if ((e = cudaMalloc(&dev, sizeof(IpcPair) * (c->size + 1))) != cudaSuccess) { close_window(c); return mlxq::cuda_fail(e, "handle staging"); }
    cudaMemcpy(dev + c->size, &mine, sizeof mine, cudaMemcpyHostToDevice);
    ncclResult_t r = nccl().AllGather(dev + c->size, dev, sizeof(IpcPair), /*ncclInt8*/ 0, c->comm, nullptr);
    if (r == ncclSuccess) e = cudaStreamSynchronize(nullptr);
    if (r == ncclSuccess && e == cudaSuccess) e = cudaMemcpy(all, dev, sizeof(IpcPair) * c->size, cudaMemcpyDeviceToHost);
    cudaFree(dev);
    if (r != ncclSuccess) { close_window(c); return nccl_fail(r, "handle exchange"); }
    if (e != cudaSuccess) { close_window(c); return mlxq::cuda_fail(e, "handle exchange"); }
    for (int p = 0; p < c->size; p++) {
        if (p == c->rank) continue;
        void* a = nullptr;
        void* b = nullptr;
        if ((e = cudaIpcOpenMemHandle(&a, all[p].window, cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess ||
            (e = cudaIpcOpenMemHandle(&b, all[p].flags, cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess) {
            if (a) cudaIpcCloseMemHandle(a);
            close_window(c);
            return mlxq::cuda_fail(e, "cudaIpcOpenMemHandle (peer window)");
        }
        w.peer[p] = static_cast<char*>(a);
        w.peer_flags[p] = static_cast<unsigned*>(b);
    }
    return MLXQ_OK;
}

int mlxq_linear_forward_gather_fused(mlxq_linear_t h, mlxq_comm_t c, mlxq_stream_t stream, const void* x, int x_dtype,
                                     int64_t x_stride, int64_t T, float** y_full) {
    if (!h || !c || !y_full) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "null argument");
    *y_full = nullptr;
    if (h->shard_count != c->size || h->shard_rank != c->rank)
        return mlxq::fail(MLXQ_INVALID_ARGUMENT, "layer is shard %d of %d but the communicator is rank %d of %d",
                          h->shard_rank, h->shard_count, c->rank, c->size);
    GatherWindow& w = c->win;
    if (!w.local) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "the communicator has no window (mlxq_comm_window)");
    if (T < 1 || static_cast<unsigned long long>(T) * h->total_out * 4ull > w.bytes)
        return mlxq::fail(MLXQ_INVALID_ARGUMENT, "%lld tokens x %lld rows do not fit the %zu-byte window", (long long)T, (long long)h->total_out, w.bytes);
    const unsigned epoch = w.epoch + 1;
    const size_t half = (epoch & 1u) * w.bytes;
    float* y = reinterpret_cast<float*>(w.local + half);
    mlxq::PeerGather pg = {};
    pg.rank = c->rank;
    pg.epoch = epoch;
    pg.my_flags = w.flags;
    pg.counter = w.counter;
    pg.epoch_ctr = w.epoch_ctr;
    {
        const char* xp = static_cast<const char*>(x);
        pg.x_is_gathered = (xp >= w.local && xp < w.local + 2 * w.bytes) ? 1 : 0;
    }
    for (int p = 0; p < c->size; p++) {
        if (p == c->rank) continue;
        pg.y[pg.n] = w.peer[p] + half + static_cast<size_t>(h->row_offset) * 4;
        pg.flag[pg.n] = w.peer_flags[p];
        pg.peer_rank[pg.n] = p;
        pg.n++;
    }
    int rc = mlxq::forward_impl(h, static_cast<cudaStream_t>(stream), x, x_dtype, x_stride, y + h->row_offset, MLXQ_F32,
                                h->total_out, T, c->size > 1 ? &pg : nullptr);
    if (rc != MLXQ_OK) return rc;
    w.epoch = epoch;          // only calls that were enqueued count: every rank takes the same decision for a shape
    *y_full = y;
    return MLXQ_OK;
}

int mlxq_comm_wait(mlxq_comm_t c, mlxq_stream_t stream) {
    if (!c) return mlxq::fail(MLXQ_INVALID_ARGUMENT, "null communicator");
    if (c->size == 1 || !c->win.local || c->win.epoch == 0) return MLXQ_OK;
    cudaError_t e = cudaSetDevice(c->device);
    if (e != cudaSuccess) return mlxq::cuda_fail(e, "cudaSetDevice");
    unsigned* err = mlxq::device_error_word(c->device);
    if (!err) return mlxq::fail(MLXQ_GPU_FAILURE, "no error word on device %d", c->device);
    PeerFlags pf = {};
    for (int p = 0; p < c->size && p <= mlxq::MAX_PEERS; p++) pf.flag[p] = c->win.peer_flags[p];
    gather_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(c->win.flags, pf, c->rank, c->size, c->win.epoch_ctr, err);
    e = cudaGetLastError();
    return e == cudaSuccess ? MLXQ_OK : mlxq::cuda_fail(e, "gather wait launch");
}

}  // extern "C"
