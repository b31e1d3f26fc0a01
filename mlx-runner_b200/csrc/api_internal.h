// Declarations shared by the host-side translation units of libmlxq (api.cu, comm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>

#include "peer_gather.h"

// The layer handle behind mlxq_linear_t: borrowed device pointers plus the facts derived from shapes.
struct mlxq_linear {
    const uint8_t* w;
    const void* s;
    const void* b;
    const void* bias;
    int64_t in_dim, out_dim;
    int bits, gs;         // bits == 0: a dense (unquantized) layer, its weights in w_dtype
    int w_dtype = 0;
    int s_dtype, bias_dtype;
    int device;
    int64_t row_offset;   // first global output row (shards)
    int64_t total_out;    // rows of the whole layer (== out_dim unless sharded)
    int shard_rank, shard_count;
    bool qmv_eligible;
    std::string name;
    // The tensor-core GEMM's staged scale/bias table (it depends on the layer only): built by mlxq_linear_prepare or
    // by the first batch that takes the GEMM, owned by the handle, freed with it.
    std::mutex table_mu;
    void* gemm_table = nullptr;
    bool table_tried = false;
};

namespace mlxq {

// Records the message for mlxq_last_error() and returns `status`.
int fail(int status, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
int cuda_fail(cudaError_t e, const char* what);
// Device address of the per-device error word (nullptr if the device cannot be selected).
unsigned* device_error_word(int device);
// `peer` (optional): also store the rows into the peers' windows and run the flag hand-shake; only the persistent
// decode kernel can do that, other paths return MLXQ_UNSUPPORTED when it is given.
int forward_impl(mlxq_linear* h, cudaStream_t st, const void* x, int x_dtype, int64_t x_stride, void* y, int y_dtype,
                 int64_t y_stride, int64_t T, const PeerGather* peer = nullptr);

}  // namespace mlxq
