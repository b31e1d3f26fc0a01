// Interface of the tensor-core dequant-GEMM (qgemm_sm100.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mlxq {

struct GemmLayer {
    const uint8_t* w;    // packed rows [O, K*bits/8]
    const void* s;       // scales [O, K/gs]
    const void* b;       // biases [O, K/gs]
    const void* bias;    // optional per-row bias [O]
    int s_dtype, bias_dtype;
    int O, K, gs, bits;
    int device;
};

struct GemmCall {
    const void* x;       // [T, K], 16-bit elements, row stride x_stride
    int x_dtype;
    long long x_stride;
    void* y;             // [T, O], row stride y_stride
    int y_dtype;
    long long y_stride;
    long long T;
    unsigned* err;       // device error word
    const void* table;   // the layer's staged scale/bias table when it has been built ahead (qgemm_build_table), else nullptr
};

// 0 when the GEMM cannot take this layer / call (the caller then uses the CUDA-core kernel), else the
// number of tokens per output tile it would use.
int qgemm_tile_tokens(const GemmLayer& L, int x_dtype, long long x_stride, const void* x, long long T);

// Enqueues the GEMM.  Returns cudaSuccess, or an error with `why` filled in.
cudaError_t launch_qgemm(const GemmLayer& L, const GemmCall& c, cudaStream_t st, const char** why);

// The same GEMM with its scratch in a fixed device array instead of pool memory: allocates nothing.
// Returns cudaErrorInvalidValue (why = "batch exceeds the static scratch") beyond qgemm_static_capacity().
size_t qgemm_static_capacity();
// Builds the layer's staged scale/bias table (qgemm_table_bytes(L) bytes at `table`, 256-byte aligned) on `st`.  The
// table depends on the layer only: a caller that keeps it passes it in GemmCall::table and saves the GEMM the work.
cudaError_t qgemm_build_table(const GemmLayer& L, void* table, cudaStream_t st);
// Bytes of the scale/bias table the GEMM stages for this layer, and the room the fixed array has for it.
size_t qgemm_table_bytes(const GemmLayer& L);
size_t qgemm_static_table_capacity();
cudaError_t launch_qgemm_static(const GemmLayer& L, const GemmCall& c, cudaStream_t st, const char** why);

}  // namespace mlxq
