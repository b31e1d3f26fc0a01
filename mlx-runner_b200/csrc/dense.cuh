// Dense (unquantized) layers through the same handle: y[t, o] = sum_k W[o, k] x[t, k] (+ bias[o]), W in f32 / f16 / bf16,
// fp32 accumulation (dmm, Sources/MLXEngine/Kernels.swift:938-999).  A CUDA-core kernel: one warp per output row, the
// row streamed once per tile of eight tokens with 16-byte loads.  It is HBM-bound for decode batches; long batches
// re-read the weights once per eight tokens (from L2 where the layer fits), which a library GEMM would avoid -- dense
// layers are the exception in a quantized checkpoint, and no long-batch path is built for them.
#pragma once

#include "mlxq_device.cuh"

namespace mlxq {

cudaError_t launch_dense(const void* w, int w_dtype, const void* bias, int bias_dtype, const void* x, int x_dtype, long long x_stride,
                         void* y, int y_dtype, long long y_stride, long long T, int O, int K, cudaStream_t st);

}  // namespace mlxq
