// Launchers of the small kernels beside the matvec / GEMM (see aux_kernels.cu).
#pragma once

#include "mlxq_device.cuh"

namespace mlxq {

cudaError_t launch_unpack_codes(const uint8_t* w, uint8_t* out, long long rows, int K, int bits, cudaStream_t st);
cudaError_t launch_lookup(const uint8_t* w, const void* scales, const void* biases, int s_dtype, const int32_t* ids,
                          float* out, long long T, int rows, int K, int gs, int bits, unsigned* err, cudaStream_t st);
cudaError_t launch_rows(const uint8_t* w, const void* scales, const void* biases, int s_dtype, const void* x, int x_dtype,
                        float* y, const uint32_t* count, const int32_t* list, long long max_rows, int rows, int K, int gs,
                        int bits, cudaStream_t st);

// First pass of the token selection (block maxima) and the greedy second pass over them.  `pairs` holds, per segment,
// the maxima as fp32 [T][nb] followed by their indices as int32 [T][nb].
constexpr int SELECT_BLOCK = 256;            // logits per block
constexpr int SELECT_NONE = 0x7fffffff;      // index of a block (or a token) with no value above -inf
cudaError_t launch_block_max(const float* logits, long long stride, long long V, long long T, int index_base, uint32_t* pairs,
                             cudaStream_t st);
cudaError_t launch_block_argmax(const uint32_t* pairs, int n_seg, long long T, int nb, int32_t* token, float* value, cudaStream_t st);

// Elementwise neighbours of the projections: out[t, i] = act(gu[t, i]) * gu[t, cols + i], and the residual add fused with
// the next RMS norm (h += r; y = RMSNorm(h) * w).
cudaError_t launch_act_mul(const float* gu, long long stride, long long cols, long long T, int act, float* out, cudaStream_t st);
cudaError_t launch_add_rms_norm(float* h, const float* r, float* y, const void* w, int w_dtype, long long dim, long long rows,
                                long long row_stride, float eps, cudaStream_t st);

}  // namespace mlxq
