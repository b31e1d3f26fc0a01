// The dense matvec / small-batch kernel (dense.cuh).
#include "dense.cuh"

namespace mlxq {

namespace {

constexpr int DENSE_WARPS = 8;
constexpr int DENSE_TOKENS = 8;      // tokens per pass over a row

// eight consecutive elements as fp32; `vec`: the address is 16-byte aligned (32 for fp32) and may be read in one piece
__device__ __forceinline__ void load8_any(const void* p, int dt, size_t idx, bool vec, float (&o)[8]) {
    if (vec) {
        if (dt == DT_F32) {
            const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx);
            const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx + 4);
            o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
            return;
        }
        const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p) + idx);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (dt == DT_F16) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                o[2 * i] = f.x; o[2 * i + 1] = f.y;
            } else {
                o[2 * i] = __uint_as_float(w[i] << 16);
                o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = load_scalar(p, dt, idx + i);
}

__global__ void __launch_bounds__(DENSE_WARPS * 32)
dense_mv_kernel(const void* __restrict__ w, int w_dtype, const void* __restrict__ bias, int bias_dtype, const void* __restrict__ x,
                int x_dtype, long long x_stride, void* __restrict__ y, int y_dtype, long long y_stride, int tt, int O, int K,
                int w_vec, int x_vec) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * DENSE_WARPS + (threadIdx.x >> 5);
    if (row >= O) return;
    float acc[DENSE_TOKENS];
#pragma unroll
    for (int t = 0; t < DENSE_TOKENS; t++) acc[t] = 0.0f;
    const size_t wrow = static_cast<size_t>(row) * K;
    const int K8 = K & ~7;
    for (int k = lane * 8; k < K8; k += 256) {
        float wv[8];
        load8_any(w, w_dtype, wrow + k, w_vec != 0, wv);
#pragma unroll
        for (int t = 0; t < DENSE_TOKENS; t++) {
            if (t < tt) {
                float xv[8];
                load8_any(x, x_dtype, static_cast<size_t>(t) * x_stride + k, x_vec != 0, xv);
#pragma unroll
                for (int i = 0; i < 8; i++) acc[t] = fmaf(wv[i], xv[i], acc[t]);
            }
        }
    }
    for (int k = K8 + lane; k < K; k += 32) {
        const float wv = load_scalar(w, w_dtype, wrow + k);
        for (int t = 0; t < tt; t++) acc[t] = fmaf(wv, load_scalar(x, x_dtype, static_cast<size_t>(t) * x_stride + k), acc[t]);
    }
#pragma unroll
    for (int t = 0; t < DENSE_TOKENS; t++) {
        float v = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && t < tt) {
            if (bias != nullptr) v += load_scalar(bias, bias_dtype, row);
            store_scalar(y, y_dtype, static_cast<size_t>(t) * y_stride + row, v);
        }
    }
}

}  // namespace

cudaError_t launch_dense(const void* w, int w_dtype, const void* bias, int bias_dtype, const void* x, int x_dtype, long long x_stride,
                         void* y, int y_dtype, long long y_stride, long long T, int O, int K, cudaStream_t st) {
    const size_t wsz = dtype_size(w_dtype), xsz = dtype_size(x_dtype);
    const int w_vec = (reinterpret_cast<uintptr_t>(w) % 16 == 0 && (static_cast<size_t>(K) * wsz) % 16 == 0) ? 1 : 0;
    const int x_vec = (reinterpret_cast<uintptr_t>(x) % 16 == 0 && (static_cast<size_t>(x_stride) * xsz) % 16 == 0) ? 1 : 0;
    const unsigned grid = static_cast<unsigned>((O + DENSE_WARPS - 1) / DENSE_WARPS);
    for (long long t0 = 0; t0 < T; t0 += DENSE_TOKENS) {
        const int tt = static_cast<int>(T - t0 < DENSE_TOKENS ? T - t0 : DENSE_TOKENS);
        dense_mv_kernel<<<grid, DENSE_WARPS * 32, 0, st>>>(
            w, w_dtype, bias, bias_dtype, static_cast<const char*>(x) + static_cast<size_t>(t0) * x_stride * xsz, x_dtype, x_stride,
            static_cast<char*>(y) + static_cast<size_t>(t0) * y_stride * dtype_size(y_dtype), y_dtype, y_stride, tt, O, K, w_vec, x_vec);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace mlxq
