// Device-side helpers shared by the libmlxq kernels: element-type loads/stores, the MLX bit-stream
// decoders and the gated-epilogue activations.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mlxq {

enum : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };

// Device-side error word bits (one word per device, read by mlxq_stream_status).
enum : unsigned { ERR_BAD_LOOKUP_ID = 1u, ERR_WAIT_TIMEOUT = 2u, ERR_GEMM_PIPELINE = 4u, ERR_PEER_FLAG = 8u };

__host__ __device__ inline int dtype_size(int dt) { return dt == DT_F32 ? 4 : 2; }

// ---- scalar loads of a runtime element type ---------------------------------------------------------
__device__ __forceinline__ float load_scalar(const void* p, int dt, size_t i) {
    if (dt == DT_F32) return __ldg(reinterpret_cast<const float*>(p) + i);
    unsigned short u = __ldg(reinterpret_cast<const unsigned short*>(p) + i);
    if (dt == DT_F16) return __half2float(__ushort_as_half(u));
    return __uint_as_float(static_cast<uint32_t>(u) << 16);
}

// Split form for software prefetching: the load returns raw bits (nothing depends on it, so the warp does not
// wait), the conversion happens where the value is used.
__device__ __forceinline__ uint32_t load_scalar_raw(const void* p, int dt, size_t i) {
    if (dt == DT_F32) return __float_as_uint(__ldg(reinterpret_cast<const float*>(p) + i));
    return __ldg(reinterpret_cast<const unsigned short*>(p) + i);
}
__device__ __forceinline__ float scalar_from_raw(uint32_t raw, int dt) {
    if (dt == DT_F32) return __uint_as_float(raw);
    if (dt == DT_F16) return __half2float(__ushort_as_half(static_cast<unsigned short>(raw)));
    return __uint_as_float(raw << 16);
}

// The same for a shared-memory (or any generic) address: plain loads, no read-only cache hint.
__device__ __forceinline__ float smem_scalar(const void* p, int dt, size_t i) {
    if (dt == DT_F32) return reinterpret_cast<const float*>(p)[i];
    const unsigned short u = reinterpret_cast<const unsigned short*>(p)[i];
    if (dt == DT_F16) return __half2float(__ushort_as_half(u));
    return __uint_as_float(static_cast<uint32_t>(u) << 16);
}

__device__ __forceinline__ void store_scalar(void* p, int dt, size_t i, float v) {
    if (dt == DT_F32) reinterpret_cast<float*>(p)[i] = v;
    else if (dt == DT_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// ---- eight consecutive activations as fp32 (x rows are 16-byte aligned, k is a multiple of 8) -------
template <typename XT> struct XLoad;
template <> struct XLoad<float> {
    static constexpr int DT = DT_F32;
    __device__ __forceinline__ static void load8(const float* p, float (&o)[8]) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p));
        const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
};
template <> struct XLoad<__half> {
    static constexpr int DT = DT_F16;
    __device__ __forceinline__ static void load8(const __half* p, float (&o)[8]) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            o[2 * i] = f.x; o[2 * i + 1] = f.y;
        }
    }
};
template <> struct XLoad<__nv_bfloat16> {
    static constexpr int DT = DT_BF16;
    __device__ __forceinline__ static void load8(const __nv_bfloat16* p, float (&o)[8]) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
};

// ---- generic decoder: eight codes from BITS bytes at any byte address --------------------------------
// Code i of the chunk is bits [i*BITS, (i+1)*BITS) of the little-endian value of those bytes.
template <int BITS>
__device__ __forceinline__ uint64_t chunk_bits(const uint8_t* p) {
    uint64_t v = 0;
#pragma unroll
    for (int i = 0; i < BITS; i++) v |= static_cast<uint64_t>(__ldg(p + i)) << (8 * i);
    return v;
}

template <int BITS>
__device__ __forceinline__ void chunk_codes(uint64_t v, uint32_t (&q)[8]) {
    constexpr uint64_t M = (1ull << BITS) - 1ull;
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = static_cast<uint32_t>((v >> (i * BITS)) & M);
}

__device__ __forceinline__ uint64_t chunk_bits_rt(const uint8_t* p, int bits) {
    uint64_t v = 0;
    for (int i = 0; i < bits; i++) v |= static_cast<uint64_t>(__ldg(p + i)) << (8 * i);
    return v;
}

// ---- gated epilogue: act(g) * u with 0 SiLU, 1 tanh-GELU, 2 exact GELU -----------------------------
// The exact GELU uses the erfc Chebyshev fit the layer's definition names (|error| < 1.2e-7).
__device__ __forceinline__ float erf_fit(float x) {
    const float z = fabsf(x), t = 1.0f / (1.0f + 0.5f * z);
    const float r = t * expf(-z * z - 1.26551223f +
                             t * (1.00002368f +
                                  t * (0.37409196f +
                                       t * (0.09678418f +
                                            t * (-0.18628806f +
                                                 t * (0.27886807f +
                                                      t * (-1.13520398f +
                                                           t * (1.48851587f + t * (-0.82215223f + t * 0.17087277f)))))))));
    return x >= 0.0f ? 1.0f - r : r - 1.0f;
}

__device__ __forceinline__ float act_mul(int act, float g, float u) {
    if (act == 0) return (g / (1.0f + expf(-g))) * u;
    if (act == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    return 0.5f * g * (1.0f + erf_fit(g * 0.7071067811865476f)) * u;
}

}  // namespace mlxq
