// Decode matvec on CUDA cores: y[t, o] = sum_k x[t, k] * (scale * q[o, k] + bias) for small token counts.
//
// One warp owns R consecutive output rows.  Per step a lane takes one 16-byte-aligned period of each
// row's bit stream with 128-bit loads (32 codes at 4 bits, 64 at 2 and 6 bits, 128 at 3 and 5 bits, two
// loads = 32 codes at 8 bits), unpacks it in registers -- including the 3/5/6-bit codes that straddle
// 32-bit words -- and accumulates in fp32.  Codes are turned into floats without integer-to-float
// conversions: a code placed at mantissa bit 16 under exponent byte 0x43 *is* the float 128 + q, so the
// inner product runs on (128 + q) and the 128 * sum(x) term is removed per group with one fma.
// Per 32-code segment the lane applies the group's scale and bias:
//     acc += scale * (sum (128+q) x  -  128 * sum x)  +  bias * sum x
// Rows are reduced with warp shuffles and lane 0 writes the result (row bias, gate and output type
// folded in).  Up to three layers that share K / bits / group size run as one launch over the
// concatenated rows [A | B | C].
#pragma once

#include "mlxq_device.cuh"
#include "peer_gather.h"

namespace mlxq {

struct QmvPart {
    const uint8_t* w;   // packed rows
    const void* s;      // scales [rows, K/gs]
    const void* b;      // biases [rows, K/gs]
    const void* bias;   // optional per-row bias [rows]
    int rows;
};

struct QmvParams {
    QmvPart part[3];
    int n_parts;
    int total_rows;
    int K, gs, T;
    long long x_stride, y_stride;   // elements
    const void* x;
    void* y;
    int x_dtype, y_dtype, s_dtype, bias_dtype;
    int has_bias;
    const float* e;     // gate input (fp32 [total_rows]) or nullptr
    int act;
    int fast;           // rows and base pointers are 16-byte aligned: 128-bit loads allowed
    int seg32;          // gs % 32 == 0: one (scale, bias) per aligned 32-code segment
    int gs_shift;       // log2(gs) when gs is a power of two, else -1
    PeerGather peer;    // sharded calls of the persistent decode kernel: peers that receive the rows too
    const float* x_up;  // gated input (persistent kernels only): x is the fp32 gate half, x_up the up half, and the
    int x_act;          // activations the layer sees are act(x) * x_up (silu_mul / gelu_*_mul folded into the staging)
};

template <int BITS> struct QmvUnit {
    static constexpr int NL = BITS == 2 ? 1 : BITS == 3 ? 3 : BITS == 4 ? 1 : BITS == 5 ? 5 : BITS == 6 ? 3 : 2;
    static constexpr int CPL = NL * 128 / BITS;   // codes per lane per step
    static constexpr int R = NL <= 2 ? 4 : 2;     // rows per warp
    static constexpr float OFF = BITS == 8 ? 0.0f : 128.0f;
};

constexpr int QMV_WARPS = 8;

__device__ __forceinline__ int group_of(int k, const QmvParams& p) {
    return p.gs_shift >= 0 ? (k >> p.gs_shift) : (k / p.gs);
}

// Eight codes (chunk c of the lane's unit) as floats OFF + q, from the unit's registers.
template <int BITS>
__device__ __forceinline__ void unit_chunk(const uint32_t* w, int c, float (&f)[8]) {
    if constexpr (BITS == 4) {
        const uint32_t v = w[c];
        const uint32_t lo = v & 0x0F0F0F0Fu, hi = (v >> 4) & 0x0F0F0F0Fu;
        f[0] = __uint_as_float(__byte_perm(lo, 0x43000000u, 0x7044));
        f[1] = __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7044));
        f[2] = __uint_as_float(__byte_perm(lo, 0x43000000u, 0x7144));
        f[3] = __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7144));
        f[4] = __uint_as_float(__byte_perm(lo, 0x43000000u, 0x7244));
        f[5] = __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7244));
        f[6] = __uint_as_float(__byte_perm(lo, 0x43000000u, 0x7344));
        f[7] = __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7344));
    } else if constexpr (BITS == 8) {
        const uint32_t a = w[2 * c], b = w[2 * c + 1];
        f[0] = __uint_as_float(__byte_perm(a, 0x4B000000u, 0x7440)) - 8388608.0f;
        f[1] = __uint_as_float(__byte_perm(a, 0x4B000000u, 0x7441)) - 8388608.0f;
        f[2] = __uint_as_float(__byte_perm(a, 0x4B000000u, 0x7442)) - 8388608.0f;
        f[3] = __uint_as_float(__byte_perm(a, 0x4B000000u, 0x7443)) - 8388608.0f;
        f[4] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7440)) - 8388608.0f;
        f[5] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7441)) - 8388608.0f;
        f[6] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7442)) - 8388608.0f;
        f[7] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7443)) - 8388608.0f;
    } else if constexpr (BITS == 2) {
        // 16 codes per word: chunk c is the low or high half of word c/2.
        const uint32_t v = (c & 1) ? (w[c >> 1] >> 16) : w[c >> 1];
        const uint32_t p0 = v & 0x0303u, p1 = (v >> 2) & 0x0303u, p2 = (v >> 4) & 0x0303u, p3 = (v >> 6) & 0x0303u;
        f[0] = __uint_as_float(__byte_perm(p0, 0x43000000u, 0x7044));
        f[1] = __uint_as_float(__byte_perm(p1, 0x43000000u, 0x7044));
        f[2] = __uint_as_float(__byte_perm(p2, 0x43000000u, 0x7044));
        f[3] = __uint_as_float(__byte_perm(p3, 0x43000000u, 0x7044));
        f[4] = __uint_as_float(__byte_perm(p0, 0x43000000u, 0x7144));
        f[5] = __uint_as_float(__byte_perm(p1, 0x43000000u, 0x7144));
        f[6] = __uint_as_float(__byte_perm(p2, 0x43000000u, 0x7144));
        f[7] = __uint_as_float(__byte_perm(p3, 0x43000000u, 0x7144));
    } else {
        // 3, 5, 6 bits: bring each code to mantissa bit 16 with one (funnel) shift, mask and set the
        // exponent with one logic op.  Codes that straddle two words take the funnel shift.
        constexpr uint32_t M = ((1u << BITS) - 1u) << 16;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int bit = (c * 8 + i) * BITS;
            const int wi = bit >> 5, sh = bit & 31;
            uint32_t v;
            if (sh + BITS <= 32) v = sh <= 16 ? (w[wi] << (16 - sh)) : (w[wi] >> (sh - 16));
            else v = __funnelshift_r(w[wi], w[wi + 1], sh - 16);
            f[i] = __uint_as_float((v & M) | 0x43000000u);
        }
    }
}

template <int BITS, typename XT, int MT>
__global__ void __launch_bounds__(QMV_WARPS * 32)
qmv_kernel(const QmvParams p) {
    using U = QmvUnit<BITS>;
    constexpr int R = U::R, NL = U::NL, CPL = U::CPL;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g_row = (blockIdx.x * QMV_WARPS + warp) * R;
    if (g_row >= p.total_rows) return;
    const int t0 = blockIdx.y * MT;
    const int nt = min(MT, p.T - t0);

    // Locate the part ([A | B | C]) this row block belongs to; blocks never straddle parts because
    // fused parts have row counts that are multiples of 8.
    int pi = 0, row0 = g_row;
    if (p.n_parts > 1 && row0 >= p.part[0].rows) {
        row0 -= p.part[0].rows; pi = 1;
        if (p.n_parts > 2 && row0 >= p.part[1].rows) { row0 -= p.part[1].rows; pi = 2; }
    }
    const QmvPart part = p.part[pi];
    const int nr = min(R, part.rows - row0);
    const size_t row_bytes = static_cast<size_t>(p.K) * BITS / 8;
    const int gpr = p.K / p.gs;

    const XT* xb = reinterpret_cast<const XT*>(p.x) + static_cast<size_t>(t0) * p.x_stride;

    float acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) acc[r][t] = 0.0f;

    const uint8_t* wrow[R];
#pragma unroll
    for (int r = 0; r < R; r++) wrow[r] = part.w + static_cast<size_t>(row0 + min(r, nr - 1)) * row_bytes;

    int k_done = 0;
    if (p.fast) {
        const int units = p.K / CPL;
        for (int u = lane; u < units; u += 32) {
            uint32_t w[R][NL * 4];
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int j = 0; j < NL; j++) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(wrow[r] + static_cast<size_t>(u) * (NL * 16)) + j);
                    w[r][4 * j] = v.x; w[r][4 * j + 1] = v.y; w[r][4 * j + 2] = v.z; w[r][4 * j + 3] = v.w;
                }
            const int k0 = u * CPL;
            if (p.seg32) {
#pragma unroll
                for (int sgm = 0; sgm < CPL / 32; sgm++) {
                    float d[R][MT], xs[MT];
#pragma unroll
                    for (int t = 0; t < MT; t++) {
                        xs[t] = 0.0f;
#pragma unroll
                        for (int r = 0; r < R; r++) d[r][t] = 0.0f;
                    }
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) {
                        const int c = sgm * 4 + cc;
                        float xv[MT][8];
#pragma unroll
                        for (int t = 0; t < MT; t++) {
                            if (t < nt) {
                                XLoad<XT>::load8(xb + static_cast<size_t>(t) * p.x_stride + k0 + c * 8, xv[t]);
                            } else {
#pragma unroll
                                for (int i = 0; i < 8; i++) xv[t][i] = 0.0f;
                            }
#pragma unroll
                            for (int i = 0; i < 8; i++) xs[t] += xv[t][i];
                        }
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            float f[8];
                            unit_chunk<BITS>(w[r], c, f);
#pragma unroll
                            for (int t = 0; t < MT; t++)
#pragma unroll
                                for (int i = 0; i < 8; i++) d[r][t] = fmaf(f[i], xv[t][i], d[r][t]);
                        }
                    }
                    const int g = group_of(k0 + sgm * 32, p);
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        const size_t gi = static_cast<size_t>(row0 + min(r, nr - 1)) * gpr + g;
                        const float s = load_scalar(part.s, p.s_dtype, gi);
                        const float b = load_scalar(part.b, p.s_dtype, gi);
#pragma unroll
                        for (int t = 0; t < MT; t++) {
                            const float dq = fmaf(-U::OFF, xs[t], d[r][t]);
                            acc[r][t] = fmaf(b, xs[t], fmaf(s, dq, acc[r][t]));
                        }
                    }
                }
            } else {
                // Any group size that is a multiple of 8: the group is looked up per 8-code chunk.
#pragma unroll
                for (int c = 0; c < CPL / 8; c++) {
                    float xv[MT][8], xs[MT];
#pragma unroll
                    for (int t = 0; t < MT; t++) {
                        if (t < nt) {
                            XLoad<XT>::load8(xb + static_cast<size_t>(t) * p.x_stride + k0 + c * 8, xv[t]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; i++) xv[t][i] = 0.0f;
                        }
                        xs[t] = 0.0f;
#pragma unroll
                        for (int i = 0; i < 8; i++) xs[t] += xv[t][i];
                    }
                    const int g = group_of(k0 + c * 8, p);
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        float f[8];
                        unit_chunk<BITS>(w[r], c, f);
                        const size_t gi = static_cast<size_t>(row0 + min(r, nr - 1)) * gpr + g;
                        const float s = load_scalar(part.s, p.s_dtype, gi);
                        const float b = load_scalar(part.b, p.s_dtype, gi);
#pragma unroll
                        for (int t = 0; t < MT; t++) {
                            float d = 0.0f;
#pragma unroll
                            for (int i = 0; i < 8; i++) d = fmaf(f[i], xv[t][i], d);
                            const float dq = fmaf(-U::OFF, xs[t], d);
                            acc[r][t] = fmaf(b, xs[t], fmaf(s, dq, acc[r][t]));
                        }
                    }
                }
            }
        }
        k_done = units * CPL;
    }

    // Remainder (K not a multiple of the unit) or rows that are not 16-byte aligned: 8-code chunks,
    // byte loads, one chunk per lane.
    for (int c = k_done / 8 + lane; c < p.K / 8; c += 32) {
        float xv[MT][8], xs[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) {
            if (t < nt) {
                XLoad<XT>::load8(xb + static_cast<size_t>(t) * p.x_stride + c * 8, xv[t]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) xv[t][i] = 0.0f;
            }
            xs[t] = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) xs[t] += xv[t][i];
        }
        const int g = group_of(c * 8, p);
#pragma unroll
        for (int r = 0; r < R; r++) {
            uint32_t q[8];
            chunk_codes<BITS>(chunk_bits<BITS>(wrow[r] + static_cast<size_t>(c) * BITS), q);
            const size_t gi = static_cast<size_t>(row0 + min(r, nr - 1)) * gpr + g;
            const float s = load_scalar(part.s, p.s_dtype, gi);
            const float b = load_scalar(part.b, p.s_dtype, gi);
#pragma unroll
            for (int t = 0; t < MT; t++) {
                float d = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) d = fmaf(static_cast<float>(q[i]), xv[t][i], d);
                acc[r][t] = fmaf(b, xs[t], fmaf(s, d, acc[r][t]));
            }
        }
    }

#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) {
            float v = acc[r][t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            acc[r][t] = v;
        }

    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (r >= nr) break;
            const float rb = p.has_bias ? load_scalar(part.bias, p.bias_dtype, row0 + r) : 0.0f;
#pragma unroll
            for (int t = 0; t < MT; t++) {
                if (t >= nt) break;
                float v = acc[r][t] + rb;
                if (p.e != nullptr) v = act_mul(p.act, v, __ldg(p.e + g_row + r));
                store_scalar(p.y, p.y_dtype, static_cast<size_t>(t0 + t) * p.y_stride + g_row + r, v);
            }
        }
    }
}

// Launchers, one translation unit per bit width (qmv_inst.cu compiled with -DMLXQ_BITS=n).
cudaError_t launch_qmv_b2(const QmvParams& p, cudaStream_t st);
cudaError_t launch_qmv_b3(const QmvParams& p, cudaStream_t st);
cudaError_t launch_qmv_b4(const QmvParams& p, cudaStream_t st);
cudaError_t launch_qmv_b5(const QmvParams& p, cudaStream_t st);
cudaError_t launch_qmv_b6(const QmvParams& p, cudaStream_t st);
cudaError_t launch_qmv_b8(const QmvParams& p, cudaStream_t st);

}  // namespace mlxq
