// Decode matvec on the tensor cores, raw codes in, fp32 scaling out:
//     y[t, o] = sum_g ( scale[o,g] * sum_{k in g} q[o,k] x[t,k]  +  bias[o,g] * sum_{k in g} x[t,k] )
//
// At HBM speed a B200 SM must retire ~40 four-bit codes per clock; turning every code into a float and
// issuing one FMA for it costs more instructions than the SM can issue (measured: the CUDA-core kernel is
// issue-bound at a quarter of the memory roofline).  Here the inner products run on mma.m16n8k16 with the
// *codes themselves* as the fp16 A operand: a masked code is the bit pattern of the subnormal half
// q * 2^-24, so two codes become one A register with a single logic op and no conversion.  Codes that sit
// at a higher bit position (the odd nibble of a byte, the upper fields of a 2-bit word) are left where
// they are and the matching activations are pre-divided by that power of two when they are staged.
//
// A warp owns 16 output rows; lane (g = lane/4, t = lane%4) loads 16 bytes (4/8/2-bit) or 24/40 bytes
// (6/3/5-bit) of rows g and g+8 per step -- the four lanes of a row read one contiguous 64/96/160-byte run
// -- and keeps several steps of loads in flight.  The 8 accumulator columns are not 8 tokens: a column
// stands for (token, quantisation group) and is fed only that group's activations (zeros otherwise), so one
// set of MMAs yields the per-group sums sum_{k in g} q x separately; with few tokens the spare columns hold
// the groups of the following steps, so the accumulators are drained -- scale and bias applied in fp32,
// exactly as the layer is defined -- once per eight (token, group) pairs.  fp32 activations ride as two fp16
// columns (hi + lo).  The CTA's four warps split K; partial sums meet in shared memory.
#pragma once

#include "mlxq_device.cuh"
#include "qmv.cuh"

namespace mlxq {

constexpr int MMA_WARPS = 4;        // K splits per 16-row block

template <int BITS> struct MmaUnit {
    // bytes a lane loads per row per step, codes in them, codes per row per step (four lanes)
    static constexpr int LB = (BITS == 2 || BITS == 4 || BITS == 8) ? 16 : (BITS == 5 ? 40 : 24);
    static constexpr int CL = LB * 8 / BITS;
    static constexpr int KB = 4 * CL;
    static constexpr int NW = LB / 4;            // 32-bit words per lane per row per step
    static constexpr int NM = CL / 4;            // MMAs per step
    static constexpr int PF = NW <= 4 ? 4 : 2;   // steps of weight loads in flight per lane
    // the staging permutation works on units of UW codes (one 32-bit word for 2/4/8 bits)
    static constexpr int UW = (BITS == 2) ? 16 : (BITS == 4) ? 8 : (BITS == 8) ? 4 : 2;
};

// Position (in halves) of code i of a unit inside the staged activations, and the power of two its
// activation is divided by.  Must mirror the A-register construction in `a_regs`.
template <int BITS> __device__ __forceinline__ int stage_pos(int i) {
    if (BITS == 4) return (i & 3) * 2 + (i >> 2);          // order 0,4,1,5,2,6,3,7
    if (BITS == 8) return (i & 1) * 2 + (i >> 1);          // order 0,2,1,3
    if (BITS == 2) return (i & 7) * 2 + (i >> 3);          // order 0,8,1,9,...,7,15
    return i;
}
template <int BITS> __device__ __forceinline__ int stage_shift(int i) {
    if (BITS == 4) return (i & 1) * 4;
    if (BITS == 2) return (i & 3) * 2;
    return 0;
}

struct MmaParams {
    QmvParams q;            // layer parts, x, y, strides, dtypes, epilogue
    int xn;                 // staged activation columns: tokens, or 2 * tokens for fp32 activations
    int split;              // 1: one column per token, 2: hi/lo columns
    int xstride;            // halves between staged columns (K + pad)
    int passes;             // accumulator sets: ceil(xn * groups-per-step / 8)
    int gstep_shift;        // log2(groups per step); 0 when a group spans one or more whole steps
    int spg_shift;          // log2(steps per group), 0 unless the group is wider than a step
    int cycle;              // consecutive group blocks that share one accumulator set (1 when passes > 1)
    unsigned* err;          // device error word (bounded waits of the persistent kernel)
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Pair registers of one row for MMA `j` of a step, from the lane's words of that row.
// lo -> slots (2t, 2t+1), hi -> slots (2t+8, 2t+9).
template <int BITS>
__device__ __forceinline__ void a_regs(const uint32_t* w, int j, uint32_t& lo, uint32_t& hi) {
    if constexpr (BITS == 4) {
        const uint32_t v = (j & 1) ? (w[j >> 1] >> 8) : w[j >> 1];
        lo = v & 0x000F000Fu;        // codes (0,4) or (2,6) of the word
        hi = v & 0x00F000F0u;        // codes (1,5) or (3,7), times 16
    } else if constexpr (BITS == 8) {
        lo = w[j] & 0x00FF00FFu;         // codes (0,2)
        hi = (w[j] >> 8) & 0x00FF00FFu;  // codes (1,3)
    } else if constexpr (BITS == 2) {
        const uint32_t v = (j & 2) ? (w[j >> 2] >> 8) : w[j >> 2];
        if (j & 1) { lo = v & 0x00300030u; hi = v & 0x00C000C0u; }   // codes (2,10)*16, (3,11)*64  [+4 when j&2]
        else       { lo = v & 0x00030003u; hi = v & 0x000C000Cu; }   // codes (0,8), (1,9)*4
    } else {
        // 3, 5, 6 bits: codes 4j..4j+3 of the lane's run, consecutive pairs, no pre-scaling.
        constexpr uint32_t M = ((1u << BITS) - 1u) * 0x00010001u;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int bit = (4 * j + 2 * h) * BITS;
            const int wi = bit >> 5, sh = bit & 31;
            uint32_t v;                                    // 2*BITS bits starting at `bit`: both codes of the pair
            if (sh == 0) v = w[wi];
            else if (sh + 2 * BITS <= 32) v = w[wi] >> sh;
            else v = __funnelshift_r(w[wi], w[wi + 1], sh);
            const uint32_t r = __byte_perm(v, v << (16 - BITS), 0x7610) & M;
            if (h == 0) lo = r; else hi = r;
        }
    }
}

// MMA j of a step uses codes starting at this offset inside the lane's run (for the group lookup).
template <int BITS> __device__ __forceinline__ int mma_code_offset(int j) {
    if (BITS == 4) return (j >> 1) * 8;
    if (BITS == 8) return j * 4;
    if (BITS == 2) return (j >> 2) * 16;
    return j * 4;
}

// Eight consecutive activations -> staged halves.  `v` are the fp32 values, `k` their first index.
template <int BITS>
__device__ __forceinline__ void stage8(__half* col, int k, const float (&v)[8]) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int u = (k + i) % MmaUnit<BITS>::UW;
        const float sc = __int_as_float((127 - stage_shift<BITS>(u)) << 23);     // 2^-shift
        col[k + i - u + stage_pos<BITS>(u)] = __float2half_rn(v[i] * sc);
    }
}

template <int BITS, int NP>
__global__ void __launch_bounds__(MMA_WARPS * 32)
qmv_mma_kernel(const MmaParams p) {
    using U = MmaUnit<BITS>;
    constexpr int LB = U::LB, CL = U::CL, KB = U::KB, NW = U::NW, NM = U::NM, PF = U::PF;
    extern __shared__ __align__(16) uint8_t smem_mma[];
    const QmvParams& q = p.q;
    const int K = q.K, gs_shift = q.gs_shift;
    const int groups = K >> gs_shift;
    __half* xs = reinterpret_cast<__half*>(smem_mma);                                   // [xn][xstride]
    float* xsum = reinterpret_cast<float*>(smem_mma + static_cast<size_t>(p.xn) * p.xstride * 2);   // [xn][groups]
    float* part = xsum + p.xn * groups;                                                 // [warps][NP][16][8]
    float* csum = part + MMA_WARPS * NP * 128;                                          // [tokens][K/8]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row_blk = blockIdx.x * 16;

    // The lane's two rows (g and g+8 of the block); each 8-row half lies inside one fused part.
    const uint8_t* wrow[2];
    const void* srow[2];
    const void* brow[2];
    const size_t row_bytes = static_cast<size_t>(K) * BITS / 8;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        int r = min(row_blk + g + 8 * h, q.total_rows - 1), pi = 0;
        if (q.n_parts > 1 && r >= q.part[0].rows) {
            r -= q.part[0].rows; pi = 1;
            if (q.n_parts > 2 && r >= q.part[1].rows) { r -= q.part[1].rows; pi = 2; }
        }
        wrow[h] = q.part[pi].w + static_cast<size_t>(r) * row_bytes + t * LB;
        const size_t off = static_cast<size_t>(r) * groups * dtype_size(q.s_dtype);
        srow[h] = static_cast<const char*>(q.part[pi].s) + off;
        brow[h] = static_cast<const char*>(q.part[pi].b) + off;
    }

    // K split: contiguous ranges of steps per warp, cut at group boundaries (a group wider than a step
    // must be finished by the warp that started it).
    const int spg_shift = p.spg_shift;
    const int chunks = (K / KB) >> spg_shift;
    const int s_begin = ((chunks * warp) / MMA_WARPS) << spg_shift;
    const int s_end = ((chunks * (warp + 1)) / MMA_WARPS) << spg_shift;

    // ---- first loads go out before anything else --------------------------------------------------------
    uint32_t wbuf[PF][2][NW];
    auto load_step = [&](int s, uint32_t (&dst)[2][NW]) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint8_t* src = wrow[h] + static_cast<size_t>(s) * (4 * LB);
            if constexpr (LB == 16) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
                dst[h][0] = v.x; dst[h][1] = v.y; dst[h][2] = v.z; dst[h][3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < NW / 2; i++) {
                    const uint2 v = __ldg(reinterpret_cast<const uint2*>(src) + i);
                    dst[h][2 * i] = v.x; dst[h][2 * i + 1] = v.y;
                }
            }
        }
    };
#pragma unroll
    for (int i = 0; i < PF; i++)
        if (s_begin + i < s_end) load_step(s_begin + i, wbuf[i]);

    // ---- stage the activations: fp16, permuted and pre-scaled to match the A registers ------------------
    // Eight consecutive activations per thread and turn; sums are formed in a fixed order (chunk of 8, then
    // the chunks of a group in order) so that a token's result never depends on scheduling.
    {
        const int cpr = K / 8;
        for (int idx = threadIdx.x; idx < q.T * cpr; idx += blockDim.x) {
            const int tok = idx / cpr, k = (idx - tok * cpr) * 8;
            float v[8];
            if (q.x_dtype == DT_F16) XLoad<__half>::load8(reinterpret_cast<const __half*>(q.x) + static_cast<size_t>(tok) * q.x_stride + k, v);
            else if (q.x_dtype == DT_BF16) XLoad<__nv_bfloat16>::load8(reinterpret_cast<const __nv_bfloat16*>(q.x) + static_cast<size_t>(tok) * q.x_stride + k, v);
            else XLoad<float>::load8(reinterpret_cast<const float*>(q.x) + static_cast<size_t>(tok) * q.x_stride + k, v);
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) sum += v[i];
            csum[idx] = sum;
            if (p.split == 1) {
                stage8<BITS>(xs + static_cast<size_t>(tok) * p.xstride, k, v);
            } else {
                float hi[8], lo[8];
#pragma unroll
                for (int i = 0; i < 8; i++) { hi[i] = __half2float(__float2half_rn(v[i])); lo[i] = v[i] - hi[i]; }
                stage8<BITS>(xs + static_cast<size_t>(2 * tok) * p.xstride, k, hi);
                stage8<BITS>(xs + static_cast<size_t>(2 * tok + 1) * p.xstride, k, lo);
            }
        }
        __syncthreads();
        const int cpg = 1 << (gs_shift - 3);                 // 8-wide chunks per group
        for (int idx = threadIdx.x; idx < p.xn * groups; idx += blockDim.x) {
            const int xc = idx / groups, gi = idx - xc * groups;
            float sum = 0.0f;
            if (p.split == 1 || (xc & 1) == 0) {             // the lo column of an fp32 token carries no bias term
                const int tok = p.split == 1 ? xc : (xc >> 1);
                for (int i = 0; i < cpg; i++) sum += csum[tok * cpr + gi * cpg + i];
            }
            xsum[idx] = sum;
        }
    }
    __syncthreads();

    // ---- column bookkeeping (all step-invariant) ----------------------------------------------------------
    // Accumulator column n of pass ps stands for (cycle, staged column, group-in-step):
    //   cycle == 1:  lin = ps*8 + n,  xc = lin >> gstep_shift,  grp = lin & (G-1)
    //   cycle  > 1:  (one pass) cyc = n / (xn*G),  rem = n % (xn*G),  xc = rem >> gstep_shift,  grp = rem & (G-1)
    const int gsh = p.gstep_shift, G = 1 << gsh, CY = p.cycle;
    const int cols_per_cycle = p.xn << gsh;
    // groups of the lane's run: first half of the step's MMAs and second half (they differ only when a
    // lane's run spans two groups)
    const int run_grp_a = ((t * CL + mma_code_offset<BITS>(0)) >> gs_shift) & (G - 1);
    const int run_grp_b = ((t * CL + mma_code_offset<BITS>(NM / 2)) >> gs_shift) & (G - 1);
    const __half* bptr[NP];          // staged column this lane feeds as B (column n = g), at the lane's run
    bool keep_a[NP], keep_b[NP];
    int b_cyc[NP];
#pragma unroll
    for (int ps = 0; ps < NP; ps++) {
        int xc, grp, cyc = 0;
        if (CY > 1) { cyc = g / cols_per_cycle; const int rem = g - cyc * cols_per_cycle; xc = rem >> gsh; grp = rem & (G - 1); }
        else { const int lin = ps * 8 + g; xc = lin >> gsh; grp = lin & (G - 1); }
        const bool valid = xc < p.xn && cyc < CY;
        bptr[ps] = xs + static_cast<size_t>(valid ? xc : 0) * p.xstride + t * CL;
        keep_a[ps] = valid && grp == run_grp_a;
        keep_b[ps] = valid && grp == run_grp_b;
        b_cyc[ps] = cyc;
    }
    // the lane's accumulator columns 2t, 2t+1: staged column, group offset inside the cycle block
    int c_xc[NP][2], c_goff[NP][2];
#pragma unroll
    for (int ps = 0; ps < NP; ps++)
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const int n = 2 * t + ci;
            int xc, grp, cyc = 0;
            if (CY > 1) { cyc = n / cols_per_cycle; const int rem = n - cyc * cols_per_cycle; xc = rem >> gsh; grp = rem & (G - 1); }
            else { const int lin = ps * 8 + n; xc = lin >> gsh; grp = lin & (G - 1); }
            c_xc[ps][ci] = (xc < p.xn && cyc < CY) ? xc : -1;
            c_goff[ps][ci] = (cyc << gsh) + grp;
        }

    float yacc[NP][4], c[NP][4];
#pragma unroll
    for (int ps = 0; ps < NP; ps++)
#pragma unroll
        for (int i = 0; i < 4; i++) { yacc[ps][i] = 0.0f; c[ps][i] = 0.0f; }

    // Applies scale and bias to the finished per-group sums.  gbase = first group of the cycle block,
    // glimit = groups completed so far (columns of cycles not reached yet are skipped).
    const int gmin = (s_begin * KB) >> gs_shift;            // groups before it belong to the previous warp
    auto drain = [&](int gbase, int glimit) {
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int ci = i & 1, h = i >> 1;
                const int gg = gbase + c_goff[ps][ci];
                if (c_xc[ps][ci] >= 0 && gg >= gmin && gg < glimit) {
                    const float sc = load_scalar(srow[h], q.s_dtype, gg) * 16777216.0f;
                    const float bi = load_scalar(brow[h], q.s_dtype, gg);
                    yacc[ps][i] += fmaf(bi, xsum[c_xc[ps][ci] * groups + gg], sc * c[ps][i]);
                }
                c[ps][i] = 0.0f;
            }
    };

    // ---- main loop: PF steps per turn so that the load ring is indexed statically ---------------------------
    const int cyc_mask = CY - 1;
    for (int s0 = s_begin; s0 < s_end; s0 += PF) {
#pragma unroll
        for (int u = 0; u < PF; u++) {
            const int s = s0 + u;
            if (s < s_end) {
                uint32_t w[2][NW];
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int k = 0; k < NW; k++) w[h][k] = wbuf[u][h][k];
                if (s + PF < s_end) load_step(s + PF, wbuf[u]);
                const int gblock = s >> spg_shift;                 // group block (one step, or several for wide groups)
                const int cyc_s = gblock & cyc_mask;
                const int koff = s * KB;
#pragma unroll
                for (int j = 0; j < NM; j += 2) {
                    uint32_t a00, a01, a02, a03, a10, a11, a12, a13;
                    a_regs<BITS>(w[0], j, a00, a02);
                    a_regs<BITS>(w[1], j, a01, a03);
                    a_regs<BITS>(w[0], j + 1, a10, a12);
                    a_regs<BITS>(w[1], j + 1, a11, a13);
#pragma unroll
                    for (int ps = 0; ps < NP; ps++) {
                        const bool keep = (j < NM / 2 ? keep_a[ps] : keep_b[ps]) && b_cyc[ps] == cyc_s;
                        uint4 bv = make_uint4(0u, 0u, 0u, 0u);
                        if (keep) bv = *reinterpret_cast<const uint4*>(bptr[ps] + koff + 4 * j);
                        mma16816(c[ps], a00, a01, a02, a03, bv.x, bv.y);
                        mma16816(c[ps], a10, a11, a12, a13, bv.z, bv.w);
                    }
                }
                // end of a group block that closes the cycle (or the warp's range): apply scales
                if (((s + 1) & ((1 << spg_shift) - 1)) == 0 && (cyc_s == cyc_mask || s + 1 == s_end)) {
                    const int gfirst = (((gblock - cyc_s) << spg_shift) * KB) >> gs_shift;
                    drain(gfirst, ((s + 1) * KB) >> gs_shift);
                }
            }
        }
    }

    // ---- reduce the K splits and the group / hi-lo columns, then the epilogue --------------------------------
#pragma unroll
    for (int ps = 0; ps < NP; ps++)
#pragma unroll
        for (int i = 0; i < 4; i++)
            part[((warp * NP + ps) * 16 + g + 8 * (i >> 1)) * 8 + 2 * t + (i & 1)] = yacc[ps][i];
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * q.T; idx += blockDim.x) {
        const int tok = idx >> 4, r = idx & 15;
        const int row = row_blk + r;
        if (row >= q.total_rows) continue;
        float v = 0.0f;
        for (int sp = 0; sp < p.split; sp++) {
            const int xc = tok * p.split + sp;
            for (int cyc = 0; cyc < CY; cyc++)
                for (int grp = 0; grp < G; grp++) {
                    int ps, col;
                    if (CY > 1) { ps = 0; col = cyc * cols_per_cycle + (xc << gsh) + grp; }
                    else { const int lin = (xc << gsh) + grp; ps = lin >> 3; col = lin & 7; }
                    for (int wv = 0; wv < MMA_WARPS; wv++) v += part[((wv * NP + ps) * 16 + r) * 8 + col];
                }
        }
        int pr = row, pi = 0;
        if (q.n_parts > 1 && pr >= q.part[0].rows) {
            pr -= q.part[0].rows; pi = 1;
            if (q.n_parts > 2 && pr >= q.part[1].rows) { pr -= q.part[1].rows; pi = 2; }
        }
        if (q.has_bias) v += load_scalar(q.part[pi].bias, q.bias_dtype, pr);
        if (q.e != nullptr) v = act_mul(q.act, v, __ldg(q.e + row));
        store_scalar(q.y, q.y_dtype, static_cast<size_t>(tok) * q.y_stride + row, v);
    }
}

// Codes per row a warp consumes per step at this bit width (K must be a multiple of it).
int qmv_mma_step_codes(int bits);
// Fills the column plan (passes, cycle, shifts) for xn staged columns; false when the call does not fit.
bool qmv_mma_plan(int bits, int K, int gs, int xn, MmaParams& p);
// Shared memory the kernel needs for a planned call.
size_t qmv_mma_smem(int K, int gs, int tokens, const MmaParams& p);
// Launch (bits, passes) instantiation; returns cudaErrorNotSupported when there is none.
cudaError_t launch_qmv_mma(int bits, const MmaParams& p, size_t smem, int device, cudaStream_t st);

}  // namespace mlxq
