// A-register construction for the widths whose codes straddle bytes (3, 5, 6 bits) in the persistent decode kernels.
//
// An A register of mma.m16n8k16 holds two fp16 values; a masked code is the subnormal half q * 2^-24, and a code that
// sits p bits up inside its half is q * 2^p * 2^-24, which the staged activation undoes (it is pre-divided by 2^p), as
// long as the code stays inside the ten mantissa bits: p + BITS <= 10.  So two codes whose bit positions in the packed
// row differ by 16 + p become one register with one shift and one logic op: code i at bit 0 of the shifted word, and
// its partner i + D, D = ceil(16 / BITS), at bit 16 + p with p = BITS * D - 16 (2 for 3 and 6 bits, 4 for 5 bits).
// The plan pairs the codes of a lane's run greedily inside 32-code sub-runs (so that a sub-run never straddles a
// quantisation group); the few codes left without a partner are taken as consecutive pairs the longer way (shift,
// shift, byte permute, mask).  Register n of the run feeds MMA n / 2 (even n: k slots 2t, 2t + 1; odd n: 2t + 8,
// 2t + 9), so code c is staged at half 2 n + (0 | 1) of the run, pre-divided by 2^p.
#pragma once

#include <type_traits>

#include "qmv_mma.cuh"

namespace mlxq {

template <int BITS, int CL> struct CodePlan {
    static constexpr int NR = CL / 2;                     // A registers (code pairs) per row and run
    static constexpr int SUB = CL < 32 ? CL : 32;
    static constexpr int D = (16 + BITS - 1) / BITS;      // partner distance
    static constexpr int P1 = BITS * D - 16;              // the partner's bit position inside the high half
    int first[NR], second[NR];
    bool cheap[NR];
    int pos[CL], shl[CL];                                 // staged half and pre-scaling shift of code c of the run
    bool ok;
    __host__ __device__ constexpr CodePlan() : first{}, second{}, cheap{}, pos{}, shl{}, ok(true) {
        bool used[CL] = {};
        int n = 0;
        for (int base = 0; base < CL; base += SUB) {
            for (int i = base; i < base + SUB; i++) {
                if (used[i]) continue;
                const int j = i + D;
                if (j < base + SUB && !used[j] && P1 + BITS <= 10) {
                    first[n] = i; second[n] = j; cheap[n] = true;
                    pos[i] = 2 * n; shl[i] = 0;
                    pos[j] = 2 * n + 1; shl[j] = P1;
                    used[i] = used[j] = true;
                } else {
                    if (i + 1 >= base + SUB || used[i + 1]) { ok = false; used[i] = true; continue; }
                    first[n] = i; second[n] = i + 1; cheap[n] = false;
                    pos[i] = 2 * n; shl[i] = 0;
                    pos[i + 1] = 2 * n + 1; shl[i + 1] = 0;
                    used[i] = used[i + 1] = true;
                }
                n++;
            }
        }
        if (n != NR) ok = false;
    }
};

template <int BITS> constexpr bool planned_width() { return BITS == 3 || BITS == 5 || BITS == 6; }

// Register n of a row's run from the lane's words of that row.
template <int BITS, int CL, int N>
__device__ __forceinline__ uint32_t plan_reg(const uint32_t* w) {
    constexpr CodePlan<BITS, CL> P{};
    static_assert(P.ok, "no register plan for this width and run length");
    constexpr uint32_t M1 = (1u << BITS) - 1u;
    constexpr int bit = P.first[N] * BITS, wi = bit >> 5, sh = bit & 31;
    if constexpr (P.cheap[N]) {
        constexpr int top = sh + 16 + P.P1 + BITS;            // bits of the shifted word that are looked at
        uint32_t v;
        if constexpr (sh == 0) v = w[wi];
        else if constexpr (top <= 32) v = w[wi] >> sh;
        else v = __funnelshift_r(w[wi], w[wi + 1], sh);
        return v & (M1 | (M1 << (16 + P.P1)));
    } else {
        uint32_t v;
        if constexpr (sh == 0) v = w[wi];
        else if constexpr (sh + 2 * BITS <= 32) v = w[wi] >> sh;
        else v = __funnelshift_r(w[wi], w[wi + 1], sh);
        return __byte_perm(v, v << (16 - BITS), 0x7610) & (M1 * 0x00010001u);
    }
}

// The pair registers of MMA j of a run of CL codes: a_regs of qmv_mma.cuh for 2, 4 and 8 bits, the plan above otherwise.
template <int BITS, int CL, int J>
__device__ __forceinline__ void a_regs_run(const uint32_t* w, uint32_t& lo, uint32_t& hi) {
    if constexpr (planned_width<BITS>()) {
        lo = plan_reg<BITS, CL, 2 * J>(w);
        hi = plan_reg<BITS, CL, 2 * J + 1>(w);
    } else {
        a_regs<BITS>(w, J, lo, hi);
    }
}

template <int I, int N, int STEP, class F>
__device__ __forceinline__ void plan_static_for(F&& f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        plan_static_for<I + STEP, N, STEP>(f);
    }
}

// Eight consecutive activations (k a multiple of eight) into the staged order of a planned width.
template <int BITS, int CL>
__device__ __forceinline__ void stage8_plan(__half* col, int k, const float (&v)[8]) {
    const int u0 = k % CL;                                    // (CL is a power of two)
    __half* run = col + (k - u0);
    plan_static_for<0, CL, 8>([&](auto uc) {
        constexpr int U0 = decltype(uc)::value;
        if (u0 == U0) {
            constexpr CodePlan<BITS, CL> P{};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float sc = __int_as_float((127 - P.shl[U0 + i]) << 23);      // 2^-shift
                run[P.pos[U0 + i]] = __float2half_rn(v[i] * sc);
            }
        }
    });
}

}  // namespace mlxq
