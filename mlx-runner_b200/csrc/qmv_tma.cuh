// Persistent decode matvec: the tensor-core inner loop of qmv_mma.cuh fed by TMA bulk copies.
//
// One CTA per SM walks the layer's 16-row blocks.  Eight consecutive rows of the packed matrix are one
// contiguous run of memory, and so are their scales and their biases, so a PRODUCER warp moves each half
// block with three large cp.async.bulk copies into a shared-memory ring (a B200 issues a bulk copy only
// every ~70 ns, so few large copies, not one per row).  The bytes in flight are bounded by shared memory
// (well over 100 KB per SM) instead of by registers, and HBM stays busy while the sixteen CONSUMER warps
// unpack, multiply and drain.  Consumers split a block along K, read their A fragments from the ring
// with 128-bit shared loads, run the raw-code MMAs against the staged activations (four independent
// accumulator chains: a dependent mma.m16n8k16 chain costs ~80 cycles per link on this part), apply the
// per-group scale and bias in fp32 from the staged scale rows, and leave their partial sums in shared
// memory.  A REDUCER warp adds the sixteen partials of a block in a fixed order and writes the outputs,
// so no consumer ever waits for another.  The activations are staged once per CTA.
//
// Hand-offs are mbarriers (full / empty per ring stage, full / empty per partial-sum slot).  Every wait is
// bounded: when one runs out the CTA raises its abort flag and the device error word; control flow does
// not change, later waits return at once, and the result is discarded by the host through the error word.
#pragma once

#include "qmv_mma.cuh"
#include "sm100_ptx.cuh"

namespace mlxq {

constexpr int TMA_CONSUMERS = 16;                      // consumer warps (K splits of a block)
constexpr int TMA_PRODUCER = TMA_CONSUMERS;            // warp index of the producer
constexpr int TMA_REDUCER = TMA_CONSUMERS + 1;         // warp index of the reducer
constexpr int TMA_THREADS = (TMA_CONSUMERS + 2) * 32;
constexpr int TMA_MAX_STAGES = 12;                     // ring stages (one stage = 8 rows)
constexpr int TMA_SLOTS = 4;                           // row blocks whose partial sums may be pending

struct TmaPlan {
    int ns;              // ring stages (half blocks)
    int w_bytes;         // 8 rows of packed weights
    int s_bytes;         // 8 rows of scales (or of biases)
    int stage_bytes;     // w_bytes + 2 * s_bytes, rounded up to 128
    int off_xsum, off_csum, off_part, off_stage, off_bars;   // shared-memory offsets
    int n_blocks;        // 16-row blocks
};

struct TmaBars {
    uint64_t full[TMA_MAX_STAGES];
    uint64_t empty[TMA_MAX_STAGES];
    uint64_t part_full[TMA_SLOTS];
    uint64_t part_empty[TMA_SLOTS];
    int abort_flag;
};

template <int BITS, int NP>
__global__ void __launch_bounds__(TMA_THREADS, 1)
qmv_tma_kernel(const MmaParams p, const TmaPlan tp) {
    using U = MmaUnit<BITS>;
    constexpr int LB = U::LB, CL = U::CL, KB = U::KB, NW = U::NW, NM = U::NM;
    extern __shared__ __align__(128) uint8_t smem_tma[];
    const QmvParams& q = p.q;
    const int K = q.K, gs_shift = q.gs_shift;
    const int groups = K >> gs_shift;
    const int sbytes = dtype_size(q.s_dtype);
    __half* xs = reinterpret_cast<__half*>(smem_tma);
    float* xsum = reinterpret_cast<float*>(smem_tma + tp.off_xsum);
    float* csum = reinterpret_cast<float*>(smem_tma + tp.off_csum);
    float* part = reinterpret_cast<float*>(smem_tma + tp.off_part);      // [TMA_SLOTS][consumers][NP][16][8]
    uint8_t* stages = smem_tma + tp.off_stage;
    TmaBars* bars = reinterpret_cast<TmaBars*>(smem_tma + tp.off_bars);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int steps_total = K / KB;
    const size_t row_bytes = static_cast<size_t>(K) * BITS / 8;

    if (threadIdx.x == 0) {
        for (int i = 0; i < tp.ns; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], TMA_CONSUMERS); }
        for (int i = 0; i < TMA_SLOTS; i++) { mbar_init(&bars->part_full[i], TMA_CONSUMERS); mbar_init(&bars->part_empty[i], 1); }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // geometry of the column plan shared by consumers and reducer (see qmv_mma.cuh)
    const int gsh = p.gstep_shift, G = 1 << gsh, CY = p.cycle, spg_shift = p.spg_shift;
    const int cols_per_cycle = p.xn << gsh;

    if (warp == TMA_PRODUCER) {
        // ---- producer: three bulk copies per half block (weights, scales, biases of 8 consecutive rows) -----
        if (lane == 0) {
            uint32_t it = 0;
            for (int blk = blockIdx.x; blk < tp.n_blocks; blk += gridDim.x) {
                for (int h = 0; h < 2; h++, it++) {
                    const int st = it % tp.ns;
                    if (it >= static_cast<uint32_t>(tp.ns))
                        mbar_wait(&bars->empty[st], ((it / tp.ns) - 1) & 1, &bars->abort_flag, p.err);
                    // the half's first row, resolved to its layer part (a missing second half re-reads the first)
                    int r = min(blk * 16 + 8 * h, q.total_rows - 8), pi = 0;
                    if (q.n_parts > 1 && r >= q.part[0].rows) {
                        r -= q.part[0].rows; pi = 1;
                        if (q.n_parts > 2 && r >= q.part[1].rows) { r -= q.part[1].rows; pi = 2; }
                    }
                    uint8_t* dst = stages + static_cast<size_t>(st) * tp.stage_bytes;
                    const size_t soff = static_cast<size_t>(r) * groups * sbytes;
                    mbar_expect_tx(&bars->full[st], tp.w_bytes + 2 * tp.s_bytes);
                    bulk_load(dst, q.part[pi].w + static_cast<size_t>(r) * row_bytes, tp.w_bytes, &bars->full[st]);
                    bulk_load(dst + tp.w_bytes, static_cast<const char*>(q.part[pi].s) + soff, tp.s_bytes, &bars->full[st]);
                    bulk_load(dst + tp.w_bytes + tp.s_bytes, static_cast<const char*>(q.part[pi].b) + soff, tp.s_bytes, &bars->full[st]);
                }
            }
            // see every copy of the last ring turn land before leaving (bounded)
            const uint32_t first = it > static_cast<uint32_t>(tp.ns) ? it - tp.ns : 0;
            for (uint32_t j = first; j < it; j++) {
                const uint64_t t0 = global_ns();
                while (!mbar_try_wait(&bars->full[j % tp.ns], (j / tp.ns) & 1))
                    if (global_ns() - t0 > WAIT_NS) break;
            }
        }
        return;
    }

    if (warp == TMA_REDUCER) {
        // ---- reducer: adds a block's sixteen partials (fixed order), epilogue, store ----------------------------
        uint32_t bi = 0;
        const int per_tok = p.split << gsh;
        for (int blk = blockIdx.x; blk < tp.n_blocks; blk += gridDim.x, bi++) {
            const int slot = bi % TMA_SLOTS;
            float* blockpart = part + static_cast<size_t>(slot) * (TMA_CONSUMERS * NP * 128);
            mbar_wait_warp(&bars->part_full[slot], (bi / TMA_SLOTS) & 1, &bars->abort_flag, p.err);
            // stage 1: entry-wise sum over the consumer warps, four entries per lane per pass
            float4 acc[NP];
#pragma unroll
            for (int ps = 0; ps < NP; ps++) {
                acc[ps] = *reinterpret_cast<const float4*>(blockpart + ps * 128 + lane * 4);
#pragma unroll
                for (int wv = 1; wv < TMA_CONSUMERS; wv++) {
                    const float4 o = *reinterpret_cast<const float4*>(blockpart + (wv * NP + ps) * 128 + lane * 4);
                    acc[ps].x += o.x; acc[ps].y += o.y; acc[ps].z += o.z; acc[ps].w += o.w;
                }
            }
            __syncwarp();
#pragma unroll
            for (int ps = 0; ps < NP; ps++) *reinterpret_cast<float4*>(blockpart + ps * 128 + lane * 4) = acc[ps];
            __syncwarp();
            // stage 2: one (row, token) per lane and turn.  A token's columns are, for every cycle, the
            // contiguous run [cyc * cols_per_cycle + tok * per_tok, + per_tok) of linear columns.
            for (int idx = lane; idx < 16 * q.T; idx += 32) {
                const int tok = idx >> 4, r = idx & 15;
                const int row = blk * 16 + r;
                float v = 0.0f;
                for (int cyc = 0; cyc < CY; cyc++) {
                    const int base = cyc * cols_per_cycle + tok * per_tok;
                    for (int j = 0; j < per_tok; j++) {
                        const int lin = base + j;
                        v += blockpart[((lin >> 3) * 16 + r) * 8 + (lin & 7)];
                    }
                }
                if (row < q.total_rows) {
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
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->part_empty[slot]);
        }
        return;
    }

    // ---- consumers --------------------------------------------------------------------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int ctid = threadIdx.x;                                        // 0 .. 32 * TMA_CONSUMERS - 1
    constexpr int CTHREADS = TMA_CONSUMERS * 32;

    // stage the activations once per CTA (see qmv_mma.cuh for the layout)
    {
        const int cpr = K / 8;
        for (int idx = ctid; idx < q.T * cpr; idx += CTHREADS) {
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
        asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
        const int cpg = 1 << (gs_shift - 3);
        for (int idx = ctid; idx < p.xn * groups; idx += CTHREADS) {
            const int xc = idx / groups, gi = idx - xc * groups;
            float sum = 0.0f;
            if (p.split == 1 || (xc & 1) == 0) {
                const int tok = p.split == 1 ? xc : (xc >> 1);
                for (int i = 0; i < cpg; i++) sum += csum[tok * cpr + gi * cpg + i];
            }
            xsum[idx] = sum;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
    }

    // column bookkeeping, identical to qmv_mma_kernel
    const int run_grp_a = ((t * CL + mma_code_offset<BITS>(0)) >> gs_shift) & (G - 1);
    const int run_grp_b = ((t * CL + mma_code_offset<BITS>(NM / 2)) >> gs_shift) & (G - 1);
    const __half* bptr[NP];
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
    const int cyc_mask = CY - 1;
    // The lane's two accumulator columns are consecutive groups of the same staged column (every layout with
    // two or more groups per cycle block), groups even-aligned, scales stored in 16 bits: loads can be paired.
    bool pair16 = q.s_dtype != DT_F32 && (groups & 1) == 0;
#pragma unroll
    for (int ps = 0; ps < NP; ps++)
        pair16 = pair16 && c_xc[ps][0] == c_xc[ps][1] && c_goff[ps][1] == c_goff[ps][0] + 1 && (c_goff[ps][0] & 1) == 0;

    // this warp's steps of every block, cut at group boundaries
    const int nblk = steps_total >> spg_shift;
    const int s_begin = ((nblk * warp) / TMA_CONSUMERS) << spg_shift;
    const int s_end = ((nblk * (warp + 1)) / TMA_CONSUMERS) << spg_shift;
    const int gmin = (s_begin * KB) >> gs_shift;
    const int frag_off = g * static_cast<int>(row_bytes) + t * LB;       // row g of a half block, this lane's run

    uint32_t it = 0, bi = 0;
    for (int blk = blockIdx.x; blk < tp.n_blocks; blk += gridDim.x, bi++, it += 2) {
        const int st0 = it % tp.ns, st1 = (it + 1) % tp.ns;
        const uint8_t* half0 = stages + static_cast<size_t>(st0) * tp.stage_bytes;   // rows 0..7: weights | scales | biases
        const uint8_t* half1 = stages + static_cast<size_t>(st1) * tp.stage_bytes;   // rows 8..15
        constexpr int NCH = NP >= 4 ? 1 : 4 / NP;          // independent accumulator chains per pass
        float yacc[NP][4], c[NP][NCH][4];
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                yacc[ps][i] = 0.0f;
#pragma unroll
                for (int k = 0; k < NCH; k++) c[ps][k][i] = 0.0f;
            }
        mbar_wait_warp(&bars->full[st0], (it / tp.ns) & 1, &bars->abort_flag, p.err);
        mbar_wait_warp(&bars->full[st1], ((it + 1) / tp.ns) & 1, &bars->abort_flag, p.err);

        const uint8_t* f0 = half0 + frag_off + s_begin * (4 * LB);
        const uint8_t* f1 = half1 + frag_off + s_begin * (4 * LB);
        for (int s = s_begin; s < s_end; s++, f0 += 4 * LB, f1 += 4 * LB) {
            uint32_t w[2][NW];
            if constexpr (LB == 16) {
                const uint4 v0 = *reinterpret_cast<const uint4*>(f0), v1 = *reinterpret_cast<const uint4*>(f1);
                w[0][0] = v0.x; w[0][1] = v0.y; w[0][2] = v0.z; w[0][3] = v0.w;
                w[1][0] = v1.x; w[1][1] = v1.y; w[1][2] = v1.z; w[1][3] = v1.w;
            } else {
#pragma unroll
                for (int i = 0; i < NW / 2; i++) {
                    const uint2 v0 = *(reinterpret_cast<const uint2*>(f0) + i), v1 = *(reinterpret_cast<const uint2*>(f1) + i);
                    w[0][2 * i] = v0.x; w[0][2 * i + 1] = v0.y;
                    w[1][2 * i] = v1.x; w[1][2 * i + 1] = v1.y;
                }
            }
            const int gblock = s >> spg_shift;
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
                    mma16816(c[ps][(j / 2) % NCH], a00, a01, a02, a03, bv.x, bv.y);
                    mma16816(c[ps][(j / 2 + (NCH > 1 ? NCH / 2 : 0)) % NCH], a10, a11, a12, a13, bv.z, bv.w);
                }
            }
            if (((s + 1) & ((1 << spg_shift) - 1)) == 0 && (cyc_s == cyc_mask || s + 1 == s_end)) {
                // end of a group block that closes the cycle (or the warp's range): scale and bias in fp32
                const int gbase = (((gblock - cyc_s) << spg_shift) * KB) >> gs_shift;
                const int glimit = ((s + 1) * KB) >> gs_shift;
#pragma unroll
                for (int ps = 0; ps < NP; ps++) {
                    float cs[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        cs[i] = c[ps][0][i];
#pragma unroll
                        for (int k = 1; k < NCH; k++) cs[i] += c[ps][k][i];
#pragma unroll
                        for (int k = 0; k < NCH; k++) c[ps][k][i] = 0.0f;
                    }
                    const int g0 = gbase + c_goff[ps][0], g1 = gbase + c_goff[ps][1];
                    const bool ok0 = c_xc[ps][0] >= 0 && g0 >= gmin && g0 < glimit;
                    const bool ok1 = c_xc[ps][1] >= 0 && g1 >= gmin && g1 < glimit;
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint8_t* srows = (h ? half1 : half0) + tp.w_bytes;      // scales [8][groups], then biases
                        const uint8_t* brows = srows + tp.s_bytes;
                        if (pair16 && ok0 && ok1) {
                            const size_t si = static_cast<size_t>(g) * groups + g0;
                            const uint32_t su = *reinterpret_cast<const uint32_t*>(srows + 2 * si);
                            const uint32_t bu = *reinterpret_cast<const uint32_t*>(brows + 2 * si);
                            float2 sf, bf;
                            if (q.s_dtype == DT_F16) {
                                sf = __half22float2(*reinterpret_cast<const __half2*>(&su));
                                bf = __half22float2(*reinterpret_cast<const __half2*>(&bu));
                            } else {
                                sf = make_float2(__uint_as_float(su << 16), __uint_as_float(su & 0xFFFF0000u));
                                bf = make_float2(__uint_as_float(bu << 16), __uint_as_float(bu & 0xFFFF0000u));
                            }
                            const float2 xv = *reinterpret_cast<const float2*>(xsum + c_xc[ps][0] * groups + g0);
                            yacc[ps][2 * h] += fmaf(bf.x, xv.x, sf.x * 16777216.0f * cs[2 * h]);
                            yacc[ps][2 * h + 1] += fmaf(bf.y, xv.y, sf.y * 16777216.0f * cs[2 * h + 1]);
                        } else {
#pragma unroll
                            for (int ci = 0; ci < 2; ci++) {
                                const int gg = ci ? g1 : g0;
                                if (ci ? ok1 : ok0) {
                                    const size_t si = static_cast<size_t>(g) * groups + gg;
                                    const float sc = smem_scalar(srows, q.s_dtype, si) * 16777216.0f;
                                    const float bs = smem_scalar(brows, q.s_dtype, si);
                                    yacc[ps][2 * h + ci] += fmaf(bs, xsum[c_xc[ps][ci] * groups + gg], sc * cs[2 * h + ci]);
                                }
                            }
                        }
                    }
                }
            }
        }
        // both half blocks are consumed (weights in registers, scales applied): hand them back
        __syncwarp();
        if (lane == 0) { mbar_arrive(&bars->empty[st0]); mbar_arrive(&bars->empty[st1]); }

        // deliver the partial sums to the reducer
        const int slot = bi % TMA_SLOTS;
        if (bi >= TMA_SLOTS) mbar_wait_warp(&bars->part_empty[slot], ((bi / TMA_SLOTS) - 1) & 1, &bars->abort_flag, p.err);
        float* mine = part + (static_cast<size_t>(slot) * TMA_CONSUMERS + warp) * (NP * 128);
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int i = 0; i < 4; i++)
                mine[(ps * 16 + g + 8 * (i >> 1)) * 8 + 2 * t + (i & 1)] = yacc[ps][i];
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->part_full[slot]);       // release semantics: the stores above are visible
    }
}

// Plans the shared-memory layout for a call; returns the bytes needed, 0 when the call does not fit.
size_t qmv_tma_plan(int bits, const MmaParams& p, int tokens, TmaPlan& tp);
cudaError_t launch_qmv_tma(int bits, const MmaParams& p, const TmaPlan& tp, size_t smem, int sms, cudaStream_t st);

}  // namespace mlxq
