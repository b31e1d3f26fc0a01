// Persistent decode matvec: the tensor-core inner loop of qmv_mma.cuh fed by TMA bulk copies.
//
// One CTA per SM walks the layer's 16-row blocks.  A producer warp streams each block's packed rows (in K
// chunks), scales and biases into a shared-memory ring with cp.async.bulk; the bytes in flight are bounded by
// shared memory (well over 100 KB per SM) instead of by registers, so HBM stays busy while the eight
// consumer warps unpack, multiply and drain.  Consumers split every chunk along K, read their A fragments
// from the ring with 128-bit shared loads (row stride padded to 64 mod 128 bytes: conflict-free), run the
// raw-code MMAs against the staged activations, apply the per-group scale and bias in fp32 from the staged
// scale rows, and meet in shared memory once per row block.  The activations are staged once per CTA.
//
// Hand-offs are mbarriers (full / empty per ring stage and per scale buffer).  Every wait is bounded: when
// one runs out the CTA raises its abort flag and the device error word; control flow does not change (so
// the consumers' named barrier always matches), later waits return at once, and the result is discarded by
// the host through the error word.
#pragma once

#include "qmv_mma.cuh"
#include "sm100_ptx.cuh"

namespace mlxq {

constexpr int TMA_CONSUMERS = 8;                       // consumer warps (K splits of a chunk)
constexpr int TMA_THREADS = (TMA_CONSUMERS + 1) * 32;  // + one producer warp
constexpr int TMA_MAX_STAGES = 8;

struct TmaPlan {
    int ns;              // ring stages
    int kc_steps;        // steps per K chunk
    int n_chunks;        // chunks per row block
    int wstride;         // bytes between rows inside a stage
    int chunk_bytes;     // bytes of one row's chunk (full chunks)
    int half_scale_bytes;// bytes of 8 rows of scales (or biases)
    int off_xsum, off_csum, off_part, off_stage, off_scale, off_bars;   // shared-memory offsets
    int stage_bytes, scale_buf_bytes;
    int n_blocks;        // 16-row blocks
};

struct TmaBars {
    uint64_t full[TMA_MAX_STAGES];
    uint64_t empty[TMA_MAX_STAGES];
    uint64_t full_s[2];
    uint64_t empty_s[2];
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
    float* part = reinterpret_cast<float*>(smem_tma + tp.off_part);      // [2][consumers][NP][16][8]
    uint8_t* stages = smem_tma + tp.off_stage;
    uint8_t* scale_bufs = smem_tma + tp.off_scale;                       // [2]{ scales[16][groups], biases[16][groups] }
    TmaBars* bars = reinterpret_cast<TmaBars*>(smem_tma + tp.off_bars);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int steps_total = K / KB;
    const size_t row_bytes = static_cast<size_t>(K) * BITS / 8;

    if (threadIdx.x == 0) {
        for (int i = 0; i < tp.ns; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], TMA_CONSUMERS); }
        for (int i = 0; i < 2; i++) { mbar_init(&bars->full_s[i], 1); mbar_init(&bars->empty_s[i], TMA_CONSUMERS); }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == TMA_CONSUMERS) {
        // ---- producer: one lane issues every bulk copy ------------------------------------------------------
        if (lane == 0) {
            uint32_t it = 0, bi = 0;
            for (int blk = blockIdx.x; blk < tp.n_blocks; blk += gridDim.x, bi++) {
                const int row0 = blk * 16;
                const int valid = min(16, q.total_rows - row0);          // 16 or 8 (parts hold multiples of 8 rows)
                // resolve the two 8-row halves to their layer parts
                const uint8_t* wbase[2]; const char* sbase[2]; const char* bbase[2];
                for (int h = 0; h < 2; h++) {
                    int r = min(row0 + 8 * h, q.total_rows - 8), pi = 0;
                    if (q.n_parts > 1 && r >= q.part[0].rows) {
                        r -= q.part[0].rows; pi = 1;
                        if (q.n_parts > 2 && r >= q.part[1].rows) { r -= q.part[1].rows; pi = 2; }
                    }
                    wbase[h] = q.part[pi].w + static_cast<size_t>(r) * row_bytes;
                    sbase[h] = static_cast<const char*>(q.part[pi].s) + static_cast<size_t>(r) * groups * sbytes;
                    bbase[h] = static_cast<const char*>(q.part[pi].b) + static_cast<size_t>(r) * groups * sbytes;
                }
                // scales and biases of the block (8 rows per copy: contiguous and 16-byte aligned)
                {
                    const int sb = bi & 1;
                    if (bi >= 2) mbar_wait(&bars->empty_s[sb], ((bi >> 1) - 1) & 1, &bars->abort_flag, p.err);
                    uint8_t* dst = scale_bufs + sb * tp.scale_buf_bytes;
                    const int halves = valid > 8 ? 2 : 1;
                    mbar_expect_tx(&bars->full_s[sb], 2u * halves * tp.half_scale_bytes);
                    for (int h = 0; h < halves; h++) {
                        bulk_load(dst + h * tp.half_scale_bytes, sbase[h], tp.half_scale_bytes, &bars->full_s[sb]);
                        bulk_load(dst + 2 * tp.half_scale_bytes + h * tp.half_scale_bytes, bbase[h], tp.half_scale_bytes, &bars->full_s[sb]);
                    }
                }
                for (int ch = 0; ch < tp.n_chunks; ch++, it++) {
                    const int st = it % tp.ns;
                    if (it >= static_cast<uint32_t>(tp.ns))
                        mbar_wait(&bars->empty[st], ((it / tp.ns) - 1) & 1, &bars->abort_flag, p.err);
                    const int step0 = ch * tp.kc_steps;
                    const int nsteps = min(tp.kc_steps, steps_total - step0);
                    const uint32_t bytes = static_cast<uint32_t>(nsteps) * (4 * LB);
                    uint8_t* dst = stages + static_cast<size_t>(st) * tp.stage_bytes;
                    mbar_expect_tx(&bars->full[st], bytes * valid);
                    for (int r = 0; r < valid; r++)
                        bulk_load(dst + r * tp.wstride, wbase[r >> 3] + static_cast<size_t>(r & 7) * row_bytes + static_cast<size_t>(step0) * (4 * LB),
                                  bytes, &bars->full[st]);
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

    // ---- consumers --------------------------------------------------------------------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int ctid = threadIdx.x;                                        // 0..255
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
    const int gsh = p.gstep_shift, G = 1 << gsh, CY = p.cycle, spg_shift = p.spg_shift;
    const int cols_per_cycle = p.xn << gsh;
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

    uint32_t it = 0, bi = 0;
    for (int blk = blockIdx.x; blk < tp.n_blocks; blk += gridDim.x, bi++) {
        const int row_blk = blk * 16;
        const int sb = bi & 1;
        const uint8_t* sc_rows = scale_bufs + sb * tp.scale_buf_bytes;               // scales [16][groups]
        const uint8_t* bi_rows = sc_rows + 2 * tp.half_scale_bytes;                  // biases [16][groups]
        float yacc[NP][4], c[NP][4];
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int i = 0; i < 4; i++) { yacc[ps][i] = 0.0f; c[ps][i] = 0.0f; }

        for (int ch = 0; ch < tp.n_chunks; ch++, it++) {
            const int st = it % tp.ns;
            const int step0 = ch * tp.kc_steps;
            const int nsteps = min(tp.kc_steps, steps_total - step0);
            // this warp's steps of the chunk, cut at group boundaries
            const int nblk = nsteps >> spg_shift;
            const int s_begin = step0 + (((nblk * warp) / TMA_CONSUMERS) << spg_shift);
            const int s_end = step0 + (((nblk * (warp + 1)) / TMA_CONSUMERS) << spg_shift);
            mbar_wait(&bars->full[st], (it / tp.ns) & 1, &bars->abort_flag, p.err);
            if (ch == 0) mbar_wait(&bars->full_s[sb], (bi >> 1) & 1, &bars->abort_flag, p.err);
            const uint8_t* wst = stages + static_cast<size_t>(st) * tp.stage_bytes + t * LB;
            const int gmin = (s_begin * KB) >> gs_shift;
            for (int s = s_begin; s < s_end; s++) {
                uint32_t w[2][NW];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint8_t* src = wst + (g + 8 * h) * tp.wstride + (s - step0) * (4 * LB);
                    if constexpr (LB == 16) {
                        const uint4 v = *reinterpret_cast<const uint4*>(src);
                        w[h][0] = v.x; w[h][1] = v.y; w[h][2] = v.z; w[h][3] = v.w;
                    } else {
#pragma unroll
                        for (int i = 0; i < NW / 2; i++) {
                            const uint2 v = *(reinterpret_cast<const uint2*>(src) + i);
                            w[h][2 * i] = v.x; w[h][2 * i + 1] = v.y;
                        }
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
                        mma16816(c[ps], a00, a01, a02, a03, bv.x, bv.y);
                        mma16816(c[ps], a10, a11, a12, a13, bv.z, bv.w);
                    }
                }
                if (((s + 1) & ((1 << spg_shift) - 1)) == 0 && (cyc_s == cyc_mask || s + 1 == s_end)) {
                    const int gbase = (((gblock - cyc_s) << spg_shift) * KB) >> gs_shift;
                    const int glimit = ((s + 1) * KB) >> gs_shift;
#pragma unroll
                    for (int ps = 0; ps < NP; ps++)
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int ci = i & 1, h = i >> 1;
                            const int gg = gbase + c_goff[ps][ci];
                            if (c_xc[ps][ci] >= 0 && gg >= gmin && gg < glimit) {
                                const size_t si = static_cast<size_t>(g + 8 * h) * groups + gg;
                                const float sc = smem_scalar(sc_rows, q.s_dtype, si) * 16777216.0f;
                                const float bs = smem_scalar(bi_rows, q.s_dtype, si);
                                yacc[ps][i] += fmaf(bs, xsum[c_xc[ps][ci] * groups + gg], sc * c[ps][i]);
                            }
                            c[ps][i] = 0.0f;
                        }
                }
            }
            // the stage's weights are in registers / consumed: hand it back to the producer
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->empty[st]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->empty_s[sb]);

        // reduce the K splits and the group / hi-lo columns, then the epilogue
        float* mypart = part + static_cast<size_t>(bi & 1) * (TMA_CONSUMERS * NP * 128);
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int i = 0; i < 4; i++)
                mypart[((warp * NP + ps) * 16 + g + 8 * (i >> 1)) * 8 + 2 * t + (i & 1)] = yacc[ps][i];
        asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
        for (int idx = ctid; idx < 16 * q.T; idx += CTHREADS) {
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
                        for (int wv = 0; wv < TMA_CONSUMERS; wv++) v += mypart[((wv * NP + ps) * 16 + r) * 8 + col];
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
}

// Plans the shared-memory layout for a call; returns the bytes needed, 0 when the call does not fit.
size_t qmv_tma_plan(int bits, const MmaParams& p, int tokens, TmaPlan& tp);
cudaError_t launch_qmv_tma(int bits, const MmaParams& p, const TmaPlan& tp, size_t smem, int sms, cudaStream_t st);

}  // namespace mlxq
