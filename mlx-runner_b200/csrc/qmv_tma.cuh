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

// A CTA has NC consumer warps (8: two CTAs per SM, each with half the shared memory; 16: one CTA per SM,
// for calls whose staged activations need the room), then the producer warp, then the reducer warp.
constexpr int TMA_MAX_CONSUMERS = 16;
constexpr int TMA_MAX_STAGES = 12;                     // ring stages (one stage = 8 rows)
constexpr int TMA_SLOTS = 8;                           // most row blocks whose partial sums may be pending

#ifdef MLXQ_TRACE
// development aid: per-CTA timestamps of the pipeline's hand-offs (64 slots per CTA)
__device__ unsigned long long g_tma_trace[148 * 64];
#define TTRACE(slot) do { if (blockIdx.x < 148) g_tma_trace[blockIdx.x * 64 + (slot)] = global_ns(); } while (0)
#else
#define TTRACE(slot) do { } while (0)
#endif

#ifndef MLXQ_ABLATE
#define MLXQ_ABLATE 0      // development aid: bit mask of kernel parts to leave out when timing (results are then wrong)
#endif

struct TmaPlan {
    int ns;              // ring stages
    int rps;             // rows per stage: 16 (a whole block: three copies per block) or 8 (half a block, long rows)
    int w_bytes;         // a stage's packed weights
    int s_bytes;         // a stage's scales (or biases)
    int stage_bytes;     // w_bytes + 2 * s_bytes, rounded up to 128
    int off_xsum, off_csum, off_part, off_stage, off_bars;   // shared-memory offsets
    int off_zero;        // 256 bytes of zeros: the B fragment of lanes whose accumulator column is idle in a step
    int n_blocks;        // 16-row blocks
    int ksplit;          // consumer warps that share one block along K (16, 8 or 4); 16 / ksplit blocks are in work at once
    int slots;           // partial-sum slots in use (<= TMA_SLOTS)
    int consumers;       // consumer warps per CTA (8 or 16)
    int grid;            // CTAs to launch
    int rowsum;          // 1: one token in one column set -- consumers hand over 16 row sums instead of 16 x 8 entries
};

struct TmaBars {
    uint64_t full[TMA_MAX_STAGES];
    uint64_t empty[TMA_MAX_STAGES];
    uint64_t part_full[TMA_SLOTS];
    uint64_t part_empty[TMA_SLOTS];
    int abort_flag;
};

// Bounded wait until a peer's flag has reached `epoch` (flags only grow; the difference is taken signed so the
// counter may wrap).  On time-out the error word is set and the caller carries on: the host discards the result.
__device__ __forceinline__ void peer_flag_wait(const unsigned* flag, unsigned epoch, unsigned* err) {
    const uint64_t t0 = global_ns();
    for (;;) {
        unsigned seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
        if (static_cast<int>(seen - epoch) >= 0) return;
        if (global_ns() - t0 > WAIT_NS) { atomicOr(err, ERR_WAIT_TIMEOUT | ERR_PEER_FLAG); return; }
    }
}

template <int BITS, int NP, int NC>
__global__ void __launch_bounds__((NC + 2) * 32, NC == 8 ? 2 : 1)
qmv_tma_kernel(const MmaParams p, const TmaPlan tp) {
    constexpr int TMA_CONSUMERS = NC, TMA_PRODUCER = NC, TMA_REDUCER = NC + 1;
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

    // barriers are set up by one thread each
    if (threadIdx.x == 0) { TTRACE(0); bars->abort_flag = 0; }
    if (threadIdx.x < tp.ns) { mbar_init(&bars->full[threadIdx.x], 1); mbar_init(&bars->empty[threadIdx.x], tp.ksplit); }
    if (threadIdx.x >= 32 && threadIdx.x < 32 + TMA_SLOTS) {
        mbar_init(&bars->part_full[threadIdx.x - 32], tp.ksplit);
        mbar_init(&bars->part_empty[threadIdx.x - 32], 1);
    }
    if (threadIdx.x < 32 + TMA_SLOTS) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (threadIdx.x >= 64 && threadIdx.x < 128) reinterpret_cast<uint32_t*>(smem_tma + tp.off_zero)[threadIdx.x - 64] = 0u;
    __syncthreads();
    // Programmatic dependent launch: the next kernel of the stream (if it was launched to allow it) may be
    // scheduled as soon as every CTA of this grid is resident, so its prologue and its weight copies overlap
    // this grid's tail.  The other half of the contract is the griddepcontrol.wait below: nothing reads the
    // activations, the row bias or the gate vector, and nothing writes y, before the previous grid is complete.
    // The packed weights, scales and biases are read earlier: they are the layer's constants.
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // geometry of the column plan shared by consumers and reducer (see qmv_mma.cuh)
    const int gsh = p.gstep_shift, G = 1 << gsh, CY = p.cycle, spg_shift = p.spg_shift;
    const int cols_per_cycle = p.xn << gsh;

    if (warp == TMA_PRODUCER) {
        // ---- producer: six lanes, one bulk copy each per block (weights, scales, biases of each 8-row half) ----
        // A bulk copy costs its issuing thread ~70 ns, so the block's six copies leave from six lanes at once.
        // The lane that copies a half's weights also posts the half's byte count on its barrier; a copy that
        // lands before that only drives the count negative for a moment, the phase cannot complete without
        // the arrival.
        uint32_t n_it = 0;
        const int nh = 16 / tp.rps;                              // stages per block
        if (lane < 3 * nh) {
            const int h = lane / 3, j = lane - 3 * h;
            if (lane == 0) TTRACE(1);
            uint32_t it = h;
            for (int blk = blockIdx.x; blk < tp.n_blocks; blk += gridDim.x, it += nh) {
                const int st = it % tp.ns;
                if (it >= static_cast<uint32_t>(tp.ns))
                    mbar_wait(&bars->empty[st], ((it / tp.ns) - 1) & 1, &bars->abort_flag, p.err);
                // the stage's first row, resolved to its layer part (8-row stages: a missing second half re-reads the first)
                int r = min(blk * 16 + 8 * h, q.total_rows - tp.rps), pi = 0;
                if (q.n_parts > 1 && r >= q.part[0].rows) {
                    r -= q.part[0].rows; pi = 1;
                    if (q.n_parts > 2 && r >= q.part[1].rows) { r -= q.part[1].rows; pi = 2; }
                }
                uint8_t* dst = stages + static_cast<size_t>(st) * tp.stage_bytes;
                const size_t soff = static_cast<size_t>(r) * groups * sbytes;
                if (j == 0) {
                    mbar_expect_tx(&bars->full[st], tp.w_bytes + 2 * tp.s_bytes);
                    bulk_load(dst, q.part[pi].w + static_cast<size_t>(r) * row_bytes, tp.w_bytes, &bars->full[st]);
                } else if (j == 1) {
                    bulk_load(dst + tp.w_bytes, static_cast<const char*>(q.part[pi].s) + soff, tp.s_bytes, &bars->full[st]);
                } else {
                    bulk_load(dst + tp.w_bytes + tp.s_bytes, static_cast<const char*>(q.part[pi].b) + soff, tp.s_bytes, &bars->full[st]);
                }
                if (j == 0 && it < 12) TTRACE(2 + it);
            }
            n_it = it - h;
        }
        n_it = __shfl_sync(0xffffffffu, n_it, 0);
        __syncwarp();
        if (lane == 0) {
            // see every copy of the last ring turn land before leaving (bounded)
            const uint32_t first = n_it > static_cast<uint32_t>(tp.ns) ? n_it - tp.ns : 0;
            for (uint32_t j = first; j < n_it; j++) {
                const uint64_t t0 = global_ns();
                while (!mbar_try_wait(&bars->full[j % tp.ns], (j / tp.ns) & 1))
                    if (global_ns() - t0 > WAIT_NS) break;
            }
        }
        return;
    }

    if (warp == TMA_REDUCER) {
        // ---- reducer: adds a block's partials (fixed order), epilogue, store -----------------------------------
        asm volatile("griddepcontrol.wait;" ::: "memory");
        uint32_t bi = 0;
        const int per_tok = p.split << gsh;
        for (int blk = blockIdx.x; blk < tp.n_blocks; blk += gridDim.x, bi++) {
            const int slot = bi % tp.slots;
            float* blockpart = part + static_cast<size_t>(slot) * (tp.ksplit * NP * 128);
            mbar_wait_warp(&bars->part_full[slot], (bi / tp.slots) & 1, &bars->abort_flag, p.err);
            if (lane == 0 && bi < 6) TTRACE(44 + 2 * bi);
            if (tp.rowsum) {
                // single token: every consumer warp left its sixteen row sums; add them in warp order
                const float* rs = part + static_cast<size_t>(slot) * (tp.ksplit * 16);
                const int r = lane & 15;
                float v = 0.0f;
#pragma unroll
                for (int wv = 0; wv < NC; wv++) if (wv < tp.ksplit) v += rs[wv * 16 + r];
                const int row = blk * 16 + r;
                if (lane < 16 && row < q.total_rows) {
                    int pr = row, pi = 0;
                    if (q.n_parts > 1 && pr >= q.part[0].rows) {
                        pr -= q.part[0].rows; pi = 1;
                        if (q.n_parts > 2 && pr >= q.part[1].rows) { pr -= q.part[1].rows; pi = 2; }
                    }
                    if (q.has_bias) v += load_scalar(q.part[pi].bias, q.bias_dtype, pr);
                    if (q.e != nullptr) v = act_mul(q.act, v, __ldg(q.e + row));
                    store_scalar(q.y, q.y_dtype, row, v);
                    for (int pp = 0; pp < q.peer.n; pp++) store_scalar(q.peer.y[pp], q.y_dtype, row, v);
                }
                __syncwarp();
                if (lane == 0 && bi < 6) TTRACE(45 + 2 * bi);
                if (lane == 0) mbar_arrive(&bars->part_empty[slot]);
                continue;
            }
            // stage 1: entry-wise sum over the consumer warps, four entries per lane per pass
            float4 acc[NP];
#pragma unroll
            for (int ps = 0; ps < NP; ps++) {
                acc[ps] = *reinterpret_cast<const float4*>(blockpart + ps * 128 + lane * 4);
#pragma unroll 4
                for (int wv = 1; wv < tp.ksplit; wv++) {
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
                    for (int pp = 0; pp < q.peer.n; pp++)
                        store_scalar(q.peer.y[pp], q.y_dtype, static_cast<size_t>(tok) * q.y_stride + row, v);
                }
            }
            __syncwarp();
            if (lane == 0 && bi < 6) TTRACE(45 + 2 * bi);
            if (lane == 0) mbar_arrive(&bars->part_empty[slot]);
        }
        if (q.peer.n > 0) {
            // Sharded call: this CTA's rows are on their way to every peer's window.  The CTA that finishes last
            // publishes this rank's epoch in every peer's flag array.  Nobody waits here: the next call on the
            // communicator (or mlxq_comm_wait) waits for the peers' flags before it reads the gathered rows,
            // and by then its own weight copies are already in flight.
            __threadfence_system();
            __syncwarp();
            unsigned last = 0;
            if (lane == 0) last = atomicInc(q.peer.counter, gridDim.x - 1) == gridDim.x - 1 ? 1u : 0u;
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence_system();
                if (lane < q.peer.n)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(q.peer.flag[lane] + q.peer.rank), "r"(q.peer.epoch) : "memory");
            }
        }
        return;
    }

    // ---- consumers --------------------------------------------------------------------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int ctid = threadIdx.x;                                        // 0 .. 32 * TMA_CONSUMERS - 1
    constexpr int CTHREADS = TMA_CONSUMERS * 32;

    // Everything that does not depend on the activations comes first: under dependent launch it runs while the
    // previous kernel of the stream is still finishing.
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
    const int kw = warp % tp.ksplit, stream = warp / tp.ksplit, n_streams = TMA_CONSUMERS / tp.ksplit;
    const int s_begin = ((nblk * kw) / tp.ksplit) << spg_shift;
    const int s_end = ((nblk * (kw + 1)) / tp.ksplit) << spg_shift;
    const int gmin = (s_begin * KB) >> gs_shift;
    const int frag_off = g * static_cast<int>(row_bytes) + t * LB;       // row g of a half block, this lane's run
    const __half* zeros = reinterpret_cast<const __half*>(smem_tma + tp.off_zero);

    // Most calls drain once per block, after the warp's last step: everything about that drain but the block's
    // scale rows is then the same for every block and is worked out here, once.
    int n_drains = 0;
    for (int s = s_begin; s < s_end; s++)
        if (((s + 1) & ((1 << spg_shift) - 1)) == 0 && ((((s >> spg_shift) & cyc_mask) == cyc_mask) || s + 1 == s_end)) n_drains++;
    bool f_ok = false;
    int f_soff = 0;
    float2 f_xv = make_float2(0.0f, 0.0f);
    int f_xoff = -1;
    bool lane_fast = NP == 1 && pair16 && n_drains == 1;
    {
        const int s = s_end - 1, gblock = s >> spg_shift, cyc_s = gblock & cyc_mask;
        const int gbase = (((gblock - cyc_s) << spg_shift) * KB) >> gs_shift;
        const int glimit = ((s + 1) * KB) >> gs_shift;
        const int g0 = gbase + c_goff[0][0], g1 = gbase + c_goff[0][1];
        const bool ok0 = c_xc[0][0] >= 0 && g0 >= gmin && g0 < glimit;
        const bool ok1 = c_xc[0][1] >= 0 && g1 >= gmin && g1 < glimit;
        // a lane with one live column of its pair needs the general path: the whole warp stays on one path
        lane_fast = lane_fast && ok0 == ok1;
        f_ok = lane_fast && ok0;
        if (f_ok) {
            f_soff = 2 * (g * groups + g0);
            f_xoff = c_xc[0][0] * groups + g0;      // the sums themselves exist only after the staging below
        }
    }
    const bool fast_drain = __all_sync(0xffffffffu, lane_fast);
    f_ok = f_ok && fast_drain;

    // stage the activations once per CTA (see qmv_mma.cuh for the layout)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (q.peer.n > 0 && q.peer.wait_epoch != 0) {
        // the activations may be the previous sharded call's gathered output: every peer must have finished it
        if (warp == 0 && lane < q.peer.n) peer_flag_wait(q.peer.my_flags + q.peer.peer_rank[lane], q.peer.wait_epoch, p.err);
        asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
    }
    if (p.split == 1) {
        // 16-bit activations: eight values per thread; the chunks of a group sit in consecutive lanes, so the
        // per-group sums come from a few shuffles and one barrier suffices
        const int cpr = K / 8, total = (MLXQ_ABLATE & 4) ? 0 : q.T * cpr;
        const int cpg = 1 << (gs_shift - 3);
        for (int base = 0; base < total; base += CTHREADS) {
            const int idx = base + ctid;
            const int tok = idx / cpr, k = (idx - tok * cpr) * 8;
            float sum = 0.0f;
            if (idx < total) {
                float v[8];
                if (q.x_dtype == DT_F16) XLoad<__half>::load8(reinterpret_cast<const __half*>(q.x) + static_cast<size_t>(tok) * q.x_stride + k, v);
                else XLoad<__nv_bfloat16>::load8(reinterpret_cast<const __nv_bfloat16*>(q.x) + static_cast<size_t>(tok) * q.x_stride + k, v);
#pragma unroll
                for (int i = 0; i < 8; i++) sum += v[i];
                stage8<BITS>(xs + static_cast<size_t>(tok) * p.xstride, k, v);
            }
            for (int o = 1; o < cpg; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (idx < total && (idx & (cpg - 1)) == 0) xsum[tok * groups + (k >> gs_shift)] = sum;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
    } else {
        const int cpr = K / 8;
        for (int idx = ctid; idx < ((MLXQ_ABLATE & 4) ? 0 : q.T * cpr); idx += CTHREADS) {
            const int tok = idx / cpr, k = (idx - tok * cpr) * 8;
            float v[8];
            XLoad<float>::load8(reinterpret_cast<const float*>(q.x) + static_cast<size_t>(tok) * q.x_stride + k, v);
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) sum += v[i];
            csum[idx] = sum;
            float hi[8], lo[8];
#pragma unroll
            for (int i = 0; i < 8; i++) { hi[i] = __half2float(__float2half_rn(v[i])); lo[i] = v[i] - hi[i]; }
            stage8<BITS>(xs + static_cast<size_t>(2 * tok) * p.xstride, k, hi);
            stage8<BITS>(xs + static_cast<size_t>(2 * tok + 1) * p.xstride, k, lo);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
        const int cpg = 1 << (gs_shift - 3);
        for (int idx = ctid; idx < p.xn * groups; idx += CTHREADS) {
            const int xc = idx / groups, gi = idx - xc * groups;
            float sum = 0.0f;
            if ((xc & 1) == 0) {
                const int tok = xc >> 1;
                for (int i = 0; i < cpg; i++) sum += csum[tok * cpr + gi * cpg + i];
            }
            xsum[idx] = sum;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
    }

    if (ctid == 0) TTRACE(16);
    if (f_ok && f_xoff >= 0) f_xv = *reinterpret_cast<const float2*>(xsum + f_xoff);
    if (ctid == 0) TTRACE(17);
    // the CTA's blocks are dealt to the consumer groups in turn: group `stream` takes blocks stream, stream + n_streams, ...
    for (uint32_t bi = stream; blockIdx.x + static_cast<long long>(bi) * gridDim.x < tp.n_blocks; bi += n_streams) {
        // the block's stage(s): rows 0..7 and 8..15 with their scale and bias rows
        const bool two = tp.rps == 8;
        const uint32_t it = two ? 2 * bi : bi;
        const int st0 = it % tp.ns, st1 = two ? (it + 1) % tp.ns : st0;
        const uint8_t* half0 = stages + static_cast<size_t>(st0) * tp.stage_bytes;
        const uint8_t* half1 = two ? stages + static_cast<size_t>(st1) * tp.stage_bytes : half0 + 8 * row_bytes;
        const int s_half = two ? 0 : tp.s_bytes / 2;            // one 16-row stage: the second half's scale rows follow the first's
        const uint8_t* s_ptr[2] = {half0 + tp.w_bytes, (two ? half1 : half0) + tp.w_bytes + s_half};
        const uint8_t* b_ptr[2] = {s_ptr[0] + tp.s_bytes, s_ptr[1] + tp.s_bytes};
        constexpr int NCH = NP >= 4 ? 1 : 4 / NP;          // independent accumulator chains per pass (eight were no faster)
        float yacc[NP][4], c[NP][NCH][4];
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                yacc[ps][i] = 0.0f;
#pragma unroll
                for (int k = 0; k < NCH; k++) c[ps][k][i] = 0.0f;
            }
        // (The ring length is a multiple of the stages the consumer groups take per round, so a stage always
        // comes back to the same group and each group sees its stages' phases in order.  An earlier version let
        // stages change hands and first waited for the previous use's phase: when the current copy had already
        // landed, that wait was for a phase of the future and ran into its time limit.)
        mbar_wait_warp(&bars->full[st0], (it / tp.ns) & 1, &bars->abort_flag, p.err);
        if (two) mbar_wait_warp(&bars->full[st1], ((it + 1) / tp.ns) & 1, &bars->abort_flag, p.err);
        if (kw == 0 && lane == 0 && bi < 6) TTRACE(20 + 4 * bi);

        const uint8_t* f0 = half0 + frag_off + s_begin * (4 * LB);
        const uint8_t* f1 = half1 + frag_off + s_begin * (4 * LB);
        // the lane's words of both rows for one step
        auto load_words = [&](const uint8_t* p0, const uint8_t* p1, uint32_t (&w)[2][NW]) {
            if constexpr (LB == 16) {
                const uint4 v0 = *reinterpret_cast<const uint4*>(p0), v1 = *reinterpret_cast<const uint4*>(p1);
                w[0][0] = v0.x; w[0][1] = v0.y; w[0][2] = v0.z; w[0][3] = v0.w;
                w[1][0] = v1.x; w[1][1] = v1.y; w[1][2] = v1.z; w[1][3] = v1.w;
            } else {
#pragma unroll
                for (int i = 0; i < NW / 2; i++) {
                    const uint2 v0 = *(reinterpret_cast<const uint2*>(p0) + i), v1 = *(reinterpret_cast<const uint2*>(p1) + i);
                    w[0][2 * i] = v0.x; w[0][2 * i + 1] = v0.y;
                    w[1][2 * i] = v1.x; w[1][2 * i + 1] = v1.y;
                }
            }
        };
        // (optionally the next step's words are fetched while this step's MMAs run)
        constexpr bool PREFETCH = false;          // measured: fetching a step ahead costs 0.3 us per launch (11.7 vs 11.4)
        uint32_t wn[2][NW];
        if (PREFETCH && s_begin < s_end) load_words(f0, f1, wn);
        for (int s = s_begin; s < ((MLXQ_ABLATE & 2) ? s_begin : s_end); s++, f0 += 4 * LB, f1 += 4 * LB) {
            uint32_t w[2][NW];
            if constexpr (PREFETCH) {
#pragma unroll
                for (int i = 0; i < NW; i++) { w[0][i] = wn[0][i]; w[1][i] = wn[1][i]; }
                if (s + 1 < s_end) load_words(f0 + 4 * LB, f1 + 4 * LB, wn);
            } else {
                load_words(f0, f1, w);
            }
            const int gblock = s >> spg_shift;
            const int cyc_s = gblock & cyc_mask;
            const int koff = s * KB;
            // lanes whose accumulator column belongs to another group (or cycle) multiply by zeros: they read
            // them from a zeroed patch of shared memory, so the loads need no branch
            const __half* pa[NP];
            const __half* pb[NP];
#pragma unroll
            for (int ps = 0; ps < NP; ps++) {
                const bool on = b_cyc[ps] == cyc_s;
                pa[ps] = (keep_a[ps] && on) ? bptr[ps] + koff : zeros;
                pb[ps] = (keep_b[ps] && on) ? bptr[ps] + koff : zeros;
            }
#pragma unroll
            for (int j = 0; j < NM; j += 2) {
                uint32_t a00, a01, a02, a03, a10, a11, a12, a13;
                a_regs<BITS>(w[0], j, a00, a02);
                a_regs<BITS>(w[1], j, a01, a03);
                a_regs<BITS>(w[0], j + 1, a10, a12);
                a_regs<BITS>(w[1], j + 1, a11, a13);
#pragma unroll
                for (int ps = 0; ps < NP; ps++) {
                    uint4 bv;
                    if (MLXQ_ABLATE & 16) bv = make_uint4(0x3c003c00u, 0x3c003c00u, 0x3c003c00u + s, 0x3c003c00u);
                    else bv = *reinterpret_cast<const uint4*>((j < NM / 2 ? pa[ps] : pb[ps]) + 4 * j);
                    if (MLXQ_ABLATE & 64) {
                        c[ps][(j / 2) % NCH][0] += __uint_as_float((a00 ^ a01 ^ a02 ^ a03) + bv.x + bv.y);
                        c[ps][(j / 2 + (NCH > 1 ? NCH / 2 : 0)) % NCH][1] += __uint_as_float((a10 ^ a11 ^ a12 ^ a13) + bv.z + bv.w);
                        continue;
                    }
                    mma16816(c[ps][(j / 2) % NCH], a00, a01, a02, a03, bv.x, bv.y);
                    mma16816(c[ps][(j / 2 + (NCH > 1 ? NCH / 2 : 0)) % NCH], a10, a11, a12, a13, bv.z, bv.w);
                }
            }
            if (kw == 0 && lane == 0 && bi == 0 && s - s_begin < 6) TTRACE(56 + (s - s_begin));
            if (!(MLXQ_ABLATE & 1) && ((s + 1) & ((1 << spg_shift) - 1)) == 0 && (cyc_s == cyc_mask || s + 1 == s_end)) {
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
                    if (MLXQ_ABLATE & 8) {          // timing aid: keep the MMAs alive, leave out the scale / bias work
#pragma unroll
                        for (int i = 0; i < 4; i++) yacc[ps][i] += cs[i];
                        continue;
                    }
                    if (fast_drain) {
                        if (f_ok) {
#pragma unroll
                            for (int h = 0; h < 2; h++) {
                                const uint32_t su = *reinterpret_cast<const uint32_t*>(s_ptr[h] + f_soff);
                                const uint32_t bu = *reinterpret_cast<const uint32_t*>(b_ptr[h] + f_soff);
                                float2 sf, bf;
                                if (q.s_dtype == DT_F16) {
                                    sf = __half22float2(*reinterpret_cast<const __half2*>(&su));
                                    bf = __half22float2(*reinterpret_cast<const __half2*>(&bu));
                                } else {
                                    sf = make_float2(__uint_as_float(su << 16), __uint_as_float(su & 0xFFFF0000u));
                                    bf = make_float2(__uint_as_float(bu << 16), __uint_as_float(bu & 0xFFFF0000u));
                                }
                                yacc[ps][2 * h] += fmaf(bf.x, f_xv.x, sf.x * 16777216.0f * cs[2 * h]);
                                yacc[ps][2 * h + 1] += fmaf(bf.y, f_xv.y, sf.y * 16777216.0f * cs[2 * h + 1]);
                            }
                        }
                        continue;
                    }
                    const int g0 = gbase + c_goff[ps][0], g1 = gbase + c_goff[ps][1];
                    const bool ok0 = c_xc[ps][0] >= 0 && g0 >= gmin && g0 < glimit;
                    const bool ok1 = c_xc[ps][1] >= 0 && g1 >= gmin && g1 < glimit;
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint8_t* srows = s_ptr[h];                              // scales [8][groups] of this half
                        const uint8_t* brows = b_ptr[h];
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
        if (kw == 0 && lane == 0 && bi < 6) TTRACE(21 + 4 * bi);
        // both half blocks are consumed (weights in registers, scales applied): hand them back
        __syncwarp();
        if (lane == 0) { mbar_arrive(&bars->empty[st0]); if (two) mbar_arrive(&bars->empty[st1]); }

        // deliver the partial sums to the reducer
        const int slot = bi % tp.slots;
        if (bi >= static_cast<uint32_t>(tp.slots)) mbar_wait_warp(&bars->part_empty[slot], ((bi / tp.slots) - 1) & 1, &bars->abort_flag, p.err);
        if (tp.rowsum) {
            // one token: the eight accumulator columns of a row all belong to it -- add them across the quad
            float lo = yacc[0][0] + yacc[0][1], hi = yacc[0][2] + yacc[0][3];
            lo += __shfl_xor_sync(0xffffffffu, lo, 1); hi += __shfl_xor_sync(0xffffffffu, hi, 1);
            lo += __shfl_xor_sync(0xffffffffu, lo, 2); hi += __shfl_xor_sync(0xffffffffu, hi, 2);
            float* mine = part + (static_cast<size_t>(slot) * tp.ksplit + kw) * 16;
            if (t == 0) { mine[g] = lo; mine[g + 8] = hi; }
        } else {
            float* mine = part + (static_cast<size_t>(slot) * tp.ksplit + kw) * (NP * 128);
#pragma unroll
            for (int ps = 0; ps < NP; ps++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    mine[(ps * 16 + g + 8 * (i >> 1)) * 8 + 2 * t + (i & 1)] = yacc[ps][i];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->part_full[slot]);       // release semantics: the stores above are visible
        if (kw == 0 && lane == 0 && bi < 6) TTRACE(22 + 4 * bi);
    }
}

// Plans the shared-memory layout for a call; returns the bytes needed, 0 when the call does not fit.
size_t qmv_tma_plan(int bits, const MmaParams& p, int tokens, int sms, TmaPlan& tp);
cudaError_t launch_qmv_tma(int bits, const MmaParams& p, const TmaPlan& tp, size_t smem, cudaStream_t st);

}  // namespace mlxq
