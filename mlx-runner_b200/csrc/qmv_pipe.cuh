// Persistent decode matvec: the raw-code tensor-core inner loop of qmv_mma.cuh, fed through warp-private
// asynchronous copies and laid out so that consecutive launches of a stream overlap.
//
// One CTA per SM walks the layer's 16-row blocks.  `ks` consecutive warps form a group that shares a block along
// K; the groups of a CTA take alternate blocks.  A warp needs exactly the same bytes of every block -- per step, 64
// (4/8/2-bit), 96 (6/3-bit) or 160 (5-bit) bytes of each of its sixteen rows, plus the (scale, bias) pairs of its
// lanes' accumulator columns when a step ends a drain cycle -- so it fetches them with cp.async into a small ring of
// its own in shared memory, several steps ahead: the rows as 16-byte pieces dealt out over the lanes (whole sectors
// per copy instruction at every width), the pairs by the lanes that use them.  At 2, 4 and 8 bits a lane's pieces
// are exactly the bytes it consumes and nothing is shared between lanes: no barrier, no mbarrier, no fence, just
// cp.async.wait_group; at 3, 5 and 6 bits a __syncwarp on either side of the read orders the lanes.  The ring is
// deep enough to run across block boundaries, and its first turn is issued before griddepcontrol.wait, i.e. while
// the previous launch of the stream is still finishing (packed weights, scales and biases are the layer's
// constants); the activations, the gate vector and y are only touched after it.  The activations are staged once
// per CTA.  At the end of a block every warp of a group leaves a compact [16 rows x tokens] partial sum in shared
// memory, the group meets on its named barrier, and its first warp adds the partials in warp order, applies row
// bias / gate / output type and stores, while the others go on.
//
// The only device-side wait on another party is the peers' flag wait of sharded calls; it is bounded (the error
// word is set, control flow does not change, and the host discards the result through the error word).
#pragma once

#include <type_traits>

#include "code_plan.cuh"
#include "qmv_mma.cuh"
#include "sm100_ptx.cuh"

namespace mlxq {

struct PipePlan {
    int ks, ks_shift;    // warps that share a block along K (1, 2, 4, 8 or 16) and its log2
    int depth;           // ring slots per warp: PIPE_DEPTH, or 2 when the full ring does not fit
    int unroll;          // steps per turn of the main loop: 2 when every warp's slice holds an even number of steps, else 1
    int grid;
    int n_blocks;        // 16-row blocks; CTA b walks base_blocks (+ 1 if b < extra_blocks) of them
    int base_blocks, extra_blocks;
    int cpr_shift;       // log2(in_dim / 8) when that is a power of two, else -1
    int xstride;         // halves between staged activation columns
    int off_xsum;        // group sums [staged column][groups] floats
    int off_zero;        // PIPE_ZERO_BYTES of zeros: the B fragments of lanes whose accumulator column is idle in a step
    int off_scratch;     // per warp: accumulator tile [passes][16][9] floats
    int scratch_bytes;
    int off_part;        // partial sums [groups of warps][2][ks][16 * tokens] floats
    int off_ring;        // per warp: depth slots of 2 x 32 lanes x lane bytes, then 4 x 32 x 4 bytes of (scale, bias) pairs
    int rowsum;          // 1: one token in one accumulator set -- partials come from two shuffles instead of the tile
    int special;         // 32 / 64 / 128: the one-token kernel compiled for that group size serves the call; 0: the general one
    int async_sb;        // 1: the drains' (scale, bias) pairs travel through the ring (see pipe_col_pairs)
    // What accumulator column n of pass ps stands for (the column plan of qmv_mma.cuh, worked out once on the host):
    // bits 0-7 staged activation column (255: none), 8-15 group offset inside the cycle block, 16-19 cycle position,
    // 20-23 group inside the step.
    uint32_t col[4][8];
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

// The flag protocol of sharded calls.  Every rank owns word r of every rank's flag array and keeps in it the number of
// its fused calls whose rows are complete and visible everywhere.  A call does not publish itself: its kernel ends
// without any system-scope fence, and the NEXT kernel of the communicator on that rank (the next fused call, or the
// wait kernel of mlxq_comm_wait) publishes it right after its own start -- by then the grid that stored the rows is
// complete, so one release store by one thread covers all of them, and its latency overlaps the new kernel's work
// instead of stretching the old kernel's tail.  Hence word r >= e - 1 also says that rank r has STARTED call e, i.e.
// that everything it enqueued before call e (the readers of call e - 2's rows, whose buffer call e overwrites) is done.
__device__ __forceinline__ void peer_publish_previous(const PeerGather& pg, unsigned epoch) {
    if (blockIdx.x == 0 && threadIdx.x < static_cast<unsigned>(pg.n))
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pg.flag[threadIdx.x] + pg.rank), "r"(epoch - 1u) : "memory");
}

// End of a sharded call's CTA: nothing crosses the link here.  The CTA that arrives last at the local counter records
// the call's number on the device for the next launch (which reads it after the grid dependency).
__device__ __forceinline__ void peer_finish(const PeerGather& pg, unsigned epoch) {
    __syncthreads();
    if (threadIdx.x == 0 && pg.epoch_ctr != nullptr && atomicInc(pg.counter, gridDim.x - 1) == gridDim.x - 1)
        *reinterpret_cast<volatile unsigned*>(pg.epoch_ctr) = epoch;
}

// Eight consecutive activations as fp32 through the coherent path (ld.global.cg).  The kernel may be resident
// while the previous grid of the stream is still writing these values (dependent launch), and on sharded calls
// peers write them over NVLink: the non-coherent read-only path is only defined for data that nobody writes
// during the kernel's lifetime.
__device__ __forceinline__ void load8_coherent(const void* x, int dt, size_t index, float (&o)[8]) {
    if (dt == DT_F32) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + index));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + index) + 1);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
        return;
    }
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + index));
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
}

// The same in two halves, so that several chunks' loads can be in flight before the first is used: the raw 16 bytes
// (16-bit types) or 32 bytes (fp32), then the conversion.
__device__ __forceinline__ void load8_raw(const void* x, int dt, size_t index, uint4& a, uint4& b) {
    if (dt == DT_F32) {
        a = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(x) + index));
        b = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(x) + index) + 1);
    } else {
        a = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + index));
        b = a;
    }
}
__device__ __forceinline__ void raw_to_float8(int dt, const uint4& a, const uint4& b, float (&o)[8]) {
    if (dt == DT_F32) {
        o[0] = __uint_as_float(a.x); o[1] = __uint_as_float(a.y); o[2] = __uint_as_float(a.z); o[3] = __uint_as_float(a.w);
        o[4] = __uint_as_float(b.x); o[5] = __uint_as_float(b.y); o[6] = __uint_as_float(b.z); o[7] = __uint_as_float(b.w);
        return;
    }
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
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
}

// asynchronous copies global -> shared of 16, 8 and 4 bytes; DOFF / SOFF are constant byte offsets added to the addresses
template <int DOFF, int SOFF>
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%3], 16;" ::"r"(dst), "l"(src), "n"(DOFF), "n"(SOFF) : "memory");
}
template <int DOFF, int SOFF>
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0+%2], [%1+%3], 8;" ::"r"(dst), "l"(src), "n"(DOFF), "n"(SOFF) : "memory");
}
template <int DOFF>
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0+%1], [%2], 4;" ::"r"(dst), "n"(DOFF), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
constexpr int PIPE_WARPS = 16;
constexpr int PIPE_DEPTH = 4;        // ring slots (steps in flight) per warp
constexpr int PIPE_ZERO_BYTES = 1024; // zeroed patch: a step's B fragments of an idle lane, for both steps of an unrolled turn

// f(integral_constant<I>), f(integral_constant<I + STEP>), ... below N: a loop whose index is a constant expression
template <int I, int N, int STEP, class F>
__device__ __forceinline__ void static_for(F&& f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + STEP, N, STEP>(f);
    }
}

// stage8 of qmv_mma.cuh for a chunk that starts at a multiple of eight: except at 2 bits the eight values stay
// inside their own 16 bytes, so they are permuted and pre-scaled in registers and leave with one 128-bit store.
template <int BITS>
__device__ __forceinline__ void stage8v(__half* col, int k, const float (&v)[8]) {
    if constexpr (BITS == 2) {
        stage8<BITS>(col, k, v);
    } else {
        constexpr int UW = MmaUnit<BITS>::UW;
        __half h[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int u = i % UW;
            const float sc = __int_as_float((127 - stage_shift<BITS>(u)) << 23);     // 2^-shift
            h[i - u + stage_pos<BITS>(u)] = __float2half_rn(v[i] * sc);
        }
        uint4 o;
        o.x = __half_as_ushort(h[0]) | (static_cast<uint32_t>(__half_as_ushort(h[1])) << 16);
        o.y = __half_as_ushort(h[2]) | (static_cast<uint32_t>(__half_as_ushort(h[3])) << 16);
        o.z = __half_as_ushort(h[4]) | (static_cast<uint32_t>(__half_as_ushort(h[5])) << 16);
        o.w = __half_as_ushort(h[6]) | (static_cast<uint32_t>(__half_as_ushort(h[7])) << 16);
        *reinterpret_cast<uint4*>(col + k) = o;
    }
}

// stage8v for fp16 activations that are staged as they are (one staged column per token): the eight halves arrive as
// four words (x0,x1)(x2,x3)(x4,x5)(x6,x7) and leave permuted by byte permutes, the pre-scaling by a power of two is a
// half2 multiply -- the same values as the fp32 route (scaling by a power of two, then one rounding to fp16).
template <int BITS>
__device__ __forceinline__ void stage8v_f16(__half* col, int k, const uint32_t (&w)[4]) {
    static_assert(BITS != 2, "2-bit units span sixteen values");
    uint4 o;
    if constexpr (BITS == 4) {
        // order 0,4,1,5,2,6,3,7; the odd codes of a byte sit four bits up: their activations are divided by 16
        const __half2 sc = __floats2half2_rn(0.0625f, 0.0625f);
        const uint32_t a = __byte_perm(w[0], w[2], 0x7632), b = __byte_perm(w[1], w[3], 0x7632);
        const __half2 as = __hmul2(*reinterpret_cast<const __half2*>(&a), sc), bs = __hmul2(*reinterpret_cast<const __half2*>(&b), sc);
        o.x = __byte_perm(w[0], w[2], 0x5410);
        o.y = *reinterpret_cast<const uint32_t*>(&as);
        o.z = __byte_perm(w[1], w[3], 0x5410);
        o.w = *reinterpret_cast<const uint32_t*>(&bs);
    } else if constexpr (BITS == 8) {
        // order 0,2,1,3 inside every four
        o.x = __byte_perm(w[0], w[1], 0x5410);
        o.y = __byte_perm(w[0], w[1], 0x7632);
        o.z = __byte_perm(w[2], w[3], 0x5410);
        o.w = __byte_perm(w[2], w[3], 0x7632);
    } else {
        o = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(col + k) = o;
}

// staging of a chunk for a kernel whose lanes take runs of CL codes
template <int BITS, int CL>
__device__ __forceinline__ void stage8r(__half* col, int k, const float (&v)[8]) {
    if constexpr (planned_width<BITS>()) stage8_plan<BITS, CL>(col, k, v);
    else stage8v<BITS>(col, k, v);
}

constexpr int pipe_log2(int v) { int s = 0; while ((1 << s) < v) s++; return s; }

// GS = 0: any call, the column plan is read from the launch parameters.  GS = 32, 64, 128: the one-token call with
// 16-bit activations and 16-bit scales at that group size -- the plan is then known at compile time (one pass, a
// drain cycle of eight consecutive groups, the lane's two accumulator columns are groups 2t and 2t + 1 of it, the
// pairs travel through the ring), and most of the bookkeeping below folds away.
template <int BITS, int NP, int UNR, int GS>
__global__ void __launch_bounds__(PIPE_WARPS * 32, 1)
qmv_pipe_kernel(const __grid_constant__ MmaParams p, const __grid_constant__ PipePlan pp) {
    using U = MmaUnit<BITS>;
    constexpr int LB = U::LB, CL = U::CL, KB = U::KB, NW = U::NW, NM = U::NM;
    constexpr bool SP = GS != 0;
    static_assert(!SP || NP == 1, "the one-token plan has one pass");
    constexpr int SP_GSH = !SP ? 0 : (KB > GS ? pipe_log2(KB / GS) : 0);      // log2(groups per step)
    constexpr int SP_SPG = !SP ? 0 : (GS > KB ? pipe_log2(GS / KB) : 0);      // log2(steps per group)
    constexpr int SP_CY = !SP ? 1 : ((8 >> SP_GSH) > 0 ? (8 >> SP_GSH) : 1);  // group blocks per drain cycle
    // One-token plan: every slice holds whole drain cycles of SP_SPC steps (the planner sees to it) and starts on a
    // multiple of UNR, so within a loop turn only the last step can close a cycle when UNR divides SP_SPC; and both halves
    // of a step's MMAs read the same group when a lane's run does not straddle groups.
    constexpr int SP_SPC = SP_CY << SP_SPG;
    constexpr bool LAST_ONLY = SP && SP_SPC % UNR == 0;
    constexpr bool SAME_AB = SP && CL <= GS;
    constexpr int NT = PIPE_WARPS * 32;
    // ring slots per warp: PIPE_DEPTH, or two where the larger ring does not fit beside many tokens' activations
    const int depth = SP ? PIPE_DEPTH : pp.depth;
    constexpr int RB = 4 * LB;                                 // bytes of a row per step
    constexpr int PPR = RB / 16, NPT = RB / 32;                // 16-byte pieces per row; pieces per lane (16 rows)
    constexpr uint32_t SB_OFF = 2 * 32 * LB;                   // (scale, bias) pairs follow the weights in a slot
    constexpr uint32_t SLOT = SB_OFF + 4 * 32 * 4;
    extern __shared__ __align__(128) uint8_t smem_pipe[];
    const QmvParams& q = p.q;
    const int K = q.K, gs_shift = SP ? pipe_log2(GS) : q.gs_shift;
    const int groups = K >> gs_shift;
    const int sbytes = SP ? 2 : dtype_size(q.s_dtype);
    const int T = SP ? 1 : q.T, xn = SP ? 1 : p.xn, split = SP ? 1 : p.split;
    const bool rowsum = SP ? true : pp.rowsum != 0;
    __half* xs = reinterpret_cast<__half*>(smem_pipe);                                   // [xn][xstride]
    float* xsum = reinterpret_cast<float*>(smem_pipe + pp.off_xsum);                     // [xn][groups]
    float* part = reinterpret_cast<float*>(smem_pipe + pp.off_part);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int steps_total = K / KB;
    const size_t row_bytes = static_cast<size_t>(K) * BITS / 8;

    // Programmatic dependent launch: the next kernel of the stream (if it was launched to allow it) may be
    // scheduled as soon as every CTA of this grid has got here, so its first weight copies overlap this grid's
    // tail.  The other half of the contract is the griddepcontrol.wait below: nothing reads the activations or the
    // gate vector, and nothing writes y, before the previous grid is complete.  The packed weights, scales, biases
    // and the row bias are read earlier: they are the layer's constants.
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x < PIPE_ZERO_BYTES / 4) reinterpret_cast<uint32_t*>(smem_pipe + pp.off_zero)[threadIdx.x] = 0u;

    // geometry of the column plan (see qmv_mma.cuh)
    const int gsh = SP ? SP_GSH : p.gstep_shift, G = 1 << gsh, CY = SP ? SP_CY : p.cycle, spg_shift = SP ? SP_SPG : p.spg_shift;
    const int cols_per_cycle = xn << gsh;
    const int cyc_mask = CY - 1;
    const int dmask = (CY << spg_shift) - 1;                   // a drain closes every (dmask + 1) steps
    // this warp's place: group `gi` of the CTA, slice `kw` of K (cut at group boundaries)
    const int ks = pp.ks, gi = warp >> pp.ks_shift, kw = warp & (ks - 1), n_groups = PIPE_WARPS >> pp.ks_shift;   // (warps per CTA are a multiple of ks)
    const int nblk = steps_total >> spg_shift;
    const int s_begin = ((nblk * kw) >> pp.ks_shift) << spg_shift;
    const int s_end = ((nblk * (kw + 1)) >> pp.ks_shift) << spg_shift;
    const int nsteps = s_end - s_begin;
    const int gmin = (s_begin * KB) >> gs_shift;
    float* scr = reinterpret_cast<float*>(smem_pipe + pp.off_scratch + static_cast<size_t>(warp) * pp.scratch_bytes);
    // the warp's ring, addressed through the lane's own cell: 16 (or 8) bytes inside every row of cells of a slot
    // A step's bytes of the warp's sixteen rows lie row after row in a slot (RB bytes each); the warp copies them as
    // 16-byte pieces, lane l the pieces l, l + 32, ..., so that every copy instruction reads whole 32-byte sectors.
    // At 2, 4 and 8 bits a lane's pieces are exactly the bytes it consumes (rows g and g + 8, 16 bytes at 16 t); at
    // the other widths it consumes 24 or 40 bytes at LB * t of those rows, which other lanes copied.
    const uint32_t ring = smem_u32(smem_pipe + pp.off_ring) + warp * (depth * SLOT) + lane * 16;
    const uint32_t ring_end = ring + depth * SLOT;
    const uint32_t sb_delta = SB_OFF + lane * 4 - lane * 16;   // from there to the lane's first pair cell
    const uint32_t rd_delta = LB == 16 ? 0u : static_cast<uint32_t>(g * RB + t * LB - lane * 16);   // ... and to the bytes it consumes
    const uint32_t zaddr0 = smem_u32(smem_pipe + pp.off_zero);

    const int run_grp_a = ((t * CL + mma_code_offset<BITS>(0)) >> gs_shift) & (G - 1);
    const int run_grp_b = ((t * CL + mma_code_offset<BITS>(NM / 2)) >> gs_shift) & (G - 1);
    uint32_t baddr[NP];         // shared address of the lane's run inside the staged column it feeds as B
    int b_on_a[NP], b_on_b[NP]; // the cycle position in which the lane's column is live (-1: never), per half of the step's MMAs
    int c_xc[NP][2], c_goff[NP][2];
#pragma unroll
    for (int ps = 0; ps < NP; ps++) {
        const uint32_t ce = SP ? 0u : pp.col[ps][g];            // the column this lane feeds as B (column n = g)
        const int xc = SP ? 0 : ce & 255, cyc = SP ? g >> SP_GSH : (ce >> 16) & 15, grp = SP ? g & ((1 << SP_GSH) - 1) : (ce >> 20) & 15;
        const bool valid = SP ? (g >> SP_GSH) < SP_CY : xc != 255;
        baddr[ps] = smem_u32(xs) + ((valid ? xc : 0) * pp.xstride + t * CL) * 2;
        b_on_a[ps] = (valid && grp == run_grp_a) ? cyc : -1;
        b_on_b[ps] = (valid && grp == run_grp_b) ? cyc : -1;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint32_t cc = SP ? 0u : pp.col[ps][2 * t + ci];   // the lane's accumulator columns 2t, 2t + 1
            c_xc[ps][ci] = SP ? (((2 * t + ci) >> SP_GSH) < SP_CY ? 0 : -1) : (cc & 255) == 255 ? -1 : static_cast<int>(cc & 255);
            c_goff[ps][ci] = SP ? 2 * t + ci : (cc >> 8) & 255;
        }
    }
    const bool async_sb = SP ? true : pp.async_sb != 0;
    const int pair_off = c_goff[0][0];

    // the lane's row g + 8h of block `blk`, resolved to a layer part (rows past the end read the last row)
    auto locate = [&](int blk, int h, int& pi) -> int {
        int r = min(blk * 16 + g + 8 * h, q.total_rows - 1);
        pi = 0;
        if (q.n_parts > 1 && r >= q.part[0].rows) {
            r -= q.part[0].rows; pi = 1;
            if (q.n_parts > 2 && r >= q.part[1].rows) { r -= q.part[1].rows; pi = 2; }
        }
        return r;
    };

    // ---- the copy stream: this warp's (block, step) pairs in order, `depth` of them in flight ------------------------
    // block j of the CTA is blockIdx.x + j * gridDim.x; group gi takes j = gi, gi + n_groups, ...
    const int cta_blocks = pp.base_blocks + (static_cast<int>(blockIdx.x) < pp.extra_blocks ? 1 : 0);
    const int my_blocks = cta_blocks > gi ? (cta_blocks - 1 - gi) / n_groups + 1 : 0;
    const int blk_stride = n_groups * gridDim.x;
    int l_left = my_blocks * nsteps;                           // steps not yet issued
    int l_s = s_begin, l_blk = blockIdx.x + gi * gridDim.x;
    const uint8_t* l_w[NPT];                                   // the lane's pieces at the cursor's step
    const char* l_sp[2] = {nullptr, nullptr};
    const char* l_bp[2] = {nullptr, nullptr};
#pragma unroll
    for (int m = 0; m < NPT; m++) l_w[m] = nullptr;
    auto load_rows = [&](int blk) {
#pragma unroll
        for (int m = 0; m < NPT; m++) {
            // piece lane + 32 m of the block's step: row (of sixteen) and 16-byte part of that row
            const int pc = lane + 32 * m, rr = pc / PPR, part16 = pc - rr * PPR;
            int r = min(blk * 16 + rr, q.total_rows - 1), pi = 0;
            if (q.n_parts > 1 && r >= q.part[0].rows) {
                r -= q.part[0].rows; pi = 1;
                if (q.n_parts > 2 && r >= q.part[1].rows) { r -= q.part[1].rows; pi = 2; }
            }
            l_w[m] = q.part[pi].w + static_cast<size_t>(r) * row_bytes + part16 * 16 + static_cast<size_t>(s_begin) * RB;
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int pi;
            const int r = locate(blk, h, pi);
            if (async_sb) {
                const size_t off = static_cast<size_t>(r) * groups * sbytes;
                l_sp[h] = static_cast<const char*>(q.part[pi].s) + off;
                l_bp[h] = static_cast<const char*>(q.part[pi].b) + off;
            }
        }
    };
    // from the end of this warp's slice of one block to its start in the group's next block, in bytes
    const long long w_jump = static_cast<long long>(blk_stride) * 16 * static_cast<long long>(row_bytes) - static_cast<long long>(nsteps) * (4 * LB);
    const long long s_jump = static_cast<long long>(blk_stride) * 16 * groups * sbytes;
    // copies of the UNR steps under the load cursor into the slots that start at `dst`, one commit group; moves the cursor on
    auto issue_turn = [&](uint32_t dst) {
        if (l_left > 0) {
            static_for<0, UNR, 1>([&](auto ic) {
                constexpr int i = decltype(ic)::value;
                static_for<0, NPT, 1>([&](auto mc) {
                    constexpr int m = decltype(mc)::value;
                    cp_async16<i * SLOT + m * 512, i * RB>(dst, l_w[m]);
                });
                const int ls = l_s + i;
                if (async_sb && (!LAST_ONLY || i == UNR - 1) && ((((ls + 1) & dmask) == 0) || (!SP && ls + 1 == s_end))) {
                    // the step closes a drain cycle: the pair (g0, g0 + 1) is fetched when either group lies inside this
                    // warp's slice up to this step
                    const int g0 = (((ls & ~dmask) * KB) >> gs_shift) + pair_off;
                    if (c_xc[0][0] >= 0 && g0 + 1 >= gmin && g0 + 1 < groups && g0 < (((ls + 1) * KB) >> gs_shift)) {
                        const uint32_t d = dst + sb_delta;
                        cp_async4<i * SLOT>(d, l_sp[0] + 2 * g0);
                        cp_async4<i * SLOT + 128>(d, l_bp[0] + 2 * g0);
                        cp_async4<i * SLOT + 256>(d, l_sp[1] + 2 * g0);
                        cp_async4<i * SLOT + 384>(d, l_bp[1] + 2 * g0);
                    }
                }
            });
            l_left -= UNR; l_s += UNR;
#pragma unroll
            for (int m = 0; m < NPT; m++) l_w[m] += UNR * RB;
            if (l_s == s_end) {
                l_s = s_begin; l_blk += blk_stride;
                if (l_left > 0) {
                    if (q.n_parts == 1 && l_blk * 16 + 16 <= q.total_rows) {
                        // one part, a whole block inside the layer: the next block's rows are a constant distance on
#pragma unroll
                        for (int m = 0; m < NPT; m++) l_w[m] += w_jump;
                        if (async_sb) { l_sp[0] += s_jump; l_sp[1] += s_jump; l_bp[0] += s_jump; l_bp[1] += s_jump; }
                    } else {
                        load_rows(l_blk);
                    }
                }
            }
        }
        cp_commit();
    };
    if (l_left > 0) load_rows(l_blk);
#pragma unroll
    for (int gq = 0; gq < depth / UNR; gq++) issue_turn(ring + gq * (UNR * SLOT));

    // ---- the activations: nothing before this line reads x, e or writes y --------------------------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    unsigned peer_epoch = q.peer.epoch;
    if (q.peer.n > 0) {
        // The call's number on the communicator: from the device-side count of completed calls when there is one (the
        // previous grid, which wrote it, is complete here), so that a launch captured in a graph stays correct on replay.
        if (q.peer.epoch_ctr != nullptr) peer_epoch = *reinterpret_cast<volatile unsigned*>(q.peer.epoch_ctr) + 1u;
        peer_publish_previous(q.peer, peer_epoch);
        if (peer_epoch != 1u && q.peer.x_is_gathered) {
            // the activations are the previous sharded call's gathered output: every peer must have finished it
            if (warp == 0 && lane < q.peer.n) peer_flag_wait(q.peer.my_flags + q.peer.peer_rank[lane], peer_epoch - 1u, p.err);
            __syncthreads();
        }
    }
    // Otherwise the peers only have to have STARTED their previous call (this call's rows go where the rows of the
    // call before the previous one were, which a peer may read until its previous call runs): that wait is put off
    // until a warp stores its first rows, and ranks in step never spend time in it.
    bool peers_ready = q.peer.n == 0 || q.peer.x_is_gathered || peer_epoch == 1u;
    {
        // staged once per CTA: fp16, permuted and pre-scaled to match the A registers (see qmv_mma.cuh), eight
        // values per thread and turn.  The chunks of a group sit in consecutive lanes, so the per-group sums come
        // from a few shuffles, in a fixed order.
        const int cpr = K >> 3, total_chunks = T * cpr;
        const int cpg = 1 << (gs_shift - 3);
        for (int base = 0; base < total_chunks; base += NT) {
            const int idx = base + threadIdx.x;
            const int tok = T == 1 ? 0 : pp.cpr_shift >= 0 ? idx >> pp.cpr_shift : idx / cpr, k = (idx - tok * cpr) * 8;
            float sum = 0.0f;
            if (idx < total_chunks && (BITS == 4 || BITS == 8) && split == 1 && q.x_dtype == DT_F16) {
                // fp16 activations stay fp16: permute and pre-scale the words, the sum alone is formed in fp32
                const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(q.x) + static_cast<size_t>(tok) * q.x_stride + k));
                const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w4[i]));
                    sum += f.x;
                    sum += f.y;
                }
                if constexpr (BITS == 4 || BITS == 8) stage8v_f16<BITS>(xs + static_cast<size_t>(tok) * pp.xstride, k, w4);
            } else if (idx < total_chunks) {
                float v[8];
                load8_coherent(q.x, q.x_dtype, static_cast<size_t>(tok) * q.x_stride + k, v);
                if (q.x_up != nullptr) {
                    // gated input: the activation the layer sees is act(gate) * up, formed here instead of by a kernel of its own
                    float u[8];
                    load8_coherent(q.x_up, DT_F32, static_cast<size_t>(tok) * q.x_stride + k, u);
#pragma unroll
                    for (int i = 0; i < 8; i++) v[i] = act_mul(q.x_act, v[i], u[i]);
                }
#pragma unroll
                for (int i = 0; i < 8; i++) sum += v[i];
                if (split == 1) {
                    stage8r<BITS, CL>(xs + static_cast<size_t>(tok) * pp.xstride, k, v);
                } else {
                    float hi[8], lo[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) { hi[i] = __half2float(__float2half_rn(v[i])); lo[i] = v[i] - hi[i]; }
                    stage8r<BITS, CL>(xs + static_cast<size_t>(2 * tok) * pp.xstride, k, hi);
                    stage8r<BITS, CL>(xs + static_cast<size_t>(2 * tok + 1) * pp.xstride, k, lo);
                }
            }
            for (int o = 1; o < cpg; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (idx < total_chunks && (idx & (cpg - 1)) == 0) {
                const int gidx = k >> gs_shift;
                if (split == 1) {
                    xsum[tok * groups + gidx] = sum;
                } else {
                    xsum[(2 * tok) * groups + gidx] = sum;          // the lo column of an fp32 token carries no bias term
                    xsum[(2 * tok + 1) * groups + gidx] = 0.0f;
                }
            }
        }
    }
    __syncthreads();
    // (from here on the staged activations are read with loads the compiler may move: tie their addresses to this point)
    uint32_t zaddr = zaddr0;
    asm volatile("" : "+r"(zaddr) :: "memory");
#pragma unroll
    for (int ps = 0; ps < NP; ps++) asm volatile("" : "+r"(baddr[ps]) :: "memory");

    const int per_tok = split << gsh;
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

    // partial sums of this warp's group: two slots (the block's parity) of ks x [16 rows x tokens] floats
    const int par_floats = ks * 16 * T;
    float* part_g = part + gi * 2 * par_floats;
    uint32_t c_src = ring;                                      // ring slot of the step in work
    int c_blk = blockIdx.x + gi * gridDim.x;
    for (int bj = 0; bj < my_blocks; bj++, c_blk += blk_stride) {
        // scale / bias rows of the block, for drains whose pairs do not travel through the ring
        const char* gs_ptr[2] = {nullptr, nullptr};
        const char* gb_ptr[2] = {nullptr, nullptr};
        if (!async_sb) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                int pi;
                const int r = locate(c_blk, h, pi);
                const size_t off = static_cast<size_t>(r) * groups * sbytes;
                gs_ptr[h] = static_cast<const char*>(q.part[pi].s) + off;
                gb_ptr[h] = static_cast<const char*>(q.part[pi].b) + off;
            }
        }
        uint32_t koff2 = s_begin * (KB * 2);                    // byte offset of the step's codes inside a staged column
        for (int s0 = s_begin; s0 < s_end; s0 += UNR, koff2 += UNR * KB * 2) {
            // the turn's UNR steps have landed: their words (and, for steps that close a drain cycle, the pairs) to registers
            if (depth == PIPE_DEPTH) asm volatile("cp.async.wait_group %0;" ::"n"(PIPE_DEPTH / UNR - 1) : "memory");
            else asm volatile("cp.async.wait_group %0;" ::"n"(2 / UNR - 1) : "memory");
            if constexpr (LB != 16) __syncwarp();               // (the bytes a lane consumes were copied by other lanes)
            uint32_t w[UNR][2][NW];
            uint32_t sbv[UNR][4];                                // (read only where drains[i] holds)
            bool drains[UNR];
            static_for<0, UNR, 1>([&](auto ic) {
                constexpr int i = decltype(ic)::value;
                if constexpr (LB == 16) {
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];"
                                 : "=r"(w[i][0][0]), "=r"(w[i][0][1]), "=r"(w[i][0][2]), "=r"(w[i][0][3]) : "r"(c_src), "n"(i * SLOT));
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];"
                                 : "=r"(w[i][1][0]), "=r"(w[i][1][1]), "=r"(w[i][1][2]), "=r"(w[i][1][3]) : "r"(c_src), "n"(i * SLOT + 512));
                } else {
                    static_for<0, LB / 8, 1>([&](auto kc) {
                        constexpr int k = decltype(kc)::value;
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];"
                                     : "=r"(w[i][0][2 * k]), "=r"(w[i][0][2 * k + 1]) : "r"(c_src + rd_delta), "n"(i * SLOT + 8 * k));
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];"
                                     : "=r"(w[i][1][2 * k]), "=r"(w[i][1][2 * k + 1]) : "r"(c_src + rd_delta), "n"(i * SLOT + 8 * RB + 8 * k));
                    });
                }
                const int s = s0 + i;
                drains[i] = (!LAST_ONLY || i == UNR - 1) && (((s + 1) & dmask) == 0 || (!SP && s + 1 == s_end));
                if (async_sb && drains[i]) {
                    const uint32_t d = c_src + sb_delta;
                    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(sbv[i][0]) : "r"(d), "n"(i * SLOT));
                    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(sbv[i][1]) : "r"(d), "n"(i * SLOT + 128));
                    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(sbv[i][2]) : "r"(d), "n"(i * SLOT + 256));
                    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(sbv[i][3]) : "r"(d), "n"(i * SLOT + 384));
                }
            });
            static_for<0, UNR, 1>([&](auto ic) {
                constexpr int i = decltype(ic)::value;
                const int s = s0 + i;
                const bool drain = drains[i];
                const int cyc_s = (s >> spg_shift) & cyc_mask;
                // lanes whose accumulator column belongs to another group (or cycle) multiply by zeros: they read
                // them from a zeroed patch of shared memory, so the loads need no branch
                uint32_t pa[NP], pb[NP];
#pragma unroll
                for (int ps = 0; ps < NP; ps++) {
                    pa[ps] = b_on_a[ps] == cyc_s ? baddr[ps] + koff2 : zaddr;
                    pb[ps] = SAME_AB ? pa[ps] : b_on_b[ps] == cyc_s ? baddr[ps] + koff2 : zaddr;
                }
                static_for<0, NM, 2>([&](auto jc) {
                    constexpr int j = decltype(jc)::value;
                    uint32_t a00, a01, a02, a03, a10, a11, a12, a13;
                    a_regs_run<BITS, CL, j>(w[i][0], a00, a02);
                    a_regs_run<BITS, CL, j>(w[i][1], a01, a03);
                    a_regs_run<BITS, CL, j + 1>(w[i][0], a10, a12);
                    a_regs_run<BITS, CL, j + 1>(w[i][1], a11, a13);
#pragma unroll
                    for (int ps = 0; ps < NP; ps++) {
                        // (not volatile: the staged activations do not change after the barrier that follows the staging,
                        // and the addresses are made to depend on that barrier, so the compiler may schedule these freely)
                        uint4 bv;
                        asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];"
                            : "=r"(bv.x), "=r"(bv.y), "=r"(bv.z), "=r"(bv.w)
                            : "r"(j < NM / 2 ? pa[ps] : pb[ps]), "n"(8 * j + i * KB * 2));
                        mma16816(c[ps][(j / 2) % NCH], a00, a01, a02, a03, bv.x, bv.y);
                        mma16816(c[ps][(j / 2 + (NCH > 1 ? NCH / 2 : 0)) % NCH], a10, a11, a12, a13, bv.z, bv.w);
                    }
                });
                if (drain) {
                    // end of a group block that closes the cycle (or the warp's range): scale and bias in fp32
                    const int gbase = ((s & ~dmask) * KB) >> gs_shift;
                    const int glimit = ((s + 1) * KB) >> gs_shift;
#pragma unroll
                    for (int ps = 0; ps < NP; ps++) {
                        float cs[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            cs[k] = c[ps][0][k];
#pragma unroll
                            for (int ch = 1; ch < NCH; ch++) cs[k] += c[ps][ch][k];
#pragma unroll
                            for (int ch = 0; ch < NCH; ch++) c[ps][ch][k] = 0.0f;
                        }
                        const int g0 = gbase + c_goff[ps][0], g1 = gbase + c_goff[ps][1];
                        const bool ok0 = c_xc[ps][0] >= 0 && g0 >= gmin && g0 < glimit;
                        const bool ok1 = c_xc[ps][1] >= 0 && g1 >= gmin && g1 < glimit;
                        if (async_sb) {
                            // pairs from the ring (same group offset in every pass); a lane with one live column keeps that one
                            if (ok0 || ok1) {
                                const float2 xv = *reinterpret_cast<const float2*>(xsum + c_xc[ps][0] * groups + g0);
#pragma unroll
                                for (int h = 0; h < 2; h++) {
                                    const uint32_t su = sbv[i][2 * h], bu = sbv[i][2 * h + 1];
                                    float2 sf, bf;
                                    if (q.s_dtype == DT_F16) {
                                        sf = __half22float2(*reinterpret_cast<const __half2*>(&su));
                                        bf = __half22float2(*reinterpret_cast<const __half2*>(&bu));
                                    } else {
                                        sf = make_float2(__uint_as_float(su << 16), __uint_as_float(su & 0xFFFF0000u));
                                        bf = make_float2(__uint_as_float(bu << 16), __uint_as_float(bu & 0xFFFF0000u));
                                    }
                                    if (ok0) yacc[ps][2 * h] += fmaf(bf.x, xv.x, sf.x * 16777216.0f * cs[2 * h]);
                                    if (ok1) yacc[ps][2 * h + 1] += fmaf(bf.y, xv.y, sf.y * 16777216.0f * cs[2 * h + 1]);
                                }
                            }
                        } else {
#pragma unroll
                            for (int h = 0; h < 2; h++) {
#pragma unroll
                                for (int ci = 0; ci < 2; ci++) {
                                    const int gg = ci ? g1 : g0;
                                    if (ci ? ok1 : ok0) {
                                        const float sc = load_scalar(gs_ptr[h], q.s_dtype, gg) * 16777216.0f;
                                        const float bs = load_scalar(gb_ptr[h], q.s_dtype, gg);
                                        yacc[ps][2 * h + ci] += fmaf(bs, xsum[c_xc[ps][ci] * groups + gg], sc * cs[2 * h + ci]);
                                    }
                                }
                            }
                        }
                    }
                }
            });
            // the turn's slots are in registers: refill them with the steps that are `depth` ahead
            if constexpr (LB != 16) __syncwarp();               // (... in every lane's registers)
            issue_turn(c_src);
            c_src += UNR * SLOT;
            if (c_src == ring_end) c_src = ring;
        }
        // ---- end of a block: this warp's partial sums, compact [16 rows][tokens], to the group's first warp ----------
        float* slot_base = part_g + ((bj & 1) ? par_floats : 0);
        float* mine = slot_base + kw * (16 * T);
        if (rowsum) {
            // one token: the eight accumulator columns of a row all belong to it -- add them across the quad
            float lo = yacc[0][0] + yacc[0][1], hi = yacc[0][2] + yacc[0][3];
            lo += __shfl_xor_sync(0xffffffffu, lo, 1); hi += __shfl_xor_sync(0xffffffffu, hi, 1);
            lo += __shfl_xor_sync(0xffffffffu, lo, 2); hi += __shfl_xor_sync(0xffffffffu, hi, 2);
            if (t == 0) { mine[g] = lo; mine[g + 8] = hi; }
        } else {
            // through the warp's private tile: a token's columns are, for every cycle, the contiguous run
            // [cyc * cols_per_cycle + tok * per_tok, + per_tok) of linear columns
#pragma unroll
            for (int ps = 0; ps < NP; ps++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    scr[(ps * 16 + g + 8 * (i >> 1)) * 9 + 2 * t + (i & 1)] = yacc[ps][i];
            __syncwarp();
            for (int idx = lane; idx < 16 * T; idx += 32) {
                const int tok = idx >> 4, r = idx & 15;
                float v = 0.0f;
                for (int cyc = 0; cyc < CY; cyc++) {
                    const int base = cyc * cols_per_cycle + tok * per_tok;
                    for (int j = 0; j < per_tok; j++) {
                        const int lin = base + j;
                        v += scr[((lin >> 3) * 16 + r) * 9 + (lin & 7)];
                    }
                }
                mine[idx] = v;
            }
            __syncwarp();
        }
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int i = 0; i < 4; i++) yacc[ps][i] = 0.0f;
        // The group meets on its own named barrier (which also orders the partial sums in shared memory); the two
        // parities of the slot keep a warp that runs ahead from overwriting sums the first warp still reads.
        if (ks > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(ks * 32) : "memory");
        else __syncwarp();
        if (kw == 0) {
            if (!peers_ready) {
                if (lane < q.peer.n) peer_flag_wait(q.peer.my_flags + q.peer.peer_rank[lane], peer_epoch - 2u, p.err);
                __syncwarp();
                peers_ready = true;
            }
            for (int idx = lane; idx < 16 * T; idx += 32) {
                const int tok = idx >> 4, r = idx & 15;
                const int row = c_blk * 16 + r;
                float v = 0.0f;
                for (int wv = 0; wv < ks; wv++) v += slot_base[wv * (16 * T) + idx];
                if (row < q.total_rows) {
                    int pr = row, pi = 0;
                    if (q.n_parts > 1 && pr >= q.part[0].rows) {
                        pr -= q.part[0].rows; pi = 1;
                        if (q.n_parts > 2 && pr >= q.part[1].rows) { pr -= q.part[1].rows; pi = 2; }
                    }
                    if (q.has_bias) v += load_scalar(q.part[pi].bias, q.bias_dtype, pr);
                    if (q.e != nullptr) v = act_mul(q.act, v, __ldcg(q.e + row));
                    const size_t at = static_cast<size_t>(tok) * q.y_stride + row;
                    store_scalar(q.y, q.y_dtype, at, v);
                    for (int pp_ = 0; pp_ < q.peer.n; pp_++) store_scalar(q.peer.y[pp_], q.y_dtype, at, v);
                }
            }
            __syncwarp();
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    if (q.peer.n > 0) peer_finish(q.peer, peer_epoch);
}

// Plans the launch and the shared-memory layout for a call; returns the bytes needed, 0 when the call does not fit.
size_t qmv_pipe_plan(int bits, const MmaParams& p, int tokens, int sms, PipePlan& pp);
cudaError_t launch_qmv_pipe(int bits, const MmaParams& p, const PipePlan& pp, size_t smem, int device, cudaStream_t st);

}  // namespace mlxq
