// Decode matvec for small batches (2 ... 16 tokens): the raw-code tensor-core inner loop of qmv_mma.cuh with the
// eight accumulator columns standing for eight TOKENS, and the quantisation groups separated in time.
//
// The one-token kernel (qmv_pipe.cuh) spends its spare accumulator columns on groups; with eight tokens there are no
// spare columns, and a step of that kernel's size mixes two or four groups in the k dimension of one MMA.  Here a
// step IS one group: lane (g, t) consumes GS / 4 codes of rows g and g + 8 (4 ... 32 bytes, the four lanes of a row
// one contiguous run of GS codes; the warp copies the sixteen rows' bytes piece-wise, see below), the group's MMAs
// accumulate into fresh registers, and the drain is four FMAs per eight tokens: yacc += scale[row, group] * c.  The bias term sum_g bias[row, g] * xsum[g, token] is a small matrix
// product of its own: eight groups at a time go through one mma.m16n8k8 in TF32 -- a 16-bit bias is exact in TF32,
// and the fp32 group sums of the activations are split into three TF32 parts (11 + 11 + 2 mantissa bits), so the
// products are exact and the sum is an fp32 sum like the FMA chain it replaces.
//
// The (scale, bias) values of a block's rows travel once per block: for every window of eight groups lane (g, t)
// copies the pairs (groups 2t, 2t + 1 of the window) of rows g and g + 8 into a cell of its own -- which is exactly
// the A fragment of the bias MMA -- and hands a group's scales to the other lanes of its row by shuffle.  Everything
// else (warp-private cp.async rings, K split over `ks` warps with a named barrier per group of warps, dependent
// launch, the peers' stores of sharded calls) is as in qmv_pipe.cuh.
#pragma once

#include "qmv_pipe.cuh"

namespace mlxq {

constexpr int TOK_WARPS = 16;

struct TokPlan {
    int ks, ks_shift;    // warps that share a block along K and its log2
    int depth;           // ring slots (groups in flight) per warp: 8, 4 or 2
    int ntab;            // buffers of the per-block (scale, bias) cells: blocks the copy cursor may run ahead, plus two
    int nwin;            // windows of eight groups per warp slice
    int slice_groups;    // groups of the longest warp slice (slices are cut at even groups: floor(pairs * kw / ks) * 2)
    int grid, n_blocks, base_blocks, extra_blocks;
    int cpr_shift;       // log2(in_dim / 8) when that is a power of two, else -1
    int xstride;         // halves between staged activation columns
    int tp;              // floats per row of a partial-sum tile (tokens + 1)
    int gpad;            // floats per staged column of a part of the group sums (groups + 8, the tail zero)
    int off_parts;       // [3][staged columns][gpad] floats: the TF32 parts of the activations' group sums
    int off_zero;        // PIPE_ZERO_BYTES of zeros (B fragments of idle columns)
    int parities;        // partial-sum slots per group of warps: 2 (alternating by block), or 1 where shared memory is short
    int off_part;        // partial sums [groups of warps][parities][ks][16 * tp] floats
    int off_tab;         // per warp: ntab x nwin cells of 32 lanes x 16 bytes
    int off_ring;        // per warp: depth slots of 2 rows x 32 lanes x group bytes
};

template <int BITS, int GS> struct TokUnit {
    static constexpr int GB = GS * BITS / 32;                                   // bytes of one group per lane and row (4 ... 32, or 6 / 10)
    static constexpr bool WORDS = GB % 4 == 0;                                  // the lane's run starts on a word of its row
    static constexpr int PS = GB % 16 == 0 ? 16 : GB % 8 == 0 ? 8 : 4;          // bytes per shared load of the run
    static constexpr int NPC = WORDS ? GB / PS : (GB + 2 + 3) / 4;              // loads per row (unaligned runs: the words that hold run + 16 bits)
    static constexpr int NW = (GB + 3) / 4;                                     // 32-bit words of a run
    static constexpr int CL = GS / 4;                                           // codes per lane and group
    static constexpr int NM = CL / 4;                                           // MMAs per group
    static constexpr int RB = 4 * GB;                                           // bytes of a row per group
    static constexpr int PIECE = RB % 16 == 0 && GB != 8 ? 16 : 8;              // bytes per asynchronous copy (8-byte runs: every lane copies its own)
    static constexpr bool SUPPORTED = (GS * BITS) % 64 == 0 && GB >= 4 && NM >= 2 && NM % 2 == 0 && (WORDS || planned_width<BITS>());
    static constexpr uint32_t SLOT = 16 * RB;
};

template <int PS, int DOFF, int SOFF>
__device__ __forceinline__ void cp_async_piece(uint32_t dst, const void* src) {
    if constexpr (PS == 16) cp_async16<DOFF, SOFF>(dst, src);
    else if constexpr (PS == 8) cp_async8<DOFF, SOFF>(dst, src);
    else asm volatile("cp.async.ca.shared.global [%0+%2], [%1+%3], 4;" ::"r"(dst), "l"(src), "n"(DOFF), "n"(SOFF) : "memory");
}

// d = a * b with a zero accumulator in, and d += a * b: m16n8k16, fp16 operands, fp32 accumulators
__device__ __forceinline__ void mma16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// d += a * b: m16n8k8, TF32 operands (fp32 bit patterns whose low 13 mantissa bits are zero), fp32 accumulators
__device__ __forceinline__ void mma1688_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// DEPTH_CT: the ring depth when it is the width's usual one (compiled in), 0 when the planner had to take a shallower ring.
template <int BITS, int GS, int NP, int DEPTH_CT>
__global__ void __launch_bounds__(TOK_WARPS * 32, 1)
qmv_tok_kernel(const __grid_constant__ MmaParams p, const __grid_constant__ TokPlan tp) {
    using U = TokUnit<BITS, GS>;
    static_assert(U::SUPPORTED, "no token-major kernel for this width and group size");
    constexpr int GB = U::GB, PS = U::PS, NPC = U::NPC, NW = U::NW, NM = U::NM, CL = U::CL;
    constexpr uint32_t SLOT = U::SLOT;
    constexpr int NT = TOK_WARPS * 32;
    constexpr int GSH = pipe_log2(GS);
    extern __shared__ __align__(128) uint8_t smem_tok[];
    const QmvParams& q = p.q;
    const int K = q.K, groups = K >> GSH;
    const int T = q.T, xn = p.xn, split = p.split;
    __half* xs = reinterpret_cast<__half*>(smem_tok);                                    // [xn][xstride]
    float* parts = reinterpret_cast<float*>(smem_tok + tp.off_parts);                    // [3][xn][gpad]
    float* part = reinterpret_cast<float*>(smem_tok + tp.off_part);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const size_t row_bytes = static_cast<size_t>(K) * BITS / 8;
    const int depth = DEPTH_CT ? DEPTH_CT : tp.depth, ntab = tp.ntab, nwin = tp.nwin, TP = tp.tp, gpad = tp.gpad;

    // Dependent launch, as in qmv_pipe.cuh: the layer's constants are fetched before griddepcontrol.wait, the
    // activations, the gate vector and y are touched after it.
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x < PIPE_ZERO_BYTES / 4) reinterpret_cast<uint32_t*>(smem_tok + tp.off_zero)[threadIdx.x] = 0u;

    // this warp's place: group `gi` of warps in the CTA, slice `kw` of K
    const int ks = tp.ks, gi = warp >> tp.ks_shift, kw = warp & (ks - 1), n_groups = TOK_WARPS >> tp.ks_shift;
    // the slice: quantisation groups [gmin, gmin + slice_groups), cut at even groups so that (scale, bias) pairs stay whole
    const int gmin = (((groups >> 1) * kw) >> tp.ks_shift) << 1;
    const int slice_groups = ((((groups >> 1) * (kw + 1)) >> tp.ks_shift) << 1) - gmin;
    // A group's bytes of the warp's sixteen rows lie row after row in a slot (RB bytes each); the warp copies them as
    // 16-byte pieces, lane l the pieces l, l + 32, ... below NPIECE, so that the copies read whole sectors whatever
    // the width; a lane then consumes GB bytes at GB * t of rows g and g + 8, which other lanes may have copied.
    // (Rows of 24 or 40 bytes per group -- 3- and 5-bit at group 64, 6-bit at group 32 -- go as 8-byte pieces, and a
    // lane's 6- or 10-byte run then starts on a half word: it loads the words around it and shifts by 0 or 16 bits.)
    constexpr int RB = U::RB, PIECE = U::PIECE, PPR = RB / PIECE, NPIECE = 16 * PPR, NPT = (NPIECE + 31) / 32;
    constexpr bool OWN_BYTES = GB == 16 || GB == 8;            // the lane's pieces are exactly the bytes it consumes
    const uint32_t ring = smem_u32(smem_tok + tp.off_ring) + warp * (depth * SLOT) + lane * PIECE;
    const uint32_t ring_end = ring + depth * SLOT;
    const uint32_t rd_delta = static_cast<uint32_t>(g * RB + ((t * GB) & ~3) - lane * PIECE);
    const uint32_t rd_shift = static_cast<uint32_t>(((t * GB) & 3) * 8);     // 0 or 16 (0 when the run starts on a word)
    const uint32_t tab = smem_u32(smem_tok + tp.off_tab) + warp * (ntab * nwin * 512) + lane * 16;
    const uint32_t zaddr0 = smem_u32(smem_tok + tp.off_zero);
    const bool s_f16 = q.s_dtype == DT_F16;
    // The lane's (scale, bias) cells start as zeros and the copies only ever fill the pairs inside the slice, so a
    // window's tail past the slice multiplies by zero.
    for (int c = 0; c < ntab * nwin; c++) asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(tab + c * 512), "r"(0u) : "memory");

    auto locate = [&](int blk, int h, int& pi) -> int {
        int r = min(blk * 16 + g + 8 * h, q.total_rows - 1);
        pi = 0;
        if (q.n_parts > 1 && r >= q.part[0].rows) {
            r -= q.part[0].rows; pi = 1;
            if (q.n_parts > 2 && r >= q.part[1].rows) { r -= q.part[1].rows; pi = 2; }
        }
        return r;
    };

    // ---- the copy stream: this warp's (block, group) pairs in order, `depth` groups in flight -------------------
    const int cta_blocks = tp.base_blocks + (static_cast<int>(blockIdx.x) < tp.extra_blocks ? 1 : 0);
    const int my_blocks = cta_blocks > gi ? (cta_blocks - 1 - gi) / n_groups + 1 : 0;
    const int blk_stride = n_groups * gridDim.x;
    int l_left = my_blocks * slice_groups;                     // groups not yet issued
    int l_g = 0, l_blk = blockIdx.x + gi * gridDim.x, l_tab = 0;
    const uint8_t* l_w[NPT];                                   // the lane's pieces at the cursor's group
#pragma unroll
    for (int m = 0; m < NPT; m++) l_w[m] = nullptr;
    const char* l_sp[2] = {nullptr, nullptr};                  // scales / biases of the two rows, at the slice's first group
    const char* l_bp[2] = {nullptr, nullptr};
    auto load_rows = [&](int blk) {
#pragma unroll
        for (int m = 0; m < NPT; m++) {
            // piece lane + 32 m of the block's group: row (of sixteen) and 16-byte part of that row
            const int pc = min(lane + 32 * m, NPIECE - 1), rr = pc / PPR, part16 = pc - rr * PPR;
            int r = min(blk * 16 + rr, q.total_rows - 1), pi = 0;
            if (q.n_parts > 1 && r >= q.part[0].rows) {
                r -= q.part[0].rows; pi = 1;
                if (q.n_parts > 2 && r >= q.part[1].rows) { r -= q.part[1].rows; pi = 2; }
            }
            l_w[m] = q.part[pi].w + static_cast<size_t>(r) * row_bytes + static_cast<size_t>(gmin) * RB + part16 * PIECE;
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int pi;
            const int r = locate(blk, h, pi);
            const size_t off = (static_cast<size_t>(r) * groups + gmin) * 2;
            l_sp[h] = static_cast<const char*>(q.part[pi].s) + off;
            l_bp[h] = static_cast<const char*>(q.part[pi].b) + off;
        }
    };
    const long long w_jump = static_cast<long long>(blk_stride) * 16 * static_cast<long long>(row_bytes) - static_cast<long long>(slice_groups) * RB;
    const long long s_jump = static_cast<long long>(blk_stride) * 16 * groups * 2;
    auto issue_turn = [&](uint32_t dst) {
        if (l_left > 0) {
            if (l_g == 0) {
                // first group of a block: the block's (scale, bias) pairs, a cell per window of eight groups
                const uint32_t cell0 = tab + l_tab * (nwin * 512);
                for (int w = 0; w < nwin; w++) {
                    const int gp = 8 * w + 2 * t;
                    if (gp < slice_groups) {
                        const uint32_t cell = cell0 + w * 512;
                        cp_async4<0>(cell, l_sp[0] + 2 * gp);
                        cp_async4<4>(cell, l_sp[1] + 2 * gp);
                        cp_async4<8>(cell, l_bp[0] + 2 * gp);
                        cp_async4<12>(cell, l_bp[1] + 2 * gp);
                    }
                }
            }
            static_for<0, NPT, 1>([&](auto mc) {
                constexpr int m = decltype(mc)::value;
                if (NPIECE % 32 == 0 || m + 1 < NPT || lane + 32 * m < NPIECE) cp_async_piece<PIECE, m * 32 * PIECE, 0>(dst, l_w[m]);
            });
            l_left--; l_g++;
#pragma unroll
            for (int m = 0; m < NPT; m++) l_w[m] += RB;
            if (l_g == slice_groups) {
                l_g = 0; l_blk += blk_stride;
                if (++l_tab == ntab) l_tab = 0;
                if (l_left > 0) {
                    if (q.n_parts == 1 && l_blk * 16 + 16 <= q.total_rows) {
#pragma unroll
                        for (int m = 0; m < NPT; m++) l_w[m] += w_jump;
                        l_sp[0] += s_jump; l_sp[1] += s_jump; l_bp[0] += s_jump; l_bp[1] += s_jump;
                    } else {
                        load_rows(l_blk);
                    }
                }
            }
        }
        cp_commit();
    };
    if (l_left > 0) load_rows(l_blk);
    for (int gq = 0; gq < depth; gq++) issue_turn(ring + gq * SLOT);

    // ---- the activations: nothing before this line reads x, e or writes y --------------------------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    unsigned peer_epoch = q.peer.epoch;
    if (q.peer.n > 0) {
        if (q.peer.epoch_ctr != nullptr) peer_epoch = *reinterpret_cast<volatile unsigned*>(q.peer.epoch_ctr) + 1u;
        peer_publish_previous(q.peer, peer_epoch);
        if (peer_epoch != 1u && q.peer.x_is_gathered) {
            if (warp == 0 && lane < q.peer.n) peer_flag_wait(q.peer.my_flags + q.peer.peer_rank[lane], peer_epoch - 1u, p.err);
            __syncthreads();
        }
    }
    bool peers_ready = q.peer.n == 0 || q.peer.x_is_gathered || peer_epoch == 1u;
    {
        // staged once per CTA, as in qmv_pipe.cuh; the group sums leave as three TF32 parts
        for (int i = threadIdx.x; i < 3 * xn * 8; i += NT) {                  // the zero tail of every column of every part
            const int col = i >> 3;
            parts[col * gpad + groups + (i & 7)] = 0.0f;
        }
        const int cpr = K >> 3, total_chunks = T * cpr;
        constexpr int cpg = GS / 8;
        constexpr int SU = 4;                                  // chunks whose loads are in flight together
        const bool f16_fast = (BITS == 4 || BITS == 8) && split == 1 && q.x_dtype == DT_F16;
        for (int base = 0; base < total_chunks; base += NT * SU) {
            uint4 ra[SU], rb[SU];
#pragma unroll
            for (int u = 0; u < SU; u++) {
                const int idx = base + u * NT + threadIdx.x;
                if (idx < total_chunks) {
                    const int tok = tp.cpr_shift >= 0 ? idx >> tp.cpr_shift : idx / cpr, k = (idx - tok * cpr) * 8;
                    load8_raw(q.x, q.x_dtype, static_cast<size_t>(tok) * q.x_stride + k, ra[u], rb[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < SU; u++) {
                const int idx = base + u * NT + threadIdx.x;
                if (base + u * NT >= total_chunks) break;      // (uniform: the shuffles below are executed by whole warps)
                const int tok = tp.cpr_shift >= 0 ? idx >> tp.cpr_shift : idx / cpr, k = (idx - tok * cpr) * 8;
                float sum = 0.0f;
                if (idx < total_chunks && f16_fast) {
                    // fp16 activations stay fp16: permute and pre-scale the words, the sum alone is formed in fp32
                    const uint32_t w4[4] = {ra[u].x, ra[u].y, ra[u].z, ra[u].w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w4[i]));
                        sum += f.x;
                        sum += f.y;
                    }
                    if constexpr (BITS == 4 || BITS == 8) stage8v_f16<BITS>(xs + static_cast<size_t>(tok) * tp.xstride, k, w4);
                } else if (idx < total_chunks) {
                    float v[8];
                    raw_to_float8(q.x_dtype, ra[u], rb[u], v);
                    if (q.x_up != nullptr) {
                        // gated input: the activation the layer sees is act(gate) * up, formed here
                        float up[8];
                        load8_coherent(q.x_up, DT_F32, static_cast<size_t>(tok) * q.x_stride + k, up);
#pragma unroll
                        for (int i = 0; i < 8; i++) v[i] = act_mul(q.x_act, v[i], up[i]);
                    }
#pragma unroll
                    for (int i = 0; i < 8; i++) sum += v[i];
                    if (split == 1) {
                        stage8r<BITS, CL>(xs + static_cast<size_t>(tok) * tp.xstride, k, v);
                    } else {
                        float hi[8], lo[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) { hi[i] = __half2float(__float2half_rn(v[i])); lo[i] = v[i] - hi[i]; }
                        stage8r<BITS, CL>(xs + static_cast<size_t>(2 * tok) * tp.xstride, k, hi);
                        stage8r<BITS, CL>(xs + static_cast<size_t>(2 * tok + 1) * tp.xstride, k, lo);
                    }
                }
#pragma unroll
                for (int o = 1; o < cpg; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (idx < total_chunks && (idx & (cpg - 1)) == 0) {
                    const int gidx = k >> GSH;
                    const int col = split == 1 ? tok : 2 * tok;
                    // sum = hi + mid + lo exactly, each part a TF32 number
                    const float hi = __uint_as_float(__float_as_uint(sum) & 0xFFFFE000u);
                    const float r1 = sum - hi;
                    const float mid = __uint_as_float(__float_as_uint(r1) & 0xFFFFE000u);
                    const float lo = r1 - mid;
                    parts[(0 * xn + col) * gpad + gidx] = hi;
                    parts[(1 * xn + col) * gpad + gidx] = mid;
                    parts[(2 * xn + col) * gpad + gidx] = lo;
                    if (split == 2) {                                         // the lo column of an fp32 token carries no bias term
                        parts[(0 * xn + col + 1) * gpad + gidx] = 0.0f;
                        parts[(1 * xn + col + 1) * gpad + gidx] = 0.0f;
                        parts[(2 * xn + col + 1) * gpad + gidx] = 0.0f;
                    }
                }
            }
        }
    }
    __syncthreads();

    // the lane feeds accumulator column g of every pass: staged column ps * 8 + g, or zeros when there is none
    uint32_t xb[NP], xinc[NP], sb_[NP], sinc[NP], pstr[NP];
#pragma unroll
    for (int ps = 0; ps < NP; ps++) {
        const int col = ps * 8 + g;
        const bool valid = col < xn;
        xb[ps] = valid ? smem_u32(xs) + (col * tp.xstride + gmin * GS + t * CL) * 2 : zaddr0;
        xinc[ps] = valid ? GS * 2 : 0;
        sb_[ps] = valid ? smem_u32(parts) + (col * gpad + gmin + 2 * t) * 4 : zaddr0;
        sinc[ps] = valid ? 32u : 0u;                            // a window of eight group sums
        pstr[ps] = valid ? static_cast<uint32_t>(xn) * gpad * 4 : 0u;   // bytes between the parts of the group sums
        asm volatile("" : "+r"(xb[ps]), "+r"(sb_[ps]) :: "memory");
    }
    const int par_floats = ks * 16 * TP;
    float* part_g = part + gi * tp.parities * par_floats;
    uint32_t c_src = ring;
    int c_tab = 0;
    int c_blk = blockIdx.x + gi * gridDim.x;
    for (int bj = 0; bj < my_blocks; bj++, c_blk += blk_stride) {
        float yacc[NP][4], yb[NP][4];
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int i = 0; i < 4; i++) { yacc[ps][i] = 0.0f; yb[ps][i] = 0.0f; }
        uint32_t xp[NP], sp[NP];
#pragma unroll
        for (int ps = 0; ps < NP; ps++) { xp[ps] = xb[ps]; sp[ps] = sb_[ps]; }
        const uint32_t cell0 = tab + c_tab * (nwin * 512);
        float sf0 = 0.0f, sf1 = 0.0f, sf2 = 0.0f, sf3 = 0.0f;  // scales of the lane's pair of the window: row g (two groups), row g + 8
        uint32_t cell = cell0;
        // (one group per turn of a plain loop: the body is issued far more often than it could be unrolled usefully,
        // and sixteen warps interleave)
#pragma unroll 1
        for (int gl = 0; gl < slice_groups; gl++) {
            const int gw = gl & 7;                              // the group's place in its window of eight
            if constexpr (DEPTH_CT != 0) asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH_CT - 1) : "memory");
            else if (depth == 8) asm volatile("cp.async.wait_group 7;" ::: "memory");
            else if (depth == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
            else asm volatile("cp.async.wait_group 1;" ::: "memory");
            if constexpr (!OWN_BYTES) __syncwarp();             // (the bytes a lane consumes were copied by other lanes)
            if (gw == 0) {
                // the window's pairs (they arrived with the block's first group, at the latest)
                uint32_t s0, s1, b0, b1;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(s0), "=r"(s1), "=r"(b0), "=r"(b1) : "r"(cell));
                cell += 512;
                // bias term of the window's eight groups: k slot t is group 2t, slot t + 4 is group 2t + 1
                uint32_t a0, a1, a2, a3;
                if (s_f16) {
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&s0)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&s1));
                    const float2 g0 = __half22float2(*reinterpret_cast<const __half2*>(&b0)), g1 = __half22float2(*reinterpret_cast<const __half2*>(&b1));
                    sf0 = f0.x; sf1 = f0.y; sf2 = f1.x; sf3 = f1.y;
                    a0 = __float_as_uint(g0.x); a2 = __float_as_uint(g0.y); a1 = __float_as_uint(g1.x); a3 = __float_as_uint(g1.y);
                } else {
                    sf0 = __uint_as_float(s0 << 16); sf1 = __uint_as_float(s0 & 0xFFFF0000u);
                    sf2 = __uint_as_float(s1 << 16); sf3 = __uint_as_float(s1 & 0xFFFF0000u);
                    a0 = b0 << 16; a2 = b0 & 0xFFFF0000u; a1 = b1 << 16; a3 = b1 & 0xFFFF0000u;
                }
#pragma unroll
                for (int ps = 0; ps < NP; ps++) {
#pragma unroll
                    for (int pt = 0; pt < 3; pt++) {
                        uint32_t x0, x1;
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(x0), "=r"(x1) : "r"(sp[ps] + pt * pstr[ps]));
                        mma1688_tf32(yb[ps], a0, a1, a2, a3, x0, x1);
                    }
                    sp[ps] += sinc[ps];
                }
            }
            uint32_t wd[2][NW];
            if constexpr (U::WORDS) {
                static_for<0, NPC, 1>([&](auto pc_) {
                    constexpr int pc = decltype(pc_)::value;
                    static_for<0, 2, 1>([&](auto hc) {
                        constexpr int h = decltype(hc)::value;
                        constexpr int off = h * 8 * RB + pc * PS;
                        constexpr int wi = pc * (PS / 4);
                        if constexpr (PS == 16)
                            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(wd[h][wi]), "=r"(wd[h][wi + 1]), "=r"(wd[h][wi + 2]), "=r"(wd[h][wi + 3]) : "r"(c_src + rd_delta), "n"(off));
                        else if constexpr (PS == 8)
                            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(wd[h][wi]), "=r"(wd[h][wi + 1]) : "r"(c_src + rd_delta), "n"(off));
                        else
                            asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(wd[h][wi]) : "r"(c_src + rd_delta), "n"(off));
                    });
                });
            } else {
                // the run starts on a half word: NPC words from the word below it, moved down by 0 or 16 bits
                static_for<0, 2, 1>([&](auto hc) {
                    constexpr int h = decltype(hc)::value;
                    uint32_t raw[NPC];
                    static_for<0, NPC, 1>([&](auto pc_) {
                        constexpr int pc = decltype(pc_)::value;
                        asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(raw[pc]) : "r"(c_src + rd_delta), "n"(h * 8 * RB + pc * 4));
                    });
#pragma unroll
                    for (int wi = 0; wi < NW; wi++)
                        wd[h][wi] = wi + 1 < NPC ? __funnelshift_r(raw[wi], raw[wi + 1], rd_shift) : raw[wi] >> rd_shift;
                });
            }
            // the slot is in registers: refill it with the group that is `depth` ahead
            if constexpr (!OWN_BYTES) __syncwarp();             // (... in every lane's registers)
            issue_turn(c_src);
            c_src += SLOT;
            if (c_src == ring_end) c_src = ring;
            float c[NP][2][4];
            static_for<0, NM, 2>([&](auto jc) {
                constexpr int j = decltype(jc)::value;
                uint32_t a00, a01, a02, a03, a10, a11, a12, a13;
                a_regs_run<BITS, CL, j>(wd[0], a00, a02);
                a_regs_run<BITS, CL, j>(wd[1], a01, a03);
                a_regs_run<BITS, CL, j + 1>(wd[0], a10, a12);
                a_regs_run<BITS, CL, j + 1>(wd[1], a11, a13);
#pragma unroll
                for (int ps = 0; ps < NP; ps++) {
                    uint4 bv;
                    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(bv.x), "=r"(bv.y), "=r"(bv.z), "=r"(bv.w) : "r"(xp[ps]), "n"(8 * j));
                    if constexpr (j == 0) {
                        mma16816_first(c[ps][0], a00, a01, a02, a03, bv.x, bv.y);
                        mma16816_first(c[ps][1], a10, a11, a12, a13, bv.z, bv.w);
                    } else {
                        mma16816(c[ps][0], a00, a01, a02, a03, bv.x, bv.y);
                        mma16816(c[ps][1], a10, a11, a12, a13, bv.z, bv.w);
                    }
                }
            });
            // the group's scales sit in lane gw / 2 of the row's four lanes
            const int src = (lane & ~3) | (gw >> 1);
            const float sg = __shfl_sync(0xffffffffu, (gw & 1) ? sf1 : sf0, src);
            const float sg8 = __shfl_sync(0xffffffffu, (gw & 1) ? sf3 : sf2, src);
#pragma unroll
            for (int ps = 0; ps < NP; ps++) {
                yacc[ps][0] = fmaf(sg, c[ps][0][0] + c[ps][1][0], yacc[ps][0]);
                yacc[ps][1] = fmaf(sg, c[ps][0][1] + c[ps][1][1], yacc[ps][1]);
                yacc[ps][2] = fmaf(sg8, c[ps][0][2] + c[ps][1][2], yacc[ps][2]);
                yacc[ps][3] = fmaf(sg8, c[ps][0][3] + c[ps][1][3], yacc[ps][3]);
                xp[ps] += xinc[ps];
            }
        }
        if (++c_tab == ntab) c_tab = 0;

        // ---- end of a block: this warp's partial sums [16 rows][tokens] to the group's first warp -------------------
        float* slot_base = part_g + ((tp.parities == 2 && (bj & 1)) ? par_floats : 0);
        float* mine = slot_base + kw * (16 * TP);
#pragma unroll
        for (int ps = 0; ps < NP; ps++) {
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = fmaf(yacc[ps][i], 16777216.0f, yb[ps][i]);
            if (split == 1) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int tok = ps * 8 + 2 * t + (i & 1);
                    if (tok < T) mine[(g + 8 * (i >> 1)) * TP + tok] = v[i];
                }
            } else {
                const int tok = ps * 4 + t;                    // columns (2t, 2t + 1) are the token's hi and lo halves
                if (tok < T) { mine[g * TP + tok] = v[0] + v[1]; mine[(g + 8) * TP + tok] = v[2] + v[3]; }
            }
        }
        if (ks > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(ks * 32) : "memory");
        else __syncwarp();
        // Every warp of the group adds up and stores a share of the block's outputs: a token's sixteen rows per half
        // warp.  (The two parities of the partial-sum slot keep a warp that runs ahead from overwriting sums still
        // being read: it meets the others at the next block's barrier before it writes this parity again.  With a
        // single slot the group meets a second time, after the reads.)
        if (2 * kw < T) {
            if (!peers_ready) {
                if (lane < q.peer.n) peer_flag_wait(q.peer.my_flags + q.peer.peer_rank[lane], peer_epoch - 2u, p.err);
                __syncwarp();
                peers_ready = true;
            }
            for (int tok = 2 * kw + (lane >> 4); tok < T; tok += 2 * ks) {
                const int r = lane & 15;
                const int row = c_blk * 16 + r;
                float v = 0.0f;
                for (int wv = 0; wv < ks; wv++) v += slot_base[wv * (16 * TP) + r * TP + tok];
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
        }
        if (tp.parities == 1 && ks > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(ks * 32) : "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    if (q.peer.n > 0) peer_finish(q.peer, peer_epoch);
}

// Plans a call of the token-major kernel; returns the shared memory it needs, 0 when the call is not one it serves.
size_t qmv_tok_plan(int bits, const MmaParams& p, int tokens, int sms, TokPlan& tp);
cudaError_t launch_qmv_tok(int bits, const MmaParams& p, const TokPlan& tp, size_t smem, int device, cudaStream_t st);

}  // namespace mlxq
