// Planner, instantiations and launcher of the persistent decode matvec fed by warp-private asynchronous copies
// (qmv_pipe.cuh).
#include "qmv_pipe.cuh"

#include <cstdlib>
#include <mutex>

namespace mlxq {

namespace {

constexpr int SMEM_WHOLE = 224 * 1024;      // of the 227 KB a CTA may opt into

template <int BITS> void unit_of(int& lb, int& kb) { lb = MmaUnit<BITS>::LB; kb = MmaUnit<BITS>::KB; }

void unit_for(int bits, int& lb, int& kb) {
    switch (bits) {
        case 2: unit_of<2>(lb, kb); break;
        case 3: unit_of<3>(lb, kb); break;
        case 4: unit_of<4>(lb, kb); break;
        case 5: unit_of<5>(lb, kb); break;
        case 6: unit_of<6>(lb, kb); break;
        default: unit_of<8>(lb, kb); break;
    }
}

int align_up(int v, int a) { return (v + a - 1) / a * a; }

// MLXQ_PDL=0 launches without the programmatic-dependent-launch attribute (see the kernel's prologue).
bool pdl_enabled() {
    static const bool v = [] { const char* e = std::getenv("MLXQ_PDL"); return !(e && e[0] == '0'); }();
    return v;
}

template <int BITS, int NP, int UNR, int GS>
cudaError_t launch_one(const MmaParams& p, const PipePlan& pp, size_t smem, int device, cudaStream_t st) {
    // The shared-memory opt-in is an attribute of the function in one device's context: once per device, with
    // that device current (the caller has selected it).
    static std::mutex mu;
    static bool done[64] = {};
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!done[device]) {
            const cudaError_t e = cudaFuncSetAttribute(qmv_pipe_kernel<BITS, NP, UNR, GS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_WHOLE);
            if (e != cudaSuccess) return e;
            done[device] = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(pp.grid));
    cfg.blockDim = dim3(PIPE_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute la[1];
    la[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    la[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = la;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, qmv_pipe_kernel<BITS, NP, UNR, GS>, p, pp);
}

template <int BITS, int UNR>
cudaError_t launch_np(const MmaParams& p, const PipePlan& pp, size_t smem, int device, cudaStream_t st) {
    // the one-token kernels with the column plan folded in at compile time
    if (pp.special == 32) return launch_one<BITS, 1, UNR, 32>(p, pp, smem, device, st);
    if (pp.special == 64) return launch_one<BITS, 1, UNR, 64>(p, pp, smem, device, st);
    if (pp.special == 128) return launch_one<BITS, 1, UNR, 128>(p, pp, smem, device, st);
    if (p.passes <= 1) return launch_one<BITS, 1, UNR, 0>(p, pp, smem, device, st);
    if (p.passes <= 2) return launch_one<BITS, 2, UNR, 0>(p, pp, smem, device, st);
    if (p.passes <= 4) return launch_one<BITS, 4, UNR, 0>(p, pp, smem, device, st);
    return cudaErrorNotSupported;
}

template <int BITS>
cudaError_t launch_bits(const MmaParams& p, const PipePlan& pp, size_t smem, int device, cudaStream_t st) {
    return pp.unroll == 2 ? launch_np<BITS, 2>(p, pp, smem, device, st) : launch_np<BITS, 1>(p, pp, smem, device, st);
}

}  // namespace

size_t qmv_pipe_plan(int bits, const MmaParams& p, int tokens, int sms, PipePlan& pp) {
    const QmvParams& q = p.q;
    if (p.passes > 4 || tokens < 1 || q.total_rows < 1) return 0;
    int lb, kb;
    unit_for(bits, lb, kb);
    const int K = q.K, groups = K / q.gs;
    // rows are copied in 16-byte (8-byte) pieces, (scale, bias) pairs in 4-byte pieces
    const long long row_b = static_cast<long long>(K) * bits / 8;
    if (row_b % 16 != 0) return 0;
    for (int i = 0; i < q.n_parts; i++) {
        if (q.n_parts > 1 && q.part[i].rows % 8 != 0) return 0;         // an 8-row half of a block lies inside one part
        if ((reinterpret_cast<uintptr_t>(q.part[i].w) & 15u) || (reinterpret_cast<uintptr_t>(q.part[i].s) & 3u) ||
            (reinterpret_cast<uintptr_t>(q.part[i].b) & 3u))
            return 0;
    }
    int np = 1;
    while (np < p.passes) np *= 2;
    const int steps_total = K / kb, nblk = steps_total >> p.spg_shift;
    pp.n_blocks = (q.total_rows + 15) / 16;
    pp.grid = pp.n_blocks < sms ? pp.n_blocks : sms;
    pp.rowsum = (tokens == 1 && np == 1) ? 1 : 0;
    const int slot_bytes = 2 * 32 * lb + 4 * 32 * 4;
    pp.xstride = K + 8;
    const int warps = PIPE_WARPS;
    // K split: the group size that leaves the longest-working warp the least to do
    const int cta_blocks = (pp.n_blocks + pp.grid - 1) / pp.grid;
    const int step_weight = bits == 4 ? 4 : bits == 8 ? 3 : bits == 2 ? 5 : bits == 6 ? 10 : 18;     // in quarters of a 4-bit step
    int best_ks = 1;
    long long best_cost = -1;
    for (int ks = 1; ks <= warps && ks <= nblk && ks <= 16; ks *= 2) {
        if (warps % ks != 0 || (ks > 1 && warps / ks > 15)) continue;      // one named barrier per group
        int slice = 0;
        for (int kw = 0; kw < ks; kw++) {
            const int a = ((nblk * kw) / ks) << p.spg_shift, b = ((nblk * (kw + 1)) / ks) << p.spg_shift;
            if (b - a > slice) slice = b - a;
        }
        const int n_groups = warps / ks;
        const long long rounds = (cta_blocks + n_groups - 1) / n_groups;
        // (measured: ending a block and meeting the group costs about as much as three 4-bit steps; a step of the
        // widths whose codes straddle bytes costs several times a 4-bit one in unpacking)
        const long long cost = rounds * (static_cast<long long>(slice) * step_weight + 12);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_ks = ks; }
    }
    pp.ks = best_ks;
    pp.ks_shift = 0;
    while ((1 << pp.ks_shift) < pp.ks) pp.ks_shift++;
    pp.base_blocks = pp.n_blocks / pp.grid;
    pp.extra_blocks = pp.n_blocks % pp.grid;
    pp.cpr_shift = -1;
    for (int sft = 0; sft < 30; sft++) if ((1 << sft) == K / 8) pp.cpr_shift = sft;
    // the column plan, per pass and accumulator column (the same arithmetic as qmv_mma_kernel's prologue)
    const int gsh = p.gstep_shift, G = 1 << gsh, CY = p.cycle, cpc = p.xn << gsh;
    bool pairs = dtype_size(q.s_dtype) == 2 && groups % 2 == 0;
    for (int ps = 0; ps < 4; ps++)
        for (int n = 0; n < 8; n++) {
            int xc, grp, cyc = 0;
            if (CY > 1) { cyc = n / cpc; const int rem = n - cyc * cpc; xc = rem >> gsh; grp = rem & (G - 1); }
            else { const int lin = ps * 8 + n; xc = lin >> gsh; grp = lin & (G - 1); }
            const bool valid = xc < p.xn && cyc < CY;
            const int goff = (cyc << gsh) + grp;
            pp.col[ps][n] = static_cast<uint32_t>(valid ? xc : 255) | (static_cast<uint32_t>(goff & 255) << 8) |
                            (static_cast<uint32_t>(cyc & 15) << 16) | (static_cast<uint32_t>(grp & 15) << 20);
        }
    // The drains' (scale, bias) pairs can travel through the ring when, for every lane, the two accumulator columns
    // are consecutive even-aligned groups of the same staged column, at the same group offset in every pass.
    for (int ps = 0; ps < np; ps++)
        for (int t = 0; t < 4; t++) {
            const uint32_t c0 = pp.col[ps][2 * t], c1 = pp.col[ps][2 * t + 1], f0 = pp.col[0][2 * t];
            const int g0 = (c0 >> 8) & 255, g1 = (c1 >> 8) & 255;
            pairs = pairs && (c0 & 255) == (c1 & 255) && g1 == g0 + 1 && (g0 & 1) == 0 && g0 == static_cast<int>((f0 >> 8) & 255);
        }
    pp.async_sb = pairs ? 1 : 0;
    // (the one-token kernels assume slices of whole drain cycles)
    bool whole_cycles = true;
    {
        const int spc = p.cycle << p.spg_shift;
        for (int kw = 0; kw < pp.ks; kw++) {
            const int a = ((nblk * kw) >> pp.ks_shift) << p.spg_shift, b = ((nblk * (kw + 1)) >> pp.ks_shift) << p.spg_shift;
            if (a % spc != 0 || b % spc != 0) whole_cycles = false;
        }
    }
    pp.special = (whole_cycles && tokens == 1 && p.split == 1 && p.xn == 1 && pp.async_sb && pp.rowsum && (q.gs == 32 || q.gs == 64 || q.gs == 128)) ? q.gs : 0;
    int off = align_up(p.xn * pp.xstride * 2, 16);
    pp.off_xsum = off; off += align_up(p.xn * groups * 4, 16);
    pp.off_zero = off; off += PIPE_ZERO_BYTES;
    pp.scratch_bytes = np * 16 * 9 * 4;
    pp.off_scratch = off; off += warps * pp.scratch_bytes;
    pp.off_part = off; off += 2 * warps * 16 * tokens * 4;
    pp.off_ring = align_up(off, 128);
    // two steps per loop turn when every warp's slice holds an even number of steps
    pp.unroll = 2;
    for (int kw = 0; kw < pp.ks; kw++) {
        const int a = ((nblk * kw) >> pp.ks_shift) << p.spg_shift, b = ((nblk * (kw + 1)) >> pp.ks_shift) << p.spg_shift;
        if ((b - a) % 2 != 0) pp.unroll = 1;
    }
    pp.depth = PIPE_DEPTH;
    long long total = static_cast<long long>(pp.off_ring) + static_cast<long long>(warps) * pp.depth * slot_bytes;
    if (total > SMEM_WHOLE && !pp.special) {
        pp.depth = 2;
        total = static_cast<long long>(pp.off_ring) + static_cast<long long>(warps) * pp.depth * slot_bytes;
    }
    return total <= SMEM_WHOLE ? static_cast<size_t>(total) : 0;
}

cudaError_t launch_qmv_pipe(int bits, const MmaParams& p, const PipePlan& pp, size_t smem, int device, cudaStream_t st) {
    switch (bits) {
        case 2: return launch_bits<2>(p, pp, smem, device, st);
        case 3: return launch_bits<3>(p, pp, smem, device, st);
        case 4: return launch_bits<4>(p, pp, smem, device, st);
        case 5: return launch_bits<5>(p, pp, smem, device, st);
        case 6: return launch_bits<6>(p, pp, smem, device, st);
        case 8: return launch_bits<8>(p, pp, smem, device, st);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace mlxq
