// Planner, instantiations and launcher of the token-major decode matvec for small batches (qmv_tok.cuh).
#include "qmv_tok.cuh"

#include <cstdlib>
#include <mutex>

namespace mlxq {

namespace {

constexpr int SMEM_WHOLE = 224 * 1024;      // of the 227 KB a CTA may opt into

int align_up(int v, int a) { return (v + a - 1) / a * a; }

bool pdl_enabled() {
    static const bool v = [] { const char* e = std::getenv("MLXQ_PDL"); return !(e && e[0] == '0'); }();
    return v;
}

bool supported(int bits, int gs) {
    const int gb_bits = gs * bits;                  // bits of a group per row
    if (gb_bits % 64 != 0 || gb_bits < 128) return false;      // four lanes, whole half words each, at least four bytes
    if (gb_bits % 128 != 0 && bits != 3 && bits != 5 && bits != 6) return false;
    const int nm = gs / 16;
    return nm >= 2 && nm % 2 == 0;
}

template <int BITS, int GS, int NP, int DEPTH_CT>
cudaError_t launch_one(const MmaParams& p, const TokPlan& tp, size_t smem, int device, cudaStream_t st) {
    if constexpr (!TokUnit<BITS, GS>::SUPPORTED) {
        return cudaErrorNotSupported;
    } else {
        // the shared-memory opt-in is an attribute of the function in one device's context
        static std::mutex mu;
        static bool done[64] = {};
        if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
        {
            std::lock_guard<std::mutex> lk(mu);
            if (!done[device]) {
                const cudaError_t e = cudaFuncSetAttribute(qmv_tok_kernel<BITS, GS, NP, DEPTH_CT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_WHOLE);
                if (e != cudaSuccess) return e;
                done[device] = true;
            }
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(tp.grid));
        cfg.blockDim = dim3(TOK_WARPS * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute la[1];
        la[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        la[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = la;
        cfg.numAttrs = pdl_enabled() ? 1 : 0;
        return cudaLaunchKernelEx(&cfg, qmv_tok_kernel<BITS, GS, NP, DEPTH_CT>, p, tp);
    }
}

template <int BITS, int GS, int NP>
cudaError_t launch_depth(const MmaParams& p, const TokPlan& tp, size_t smem, int device, cudaStream_t st) {
    // the width's usual ring depth is compiled in; a shallower ring (shared memory short) takes the general instance
    constexpr int usual = GS * BITS / 32 >= 16 ? 4 : 8;
    return tp.depth == usual ? launch_one<BITS, GS, NP, usual>(p, tp, smem, device, st) : launch_one<BITS, GS, NP, 0>(p, tp, smem, device, st);
}

template <int BITS, int GS>
cudaError_t launch_np(const MmaParams& p, const TokPlan& tp, size_t smem, int device, cudaStream_t st) {
    return p.xn <= 8 ? launch_depth<BITS, GS, 1>(p, tp, smem, device, st) : launch_depth<BITS, GS, 2>(p, tp, smem, device, st);
}

template <int BITS>
cudaError_t launch_gs(const MmaParams& p, const TokPlan& tp, size_t smem, int device, cudaStream_t st) {
    switch (p.q.gs) {
        case 32: return launch_np<BITS, 32>(p, tp, smem, device, st);
        case 64: return launch_np<BITS, 64>(p, tp, smem, device, st);
        case 128: return launch_np<BITS, 128>(p, tp, smem, device, st);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace

size_t qmv_tok_plan(int bits, const MmaParams& p, int tokens, int sms, TokPlan& tp) {
    const QmvParams& q = p.q;
    if (tokens < 1 || q.total_rows < 1 || p.xn < 1 || p.xn > 16) return 0;
    if (q.gs != 32 && q.gs != 64 && q.gs != 128) return 0;
    if (!supported(bits, q.gs)) return 0;
    if (q.s_dtype != DT_F16 && q.s_dtype != DT_BF16) return 0;     // a 16-bit bias is exact in TF32; an fp32 one is not
    const int K = q.K, groups = K / q.gs;
    if (K % q.gs != 0 || groups % 2 != 0) return 0;
    const long long row_b = static_cast<long long>(K) * bits / 8;
    if (row_b % 16 != 0) return 0;
    for (int i = 0; i < q.n_parts; i++) {
        if (q.n_parts > 1 && q.part[i].rows % 8 != 0) return 0;         // an 8-row half of a block lies inside one part
        if ((reinterpret_cast<uintptr_t>(q.part[i].w) & 15u) || (reinterpret_cast<uintptr_t>(q.part[i].s) & 3u) ||
            (reinterpret_cast<uintptr_t>(q.part[i].b) & 3u))
            return 0;
    }
    const int gb = q.gs * bits / 32;                 // bytes of a group per lane and row
    const int slot_bytes = 2 * 32 * gb;
    const int warps = TOK_WARPS;
    tp.n_blocks = (q.total_rows + 15) / 16;
    tp.grid = tp.n_blocks < sms ? tp.n_blocks : sms;
    tp.base_blocks = tp.n_blocks / tp.grid;
    tp.extra_blocks = tp.n_blocks % tp.grid;
    tp.xstride = K + 8;
    tp.cpr_shift = -1;
    for (int sft = 0; sft < 30; sft++) if ((1 << sft) == K / 8) tp.cpr_shift = sft;
    tp.tp = tokens + 1;
    tp.gpad = groups + 8;
    // fixed part of the layout
    int off = align_up(p.xn * tp.xstride * 2, 16);
    tp.off_parts = off; off += align_up(3 * p.xn * tp.gpad * 4, 16);
    tp.off_zero = off; off += PIPE_ZERO_BYTES;
    tp.off_part = off;
    const int off_fixed = off;
    // K split and ring depth: the split that leaves the longest-working warp the least to do, among those whose
    // slices are equal, even, and at least two groups long; the deepest ring that fits.
    const int cta_blocks = (tp.n_blocks + tp.grid - 1) / tp.grid;
    long long best_cost = -1;
    size_t best_total = 0;
    for (int parities = 2; parities >= 1 && best_cost < 0; parities--)
    for (int ks = 1; ks <= warps; ks *= 2) {
        const int off_tab = align_up(off_fixed + parities * warps * 16 * tp.tp * 4, 128);
        // slices are cut at even groups; the shortest must hold a pair, the longest sets the tables' size
        int slice = 0, slice_min = groups;
        for (int kw = 0; kw < ks; kw++) {
            const int a = (((groups / 2) * kw) / ks) * 2, b = (((groups / 2) * (kw + 1)) / ks) * 2;
            if (b - a > slice) slice = b - a;
            if (b - a < slice_min) slice_min = b - a;
        }
        if (slice_min < 2) break;
        if (ks > 1 && warps / ks > 15) continue;                       // one named barrier per group of warps
        const int n_groups = warps / ks;
        const long long rounds = (cta_blocks + n_groups - 1) / n_groups;
        const long long cost = rounds * (slice + 2);                   // (ending a block and meeting the group: about two groups' work)
        const int nwin = (slice + 7) / 8;
        for (int depth = gb >= 16 ? 4 : 8; depth >= 2; depth /= 2) {
            const int ntab = depth / slice_min + 2;
            const long long total = static_cast<long long>(off_tab) + static_cast<long long>(warps) * ntab * nwin * 512;
            const long long ring_at = (total + 127) / 128 * 128;
            const long long end = ring_at + static_cast<long long>(warps) * depth * slot_bytes;
            if (end > SMEM_WHOLE) continue;
            // a shallower ring costs: count it as a quarter more work per halving
            const long long c = cost * (depth >= 4 || gb >= 16 ? 4 : 5);
            if (best_cost < 0 || c < best_cost) {
                best_cost = c; best_total = static_cast<size_t>(end);
                tp.ks = ks; tp.depth = depth; tp.ntab = ntab; tp.nwin = nwin; tp.slice_groups = slice;
                tp.off_ring = static_cast<int>(ring_at); tp.off_tab = off_tab; tp.parities = parities;
            }
            break;
        }
    }
    if (best_cost < 0) return 0;
    tp.ks_shift = 0;
    while ((1 << tp.ks_shift) < tp.ks) tp.ks_shift++;
    return best_total;
}

cudaError_t launch_qmv_tok(int bits, const MmaParams& p, const TokPlan& tp, size_t smem, int device, cudaStream_t st) {
    switch (bits) {
        case 2: return launch_gs<2>(p, tp, smem, device, st);
        case 3: return launch_gs<3>(p, tp, smem, device, st);
        case 4: return launch_gs<4>(p, tp, smem, device, st);
        case 5: return launch_gs<5>(p, tp, smem, device, st);
        case 6: return launch_gs<6>(p, tp, smem, device, st);
        case 8: return launch_gs<8>(p, tp, smem, device, st);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace mlxq
