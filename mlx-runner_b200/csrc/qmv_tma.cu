// Planner, instantiations and launcher of the persistent TMA-fed decode matvec (qmv_tma.cuh).
#include "qmv_tma.cuh"

#include <cstdlib>
#include <mutex>

namespace mlxq {

namespace {

constexpr int SMEM_BUDGET = 224 * 1024;     // of the 227 KB a CTA may opt into
constexpr int SMEM_HALF = 112 * 1024;       // two CTAs per SM (each also pays 1 KB of system shared memory)

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

// MLXQ_TMA_CONSUMERS=8|16 fixes the CTA layout (tuning aid); anything else = automatic.
int consumers_override() {
    static const int v = [] {
        const char* e = std::getenv("MLXQ_TMA_CONSUMERS");
        const int k = e ? std::atoi(e) : 0;
        return (k == 8 || k == 16) ? k : 0;
    }();
    return v;
}

// MLXQ_PDL=0 launches without the programmatic-dependent-launch attribute (see the kernel's prologue).
bool pdl_enabled() {
    static const bool v = [] { const char* e = std::getenv("MLXQ_PDL"); return !(e && e[0] == '0'); }();
    return v;
}

template <int BITS, int NP, int NC>
cudaError_t launch_one(const MmaParams& p, const TmaPlan& tp, size_t smem, cudaStream_t st) {
    static std::once_flag once;
    static cudaError_t attr = cudaSuccess;
    std::call_once(once, [] {
        attr = cudaFuncSetAttribute(qmv_tma_kernel<BITS, NP, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    NC == 8 ? SMEM_HALF : SMEM_BUDGET);
    });
    if (attr != cudaSuccess) return attr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(tp.grid));
    cfg.blockDim = dim3((NC + 2) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute la[1];
    la[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    la[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = la;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, qmv_tma_kernel<BITS, NP, NC>, p, tp);
}

template <int BITS, int NC>
cudaError_t launch_np(const MmaParams& p, const TmaPlan& tp, size_t smem, cudaStream_t st) {
    if (p.passes <= 1) return launch_one<BITS, 1, NC>(p, tp, smem, st);
    if (p.passes <= 2) return launch_one<BITS, 2, NC>(p, tp, smem, st);
    if (p.passes <= 4) return launch_one<BITS, 4, NC>(p, tp, smem, st);
    return cudaErrorNotSupported;
}

template <int BITS>
cudaError_t launch_bits(const MmaParams& p, const TmaPlan& tp, size_t smem, cudaStream_t st) {
    return tp.consumers == 8 ? launch_np<BITS, 8>(p, tp, smem, st) : launch_np<BITS, 16>(p, tp, smem, st);
}

}  // namespace

size_t qmv_tma_plan(int bits, const MmaParams& p, int tokens, int sms, TmaPlan& tp) {
    const QmvParams& q = p.q;
    if (p.passes > 4) return 0;
    int lb, kb;
    unit_for(bits, lb, kb);
    (void)lb;
    const int K = q.K, groups = K / q.gs, sbytes = dtype_size(q.s_dtype);
    // Eight consecutive rows are copied as one run: parts must hold multiples of 8 rows and be 16-byte aligned.
    if (q.total_rows < 8) return 0;
    for (int i = 0; i < q.n_parts; i++) {
        if (q.part[i].rows % 8 != 0) return 0;
        if ((reinterpret_cast<uintptr_t>(q.part[i].w) & 15u) || (reinterpret_cast<uintptr_t>(q.part[i].s) & 15u) ||
            (reinterpret_cast<uintptr_t>(q.part[i].b) & 15u))
            return 0;
    }
    // Stage granularity: a whole 16-row block per stage (three copies per block -- a bulk copy costs the issuing
    // thread ~100 ns, so fewer and larger copies) when every part holds a multiple of 16 rows and four such stages
    // fit; otherwise 8-row stages (long rows).
    bool rows16 = q.total_rows >= 16;
    for (int i = 0; i < q.n_parts; i++) rows16 = rows16 && q.part[i].rows % 16 == 0;
    const long long row_b = static_cast<long long>(K) * bits / 8;
    if (rows16 && align_up(static_cast<int>(16 * row_b + 2 * 16 * groups * sbytes), 128) * 4LL > 150 * 1024) rows16 = false;
    tp.rps = rows16 ? 16 : 8;
    const long long w_bytes = tp.rps * row_b;
    if (w_bytes > 96 * 1024) return 0;
    tp.w_bytes = static_cast<int>(w_bytes);
    tp.s_bytes = tp.rps * groups * sbytes;
    tp.stage_bytes = align_up(tp.w_bytes + 2 * tp.s_bytes, 128);
    tp.n_blocks = (q.total_rows + 15) / 16;
    int np = 1;
    while (np < p.passes) np *= 2;
    int off = align_up(p.xn * p.xstride * 2, 16);
    tp.off_xsum = off; off += align_up(p.xn * groups * 4, 16);
    // (16-bit activations get their group sums from shuffles: the per-chunk sums are only staged for fp32 ones)
    tp.off_csum = off; off += p.split == 1 ? 0 : align_up(tokens * (K / 8) * 4, 16);
    // Two layouts: 16 consumer warps (two groups of 8 working on alternate blocks) on a whole SM, or 8
    // consumer warps with half the shared memory and two CTAs per SM.  The first measured faster on the
    // benchmark shapes (10.7 vs 11.9 us per 11008x4096 4-bit launch) and is the default;
    // MLXQ_TMA_CONSUMERS=8 selects the second.
    (void)kb;
    const int fixed = off;
    for (int consumers = consumers_override() > 0 ? consumers_override() : 16; consumers <= TMA_MAX_CONSUMERS; consumers *= 2) {
        const int ksplit = 8;                       // warps that share a block along K
        off = fixed;
        tp.consumers = consumers;
        tp.ksplit = ksplit;
        tp.rowsum = (tokens == 1 && np == 1) ? 1 : 0;
        tp.slots = tp.rowsum ? TMA_SLOTS : 4;          // full partial sums are 4 KB per warp: fewer slots leave room for the ring
        tp.off_part = off; off += tp.slots * ksplit * (tp.rowsum ? 16 : np * 128) * 4;
        tp.off_zero = align_up(off, 16); off = tp.off_zero + 256;
        tp.off_bars = align_up(off, 16); off = tp.off_bars + static_cast<int>(sizeof(TmaBars));
        tp.off_stage = align_up(off, 128);
        const int room = (consumers == 8 ? SMEM_HALF : SMEM_BUDGET) - tp.off_stage;
        int ns = room > 0 ? room / tp.stage_bytes : 0;
        if (ns > TMA_MAX_STAGES) ns = TMA_MAX_STAGES;
        // the ring holds at least the blocks in work (see the consumers' double wait), and the half-size layout
        // is only worth it with two blocks in flight
        const int per_block = 16 / tp.rps;
        const int round = per_block * (consumers / ksplit);     // stages the consumer groups take per round of blocks
        const int per_sm = consumers == 8 ? 2 : 1;
        tp.grid = tp.n_blocks < sms * per_sm ? tp.n_blocks : sms * per_sm;
        const int blocks_per_cta = (tp.n_blocks + tp.grid - 1) / tp.grid;
        if (blocks_per_cta * per_block > ns) {
            // stages are reused inside the launch: a stage must always return to the same consumer group
            static const bool no_wrap = [] { const char* e = std::getenv("MLXQ_TMA_WRAP"); return e && e[0] == '0'; }();
            if (no_wrap) continue;                               // MLXQ_TMA_WRAP=0: such calls go to the register-fed kernel
            ns -= ns % round;
        }
        if (ns < round || (consumers == 8 && ns < 2 * per_block)) continue;
        tp.ns = ns;
        return static_cast<size_t>(tp.off_stage) + static_cast<size_t>(ns) * tp.stage_bytes;
    }
    return 0;
}

cudaError_t launch_qmv_tma(int bits, const MmaParams& p, const TmaPlan& tp, size_t smem, cudaStream_t st) {
    switch (bits) {
        case 2: return launch_bits<2>(p, tp, smem, st);
        case 3: return launch_bits<3>(p, tp, smem, st);
        case 4: return launch_bits<4>(p, tp, smem, st);
        case 5: return launch_bits<5>(p, tp, smem, st);
        case 6: return launch_bits<6>(p, tp, smem, st);
        case 8: return launch_bits<8>(p, tp, smem, st);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace mlxq
