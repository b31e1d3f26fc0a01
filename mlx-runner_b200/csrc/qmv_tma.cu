// Planner, instantiations and launcher of the persistent TMA-fed decode matvec (qmv_tma.cuh).
#include "qmv_tma.cuh"

#include <mutex>

namespace mlxq {

namespace {

constexpr int SMEM_BUDGET = 224 * 1024;     // of the 227 KB a CTA may opt into

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

template <int BITS, int NP>
cudaError_t launch_one(const MmaParams& p, const TmaPlan& tp, size_t smem, int sms, cudaStream_t st) {
    static std::once_flag once;
    static cudaError_t attr = cudaSuccess;
    std::call_once(once, [] {
        attr = cudaFuncSetAttribute(qmv_tma_kernel<BITS, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET);
    });
    if (attr != cudaSuccess) return attr;
    const unsigned grid = static_cast<unsigned>(tp.n_blocks < sms ? tp.n_blocks : sms);
    qmv_tma_kernel<BITS, NP><<<grid, TMA_THREADS, smem, st>>>(p, tp);
    return cudaGetLastError();
}

template <int BITS>
cudaError_t launch_bits(const MmaParams& p, const TmaPlan& tp, size_t smem, int sms, cudaStream_t st) {
    if (p.passes <= 1) return launch_one<BITS, 1>(p, tp, smem, sms, st);
    if (p.passes <= 2) return launch_one<BITS, 2>(p, tp, smem, sms, st);
    if (p.passes <= 4) return launch_one<BITS, 4>(p, tp, smem, sms, st);
    return cudaErrorNotSupported;
}

}  // namespace

size_t qmv_tma_plan(int bits, const MmaParams& p, int tokens, TmaPlan& tp) {
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
    const long long w_bytes = 8LL * K * bits / 8;
    if (w_bytes > 96 * 1024) return 0;
    tp.w_bytes = static_cast<int>(w_bytes);
    tp.s_bytes = 8 * groups * sbytes;
    tp.stage_bytes = align_up(tp.w_bytes + 2 * tp.s_bytes, 128);
    tp.n_blocks = (q.total_rows + 15) / 16;
    int np = 1;
    while (np < p.passes) np *= 2;
    int off = align_up(p.xn * p.xstride * 2, 16);
    tp.off_xsum = off; off += align_up(p.xn * groups * 4, 16);
    tp.off_csum = off; off += align_up(tokens * (K / 8) * 4, 16);
    tp.off_part = off; off += TMA_SLOTS * TMA_CONSUMERS * np * 128 * 4;
    tp.off_bars = align_up(off, 16); off = tp.off_bars + static_cast<int>(sizeof(TmaBars));
    tp.off_stage = align_up(off, 128);
    const int room = SMEM_BUDGET - tp.off_stage;
    int ns = room / tp.stage_bytes;
    if (ns > TMA_MAX_STAGES) ns = TMA_MAX_STAGES;
    if (ns < 2) return 0;
    tp.ns = ns;
    return static_cast<size_t>(tp.off_stage) + static_cast<size_t>(ns) * tp.stage_bytes;
}

cudaError_t launch_qmv_tma(int bits, const MmaParams& p, const TmaPlan& tp, size_t smem, int sms, cudaStream_t st) {
    switch (bits) {
        case 2: return launch_bits<2>(p, tp, smem, sms, st);
        case 3: return launch_bits<3>(p, tp, smem, sms, st);
        case 4: return launch_bits<4>(p, tp, smem, sms, st);
        case 5: return launch_bits<5>(p, tp, smem, sms, st);
        case 6: return launch_bits<6>(p, tp, smem, sms, st);
        case 8: return launch_bits<8>(p, tp, smem, sms, st);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace mlxq
