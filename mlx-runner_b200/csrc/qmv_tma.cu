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
    const int K = q.K, groups = K / q.gs, sbytes = dtype_size(q.s_dtype);
    const int steps = K / kb, step_bytes = 4 * lb;
    // parts must hold multiples of 8 rows (the 8-row halves of a block are copied whole) and be aligned
    for (int i = 0; i < q.n_parts; i++) {
        if (q.part[i].rows % 8 != 0) return 0;
        if ((reinterpret_cast<uintptr_t>(q.part[i].s) & 15u) || (reinterpret_cast<uintptr_t>(q.part[i].b) & 15u)) return 0;
    }
    const int unit = TMA_CONSUMERS << p.spg_shift;          // keep every consumer busy and groups whole
    int kc = (36 * 1024 / 16 - 64) / step_bytes;
    kc = kc / unit * unit;
    if (kc < unit) kc = unit;
    if (kc > steps) kc = align_up(steps, 1 << p.spg_shift);
    tp.kc_steps = kc;
    tp.n_chunks = (steps + kc - 1) / kc;
    tp.chunk_bytes = kc * step_bytes;
    const int rem = tp.chunk_bytes % 128;
    tp.wstride = tp.chunk_bytes + (rem == 64 ? 0 : (64 - rem + 128) % 128);
    tp.stage_bytes = align_up(16 * tp.wstride, 128);
    tp.half_scale_bytes = 8 * groups * sbytes;
    tp.scale_buf_bytes = align_up(4 * tp.half_scale_bytes, 128);
    tp.n_blocks = (q.total_rows + 15) / 16;
    int np = 1;
    while (np < p.passes) np *= 2;
    int off = align_up(p.xn * p.xstride * 2, 16);
    tp.off_xsum = off; off += align_up(p.xn * groups * 4, 16);
    tp.off_csum = off; off += align_up(tokens * (K / 8) * 4, 16);
    tp.off_part = off; off += 2 * TMA_CONSUMERS * np * 128 * 4;
    tp.off_scale = align_up(off, 128); off = tp.off_scale + 2 * tp.scale_buf_bytes;
    tp.off_bars = align_up(off, 16); off = tp.off_bars + static_cast<int>(sizeof(TmaBars));
    tp.off_stage = align_up(off, 128);
    const int room = SMEM_BUDGET - tp.off_stage;
    if (room < 2 * tp.stage_bytes) return 0;
    tp.ns = room / tp.stage_bytes;
    if (tp.ns > TMA_MAX_STAGES) tp.ns = TMA_MAX_STAGES;
    return static_cast<size_t>(tp.off_stage) + static_cast<size_t>(tp.ns) * tp.stage_bytes;
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
