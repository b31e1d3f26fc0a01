// Instantiations and launcher of the tensor-core decode matvec (qmv_mma.cuh).
#include "qmv_mma.cuh"

#include <mutex>

namespace mlxq {

namespace {

template <int BITS> constexpr int kb_of() { return MmaUnit<BITS>::KB; }

int kb_for(int bits) {
    switch (bits) {
        case 2: return kb_of<2>();
        case 3: return kb_of<3>();
        case 4: return kb_of<4>();
        case 5: return kb_of<5>();
        case 6: return kb_of<6>();
        default: return kb_of<8>();
    }
}

template <int BITS, int NP>
cudaError_t launch_one(const MmaParams& p, size_t smem, int device, cudaStream_t st) {
    // the shared-memory opt-in belongs to one device's context: once per device, with that device current
    static std::mutex mu;
    static bool done[64] = {};
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!done[device]) {
            const cudaError_t e = cudaFuncSetAttribute(qmv_mma_kernel<BITS, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            done[device] = true;
        }
    }
    const unsigned grid = static_cast<unsigned>((p.q.total_rows + 15) / 16);
    qmv_mma_kernel<BITS, NP><<<grid, MMA_WARPS * 32, smem, st>>>(p);
    return cudaGetLastError();
}

template <int BITS>
cudaError_t launch_bits(const MmaParams& p, size_t smem, int device, cudaStream_t st) {
    if (p.passes <= 1) return launch_one<BITS, 1>(p, smem, device, st);
    if (p.passes <= 2) return launch_one<BITS, 2>(p, smem, device, st);
    if (p.passes <= 4) return launch_one<BITS, 4>(p, smem, device, st);
    if (p.passes <= 8) return launch_one<BITS, 8>(p, smem, device, st);
    return cudaErrorNotSupported;
}

}  // namespace

int qmv_mma_step_codes(int bits) { return kb_for(bits); }

static int ilog2(int v) { int s = 0; while ((1 << s) < v) s++; return s; }

bool qmv_mma_plan(int bits, int K, int gs, int xn, MmaParams& p) {
    if (gs != 32 && gs != 64 && gs != 128) return false;
    const int kb = kb_for(bits);
    if (K % kb != 0 || K < kb || xn < 1) return false;
    const int gstep = gs <= kb ? kb / gs : 1;
    p.gstep_shift = ilog2(gstep);
    p.spg_shift = gs > kb ? ilog2(gs / kb) : 0;
    if (gs > kb && (K / kb) % (gs / kb) != 0) return false;
    const int cols = xn * gstep;
    p.passes = (cols + 7) / 8;
    if (p.passes > 8) return false;
    p.cycle = 1;
    if (p.passes == 1) while (p.cycle * 2 * cols <= 8) p.cycle *= 2;
    p.xn = xn;
    p.xstride = K + 8;
    return true;
}

size_t qmv_mma_smem(int K, int gs, int tokens, const MmaParams& p) {
    int np = 1;
    while (np < p.passes) np *= 2;
    const size_t xs = static_cast<size_t>(p.xn) * p.xstride * 2;
    const size_t xsum = static_cast<size_t>(p.xn) * (K / gs) * 4;
    const size_t part = static_cast<size_t>(MMA_WARPS) * np * 128 * 4;
    const size_t csum = static_cast<size_t>(tokens) * (K / 8) * 4;
    const size_t total = xs + xsum + part + csum;
    return total <= 200 * 1024 ? total : 0;
}

cudaError_t launch_qmv_mma(int bits, const MmaParams& p, size_t smem, int device, cudaStream_t st) {
    switch (bits) {
        case 2: return launch_bits<2>(p, smem, device, st);
        case 3: return launch_bits<3>(p, smem, device, st);
        case 4: return launch_bits<4>(p, smem, device, st);
        case 5: return launch_bits<5>(p, smem, device, st);
        case 6: return launch_bits<6>(p, smem, device, st);
        case 8: return launch_bits<8>(p, smem, device, st);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace mlxq
