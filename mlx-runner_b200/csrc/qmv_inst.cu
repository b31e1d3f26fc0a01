// One instantiation set of the decode matvec per bit width: compiled six times with -DMLXQ_BITS=n so the
// translation units build in parallel.
#include "qmv.cuh"

#ifndef MLXQ_BITS
#error "compile with -DMLXQ_BITS=2|3|4|5|6|8"
#endif

#define MLXQ_CAT2(a, b) a##b
#define MLXQ_CAT(a, b) MLXQ_CAT2(a, b)

namespace mlxq {

template <typename XT>
static cudaError_t launch_typed(const QmvParams& p, cudaStream_t st) {
    constexpr int R = QmvUnit<MLXQ_BITS>::R;
    const dim3 block(QMV_WARPS * 32);
    const int rows_per_block = QMV_WARPS * R;
    const unsigned gx = static_cast<unsigned>((p.total_rows + rows_per_block - 1) / rows_per_block);
    if (p.T == 1) {
        qmv_kernel<MLXQ_BITS, XT, 1><<<dim3(gx, 1), block, 0, st>>>(p);
    } else if (p.T == 2) {
        qmv_kernel<MLXQ_BITS, XT, 2><<<dim3(gx, 1), block, 0, st>>>(p);
    } else {
        qmv_kernel<MLXQ_BITS, XT, 4><<<dim3(gx, static_cast<unsigned>((p.T + 3) / 4)), block, 0, st>>>(p);
    }
    return cudaGetLastError();
}

cudaError_t MLXQ_CAT(launch_qmv_b, MLXQ_BITS)(const QmvParams& p, cudaStream_t st) {
    switch (p.x_dtype) {
        case DT_F32: return launch_typed<float>(p, st);
        case DT_F16: return launch_typed<__half>(p, st);
        default: return launch_typed<__nv_bfloat16>(p, st);
    }
}

}  // namespace mlxq
