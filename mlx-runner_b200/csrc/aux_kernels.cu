// Small kernels beside the matvec / GEMM: code unpack (the bit-exact format check), embedding-row lookup
// and the row-list matvec.  All three walk the bit stream in 8-code chunks (BITS bytes each, byte
// aligned for every bit width).
#include "aux_kernels.cuh"

namespace mlxq {

// out[r, k] = code k of row r, one byte each.  One thread per 8-code chunk.
__global__ void unpack_codes_kernel(const uint8_t* __restrict__ w, uint8_t* __restrict__ out, long long rows, int K,
                                    int bits) {
    const long long chunks_per_row = K / 8;
    const long long n = rows * chunks_per_row;
    const unsigned mask = (1u << bits) - 1u;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / chunks_per_row, c = i - r * chunks_per_row;
        const uint64_t v = chunk_bits_rt(w + (static_cast<size_t>(r) * K / 8 + c) * bits, bits);
        uint64_t packed = 0;
        for (int j = 0; j < 8; j++) packed |= static_cast<uint64_t>((v >> (j * bits)) & mask) << (8 * j);
        *reinterpret_cast<uint64_t*>(out + static_cast<size_t>(r) * K + c * 8) = packed;
    }
}

// out[t, k] = scale * q[ids[t], k] + bias, fp32.  Grid (chunks, T).
__global__ void lookup_kernel(const uint8_t* __restrict__ w, const void* __restrict__ scales, const void* __restrict__ biases,
                              int s_dtype, const int32_t* __restrict__ ids, float* __restrict__ out, int rows, int K, int gs,
                              int bits, unsigned* err) {
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= K / 8) return;
    const int row = __ldg(ids + t);
    float* o = out + static_cast<size_t>(t) * K + c * 8;
    if (row < 0 || row >= rows) {
        if (c == 0) atomicOr(err, ERR_BAD_LOOKUP_ID);
        for (int j = 0; j < 8; j++) o[j] = 0.0f;
        return;
    }
    const size_t row_bytes = static_cast<size_t>(K) * bits / 8;
    const uint64_t v = chunk_bits_rt(w + row * row_bytes + static_cast<size_t>(c) * bits, bits);
    const unsigned mask = (1u << bits) - 1u;
    const size_t gi = static_cast<size_t>(row) * (K / gs) + (c * 8) / gs;
    const float s = load_scalar(scales, s_dtype, gi), b = load_scalar(biases, s_dtype, gi);
    for (int j = 0; j < 8; j++) {
        // multiply then add, two roundings: the layer's definition evaluates q*scale + bias unfused
        o[j] = __fadd_rn(__fmul_rn(static_cast<float>((v >> (j * bits)) & mask), s), b);
    }
}

// y[list[i]] = W[list[i]] . x for i < *count, one warp per listed row.
__global__ void rows_kernel(const uint8_t* __restrict__ w, const void* __restrict__ scales, const void* __restrict__ biases,
                            int s_dtype, const void* __restrict__ x, int x_dtype, float* __restrict__ y,
                            const uint32_t* __restrict__ count, const int32_t* __restrict__ list, int rows, int K, int gs,
                            int bits) {
    const unsigned e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (e >= __ldg(count)) return;
    const int row = __ldg(list + e);
    if (row < 0 || row >= rows) return;
    const size_t row_bytes = static_cast<size_t>(K) * bits / 8;
    const uint8_t* wr = w + row * row_bytes;
    const int gpr = K / gs;
    const unsigned mask = (1u << bits) - 1u;
    float acc = 0.0f;
    for (int c = lane; c < K / 8; c += 32) {
        const uint64_t v = chunk_bits_rt(wr + static_cast<size_t>(c) * bits, bits);
        float d = 0.0f, xs = 0.0f;
        for (int j = 0; j < 8; j++) {
            const float xv = load_scalar(x, x_dtype, c * 8 + j);
            d = fmaf(static_cast<float>((v >> (j * bits)) & mask), xv, d);
            xs += xv;
        }
        const size_t gi = static_cast<size_t>(row) * gpr + (c * 8) / gs;
        acc = fmaf(load_scalar(biases, s_dtype, gi), xs, fmaf(load_scalar(scales, s_dtype, gi), d, acc));
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) y[row] = acc;
}

cudaError_t launch_unpack_codes(const uint8_t* w, uint8_t* out, long long rows, int K, int bits, cudaStream_t st) {
    const long long n = rows * (K / 8);
    if (n == 0) return cudaSuccess;
    const int block = 256;
    const long long want = (n + block - 1) / block;
    const unsigned grid = static_cast<unsigned>(want < 148LL * 16 ? want : 148LL * 16);
    unpack_codes_kernel<<<grid, block, 0, st>>>(w, out, rows, K, bits);
    return cudaGetLastError();
}

cudaError_t launch_lookup(const uint8_t* w, const void* scales, const void* biases, int s_dtype, const int32_t* ids,
                          float* out, long long T, int rows, int K, int gs, int bits, unsigned* err, cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    const int chunks = K / 8;
    const int block = chunks < 256 ? ((chunks + 31) / 32) * 32 : 256;
    // gridDim.y is limited to 65535: walk longer id lists in slices.
    for (long long t0 = 0; t0 < T; t0 += 65535) {
        const unsigned ty = static_cast<unsigned>(T - t0 < 65535 ? T - t0 : 65535);
        lookup_kernel<<<dim3((chunks + block - 1) / block, ty), block, 0, st>>>(
            w, scales, biases, s_dtype, ids + t0, out + static_cast<size_t>(t0) * K, rows, K, gs, bits, err);
    }
    return cudaGetLastError();
}

cudaError_t launch_rows(const uint8_t* w, const void* scales, const void* biases, int s_dtype, const void* x, int x_dtype,
                        float* y, const uint32_t* count, const int32_t* list, long long max_rows, int rows, int K, int gs,
                        int bits, cudaStream_t st) {
    if (max_rows == 0) return cudaSuccess;
    const int warps = 4;
    rows_kernel<<<static_cast<unsigned>((max_rows + warps - 1) / warps), warps * 32, 0, st>>>(
        w, scales, biases, s_dtype, x, x_dtype, y, count, list, rows, K, gs, bits);
    return cudaGetLastError();
}

// ---- token selection, first pass (sample_blocks, Kernels.swift:2339-2377) -------------------------------------------
// One warp per block of 256 logits: lane l scans eight contiguous values in index order with a strict `>` (so a NaN
// never wins and the lowest index of equal values does), then the warp takes the maximum and, among the lanes that
// hold it, the lowest index.  bmax[t][b] / barg[t][b]; a block without any value above -inf reports SELECT_NONE.
__global__ void block_max_kernel(const float* __restrict__ logits, long long stride, long long V, int nb, long long T,
                                 int index_base, float* __restrict__ bmax, int* __restrict__ barg, int vec_ok) {
    const int lane = threadIdx.x & 31;
    const long long wid = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= T * nb) return;
    const long long t = wid / nb;
    const int b = static_cast<int>(wid - t * nb);
    const float* row = logits + t * stride;
    const long long i0 = static_cast<long long>(b) * SELECT_BLOCK + lane * 8;
    float best = -INFINITY;
    int bi = SELECT_NONE;
    if (vec_ok && i0 + 8 <= V) {
        const float4 a = *reinterpret_cast<const float4*>(row + i0), c = *reinterpret_cast<const float4*>(row + i0 + 4);
        const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
        for (int j = 0; j < 8; j++) if (v[j] > best) { best = v[j]; bi = static_cast<int>(i0) + j; }
    } else {
        for (long long i = i0; i < V && i < i0 + 8; i++) { const float v = row[i]; if (v > best) { best = v; bi = static_cast<int>(i); } }
    }
    float m = best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    int idx = best == m ? bi : SELECT_NONE;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) idx = min(idx, __shfl_xor_sync(0xffffffffu, idx, o));
    if (lane == 0) {
        bmax[t * nb + b] = m;
        barg[t * nb + b] = idx == SELECT_NONE ? SELECT_NONE : idx + index_base;
    }
}

// ---- token selection, greedy second pass: the maximum over the blocks of every segment and the lowest index that
// holds it (the argmax branch of sample_token, Kernels.swift:2379 ff.) -- one CTA per token --------------------------
__global__ void block_argmax_kernel(const uint32_t* __restrict__ pairs, int n_seg, long long T, int nb, int* __restrict__ token,
                                    float* __restrict__ value) {
    __shared__ float sm[8];
    __shared__ int si[8];
    const long long t = blockIdx.x;
    const long long seg_words = 2 * T * nb;
    float best = -INFINITY;
    int bi = SELECT_NONE;
    for (int i = threadIdx.x; i < n_seg * nb; i += blockDim.x) {
        const int seg = i / nb, b = i - seg * nb;
        const uint32_t* base = pairs + seg * seg_words;
        const float m = __uint_as_float(base[t * nb + b]);
        const int ix = static_cast<int>(base[T * nb + t * nb + b]);
        if (m > best || (m == best && ix < bi)) { best = m; bi = ix; }
    }
    float m = best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    int idx = best == m ? bi : SELECT_NONE;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) idx = min(idx, __shfl_xor_sync(0xffffffffu, idx, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sm[warp] = m; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        float mm = lane < nw ? sm[lane] : -INFINITY;
        const int ii = lane < nw ? si[lane] : SELECT_NONE;
        float top = mm;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
        int idx2 = mm == top ? ii : SELECT_NONE;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) idx2 = min(idx2, __shfl_xor_sync(0xffffffffu, idx2, o));
        if (lane == 0) { token[t] = idx2; if (value) value[t] = top; }
    }
}

cudaError_t launch_block_max(const float* logits, long long stride, long long V, long long T, int index_base, uint32_t* pairs,
                             cudaStream_t st) {
    if (T == 0 || V == 0) return cudaSuccess;
    const int nb = static_cast<int>((V + SELECT_BLOCK - 1) / SELECT_BLOCK);
    const int warps = 8;
    const long long n = T * nb;
    const int vec_ok = (reinterpret_cast<uintptr_t>(logits) % 16 == 0 && stride % 4 == 0) ? 1 : 0;
    block_max_kernel<<<static_cast<unsigned>((n + warps - 1) / warps), warps * 32, 0, st>>>(
        logits, stride, V, nb, T, index_base, reinterpret_cast<float*>(pairs), reinterpret_cast<int*>(pairs) + T * nb, vec_ok);
    return cudaGetLastError();
}

cudaError_t launch_block_argmax(const uint32_t* pairs, int n_seg, long long T, int nb, int32_t* token, float* value, cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    block_argmax_kernel<<<static_cast<unsigned>(T), 256, 0, st>>>(pairs, n_seg, T, nb, token, value);
    return cudaGetLastError();
}

// ---- silu_mul / gelu_tanh_mul (Kernels.swift:2004-2030): out[t, i] = act(gu[t, i]) * gu[t, cols + i] ----------------
__global__ void act_mul_kernel(const float* __restrict__ gu, long long stride, long long cols, int act, float* __restrict__ out) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long t = blockIdx.y;
    if (i >= cols) return;
    const float g = gu[t * stride + i], u = gu[t * stride + cols + i];
    out[t * cols + i] = act_mul(act, g, u);
}

// ---- add_rms_norm (Kernels.swift:1141-1175): h += r; y = RMSNorm(h) * w, one CTA per row.  The sum of squares is
// taken per thread over float4s in a strided order, then per warp, then over the warps in order, as the reference's
// threadgroup does; dim is a multiple of 4 and the rows are 16-byte aligned (checked on the host). -------------------
__global__ void add_rms_norm_kernel(float* __restrict__ hbuf, const float* __restrict__ r, float* __restrict__ y, const void* __restrict__ w,
                                    int w_dtype, int dim, long long row_stride, float eps) {
    __shared__ float buf[32];
    const long long row = blockIdx.x;
    float4* hr = reinterpret_cast<float4*>(hbuf + row * row_stride);
    const float4* rr = reinterpret_cast<const float4*>(r + row * row_stride);
    float4* yr = reinterpret_cast<float4*>(y + row * row_stride);
    const int n4 = dim / 4;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        const float4 a = hr[i], b = rr[i];
        const float4 v = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
        hr[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) buf[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
    for (int s = 0; s < nw; s++) tot += buf[s];
    const float inv = rsqrtf(tot / static_cast<float>(dim) + eps);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        const float4 v = hr[i];
        const float w0 = load_scalar(w, w_dtype, 4 * i), w1 = load_scalar(w, w_dtype, 4 * i + 1), w2 = load_scalar(w, w_dtype, 4 * i + 2),
                    w3 = load_scalar(w, w_dtype, 4 * i + 3);
        yr[i] = make_float4(v.x * inv * w0, v.y * inv * w1, v.z * inv * w2, v.w * inv * w3);
    }
}

cudaError_t launch_act_mul(const float* gu, long long stride, long long cols, long long T, int act, float* out, cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    if (T > 65535) return cudaErrorInvalidValue;
    act_mul_kernel<<<dim3(static_cast<unsigned>((cols + 255) / 256), static_cast<unsigned>(T)), 256, 0, st>>>(gu, stride, cols, act, out);
    return cudaGetLastError();
}

cudaError_t launch_add_rms_norm(float* h, const float* r, float* y, const void* w, int w_dtype, long long dim, long long rows,
                                long long row_stride, float eps, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    add_rms_norm_kernel<<<static_cast<unsigned>(rows), 256, 0, st>>>(h, r, y, w, w_dtype, static_cast<int>(dim), row_stride, eps);
    return cudaGetLastError();
}

}  // namespace mlxq
