/*
 * CPU oracle for the MLX affine quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the CPU algorithms the reference project (BackendStack21/mlx-runner,
 * Swift) uses to define and check its quantized-linear layer.  It is the checker the CUDA library is
 * compared with; it is never linked into, called from, or shipped with the product library.  Only the
 * test suite, the smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * Pinning: the reference holds no stored input/output vectors for this path (every expected value in
 * its tests is recomputed on the CPU from a seeded xorshift generator), and its Swift sources cannot
 * be compiled here.  The oracle is therefore pinned against the literal known-answer material the
 * reference's tests do contain -- the f16 bit patterns of Tests/MLXEngineTests/EngineTests.swift:213,
 * the float->half round trip of Tests/MLXEngineTests/SieveTests.swift:113-126, the quantize4 ->
 * dequantize bound of SieveTests.swift:288-306 and the useGemm64 truth table of
 * Tests/MLXEngineTests/KernelTests.swift:153-156,179 -- and against an independent bit-by-bit Python
 * restatement of the packer.  Matvec outputs are pinned by algorithm, not by stored numbers.
 *
 * Each function cites the reference file:line it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ---- seeded generator: Tests/MLXEngineTests/KernelTests.swift:8-14 (struct RNG) ------------------ */
ORACLE_API uint64_t mlxq_o_rng_next(uint64_t* s) {
    uint64_t v = *s;
    v ^= v << 13;
    v ^= v >> 7;
    v ^= v << 17;
    *s = v;
    return v;
}

/* RNG.float(lo, hi): lo + (hi - lo) * Float(next() % 1_000_000) / 1_000_000, all in Float. */
ORACLE_API float mlxq_o_rng_float(uint64_t* s, float lo, float hi) {
    float r = (float)(mlxq_o_rng_next(s) % 1000000ull);
    float w = hi - lo;
    float p = w * r;
    return lo + p / 1000000.0f;
}

/* Bulk draws, in stream order (QuantFixture draws O*K codes, then (scale, bias) pairs: KernelTests.swift:57-61). */
ORACLE_API void mlxq_o_rng_fill_codes(uint64_t* s, size_t n, int bits, uint8_t* out) {
    for (size_t i = 0; i < n; i++) out[i] = (uint8_t)(mlxq_o_rng_next(s) % (1ull << bits));
}
ORACLE_API void mlxq_o_rng_fill_floats(uint64_t* s, size_t n, float lo, float hi, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = mlxq_o_rng_float(s, lo, hi);
}
/* n pairs (a in [lo0,hi0), b in [lo1,hi1)) drawn alternately. */
ORACLE_API void mlxq_o_rng_fill_pairs(uint64_t* s, size_t n, float lo0, float hi0, float lo1, float hi1, float* a, float* b) {
    for (size_t i = 0; i < n; i++) { a[i] = mlxq_o_rng_float(s, lo0, hi0); b[i] = mlxq_o_rng_float(s, lo1, hi1); }
}

/* ---- half / bf16 conversions ------------------------------------------------------------------------ */

static inline float bits_to_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t float_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* Tensor.halfToFloat: Sources/MLXEngine/GPU.swift:170-183. */
ORACLE_API float mlxq_o_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    int exp = (h >> 10) & 0x1F;
    uint32_t frac = h & 0x3FFu;
    if (exp == 0) {
        if (frac == 0) return bits_to_float(sign);
        int e = 127 - 15 + 1;
        uint32_t f = frac;
        while ((f & 0x400u) == 0) { f <<= 1; e -= 1; }
        return bits_to_float(sign | ((uint32_t)e << 23) | ((f & 0x3FFu) << 13));
    }
    if (exp == 31) return bits_to_float(sign | 0x7F800000u | (frac << 13));
    return bits_to_float(sign | ((uint32_t)(exp + 127 - 15) << 23) | (frac << 13));
}

/* SieveImporter.halfBits (round to nearest even): Sources/MLXEngine/SieveImport.swift:65-86. */
ORACLE_API uint16_t mlxq_o_float_to_half(float f) {
    uint32_t x = float_to_bits(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    int e = (int)((x >> 23) & 0xFF);
    uint32_t man = x & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (man != 0 ? 0x200u : 0u));
    int exp = e - 127 + 15;
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t h = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1u))) h += 1;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h += 1;
    return (uint16_t)(sign | h); /* a mantissa carry has already walked into the exponent field of h */
}

/* bf16 by truncation: Tests/MLXEngineTests/KernelTests.swift:45-46 (the reference's test helper). */
ORACLE_API uint16_t mlxq_o_float_to_bf16_trunc(float f) { return (uint16_t)(float_to_bits(f) >> 16); }
ORACLE_API float mlxq_o_bf16_to_float(uint16_t u) { return bits_to_float((uint32_t)u << 16); }
/* bf16 round-to-nearest-even: what numpy/torch produce; used for the benchmark-shaped inputs. */
ORACLE_API uint16_t mlxq_o_float_to_bf16_rne(float f) {
    uint32_t x = float_to_bits(f);
    if ((x & 0x7F800000u) == 0x7F800000u && (x & 0x7FFFFFu)) return (uint16_t)((x >> 16) | 0x40u);
    x += 0x7FFFu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

/* Scale / bias / activation storage types shared with the C ABI: 0 = f32, 1 = f16, 2 = bf16. */
static inline float load_as_float(const void* p, int dtype, size_t i) {
    switch (dtype) {
        case 0: return ((const float*)p)[i];
        case 1: return mlxq_o_half_to_float(((const uint16_t*)p)[i]);
        default: return mlxq_o_bf16_to_float(((const uint16_t*)p)[i]);
    }
}

ORACLE_API void mlxq_o_to_float(const void* src, int dtype, size_t n, float* dst) {
    for (size_t i = 0; i < n; i++) dst[i] = load_as_float(src, dtype, i);
}

/* ---- the packed format ------------------------------------------------------------------------------ */

/* pack(): Tests/MLXEngineTests/KernelTests.swift:34-43.  Bit j of code i goes to bit i*bits+j of the
 * little-endian byte stream. `out` holds (n*bits+7)/8 bytes and is cleared first. */
ORACLE_API void mlxq_o_pack(const uint8_t* q, size_t n, int bits, uint8_t* out) {
    memset(out, 0, (n * (size_t)bits + 7) / 8);
    for (size_t i = 0; i < n; i++)
        for (int b = 0; b < bits; b++)
            if ((q[i] >> b) & 1) {
                size_t bit = i * (size_t)bits + (size_t)b;
                out[bit / 8] |= (uint8_t)(1u << (bit % 8));
            }
}

/* Code j of a row: SieveImporter.dequantize, Sources/MLXEngine/SieveImport.swift:104-108
 * (two-byte window, shift, mask). */
static inline uint32_t code_at(const uint8_t* row, size_t j, int bits) {
    size_t bit = j * (size_t)bits, at = bit / 8;
    unsigned sh = (unsigned)(bit % 8);
    uint32_t v = row[at];
    if (sh + (unsigned)bits > 8) v |= (uint32_t)row[at + 1] << 8;
    return (v >> sh) & ((1u << bits) - 1u);
}

/* Unpack O rows of K codes each (row r starts at byte r*K*bits/8) into one byte per code. */
ORACLE_API void mlxq_o_unpack(const uint8_t* packed, size_t O, size_t K, int bits, uint8_t* q) {
    size_t row_bytes = K * (size_t)bits / 8;
    for (size_t r = 0; r < O; r++)
        for (size_t j = 0; j < K; j++) q[r * K + j] = (uint8_t)code_at(packed + r * row_bytes, j, bits);
}

/* SieveImporter.dequantize: SieveImport.swift:90-112.  out[r,j] = Float(q)*scale + bias in fp32
 * (multiply then add, two roundings, as Swift evaluates it). */
ORACLE_API void mlxq_o_dequantize(const uint8_t* packed, const void* scales, const void* biases, int sdtype,
                                  size_t O, size_t K, int bits, size_t gs, float* out) {
    size_t row_bytes = K * (size_t)bits / 8, groups = K / gs;
    for (size_t r = 0; r < O; r++) {
        const uint8_t* row = packed + r * row_bytes;
        for (size_t j = 0; j < K; j++) {
            size_t g = r * groups + j / gs;
            volatile float prod = (float)code_at(row, j, bits) * load_as_float(scales, sdtype, g);
            out[r * K + j] = prod + load_as_float(biases, sdtype, g);
        }
    }
}

/* QuantFixture.reference: KernelTests.swift:102-113.  y[t,o] = Float(sum_k Double(w)*Double(x)) + bias[o].
 * `dense` is the fp32 dequantised table [O][K]; bias may be NULL. */
ORACLE_API void mlxq_o_matmul_dense(const float* dense, const float* x, const float* bias, size_t T, size_t O,
                                    size_t K, float* y) {
    for (size_t t = 0; t < T; t++)
        for (size_t o = 0; o < O; o++) {
            double acc = 0;
            for (size_t k = 0; k < K; k++) acc += (double)dense[o * K + k] * (double)x[t * K + k];
            y[t * O + o] = (float)acc + (bias ? bias[o] : 0.0f);
        }
}

/* The same result without materialising the dense table (for shapes where [O][K] floats is too much):
 * unpack + fp32 dequant + double accumulate per row, OpenMP over output rows.  x is fp32 [T, x_stride],
 * y fp32 [T, y_stride]; row bias (fp32, optional) is added after the cast, as KernelTests.swift:109 does.
 * accumulate_double = 0 gives the fp32-accumulate variant timed as the CPU baseline (the reference's
 * production CPU path is dequantize-to-fp32 followed by sgemm, SieveImport.swift:90-112, :346). */
ORACLE_API void mlxq_o_qmatmul(const uint8_t* packed, const void* scales, const void* biases, int sdtype,
                               const float* bias, const float* x, size_t x_stride, float* y, size_t y_stride,
                               size_t T, size_t O, size_t K, int bits, size_t gs, int accumulate_double,
                               int threads) {
    size_t row_bytes = K * (size_t)bits / 8, groups = K / gs;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
#pragma omp parallel
    {
        float* w = (float*)malloc(K * sizeof(float));
#pragma omp for schedule(static)
        for (long long ro = 0; ro < (long long)O; ro++) {
            size_t o = (size_t)ro;
            const uint8_t* row = packed + o * row_bytes;
            for (size_t j = 0; j < K; j++) {
                size_t g = o * groups + j / gs;
                volatile float prod = (float)code_at(row, j, bits) * load_as_float(scales, sdtype, g);
                w[j] = prod + load_as_float(biases, sdtype, g);
            }
            for (size_t t = 0; t < T; t++) {
                const float* xt = x + t * x_stride;
                float v;
                if (accumulate_double) {
                    double acc = 0;
                    for (size_t k = 0; k < K; k++) acc += (double)w[k] * (double)xt[k];
                    v = (float)acc;
                } else {
                    float acc = 0;
                    for (size_t k = 0; k < K; k++) acc += w[k] * xt[k];
                    v = acc;
                }
                y[t * y_stride + o] = v + (bias ? bias[o] : 0.0f);
            }
        }
        free(w);
    }
}

ORACLE_API int mlxq_o_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- gated epilogue: Sources/MLXEngine/Kernels.swift:116-130 (erf_nr, act_mul) --------------------- */
static float erf_nr(float x) {
    const float z = fabsf(x), t = 1.0f / (1.0f + 0.5f * z);
    const float r = t * expf(-z * z - 1.26551223f +
                             t * (1.00002368f +
                                  t * (0.37409196f +
                                       t * (0.09678418f +
                                            t * (-0.18628806f +
                                                 t * (0.27886807f +
                                                      t * (-1.13520398f +
                                                           t * (1.48851587f + t * (-0.82215223f + t * 0.17087277f)))))))));
    return x >= 0.0f ? 1.0f - r : r - 1.0f;
}

ORACLE_API float mlxq_o_act_mul(int act, float g, float u) {
    if (act == 0) return (g / (1.0f + expf(-g))) * u;
    if (act == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    return 0.5f * g * (1.0f + erf_nr(g * 0.7071067811865476f)) * u;
}

/* ---- quantize4: Sources/MLXEngine/SieveImport.swift:244-265 -------------------------------------- */
/* s [V x r] is overwritten with the values the kernel will compute with; codes u32 [V*r/8], scales and
 * biases f16 bits [V*r/64]. */
ORACLE_API void mlxq_o_quantize4(float* s, size_t V, size_t r, uint32_t* codes, uint16_t* scales, uint16_t* biases) {
    size_t groups = r / 64;
    memset(codes, 0, V * r / 8 * sizeof(uint32_t));
    for (size_t row = 0; row < V; row++) {
        float* p = s + row * r;
        for (size_t g = 0; g < groups; g++) {
            float lo = INFINITY, hi = -INFINITY;
            for (size_t j = g * 64; j < g * 64 + 64; j++) { lo = fminf(lo, p[j]); hi = fmaxf(hi, p[j]); }
            uint16_t sb = mlxq_o_float_to_half((hi - lo) / 15.0f), bb = mlxq_o_float_to_half(lo);
            float sc = mlxq_o_half_to_float(sb), bi = mlxq_o_half_to_float(bb);
            scales[row * groups + g] = sb;
            biases[row * groups + g] = bb;
            for (size_t j = g * 64; j < g * 64 + 64; j++) {
                float q = 0.0f;
                if (sc > 0) {
                    /* Swift's .rounded() is round-half-away-from-zero, which is roundf(). */
                    q = fminf(15.0f, fmaxf(0.0f, roundf((p[j] - bi) / sc)));
                }
                codes[(row * r + j) / 8] |= (uint32_t)q << (4 * (j % 8));
                volatile float prod = q * sc;
                p[j] = prod + bi;
            }
        }
    }
}

/* ---- host policy functions the reference tests pin ------------------------------------------------ */

/* Linear.useGemm64: Sources/MLXEngine/Transformer.swift:266-269. */
ORACLE_API int mlxq_o_use_gemm64(int T, int outDim) {
    int rows64 = (T + 63) / 64 * 64, rows32 = (T + 31) / 32 * 32;
    return rows64 * 5 <= rows32 * 6 && (T + 63) / 64 * ((outDim + 63) / 64) >= 64;
}

/* assertClose metric: KernelTests.swift:116-124.  max |a-b| / max(1, |b|). */
ORACLE_API float mlxq_o_max_rel_err(const float* a, const float* b, size_t n) {
    float worst = 0;
    for (size_t i = 0; i < n; i++) {
        float err = fabsf(a[i] - b[i]) / fmaxf(1.0f, fabsf(b[i]));
        if (!(err <= worst)) worst = err; /* NaN propagates as "worst" */
    }
    return worst;
}
