// The C ABI of libmlxq (include/mlxq.h): validation, kernel selection and launch geometry.
// Host-side only; the kernels live in qmv.cuh, aux_kernels.cu and qgemm_sm100.cu.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include "../../include/mlxq.h"
#include "api_internal.h"
#include "aux_kernels.cuh"
#include "qgemm.cuh"
#include "qmv.cuh"
#include "qmv_mma.cuh"
#include "qmv_pipe.cuh"
#include "dense.cuh"
#include "qmv_tok.cuh"

namespace mlxq {

static thread_local std::string t_last_error;

int fail(int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    t_last_error = buf;
    return status;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(e == cudaErrorMemoryAllocation ? MLXQ_OUT_OF_MEMORY : MLXQ_GPU_FAILURE, "%s: %s", what,
                cudaGetErrorString(e));
}

// One error word per device, written by kernels (bad lookup id, a bounded wait that ran out).
__device__ unsigned g_err_word;
static std::mutex g_err_mu;
static unsigned* g_err_ptr[64] = {};

unsigned* device_error_word(int device) {
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_err_mu);
    if (!g_err_ptr[device]) {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != device) cudaSetDevice(device);
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_err_word) == cudaSuccess) g_err_ptr[device] = static_cast<unsigned*>(p);
        if (cur != device) cudaSetDevice(cur);
    }
    return g_err_ptr[device];
}

int device_sm_count(int device) {
    static int cached[64] = {};
    if (device < 0 || device >= 64) return 148;
    if (!cached[device]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cached[device] = n;
    }
    return cached[device];
}

static bool valid_dtype(int dt) { return dt == MLXQ_F32 || dt == MLXQ_F16 || dt == MLXQ_BF16; }

static long env_long(const char* name, long dflt) {
    const char* v = getenv(name);
    if (!v || !*v) return dflt;
    char* end = nullptr;
    long r = strtol(v, &end, 10);
    return end && *end == 0 ? r : dflt;
}

class DeviceGuard {
public:
    explicit DeviceGuard(int device) {
        ok_ = cudaGetDevice(&prev_) == cudaSuccess;
        if (ok_ && prev_ != device) ok_ = cudaSetDevice(device) == cudaSuccess; else prev_ = -1;
    }
    ~DeviceGuard() { if (prev_ >= 0) cudaSetDevice(prev_); }
    bool ok() const { return ok_; }
private:
    int prev_ = -1;
    bool ok_ = false;
};

static int validate_desc(const mlxq_linear_desc* d, int* bits_out, int* gs_out) {
    const char* name = d->name ? d->name : "linear";
    // Shapes come from an untrusted file: reject anything a kernel could index out of bounds with.
    if (!d->weight || d->weight_rows <= 0 || d->weight_cols <= 0 || d->in_dim <= 0)
        return fail(MLXQ_INVALID_FILE, "%s: weight must be a 2-D tensor", name);
    if (d->expect_out > 0 && d->weight_rows != d->expect_out)
        return fail(MLXQ_INVALID_FILE, "%s: expected %lld output rows, found %lld", name, (long long)d->expect_out,
                    (long long)d->weight_rows);
    if (d->bias && d->bias_len != d->weight_rows)
        return fail(MLXQ_INVALID_FILE, "%s: bias shape [%lld]", name, (long long)d->bias_len);
    if (d->scales && !d->biases) return fail(MLXQ_MISSING_TENSOR, "%s.biases", name);
    if (!d->scales) {
        // dense layer (Transformer.swift:103-112): weights of a floating type, as many columns as inputs
        const int wdt = d->reserved - 1;
        if (d->biases) return fail(MLXQ_INVALID_FILE, "%s: inconsistent quantization tensors", name);
        if (!valid_dtype(wdt)) return fail(MLXQ_UNSUPPORTED, "%s: weight dtype of a dense layer not given or not floating", name);
        if (d->weight_cols != d->in_dim)
            return fail(MLXQ_INVALID_FILE, "%s: expected %lld input columns, found %lld", name, (long long)d->in_dim, (long long)d->weight_cols);
        if (d->in_dim % 4 != 0) return fail(MLXQ_UNSUPPORTED, "%s: input dim %lld", name, (long long)d->in_dim);
        if (d->bias && !valid_dtype(d->bias_dtype)) return fail(MLXQ_UNSUPPORTED, "%s: bias dtype %d", name, d->bias_dtype);
        if (d->in_dim > (1LL << 30) || d->weight_rows > (1LL << 30)) return fail(MLXQ_UNSUPPORTED, "%s: dimensions beyond 2^30", name);
        if (d->device < 0 || d->device >= 64) return fail(MLXQ_INVALID_ARGUMENT, "%s: device %d", name, d->device);
        *bits_out = 0;
        *gs_out = 0;
        return MLXQ_OK;
    }
    if (d->scales_rows != d->weight_rows || d->scales_cols <= 0 || d->in_dim % d->scales_cols != 0 ||
        d->biases_rows != d->scales_rows || d->biases_cols != d->scales_cols ||
        (d->weight_cols * 32) % d->in_dim != 0)
        return fail(MLXQ_INVALID_FILE, "%s: inconsistent quantization tensors", name);
    const long long bits = d->weight_cols * 32 / d->in_dim, gs = d->in_dim / d->scales_cols;
    const bool bits_ok = bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8;
    if (!bits_ok || gs % 8 != 0 || d->in_dim % 8 != 0)
        return fail(MLXQ_UNSUPPORTED, "%s: %lld-bit / group %lld quantization", name, bits, gs);
    if (!valid_dtype(d->scale_dtype)) return fail(MLXQ_UNSUPPORTED, "%s: scales dtype %d", name, d->scale_dtype);
    if (d->bias && !valid_dtype(d->bias_dtype)) return fail(MLXQ_UNSUPPORTED, "%s: bias dtype %d", name, d->bias_dtype);
    if (d->in_dim > (1LL << 30) || d->weight_rows > (1LL << 30))
        return fail(MLXQ_UNSUPPORTED, "%s: dimensions beyond 2^30", name);
    if (d->device < 0 || d->device >= 64) return fail(MLXQ_INVALID_ARGUMENT, "%s: device %d", name, d->device);
    *bits_out = static_cast<int>(bits);
    *gs_out = static_cast<int>(gs);
    return MLXQ_OK;
}

static mlxq_linear* make_handle(const mlxq_linear_desc* d, int bits, int gs) {
    auto* h = new (std::nothrow) mlxq_linear();
    if (!h) return nullptr;
    h->w = static_cast<const uint8_t*>(d->weight);
    h->s = d->scales;
    h->b = d->biases;
    h->bias = d->bias;
    h->in_dim = d->in_dim;
    h->out_dim = d->weight_rows;
    h->bits = bits;
    h->gs = gs;
    h->s_dtype = d->scale_dtype;
    h->bias_dtype = d->bias ? d->bias_dtype : d->scale_dtype;
    h->w_dtype = bits == 0 ? d->reserved - 1 : 0;
    h->device = d->device;
    h->row_offset = 0;
    h->total_out = d->weight_rows;
    h->shard_rank = 0;
    h->shard_count = 1;
    h->name = d->name ? d->name : "linear";
    // The reference resolves its fused decode kernel only under these conditions (Transformer.swift:76-77);
    // fusable() and canFuse() report them unchanged.
    const int align = bits == 4 ? 32 : 16;
    h->qmv_eligible = bits != 0 && d->in_dim % align == 0 && gs % align == 0 && (!d->bias || h->bias_dtype == h->s_dtype);
    return h;
}

static size_t row_bytes(const mlxq_linear* h) { return static_cast<size_t>(h->in_dim) * h->bits / 8; }

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_x(const void* x, int x_dtype, int64_t x_stride, int64_t K, int64_t T) {
    if (!x) return fail(MLXQ_INVALID_ARGUMENT, "x is null");
    if (!valid_dtype(x_dtype)) return fail(MLXQ_INVALID_ARGUMENT, "x dtype %d", x_dtype);
    if (T > 1 && x_stride < K) return fail(MLXQ_INVALID_ARGUMENT, "x stride %lld < in_dim %lld", (long long)x_stride, (long long)K);
    if (!aligned16(x) || (T > 1 && (x_stride * dtype_size(x_dtype)) % 16 != 0))
        return fail(MLXQ_INVALID_ARGUMENT, "x rows must start on 16-byte boundaries");
    return MLXQ_OK;
}

static cudaError_t launch_qmv_bits(int bits, const QmvParams& p, cudaStream_t st) {
    switch (bits) {
        case 2: return launch_qmv_b2(p, st);
        case 3: return launch_qmv_b3(p, st);
        case 4: return launch_qmv_b4(p, st);
        case 5: return launch_qmv_b5(p, st);
        case 6: return launch_qmv_b6(p, st);
        default: return launch_qmv_b8(p, st);
    }
}

// Fills the launch description of the CUDA-core kernel for up to three layers that share K/bits/gs.
static void fill_qmv(QmvParams& p, const mlxq_linear_t* parts, int n) {
    memset(&p, 0, sizeof p);
    const mlxq_linear* f = parts[0];
    p.n_parts = n;
    bool fast = true;
    int total = 0;
    for (int i = 0; i < 3; i++) {
        const mlxq_linear* h = parts[i < n ? i : n - 1];
        p.part[i].w = h->w;
        p.part[i].s = h->s;
        p.part[i].b = h->b;
        p.part[i].bias = h->bias;
        p.part[i].rows = static_cast<int>(h->out_dim);
        if (i < n) {
            total += static_cast<int>(h->out_dim);
            fast = fast && aligned16(h->w);
        }
    }
    p.total_rows = total;
    p.K = static_cast<int>(f->in_dim);
    p.gs = f->gs;
    p.s_dtype = f->s_dtype;
    p.bias_dtype = f->bias_dtype;
    p.has_bias = f->bias != nullptr;
    p.fast = fast && row_bytes(f) % 16 == 0;
    p.seg32 = f->gs % 32 == 0;
    p.gs_shift = -1;
    for (int s = 3; s < 31; s++) if ((1 << s) == f->gs) p.gs_shift = s;
}

// The tensor-core decode kernel takes a call when the batch is small, the group size is 32/64/128, K is a
// multiple of the kernel's step and the rows are aligned for vector loads.  MLXQ_DECODE=cuda forces the
// CUDA-core kernel (which handles every shape).  Returns the shared memory needed, 0 when not eligible.
static size_t mma_plan(const mlxq_linear_t* parts, int n, int x_dtype, int64_t T, MmaParams& mp, bool* planned = nullptr) {
    if (planned) *planned = false;
    const mlxq_linear* f = parts[0];
    const char* mode = getenv("MLXQ_DECODE");
    if (mode && strcmp(mode, "cuda") == 0) return 0;
    if (T > 16 || (f->gs != 32 && f->gs != 64 && f->gs != 128)) return 0;
    const int kb = qmv_mma_step_codes(f->bits);
    if (f->in_dim % kb != 0) return 0;
    for (int i = 0; i < n; i++)
        if (!aligned16(parts[i]->w)) return 0;
    mp.split = x_dtype == MLXQ_F32 ? 2 : 1;
    if (!qmv_mma_plan(f->bits, static_cast<int>(f->in_dim), f->gs, static_cast<int>(T) * mp.split, mp)) return 0;
    if (planned) *planned = true;       // (the column plan exists; the register-fed kernel may still not fit: 0)
    return qmv_mma_smem(static_cast<int>(f->in_dim), f->gs, static_cast<int>(T), mp);
}

static int run_qmv(const mlxq_linear_t* parts, int n, cudaStream_t st, const void* x, int x_dtype, int64_t x_stride,
                   void* y, int y_dtype, int64_t y_stride, int64_t T, const float* e, int act,
                   const PeerGather* peer = nullptr, const float* x_up = nullptr, int x_act = 0) {
    for (int i = 0; i < n; i++)
        if (parts[i]->bits == 0) return fail(MLXQ_UNSUPPORTED, "%s is a dense layer: only mlxq_linear_forward serves it", parts[i]->name.c_str());
    QmvParams p;
    fill_qmv(p, parts, n);
    p.x_up = x_up;
    p.x_act = x_act;
    if (peer) p.peer = *peer; else p.peer.n = 0;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    p.x_stride = x_stride;
    p.y_stride = y_stride;
    p.e = e;
    p.act = act;
    if (T > 16 && !peer && !x_up && !e) {
        // A long batch on a layer the tensor-core GEMM does not take (anything but 4-bit, or unaligned): sixteen (or
        // eight) tokens at a time on the token-major kernel -- the weights are then read once per sixteen tokens through
        // the tensor cores instead of once per four through the CUDA cores.
        for (int chunk = 16; chunk >= 8; chunk /= 2) {
            MmaParams mc;
            bool okc = false;
            mma_plan(parts, n, x_dtype, chunk, mc, &okc);
            if (!okc) continue;
            p.T = chunk; p.x = x; p.y = y;
            mc.q = p;
            mc.err = device_error_word(parts[0]->device);
            TokPlan tc;
            const char* mode = getenv("MLXQ_DECODE");
            if (!mc.err || (mode && (strcmp(mode, "mma") == 0 || strcmp(mode, "pipe") == 0)) ||
                !qmv_tok_plan(parts[0]->bits, mc, chunk, device_sm_count(parts[0]->device), tc))
                continue;
            // (every call takes exactly `chunk` tokens -- the last one reaches back over tokens already done -- so a token's
            // result does not depend on the batch it came in)
            for (int64_t t0 = 0; t0 < T; t0 += chunk) {
                const int64_t at = t0 + chunk <= T ? t0 : T - chunk;
                const int rc = run_qmv(parts, n, st, static_cast<const char*>(x) + static_cast<size_t>(at) * x_stride * dtype_size(x_dtype), x_dtype,
                                       x_stride, static_cast<char*>(y) + static_cast<size_t>(at) * y_stride * dtype_size(y_dtype), y_dtype, y_stride,
                                       chunk, nullptr, act, nullptr);
                if (rc != MLXQ_OK) return rc;
            }
            return MLXQ_OK;
        }
    }
    MmaParams mp;
    bool planned = false;
    const size_t smem = mma_plan(parts, n, x_dtype, T, mp, &planned);
    if (planned) {
        p.T = static_cast<int>(T);
        p.x = x;
        p.y = y;
        mp.q = p;
        mp.err = device_error_word(parts[0]->device);
        // Preferred: the persistent kernel fed by asynchronous copies (MLXQ_DECODE=mma keeps the register-fed one).
        const char* mode = getenv("MLXQ_DECODE");
        const bool persistent = !(mode && strcmp(mode, "mma") == 0) && mp.err;
        if (persistent && T >= 2 && !(mode && strcmp(mode, "pipe") == 0)) {
            // two or more tokens: the token-major kernel where it serves the call (MLXQ_DECODE=pipe keeps the other)
            TokPlan tp;
            const size_t tsmem = qmv_tok_plan(parts[0]->bits, mp, static_cast<int>(T), device_sm_count(parts[0]->device), tp);
            if (tsmem) {
                const cudaError_t err = launch_qmv_tok(parts[0]->bits, mp, tp, tsmem, parts[0]->device, st);
                if (err != cudaSuccess) return cuda_fail(err, "qmv (token-major) launch");
                return MLXQ_OK;
            }
        }
        PipePlan pp;
        const size_t rsmem = !persistent ? 0 : qmv_pipe_plan(parts[0]->bits, mp, static_cast<int>(T), device_sm_count(parts[0]->device), pp);
        if (peer && !rsmem) return fail(MLXQ_UNSUPPORTED, "this shape does not run on the persistent decode kernel: no fused gather");
        // does a call of `t` tokens run on one of the persistent kernels?
        auto fits_persistent = [&](int64_t t) {
            MmaParams m2;
            bool ok2 = false;
            mma_plan(parts, n, x_dtype, t, m2, &ok2);
            if (!ok2) return false;
            m2.q = p;
            m2.q.T = static_cast<int>(t);
            m2.err = mp.err;
            TokPlan t2;
            PipePlan p2;
            const int sms = device_sm_count(parts[0]->device);
            return (t >= 2 && qmv_tok_plan(parts[0]->bits, m2, static_cast<int>(t), sms, t2) != 0) || qmv_pipe_plan(parts[0]->bits, m2, static_cast<int>(t), sms, p2) != 0;
        };
        const int64_t h0 = T / 2;
        if (persistent && !rsmem && T >= 4 && fits_persistent(h0) && fits_persistent(T - h0)) {
            // Too many staged activation columns for a CTA's shared memory (long rows): two calls of half the tokens,
            // each on a persistent kernel, beat the register-fed kernel although the weights are read twice.
            const int rc = run_qmv(parts, n, st, x, x_dtype, x_stride, y, y_dtype, y_stride, h0, e, act, nullptr, x_up, x_act);
            if (rc != MLXQ_OK) return rc;
            return run_qmv(parts, n, st, static_cast<const char*>(x) + static_cast<size_t>(h0) * x_stride * dtype_size(x_dtype), x_dtype, x_stride,
                           static_cast<char*>(y) + static_cast<size_t>(h0) * y_stride * dtype_size(y_dtype), y_dtype, y_stride, T - h0, e, act, nullptr,
                           x_up ? x_up + static_cast<size_t>(h0) * x_stride : nullptr, x_act);
        }
        if (x_up && !rsmem) return fail(MLXQ_UNSUPPORTED, "this shape does not run on the persistent decode kernels: no gated input");
        if (rsmem || smem) {
            cudaError_t err = rsmem ? launch_qmv_pipe(parts[0]->bits, mp, pp, rsmem, parts[0]->device, st)
                                    : launch_qmv_mma(parts[0]->bits, mp, smem, parts[0]->device, st);
            if (err != cudaSuccess) return cuda_fail(err, "qmv (tensor-core) launch");
            return MLXQ_OK;
        }
    }
    if (peer) return fail(MLXQ_UNSUPPORTED, "this shape does not run on the persistent decode kernel: no fused gather");
    if (x_up) return fail(MLXQ_UNSUPPORTED, "this shape does not run on the persistent decode kernels: no gated input");
    // gridDim.y carries token tiles of four; walk very long batches in slices.
    const int64_t slice = 4 * 65535;
    for (int64_t t0 = 0; t0 < T; t0 += slice) {
        const int64_t nt = T - t0 < slice ? T - t0 : slice;
        p.T = static_cast<int>(nt);
        p.x = static_cast<const char*>(x) + static_cast<size_t>(t0) * x_stride * dtype_size(x_dtype);
        p.y = static_cast<char*>(y) + static_cast<size_t>(t0) * y_stride * dtype_size(y_dtype);
        cudaError_t err = launch_qmv_bits(parts[0]->bits, p, st);
        if (err != cudaSuccess) return cuda_fail(err, "qmv launch");
    }
    return MLXQ_OK;
}

static GemmLayer gemm_layer(const mlxq_linear* h) {
    GemmLayer L;
    L.w = h->w; L.s = h->s; L.b = h->b; L.bias = h->bias;
    L.s_dtype = h->s_dtype; L.bias_dtype = h->bias_dtype;
    L.O = static_cast<int>(h->out_dim); L.K = static_cast<int>(h->in_dim); L.gs = h->gs; L.bits = h->bits;
    L.device = h->device;
    return L;
}

// Token count from which a batch goes to the tensor-core GEMM (when the layer qualifies).
static int64_t gemm_min_tokens() { return env_long("MLXQ_GEMM_MIN_T", 17); }

static int gemm_tile_for(const mlxq_linear* h, int x_dtype, int64_t x_stride, const void* x, int64_t T) {
    if (T < gemm_min_tokens()) return 0;
    return qgemm_tile_tokens(gemm_layer(h), x_dtype, x_stride, x, T);
}

// The layer's GEMM table, built once (device memory owned by the handle).  Returns nullptr when it cannot be kept --
// the stream is being captured, or the allocation failed -- and the GEMM then stages the table per call as before.
// `allow_build` is false on the path that must not allocate.
static const void* gemm_table_of(mlxq_linear* h, cudaStream_t st, bool allow_build) {
    std::lock_guard<std::mutex> lk(h->table_mu);
    if (h->gemm_table || h->table_tried || !allow_build) return h->gemm_table;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    h->table_tried = true;
    const GemmLayer L = gemm_layer(h);
    void* t = nullptr;
    if (cudaMalloc(&t, qgemm_table_bytes(L)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    // built on the caller's stream and awaited once, so that calls on other streams may use it at once
    if (qgemm_build_table(L, t, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(t);
        return nullptr;
    }
    h->gemm_table = t;
    return t;
}

int forward_impl(mlxq_linear_t h, cudaStream_t st, const void* x, int x_dtype, int64_t x_stride, void* y, int y_dtype,
                 int64_t y_stride, int64_t T, const PeerGather* peer) {
    if (!h) return fail(MLXQ_INVALID_ARGUMENT, "null layer");
    if (T < 1) return fail(MLXQ_INVALID_ARGUMENT, "T = %lld", (long long)T);
    if (int rc = check_x(x, x_dtype, x_stride, h->in_dim, T)) return rc;
    if (!y || !valid_dtype(y_dtype)) return fail(MLXQ_INVALID_ARGUMENT, "y is null or has dtype %d", y_dtype);
    if (T > 1 && y_stride < h->out_dim) return fail(MLXQ_INVALID_ARGUMENT, "y stride %lld < out_dim", (long long)y_stride);
    DeviceGuard guard(h->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", h->device);
    if (h->bits == 0) {
        if (peer) return fail(MLXQ_UNSUPPORTED, "%s is a dense layer: no fused gather", h->name.c_str());
        const cudaError_t err = launch_dense(h->w, h->w_dtype, h->bias, h->bias_dtype, x, x_dtype, x_stride, y, y_dtype, y_stride, T,
                                             static_cast<int>(h->out_dim), static_cast<int>(h->in_dim), st);
        return err == cudaSuccess ? MLXQ_OK : cuda_fail(err, "dense launch");
    }
    if (gemm_tile_for(h, x_dtype, x_stride, x, T) > 0) {
        if (peer) return fail(MLXQ_UNSUPPORTED, "batches of %lld tokens take the GEMM: no fused gather", (long long)T);
        GemmCall c;
        c.x = x; c.x_dtype = x_dtype; c.x_stride = x_stride; c.y = y; c.y_dtype = y_dtype; c.y_stride = y_stride; c.T = T;
        c.err = device_error_word(h->device);
        if (!c.err) return fail(MLXQ_GPU_FAILURE, "no error word on device %d", h->device);
        c.table = gemm_table_of(h, st, true);
        const char* why = "";
        cudaError_t err = launch_qgemm(gemm_layer(h), c, st, &why);
        if (err != cudaSuccess) return fail(MLXQ_GPU_FAILURE, "qgemm launch: %s (%s)", cudaGetErrorString(err), why);
        return MLXQ_OK;
    }
    return run_qmv(&h, 1, st, x, x_dtype, x_stride, y, y_dtype, y_stride, T, nullptr, 0, peer);
}

}  // namespace mlxq

using namespace mlxq;

extern "C" {

int mlxq_version(void) { return 100; }

const char* mlxq_status_string(int status) {
    switch (status) {
        case MLXQ_OK: return "ok";
        case MLXQ_INVALID_FILE: return "Invalid model file";
        case MLXQ_UNSUPPORTED: return "Unsupported model";
        case MLXQ_MISSING_TENSOR: return "Missing tensor";
        case MLXQ_OUT_OF_MEMORY: return "Not enough memory";
        case MLXQ_GPU_FAILURE: return "GPU error";
        case MLXQ_INVALID_ARGUMENT: return "Invalid argument";
        case MLXQ_NCCL_FAILURE: return "Collective error";
        case MLXQ_TIMEOUT: return "A bounded device-side wait ran out";
        default: return "unknown status";
    }
}

const char* mlxq_last_error(void) { return t_last_error.c_str(); }

int mlxq_linear_create(const mlxq_linear_desc* desc, mlxq_linear_t* out) {
    if (!desc || !out) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    int bits = 0, gs = 0;
    if (int rc = validate_desc(desc, &bits, &gs)) return rc;
    mlxq_linear* h = make_handle(desc, bits, gs);
    if (!h) return fail(MLXQ_OUT_OF_MEMORY, "handle allocation");
    *out = h;
    return MLXQ_OK;
}

int mlxq_linear_create_shard(const mlxq_linear_desc* desc, int rank, int nranks, int desc_is_full, mlxq_linear_t* out) {
    if (!desc || !out) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (nranks < 1 || rank < 0 || rank >= nranks) return fail(MLXQ_INVALID_ARGUMENT, "rank %d of %d", rank, nranks);
    int bits = 0, gs = 0;
    if (int rc = validate_desc(desc, &bits, &gs)) return rc;
    if (bits == 0) return fail(MLXQ_UNSUPPORTED, "%s: dense layers are not sharded", desc->name ? desc->name : "linear");
    mlxq_linear_desc d = *desc;
    int64_t total = desc->weight_rows;
    if (desc_is_full) {
        if (total % (8LL * nranks) != 0)
            return fail(MLXQ_UNSUPPORTED, "%s: %lld output rows do not split into %d shards of a multiple of 8 rows",
                        desc->name ? desc->name : "linear", (long long)total, nranks);
        const int64_t rows = total / nranks, r0 = rows * rank;
        const size_t sb = dtype_size(desc->scale_dtype);
        d.weight = static_cast<const char*>(desc->weight) + static_cast<size_t>(r0) * desc->weight_cols * 4;
        d.scales = static_cast<const char*>(desc->scales) + static_cast<size_t>(r0) * desc->scales_cols * sb;
        d.biases = static_cast<const char*>(desc->biases) + static_cast<size_t>(r0) * desc->biases_cols * sb;
        if (desc->bias) d.bias = static_cast<const char*>(desc->bias) + static_cast<size_t>(r0) * dtype_size(desc->bias_dtype);
        d.weight_rows = d.scales_rows = d.biases_rows = rows;
        if (desc->bias) d.bias_len = rows;
        d.expect_out = 0;
    } else {
        if (desc->weight_rows % 8 != 0)
            return fail(MLXQ_UNSUPPORTED, "%s: a shard must hold a multiple of 8 rows", desc->name ? desc->name : "linear");
        total = desc->weight_rows * nranks;
    }
    mlxq_linear* h = make_handle(&d, bits, gs);
    if (!h) return fail(MLXQ_OUT_OF_MEMORY, "handle allocation");
    h->row_offset = h->out_dim * rank;
    h->total_out = total;
    h->shard_rank = rank;
    h->shard_count = nranks;
    *out = h;
    return MLXQ_OK;
}

void mlxq_linear_destroy(mlxq_linear_t h) {
    if (!h) return;
    if (h->gemm_table) {
        DeviceGuard guard(h->device);
        cudaFree(h->gemm_table);
    }
    delete h;
}

int mlxq_linear_prepare(mlxq_linear_t h, mlxq_stream_t stream) {
    if (!h) return fail(MLXQ_INVALID_ARGUMENT, "null layer");
    if (h->bits == 0) return MLXQ_OK;
    DeviceGuard guard(h->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", h->device);
    if (qgemm_tile_tokens(gemm_layer(h), MLXQ_BF16, h->in_dim, nullptr, 1024) == 0) return MLXQ_OK;      // the GEMM never takes this layer
    if (!gemm_table_of(h, static_cast<cudaStream_t>(stream), true))
        return fail(MLXQ_OUT_OF_MEMORY, "%s: the GEMM's scale table (%zu bytes) could not be built ahead", h->name.c_str(),
                    qgemm_table_bytes(gemm_layer(h)));
    return MLXQ_OK;
}

int64_t mlxq_linear_in_dim(mlxq_linear_t h) { return h ? h->in_dim : 0; }
int64_t mlxq_linear_out_dim(mlxq_linear_t h) { return h ? h->out_dim : 0; }
int mlxq_linear_bits(mlxq_linear_t h) { return h ? h->bits : 0; }
int mlxq_linear_group_size(mlxq_linear_t h) { return h ? h->gs : 0; }
int64_t mlxq_linear_row_offset(mlxq_linear_t h) { return h ? h->row_offset : 0; }
int64_t mlxq_linear_total_rows(mlxq_linear_t h) { return h ? h->total_out : 0; }

int mlxq_linear_forward(mlxq_linear_t h, mlxq_stream_t stream, const void* x, int x_dtype, int64_t x_stride, void* y,
                        int y_dtype, int64_t y_stride, int64_t T) {
    return forward_impl(h, static_cast<cudaStream_t>(stream), x, x_dtype, x_stride, y, y_dtype, y_stride, T);
}

int mlxq_linear_forward_static(mlxq_linear_t h, mlxq_stream_t stream, const void* x, int x_dtype, int64_t x_stride, void* y,
                               int y_dtype, int64_t y_stride, int64_t T) {
    if (!h) return fail(MLXQ_INVALID_ARGUMENT, "null layer");
    if (h->bits == 0) return fail(MLXQ_UNSUPPORTED, "%s is a dense layer: only mlxq_linear_forward serves it", h->name.c_str());
    if (T < 1) return fail(MLXQ_INVALID_ARGUMENT, "T = %lld", (long long)T);
    if (int rc = check_x(x, x_dtype, x_stride, h->in_dim, T)) return rc;
    if (!y || !valid_dtype(y_dtype)) return fail(MLXQ_INVALID_ARGUMENT, "y is null or has dtype %d", y_dtype);
    if (T > 1 && y_stride < h->out_dim) return fail(MLXQ_INVALID_ARGUMENT, "y stride %lld < out_dim", (long long)y_stride);
    DeviceGuard guard(h->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", h->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (gemm_tile_for(h, x_dtype, x_stride, x, T) > 0) {
        const unsigned long long need = static_cast<unsigned long long>(T) * static_cast<unsigned long long>(h->in_dim) * 2ull;
        if (need > qgemm_static_capacity())
            return fail(MLXQ_INVALID_ARGUMENT, "%s: T * in_dim * 2 = %llu bytes of staged activations exceed the %zu-byte static scratch; "
                        "split the batch or use mlxq_linear_forward", h->name.c_str(), need, qgemm_static_capacity());
        const void* kept = gemm_table_of(h, st, false);          // a table built ahead (mlxq_linear_prepare) needs no room
        const size_t table = kept ? 0 : qgemm_table_bytes(gemm_layer(h));
        if (table > qgemm_static_table_capacity())
            return fail(MLXQ_INVALID_ARGUMENT, "%s: the layer's staged scale table (%zu bytes, out_dim * in_dim / 8 with rows rounded up to 256) "
                        "exceeds the %zu-byte static scratch; shard the layer or use mlxq_linear_forward", h->name.c_str(), table,
                        qgemm_static_table_capacity());
        GemmCall c;
        c.x = x; c.x_dtype = x_dtype; c.x_stride = x_stride; c.y = y; c.y_dtype = y_dtype; c.y_stride = y_stride; c.T = T;
        c.err = device_error_word(h->device);
        if (!c.err) return fail(MLXQ_GPU_FAILURE, "no error word on device %d", h->device);
        c.table = kept;
        const char* why = "";
        cudaError_t err = launch_qgemm_static(gemm_layer(h), c, st, &why);
        if (err != cudaSuccess) return fail(MLXQ_GPU_FAILURE, "qgemm launch: %s (%s)", cudaGetErrorString(err), why);
        return MLXQ_OK;
    }
    // batches the GEMM does not take run on kernels that use no scratch memory at all
    return run_qmv(&h, 1, st, x, x_dtype, x_stride, y, y_dtype, y_stride, T, nullptr, 0);
}

int mlxq_fusable(const mlxq_linear_t* parts, int n) {
    if (!parts || n < 1 || n > 3 || !parts[0]) return 0;
    const mlxq_linear* f = parts[0];
    const bool has_bias = f->bias != nullptr;
    for (int i = 0; i < n; i++) {
        const mlxq_linear* p = parts[i];
        if (!p || !p->qmv_eligible || p->bits != f->bits || p->gs != f->gs || p->in_dim != f->in_dim ||
            p->s_dtype != f->s_dtype || p->out_dim % 8 != 0 || (p->bias != nullptr) != has_bias)
            return 0;
    }
    return 1;
}

int mlxq_can_fuse(const mlxq_linear_t* parts, int n, int64_t T) {
    if (!parts || n < 1) return 0;
    for (int i = 0; i < n; i++) {
        if (!parts[i] || !parts[i]->qmv_eligible) return 0;
        if (T != 1 && (T > 8 || parts[i]->bits != 4)) return 0;
    }
    return T >= 1;
}

int mlxq_use_gemm64(int64_t T, int64_t out_dim) {
    const int64_t rows64 = (T + 63) / 64 * 64, rows32 = (T + 31) / 32 * 32;
    return rows64 * 5 <= rows32 * 6 && (T + 63) / 64 * ((out_dim + 63) / 64) >= 64;
}

int mlxq_gemm_tile_tokens(mlxq_linear_t h, int64_t T) {
    if (!h || T < 1 || h->bits == 0) return 0;
    return gemm_tile_for(h, MLXQ_BF16, h->in_dim, nullptr, T);
}

const char* mlxq_kernel_for(mlxq_linear_t h, int x_dtype, int y_dtype, int64_t T) {
    (void)y_dtype;
    if (!h || T < 1) return "";
    if (h->bits == 0) return "dmm";
    if (gemm_tile_for(h, x_dtype, h->in_dim, nullptr, T) > 0) return "qgemm";
    return T <= 16 ? "qmv" : "qmm";
}

int mlxq_fused_forward(const mlxq_linear_t* parts, int n, mlxq_stream_t stream, const void* x, int x_dtype,
                       int64_t x_stride, void* y, int y_dtype, int64_t y_stride, int64_t T) {
    if (!parts || n < 1 || n > 3) return fail(MLXQ_INVALID_ARGUMENT, "1 to 3 layers can be fused, got %d", n);
    const mlxq_linear* f = parts[0];
    if (!f) return fail(MLXQ_INVALID_ARGUMENT, "null layer");
    int64_t total = 0;
    for (int i = 0; i < n; i++) {
        const mlxq_linear* p = parts[i];
        if (!p) return fail(MLXQ_INVALID_ARGUMENT, "null layer");
        if (p->bits != f->bits || p->gs != f->gs || p->in_dim != f->in_dim || p->s_dtype != f->s_dtype ||
            p->device != f->device || (p->bias != nullptr) != (f->bias != nullptr) || p->bias_dtype != f->bias_dtype ||
            (n > 1 && p->out_dim % 8 != 0))
            return fail(MLXQ_INVALID_ARGUMENT, "%s and %s cannot share one launch", f->name.c_str(), p->name.c_str());
        total += p->out_dim;
    }
    if (T < 1) return fail(MLXQ_INVALID_ARGUMENT, "T = %lld", (long long)T);
    if (int rc = check_x(x, x_dtype, x_stride, f->in_dim, T)) return rc;
    if (!y || !valid_dtype(y_dtype)) return fail(MLXQ_INVALID_ARGUMENT, "y is null or has dtype %d", y_dtype);
    if (T > 1 && y_stride < total) return fail(MLXQ_INVALID_ARGUMENT, "y stride %lld < %lld rows", (long long)y_stride, (long long)total);
    DeviceGuard guard(f->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", f->device);
    return run_qmv(parts, n, static_cast<cudaStream_t>(stream), x, x_dtype, x_stride, y, y_dtype, y_stride, T, nullptr, 0);
}

int mlxq_linear_forward_gated(mlxq_linear_t h, mlxq_stream_t stream, const void* x, int x_dtype, void* y, int y_dtype,
                              const float* e, int act) {
    if (!h) return fail(MLXQ_INVALID_ARGUMENT, "null layer");
    if (!e) return fail(MLXQ_INVALID_ARGUMENT, "e is null");
    if (act < 0 || act > 2) return fail(MLXQ_INVALID_ARGUMENT, "act %d", act);
    if (int rc = check_x(x, x_dtype, h->in_dim, h->in_dim, 1)) return rc;
    if (!y || !valid_dtype(y_dtype)) return fail(MLXQ_INVALID_ARGUMENT, "y is null or has dtype %d", y_dtype);
    DeviceGuard guard(h->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", h->device);
    return run_qmv(&h, 1, static_cast<cudaStream_t>(stream), x, x_dtype, h->in_dim, y, y_dtype, h->out_dim, 1, e, act);
}

int mlxq_linear_forward_glu(mlxq_linear_t h, mlxq_stream_t stream, const float* gu, int64_t gu_stride, int act, void* y,
                            int y_dtype, int64_t y_stride, int64_t T) {
    if (!h || !gu) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (act < 0 || act > 2) return fail(MLXQ_INVALID_ARGUMENT, "act %d", act);
    if (T < 1 || T > 8) return fail(MLXQ_UNSUPPORTED, "gated input serves 1 to 8 tokens (T = %lld)", (long long)T);
    if (gu_stride < 2 * h->in_dim) return fail(MLXQ_INVALID_ARGUMENT, "gate|up stride %lld < 2 x in_dim", (long long)gu_stride);
    if (int rc = check_x(gu, MLXQ_F32, gu_stride, h->in_dim, T)) return rc;
    if (int rc = check_x(gu + h->in_dim, MLXQ_F32, gu_stride, h->in_dim, T)) return rc;
    if (!y || !valid_dtype(y_dtype)) return fail(MLXQ_INVALID_ARGUMENT, "y is null or has dtype %d", y_dtype);
    if (T > 1 && y_stride < h->out_dim) return fail(MLXQ_INVALID_ARGUMENT, "y stride %lld < out_dim", (long long)y_stride);
    DeviceGuard guard(h->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", h->device);
    return run_qmv(&h, 1, static_cast<cudaStream_t>(stream), gu, MLXQ_F32, gu_stride, y, y_dtype, y_stride, T, nullptr, 0, nullptr,
                   gu + h->in_dim, act);
}

int mlxq_act_mul(mlxq_stream_t stream, int device, const float* gu, int64_t stride, int64_t cols, int64_t T, int act, float* out) {
    if (!gu || !out) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (act < 0 || act > 2 || cols < 1 || T < 0 || stride < 2 * cols) return fail(MLXQ_INVALID_ARGUMENT, "act %d, cols %lld, T %lld, stride %lld", act, (long long)cols, (long long)T, (long long)stride);
    DeviceGuard guard(device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", device);
    cudaError_t err = launch_act_mul(gu, stride, cols, T, act, out, static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? MLXQ_OK : cuda_fail(err, "act_mul launch");
}

int mlxq_add_rms_norm(mlxq_stream_t stream, int device, float* h, const float* r, float* y, const void* w, int w_dtype,
                      int64_t dim, int64_t rows, int64_t row_stride, float eps) {
    if (!h || !r || !y || !w) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (!valid_dtype(w_dtype) || dim < 4 || dim % 4 != 0 || rows < 0 || row_stride < dim || row_stride % 4 != 0)
        return fail(MLXQ_INVALID_ARGUMENT, "dim %lld, rows %lld, row stride %lld, weight dtype %d", (long long)dim, (long long)rows, (long long)row_stride, w_dtype);
    if (!aligned16(h) || !aligned16(r) || !aligned16(y)) return fail(MLXQ_INVALID_ARGUMENT, "rows must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", device);
    cudaError_t err = launch_add_rms_norm(h, r, y, w, w_dtype, dim, rows, row_stride, eps, static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? MLXQ_OK : cuda_fail(err, "add_rms_norm launch");
}

int mlxq_linear_lookup(mlxq_linear_t h, mlxq_stream_t stream, const int32_t* ids, float* out, int64_t T) {
    if (!h || !ids || !out) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (h->bits == 0) return fail(MLXQ_UNSUPPORTED, "%s is a dense layer: only mlxq_linear_forward serves it", h->name.c_str());
    if (T < 0) return fail(MLXQ_INVALID_ARGUMENT, "T = %lld", (long long)T);
    DeviceGuard guard(h->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", h->device);
    unsigned* errw = device_error_word(h->device);
    if (!errw) return fail(MLXQ_GPU_FAILURE, "no error word on device %d", h->device);
    cudaError_t err = launch_lookup(h->w, h->s, h->b, h->s_dtype, ids, out, T, static_cast<int>(h->out_dim),
                                    static_cast<int>(h->in_dim), h->gs, h->bits, errw,
                                    static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? MLXQ_OK : cuda_fail(err, "lookup launch");
}

int mlxq_linear_forward_rows(mlxq_linear_t h, mlxq_stream_t stream, const void* x, int x_dtype, float* y,
                             const uint32_t* count, const int32_t* list, int64_t max_rows) {
    if (!h || !x || !y || !count || !list) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (h->bits == 0) return fail(MLXQ_UNSUPPORTED, "%s is a dense layer: only mlxq_linear_forward serves it", h->name.c_str());
    if (!valid_dtype(x_dtype) || max_rows < 0) return fail(MLXQ_INVALID_ARGUMENT, "x dtype %d, max_rows %lld", x_dtype, (long long)max_rows);
    DeviceGuard guard(h->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", h->device);
    cudaError_t err = launch_rows(h->w, h->s, h->b, h->s_dtype, x, x_dtype, y, count, list, max_rows,
                                  static_cast<int>(h->out_dim), static_cast<int>(h->in_dim), h->gs, h->bits,
                                  static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? MLXQ_OK : cuda_fail(err, "row-list launch");
}

int mlxq_block_max(mlxq_stream_t stream, int device, const float* logits, int64_t stride, int64_t V, int64_t T,
                   int32_t index_base, uint32_t* pairs) {
    if (!logits || !pairs) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (V < 1 || T < 0 || stride < V || V > 0x7fffff00ll || index_base < 0 || static_cast<int64_t>(index_base) + V > 0x7fffff00ll)
        return fail(MLXQ_INVALID_ARGUMENT, "V %lld, T %lld, stride %lld, index base %d", (long long)V, (long long)T, (long long)stride, index_base);
    DeviceGuard guard(device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", device);
    cudaError_t err = launch_block_max(logits, stride, V, T, index_base, pairs, static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? MLXQ_OK : cuda_fail(err, "block maxima launch");
}

int mlxq_block_argmax(mlxq_stream_t stream, int device, const uint32_t* pairs, int n_seg, int64_t T, int64_t nb,
                      int32_t* token, float* value) {
    if (!pairs || !token) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (n_seg < 1 || T < 0 || nb < 1 || nb * n_seg > 0x7fffffffll) return fail(MLXQ_INVALID_ARGUMENT, "%d segments of %lld blocks, T %lld", n_seg, (long long)nb, (long long)T);
    DeviceGuard guard(device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", device);
    cudaError_t err = launch_block_argmax(pairs, n_seg, T, static_cast<int>(nb), token, value, static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? MLXQ_OK : cuda_fail(err, "block argmax launch");
}

int mlxq_unpack_codes(mlxq_linear_t h, mlxq_stream_t stream, uint8_t* out) {
    if (!h || !out) return fail(MLXQ_INVALID_ARGUMENT, "null argument");
    if (h->bits == 0) return fail(MLXQ_UNSUPPORTED, "%s is a dense layer: only mlxq_linear_forward serves it", h->name.c_str());
    if (reinterpret_cast<uintptr_t>(out) % 8 != 0) return fail(MLXQ_INVALID_ARGUMENT, "out must be 8-byte aligned");
    DeviceGuard guard(h->device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", h->device);
    cudaError_t err = launch_unpack_codes(h->w, out, h->out_dim, static_cast<int>(h->in_dim), h->bits,
                                          static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? MLXQ_OK : cuda_fail(err, "unpack launch");
}

int mlxq_stream_status(mlxq_stream_t stream, int device) {
    DeviceGuard guard(device);
    if (!guard.ok()) return fail(MLXQ_GPU_FAILURE, "cannot select device %d", device);
    cudaError_t err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return cuda_fail(err, "stream");
    unsigned* wp = device_error_word(device);
    if (!wp) return fail(MLXQ_GPU_FAILURE, "no error word on device %d", device);
    unsigned word = 0;
    err = cudaMemcpy(&word, wp, sizeof word, cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) return cuda_fail(err, "error word read");
    if (word) {
        unsigned zero = 0;
        cudaMemcpy(wp, &zero, sizeof zero, cudaMemcpyHostToDevice);
        if (word & ERR_WAIT_TIMEOUT) return fail(MLXQ_TIMEOUT, "a device-side wait ran out (error word 0x%x)", word);
        if (word & ERR_BAD_LOOKUP_ID) return fail(MLXQ_GPU_FAILURE, "lookup id outside the table (error word 0x%x)", word);
        return fail(MLXQ_GPU_FAILURE, "kernel reported error word 0x%x", word);
    }
    return MLXQ_OK;
}

}  // extern "C"
