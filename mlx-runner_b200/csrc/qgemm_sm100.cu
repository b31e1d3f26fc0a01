// Prefill dequant-GEMM for sm_100a: Y[T, O] = X[T, K] . W[O, K]^T with W in the 4-bit MLX affine format.
//
// Mapping onto the 5th-generation tensor cores (tcgen05):
//   * The weights are the A operand and live in TENSOR MEMORY, not shared memory.  A thread owns half a
//     weight row of the tile's current 64-wide K slice: it reads the 16 packed bytes from shared memory
//     (staged there by TMA), dequantises the 32 codes to fp16 (w = scale*q + bias, the group's scale and
//     bias in registers) and writes them to its own TMEM lane with one tcgen05.st.  A in TMEM needs no
//     swizzled shared-memory tile and costs no shared-memory bandwidth on the MMA side.
//   * Dequantisation is three logic/shift ops and four half2 FMAs per eight codes: a masked nibble left at
//     bits 4..7 of a half is the subnormal q * 2^-20, so w = fma(nibble, scale * 2^20, bias) needs no
//     conversion.  (Scales of 2^-4 and above, where scale * 2^20 would leave fp16, take an exact two-step
//     path.)  The mask pairs codes (i, i+4) of each eight, so the activations are staged with the matching
//     order 0,4,1,5,2,6,3,7 inside every eight.
//   * The activations are the B operand: TMA loads [128 tokens x 64] 16-bit tiles with the 128-byte swizzle
//     and tcgen05.mma reads them through a shared-memory descriptor.  Both operands are fp16: a kind::f16
//     MMA whose descriptor names fp16 for A and bf16 for B raises an illegal-instruction error on B200, and
//     bf16 weights would cost 2^-9 per weight, so a small kernel first writes the activations as fp16 (bf16
//     input: exact for |x| in [6.1e-5, 65504], clamped above) in the staged order into stream-ordered
//     scratch memory.
//   * One CTA computes a 256 (rows) x 128 (tokens) output tile as two M=128 MMAs that share every B tile,
//     accumulating in fp32 in TMEM (2 x 128 columns), K = 16 per instruction, issued by one thread.
//   * Warp roles: warp 0 TMA producer of activation tiles, warp 1 MMA issuer (and TMEM allocator), warp 2 TMA
//     producer of weight slabs (its own warp, so weights run ahead of the activation ring), warps 4-19
//     dequantisers (row half x K half x lane quadrant).  The same sixteen warps run the epilogue
//     (tcgen05.ld -> row bias -> store, a quarter of the tile's columns per warp): a tile's epilogue is done
//     after the first A stages of the NEXT tile are written, so the MMAs restart on a full ring.
//   * Rings: 6 shared-memory stages of activations (16 KB), 3 slabs of packed weights (256 rows x 128 bytes =
//     four K stages per TMA copy: a tile of 32-byte rows costs the TMA unit as many requests as one of
//     128-byte rows and starved the MMAs) and 4 TMEM stages for A.
//     All hand-offs are mbarriers; MMA completion is signalled with tcgen05.commit.
//   * The kernel is persistent: min(#tiles, #SMs) CTAs walk the tile list; row tiles vary fastest so the
//     CTAs running together share activation tiles in L2.
// Every wait is bounded: a wait that runs out sets the device error word, raises the CTA's abort flag and
// all roles fall through to the common exit, where TMEM is released.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>

#include "mlxq_device.cuh"
#include "qgemm.cuh"
#include "sm100_ptx.cuh"

namespace mlxq {

namespace {

constexpr int BM = 256;                 // weight rows per CTA tile (two M=128 MMA tiles)
constexpr int BN = 128;                 // tokens per tile
constexpr int BK = 64;                  // K slice per stage
constexpr int S_X = 6;                  // shared-memory stages of the activation tile
constexpr int S_W = 3;                  // shared-memory slabs of packed weights (one slab = W_SPAN stages of K)
constexpr int W_SPAN = 4;               // K stages per weight slab: 256 codes = 128 bytes per row and TMA request
constexpr int S_A = 4;                  // TMEM stages of the A operand
constexpr int X_STAGE = BN * BK * 2;    // 16384 bytes
constexpr int W_SLAB = BM * 128;        // 32768 bytes: 256 rows x 128 bytes, 128-byte swizzle
constexpr int NUM_THREADS = 20 * 32;
constexpr int W_PRODUCER = 2;           // warp that streams the packed weight slabs
// Two warps issue the MMAs, one per 128-row half of the tile (lane 0 of each).  A single thread needs ~110 cycles
// per tcgen05.mma (operands travel through uniform registers) while an M128 N128 K16 MMA executes in 64: with one
// issuer the tensor pipe was busy a third of the time.  The halves use separate accumulators and separate A
// columns, so nothing orders the two issuers against each other; stage and accumulator barriers count both.
constexpr int MMA_WARP = 1;             // issuer of half 0; it also owns the tensor-memory allocation
constexpr int MMA_WARP2 = 3;            // issuer of half 1
constexpr int DEQ_WARP0 = 4, DEQ_WARPS = 16;
constexpr int TMEM_COLS = 512;
constexpr uint32_t SCALE_MARKER = 0x7E00u;   // fp16 NaN in a staged entry: scale * 2^20 does not fit fp16
constexpr int D_COL0 = 0;               // two fp32 accumulators of BN columns each
constexpr int A_COL0 = 2 * BN;          // A ring: S_A stages x 2 halves x 32 columns
// First tensor-memory column of the 16 columns (32 fp16) that one dequantising warp stores for ring stage `sa`,
// row half `half`, K half `khalf`.
__host__ __device__ constexpr uint32_t a_col(int sa, int half, int khalf) {
    return A_COL0 + static_cast<uint32_t>((sa * 2 + half) * (BK / 2) + khalf * 16);
}

struct Barriers {
    uint64_t full_x[S_X];
    uint64_t empty_x[S_X];
    uint64_t full_w[S_W];
    uint64_t empty_w[S_W];
    uint64_t full_a[S_A];
    uint64_t empty_a[S_A];
    uint64_t d_full;
    uint64_t d_empty[2];     // per 128-row half: its issuer restarts as soon as its eight epilogue warps have read
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int SMEM_BYTES = S_X * X_STAGE + S_W * W_SLAB + sizeof(Barriers) + 1024;   // + alignment slack

struct GemmArgs {
    const void* s;
    const void* b;
    const void* bias;
    void* y;
    unsigned* err;
    long long y_stride;
    int s_dtype, bias_dtype, y_dtype;
    int O, K, gs, T;
    int gs_shift;        // log2(gs): group sizes are powers of two here
    int m_tiles, n_tiles;
    uint32_t idesc;
    const uint4* pairs;  // staged scales and biases, see stage_scales_kernel
    int o_pad;           // rows of the staged table: m_tiles * BM
};

// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle: rows of 128 bytes, 8-row
// groups 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ __half2 scale_pair(const void* p, int dt, size_t i) {
    return __float2half2_rn(load_scalar(p, dt, i));
}

// ---- the kernel -------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NUM_THREADS, 1)
qgemm4_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* x_tiles = smem;                                   // S_X x 16 KB, each 1024-byte aligned
    uint8_t* w_slabs = smem + S_X * X_STAGE;                   // S_W x 32 KB, each 1024-byte aligned
    Barriers* bars = reinterpret_cast<Barriers*>(smem + S_X * X_STAGE + S_W * W_SLAB);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_stages = a.K / BK;
    const int total_tiles = a.m_tiles * a.n_tiles;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S_X; i++) { mbar_init(&bars->full_x[i], 1); mbar_init(&bars->empty_x[i], 2); }
        for (int i = 0; i < S_W; i++) { mbar_init(&bars->full_w[i], 1); mbar_init(&bars->empty_w[i], DEQ_WARPS); }
        for (int i = 0; i < S_A; i++) { mbar_init(&bars->full_a[i], DEQ_WARPS); mbar_init(&bars->empty_a[i], 2); }
        mbar_init(&bars->d_full, 2);
        mbar_init(&bars->d_empty[0], DEQ_WARPS / 2);
        mbar_init(&bars->d_empty[1], DEQ_WARPS / 2);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
    // Launched as a programmatic dependent of the pre-pass: the set-up above and the weight producer's first slabs
    // (the layer's constants) run while it finishes; every other role first waits for it (staged activations, the
    // scale/bias table, and -- through the pre-pass's own ordering -- everything earlier in the stream).
    if (warp != W_PRODUCER) asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        // ---- TMA producer ----------------------------------------------------------------------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int tok0 = (tile / a.m_tiles) * BN, m_tile = tile % a.m_tiles;
                for (int ks = 0; ks < k_stages; ks++, it++) {
                    const int s = it % S_X;
                    if (it >= S_X && !mbar_wait(&bars->empty_x[s], ((it / S_X) - 1) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    mbar_expect_tx(&bars->full_x[s], X_STAGE);
                    tma_load_2d(x_tiles + s * X_STAGE, &map_x, &bars->full_x[s], ks * BK, tok0);
                }
            }
            // Before leaving, see every copy this thread issued land (bounded), so that no bulk copy is in
            // flight into the shared memory of a CTA that has exited.
            for (uint32_t j = it > S_X ? it - S_X : 0; j < it; j++) {
                const uint64_t t0 = global_ns();
                while (!mbar_try_wait(&bars->full_x[j % S_X], (j / S_X) & 1))
                    if (global_ns() - t0 > WAIT_NS) break;
            }
        }
    } else if (warp == W_PRODUCER) {
        // ---- TMA producer of packed weights: one slab (256 rows x 128 bytes = W_SPAN stages of K) per copy ------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
            uint32_t wi = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int row0 = (tile % a.m_tiles) * BM;
                for (int ks = 0; ks < k_stages; ks += W_SPAN, wi++) {
                    const int sw = wi % S_W;
                    if (wi >= S_W && !mbar_wait(&bars->empty_w[sw], ((wi / S_W) - 1) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    mbar_expect_tx(&bars->full_w[sw], W_SLAB);
                    tma_load_2d(w_slabs + sw * W_SLAB, &map_w, &bars->full_w[sw], ks * (BK / 2), row0);
                }
            }
            for (uint32_t j = wi > S_W ? wi - S_W : 0; j < wi; j++) {
                const uint64_t t0 = global_ns();
                while (!mbar_try_wait(&bars->full_w[j % S_W], (j / S_W) & 1))
                    if (global_ns() - t0 > WAIT_NS) break;
            }
        }
    } else if (warp == MMA_WARP || warp == MMA_WARP2) {
        // ---- MMA issuers ------------------------------------------------------------------------------------
        if (lane == 0) {
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, tile_i++) {
                if (tile_i > 0 && !mbar_wait(&bars->d_empty[warp == MMA_WARP ? 0 : 1], (tile_i - 1) & 1, &bars->abort_flag, a.err)) break;
                tc_fence_after();
                for (int ks = 0; ks < k_stages; ks++, it++) {
                    const int s = it % S_X, sa = it % S_A;
                    if (!mbar_wait(&bars->full_x[s], (it / S_X) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    if (!mbar_wait(&bars->full_a[sa], (it / S_A) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t bdesc = smem_desc_sw128(smem_u32(x_tiles + s * X_STAGE));
                    {
                        const int half = warp == MMA_WARP ? 0 : 1;
                        const uint32_t d_addr = tmem + D_COL0 + half * BN;
#pragma unroll
                        for (int kk = 0; kk < BK / 16; kk++)
                            tc_mma_ts(d_addr, tmem + a_col(sa, half, kk >> 1) + (kk & 1) * 8, bdesc + static_cast<uint64_t>(kk * 2), a.idesc, (ks | kk) != 0);
                    }
                    tc_commit(&bars->empty_x[s]);      // the activation tile of stage s is free again
                    tc_commit(&bars->empty_a[sa]);     // so is the A stage in tensor memory
                }
                if (ok) tc_commit(&bars->d_full);      // accumulators of this tile are complete
            }
        }
    } else if (warp >= DEQ_WARP0) {
        // ---- dequantisers: one thread per (weight row, half of the 64-wide K slice) ---------------------------
        const int dw = warp - DEQ_WARP0;
        const int khalf = dw >> 3;                              // which 32 codes of the slice
        const int half = (dw >> 2) & 1;                         // which 128-row MMA tile
        const int quad = warp & 3;                              // TMEM lane quadrant this warp may touch
        const int r = quad * 32 + lane;                         // row within the 128-row tile
        const int gpr = a.K >> a.gs_shift;
        const __half2 kMul = __halves2half2(__float2half(0.0625f), __float2half(0.0625f));
        const __half2 kSub = __halves2half2(__float2half(-64.0f), __float2half(-64.0f));
        uint32_t it = 0, wi = 0, tile_i = 0;
        bool ok = true;
        // Epilogue of one tile: this warp drains its lane quadrant of one row half, 64 of the 128 token columns.
        const int e_half = (dw >> 2) & 1, e_cols = (dw >> 3) * 64;
        auto epilogue = [&](int tile, uint32_t index) {
            const int row = (tile % a.m_tiles) * BM + e_half * 128 + r;
            const int tok0 = (tile / a.m_tiles) * BN + e_cols;
            if (!mbar_wait_warp(&bars->d_full, index & 1, &bars->abort_flag, a.err)) return;
            tc_fence_after();
            const float rb = (a.bias != nullptr && row < a.O) ? load_scalar(a.bias, a.bias_dtype, row) : 0.0f;
#pragma unroll 1
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                __syncwarp();                                   // rows past O skip the stores below
                tc_ld32(tmem + (static_cast<uint32_t>(quad * 32) << 16) + D_COL0 + e_half * BN + e_cols + c * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c == 1) {
                    // last read of the accumulators by this warp: the MMA warp may start the next tile
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->d_empty[e_half]);
                }
                if (row < a.O) {
                    const int tok = tok0 + c * 32;
                    const int nt = min(32, a.T - tok);
                    if (a.y_dtype == DT_BF16) {
                        __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(a.y) + static_cast<size_t>(tok) * a.y_stride + row;
#pragma unroll
                        for (int j = 0; j < 32; j++, yp += a.y_stride) if (j < nt) *yp = __float2bfloat16_rn(__uint_as_float(v[j]) + rb);
                    } else if (a.y_dtype == DT_F16) {
                        __half* yp = reinterpret_cast<__half*>(a.y) + static_cast<size_t>(tok) * a.y_stride + row;
#pragma unroll
                        for (int j = 0; j < 32; j++, yp += a.y_stride) if (j < nt) *yp = __float2half_rn(__uint_as_float(v[j]) + rb);
                    } else {
                        float* yp = reinterpret_cast<float*>(a.y) + static_cast<size_t>(tok) * a.y_stride + row;
#pragma unroll
                        for (int j = 0; j < 32; j++, yp += a.y_stride) if (j < nt) *yp = __uint_as_float(v[j]) + rb;
                    }
                }
            }
        };
        int pending_tile = -1;
        // A stage's tensor-memory store is published to the MMA issuers: wait for the store, fence, one arrival per warp.
        int stored_sa = -1;
        auto publish = [&]() {
            if (stored_sa < 0) return;
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->full_a[stored_sa]);
            stored_sa = -1;
        };
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, tile_i++) {
            const int m_tile = tile % a.m_tiles;
            const int row0 = m_tile * BM + half * 128;
            const int row = min(row0 + r, a.O - 1);            // rows past the end read a valid row; never stored
            const size_t srow = static_cast<size_t>(row) * gpr;
            // Scales and biases come from the table stage_scales_kernel wrote for this call: one 16-byte entry per
            // (weight slab, K half, row) holding, for the slab's four stages, fp16(scale * 2^20) and fp16(bias).  A
            // warp's 32 rows are 512 contiguous bytes, and the entry is fetched a whole slab ahead (volatile asm,
            // so that the load is issued here and not re-materialised next to its use): the original tensors
            // would cost every warp 32 separate sectors per load, and a conversion per stage.
            const uint4* ptab = a.pairs + static_cast<size_t>(khalf) * a.o_pad + (m_tile * BM + half * 128 + r);
            uint32_t p_nxt[4], p_cur[4] = {0u, 0u, 0u, 0u};
            auto fetch_slab = [&](int slab) {
                const uint4* e = ptab + static_cast<size_t>(slab) * 2 * a.o_pad;
                asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(p_nxt[0]), "=r"(p_nxt[1]), "=r"(p_nxt[2]), "=r"(p_nxt[3]) : "l"(e));
            };
            fetch_slab(0);
            for (int ks = 0; ks < k_stages; ks++, it++) {
                if (ks == S_A && pending_tile >= 0) {
                    // The A ring now holds this tile's first stages; the MMAs wait for the previous tile's
                    // accumulators to be read, which is what this does.
                    publish();
                    epilogue(pending_tile, tile_i - 1);
                    pending_tile = -1;
                }
                const int sa = it % S_A;
                const int sub = ks % W_SPAN;                    // stage inside the weight slab
                if (sub == 0) {
                    wi++;                                       // same count as the producer: a new slab per W_SPAN stages of a tile
#pragma unroll
                    for (int j = 0; j < 4; j++) p_cur[j] = p_nxt[j];
                    if (ks + W_SPAN < k_stages) fetch_slab(ks / W_SPAN + 1);
                }
                const int sw = (wi - 1) % S_W;
                // this stage's entry: low half fp16(scale * 2^20), or the marker when the scale is too large for
                // that; high half fp16(bias)
                uint32_t entry = p_cur[0];
#pragma unroll
                for (int j = 1; j < 4; j++) if (sub == j) entry = p_cur[j];
                const bool small = (entry & 0xFFFFu) != SCALE_MARKER;
                const uint32_t bi_bits = __byte_perm(entry, entry, 0x3232);
                const __half2 bi = *reinterpret_cast<const __half2*>(&bi_bits);
                uint32_t sc_bits = __byte_perm(entry, entry, 0x1010);
                if (!small) {
                    // rare: the scale itself (times one), from the layer's tensor
                    const int grp = min((ks * BK + khalf * 32) >> a.gs_shift, gpr - 1);
                    const __half2 s2 = __float2half2_rn(load_scalar(a.s, a.s_dtype, srow + grp));
                    sc_bits = *reinterpret_cast<const uint32_t*>(&s2);
                }
                const __half2 sc = *reinterpret_cast<const __half2*>(&sc_bits);
                if (sub == 0 && !mbar_wait_warp(&bars->full_w[sw], ((wi - 1) / S_W) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                // row of 128 bytes, 16-byte chunk (sub*2 + khalf), stored with the 128-byte swizzle (chunk ^ row%8)
                // (fetching the next stage's chunk a stage early was tried: slower, 660 vs 690 TFLOP/s)
                const int wr = half * 128 + r;
                const uint4 pk = *reinterpret_cast<const uint4*>(w_slabs + sw * W_SLAB + wr * 128 + (((sub * 2 + khalf) ^ (wr & 7)) << 4));
                if (sub == W_SPAN - 1 || ks == k_stages - 1) {
                    // last read of the slab by this warp
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->empty_w[sw]);
                }
                const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
                uint32_t v[16];
                // One decision per warp and stage, outside the unrolled loops: left per lane inside them, the
                // compiler evaluated both dequant forms for every value (3x the half-precision FMAs).
                if (__all_sync(0xffffffffu, small)) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        // nibbles (0,4), (1,5), (2,6), (3,7) of the word, each pair brought to bits 4..7 of its half:
                        // the masked nibble is the fp16 subnormal q * 2^-20 and the scale carries the 2^20
                        const uint32_t n[4] = {(words[i] << 4) & 0x00F000F0u, words[i] & 0x00F000F0u,
                                               (words[i] >> 4) & 0x00F000F0u, (words[i] >> 8) & 0x00F000F0u};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const __half2 wv = __hfma2(*reinterpret_cast<const __half2*>(&n[j]), sc, bi);
                            v[i * 4 + j] = *reinterpret_cast<const uint32_t*>(&wv);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t n[4] = {(words[i] << 4) & 0x00F000F0u, words[i] & 0x00F000F0u,
                                               (words[i] >> 4) & 0x00F000F0u, (words[i] >> 8) & 0x00F000F0u};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            __half2 wv;
                            if (small) {
                                wv = __hfma2(*reinterpret_cast<const __half2*>(&n[j]), sc, bi);
                            } else {
                                // large scale: (1024 + 16 q) / 16 - 64 = q exactly, then q * scale + bias
                                const uint32_t h = n[j] | 0x64006400u;
                                wv = __hfma2(__hfma2(*reinterpret_cast<const __half2*>(&h), kMul, kSub), sc, bi);
                            }
                            v[i * 4 + j] = *reinterpret_cast<const uint32_t*>(&wv);
                        }
                    }
                }
                if (it >= S_A && !mbar_wait_warp(&bars->empty_a[sa], ((it / S_A) - 1) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                __syncwarp();                                   // the per-lane dequant branches end here
                tc_fence_after();
                tc_st16(tmem + (static_cast<uint32_t>(quad * 32) << 16) + a_col(sa, half, khalf), v);
                stored_sa = sa;
                publish();                                      // (publishing a stage late was tried: 1 % slower)
            }
            publish();                                          // the tile's last stage
            if (ok) pending_tile = tile;
        }
        if (pending_tile >= 0) epilogue(pending_tile, tile_i - 1);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        __syncwarp();                                           // lane 0 issued the MMAs alone
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}


// ---- the wide tile: 128 weight rows x 256 tokens -----------------------------------------------------------------
// Same pipeline, other tile.  Every dequantised weight now meets 256 tokens instead of 128, so the dequantisers
// (the limiter of the 256 x 128 tile) do half the work per flop: a K stage is 128 rows x 64 codes, stored by
// eight warps, and the sixteen dequantising warps take alternate stages.  Only one A block per stage lives in
// tensor memory, so the A ring holds eight stages where the tall tile has four.  The accumulator is one
// 128 x 256 fp32 block; two threads issue the MMAs, one per 128-token half (N = 128 each, separate columns,
// separate halves of the activation tile).  Costs: 36 KB of operands per stage instead of 24 KB (L2 traffic),
// and batches are padded to 256 tokens, so the tall tile stays in use for short batches.
namespace wide {

constexpr int BM = 128, BN = 256;
constexpr int S_X = 4;                  // activation stages of 32 KB
constexpr int S_W = 3;                  // weight slabs of 16 KB (128 rows x 128 bytes = W_SPAN stages)
constexpr int S_A = 8;                  // TMEM stages of the A operand, 32 columns each
constexpr int X_STAGE = BN * BK * 2;    // 32768
constexpr int W_SLAB = BM * 128;        // 16384
constexpr int D_COL0 = 0, A_COL0 = 256;
constexpr int STAGE_WARPS = DEQ_WARPS / 2;   // warps that store one stage

__host__ __device__ constexpr uint32_t a_col(int sa, int khalf) { return A_COL0 + static_cast<uint32_t>(sa * 32 + khalf * 16); }

struct Barriers {
    uint64_t full_x[S_X];
    uint64_t empty_x[S_X];
    uint64_t full_w[S_W];
    uint64_t empty_w[S_W];
    uint64_t full_a[S_A];
    uint64_t empty_a[S_A];
    uint64_t d_full;
    uint64_t d_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int SMEM_BYTES = S_X * X_STAGE + S_W * W_SLAB + sizeof(Barriers) + 1024;

__global__ void __launch_bounds__(NUM_THREADS, 1)
qgemm4w_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* x_tiles = smem;
    uint8_t* w_slabs = smem + S_X * X_STAGE;
    Barriers* bars = reinterpret_cast<Barriers*>(smem + S_X * X_STAGE + S_W * W_SLAB);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_stages = a.K / BK;
    const int total_tiles = a.m_tiles * a.n_tiles;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S_X; i++) { mbar_init(&bars->full_x[i], 1); mbar_init(&bars->empty_x[i], 2); }
        for (int i = 0; i < S_W; i++) { mbar_init(&bars->full_w[i], 1); mbar_init(&bars->empty_w[i], DEQ_WARPS); }
        for (int i = 0; i < S_A; i++) { mbar_init(&bars->full_a[i], STAGE_WARPS); mbar_init(&bars->empty_a[i], 2); }
        mbar_init(&bars->d_full, 2);
        mbar_init(&bars->d_empty[0], DEQ_WARPS / 2);
        mbar_init(&bars->d_empty[1], DEQ_WARPS / 2);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
    // Launched as a programmatic dependent of the pre-pass: the set-up above and the weight producer's first slabs
    // (the layer's constants) run while it finishes; every other role first waits for it (staged activations, the
    // scale/bias table, and -- through the pre-pass's own ordering -- everything earlier in the stream).
    if (warp != W_PRODUCER) asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        // ---- TMA producer of the activations: one 256-token x 64 box per stage --------------------------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int tok0 = (tile / a.m_tiles) * BN;
                for (int ks = 0; ks < k_stages; ks++, it++) {
                    const int s = it % S_X;
                    if (it >= S_X && !mbar_wait(&bars->empty_x[s], ((it / S_X) - 1) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    mbar_expect_tx(&bars->full_x[s], X_STAGE);
                    tma_load_2d(x_tiles + s * X_STAGE, &map_x, &bars->full_x[s], ks * BK, tok0);
                }
            }
            for (uint32_t j = it > S_X ? it - S_X : 0; j < it; j++) {
                const uint64_t t0 = global_ns();
                while (!mbar_try_wait(&bars->full_x[j % S_X], (j / S_X) & 1))
                    if (global_ns() - t0 > WAIT_NS) break;
            }
        }
    } else if (warp == W_PRODUCER) {
        // ---- TMA producer of packed weights: one slab (128 rows x 128 bytes = W_SPAN stages of K) per copy --------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
            uint32_t wi = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int row0 = (tile % a.m_tiles) * BM;
                for (int ks = 0; ks < k_stages; ks += W_SPAN, wi++) {
                    const int sw = wi % S_W;
                    if (wi >= S_W && !mbar_wait(&bars->empty_w[sw], ((wi / S_W) - 1) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    mbar_expect_tx(&bars->full_w[sw], W_SLAB);
                    tma_load_2d(w_slabs + sw * W_SLAB, &map_w, &bars->full_w[sw], ks * (BK / 2), row0);
                }
            }
            for (uint32_t j = wi > S_W ? wi - S_W : 0; j < wi; j++) {
                const uint64_t t0 = global_ns();
                while (!mbar_try_wait(&bars->full_w[j % S_W], (j / S_W) & 1))
                    if (global_ns() - t0 > WAIT_NS) break;
            }
        }
    } else if (warp == MMA_WARP || warp == MMA_WARP2) {
        // ---- MMA issuers: one per 128-token half of the tile ------------------------------------------------------------
        if (lane == 0) {
            const int nh = warp == MMA_WARP ? 0 : 1;
            const uint32_t d_addr = tmem + D_COL0 + nh * 128;
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, tile_i++) {
                if (tile_i > 0 && !mbar_wait(&bars->d_empty[nh], (tile_i - 1) & 1, &bars->abort_flag, a.err)) break;
                tc_fence_after();
                for (int ks = 0; ks < k_stages; ks++, it++) {
                    const int s = it % S_X, sa = it % S_A;
                    if (!mbar_wait(&bars->full_x[s], (it / S_X) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    if (!mbar_wait(&bars->full_a[sa], (it / S_A) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    tc_fence_after();
                    // this half's 128 tokens are the second 16 KB of the stage (rows of 128 bytes, same swizzle phase)
                    const uint64_t bdesc = smem_desc_sw128(smem_u32(x_tiles + s * X_STAGE + nh * (128 * 128)));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; kk++)
                        tc_mma_ts(d_addr, tmem + a_col(sa, kk >> 1) + (kk & 1) * 8, bdesc + static_cast<uint64_t>(kk * 2), a.idesc, (ks | kk) != 0);
                    tc_commit(&bars->empty_x[s]);
                    tc_commit(&bars->empty_a[sa]);
                }
                if (ok) tc_commit(&bars->d_full);
            }
        }
    } else if (warp >= DEQ_WARP0) {
        // ---- dequantisers: one thread per (weight row, half of the 64-wide K slice), alternate stages ---------------------
        const int dw = warp - DEQ_WARP0;
        const int quad = warp & 3;                              // TMEM lane quadrant this warp may touch
        const int khalf = (dw >> 2) & 1;                        // which 32 codes of the slice
        const int par = dw >> 3;                                // the stages (by parity of the tile's stage index) this warp stores
        const int r = quad * 32 + lane;                         // row within the tile
        const int gpr = a.K >> a.gs_shift;
        const __half2 kMul = __halves2half2(__float2half(0.0625f), __float2half(0.0625f));
        const __half2 kSub = __halves2half2(__float2half(-64.0f), __float2half(-64.0f));
        uint32_t it = 0, wi = 0, tile_i = 0;
        bool ok = true;
        // Epilogue: this warp drains its lane quadrant for 64 of the 256 token columns.
        const int e_cols = (dw >> 2) * 64, e_nh = dw >> 3;
        auto epilogue = [&](int tile, uint32_t index) {
            const int row = (tile % a.m_tiles) * BM + r;
            const int tok0 = (tile / a.m_tiles) * BN + e_cols;
            if (!mbar_wait_warp(&bars->d_full, index & 1, &bars->abort_flag, a.err)) return;
            tc_fence_after();
            const float rb = (a.bias != nullptr && row < a.O) ? load_scalar(a.bias, a.bias_dtype, row) : 0.0f;
#pragma unroll 1
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                __syncwarp();
                tc_ld32(tmem + (static_cast<uint32_t>(quad * 32) << 16) + D_COL0 + e_cols + c * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c == 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->d_empty[e_nh]);
                }
                if (row < a.O) {
                    const int tok = tok0 + c * 32;
                    const int nt = min(32, a.T - tok);
                    if (a.y_dtype == DT_BF16) {
                        __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(a.y) + static_cast<size_t>(tok) * a.y_stride + row;
#pragma unroll
                        for (int j = 0; j < 32; j++, yp += a.y_stride) if (j < nt) *yp = __float2bfloat16_rn(__uint_as_float(v[j]) + rb);
                    } else if (a.y_dtype == DT_F16) {
                        __half* yp = reinterpret_cast<__half*>(a.y) + static_cast<size_t>(tok) * a.y_stride + row;
#pragma unroll
                        for (int j = 0; j < 32; j++, yp += a.y_stride) if (j < nt) *yp = __float2half_rn(__uint_as_float(v[j]) + rb);
                    } else {
                        float* yp = reinterpret_cast<float*>(a.y) + static_cast<size_t>(tok) * a.y_stride + row;
#pragma unroll
                        for (int j = 0; j < 32; j++, yp += a.y_stride) if (j < nt) *yp = __uint_as_float(v[j]) + rb;
                    }
                }
            }
        };
        int pending_tile = -1;
        // the accumulators of the previous tile are drained once this tile's A ring is full (short K: at once)
        const int epi_at = k_stages > S_A ? S_A : 0;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, tile_i++) {
            const int m_tile = tile % a.m_tiles;
            const int row = min(m_tile * BM + r, a.O - 1);
            const size_t srow = static_cast<size_t>(row) * gpr;
            const uint4* ptab = a.pairs + static_cast<size_t>(khalf) * a.o_pad + (m_tile * BM + r);
            uint32_t p_nxt[4], p_cur[4] = {0u, 0u, 0u, 0u};
            auto fetch_slab = [&](int slab) {
                const uint4* e = ptab + static_cast<size_t>(slab) * 2 * a.o_pad;
                asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(p_nxt[0]), "=r"(p_nxt[1]), "=r"(p_nxt[2]), "=r"(p_nxt[3]) : "l"(e));
            };
            fetch_slab(0);
            for (int ks = 0; ks < k_stages; ks++, it++) {
                if (ks == epi_at && pending_tile >= 0) {
                    epilogue(pending_tile, tile_i - 1);
                    pending_tile = -1;
                }
                const int sa = it % S_A;
                const int sub = ks % W_SPAN;
                const bool last_of_slab = sub == W_SPAN - 1 || ks == k_stages - 1;
                if (sub == 0) {
                    wi++;
#pragma unroll
                    for (int j = 0; j < 4; j++) p_cur[j] = p_nxt[j];
                    if (ks + W_SPAN < k_stages) fetch_slab(ks / W_SPAN + 1);
                    if (!mbar_wait_warp(&bars->full_w[(wi - 1) % S_W], ((wi - 1) / S_W) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                }
                const int sw = (wi - 1) % S_W;
                if ((ks & 1) == par) {
                    uint32_t entry = p_cur[0];
#pragma unroll
                    for (int j = 1; j < 4; j++) if (sub == j) entry = p_cur[j];
                    const bool small = (entry & 0xFFFFu) != SCALE_MARKER;
                    const uint32_t bi_bits = __byte_perm(entry, entry, 0x3232);
                    const __half2 bi = *reinterpret_cast<const __half2*>(&bi_bits);
                    uint32_t sc_bits = __byte_perm(entry, entry, 0x1010);
                    if (!small) {
                        const int grp = min((ks * BK + khalf * 32) >> a.gs_shift, gpr - 1);
                        const __half2 s2 = __float2half2_rn(load_scalar(a.s, a.s_dtype, srow + grp));
                        sc_bits = *reinterpret_cast<const uint32_t*>(&s2);
                    }
                    const __half2 sc = *reinterpret_cast<const __half2*>(&sc_bits);
                    const uint4 pk = *reinterpret_cast<const uint4*>(w_slabs + sw * W_SLAB + r * 128 + (((sub * 2 + khalf) ^ (r & 7)) << 4));
                    const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
                    uint32_t v[16];
                    if (__all_sync(0xffffffffu, small)) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint32_t n[4] = {(words[i] << 4) & 0x00F000F0u, words[i] & 0x00F000F0u,
                                                   (words[i] >> 4) & 0x00F000F0u, (words[i] >> 8) & 0x00F000F0u};
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const __half2 wv = __hfma2(*reinterpret_cast<const __half2*>(&n[j]), sc, bi);
                                v[i * 4 + j] = *reinterpret_cast<const uint32_t*>(&wv);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint32_t n[4] = {(words[i] << 4) & 0x00F000F0u, words[i] & 0x00F000F0u,
                                                   (words[i] >> 4) & 0x00F000F0u, (words[i] >> 8) & 0x00F000F0u};
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                __half2 wv;
                                if (small) {
                                    wv = __hfma2(*reinterpret_cast<const __half2*>(&n[j]), sc, bi);
                                } else {
                                    const uint32_t h = n[j] | 0x64006400u;
                                    wv = __hfma2(__hfma2(*reinterpret_cast<const __half2*>(&h), kMul, kSub), sc, bi);
                                }
                                v[i * 4 + j] = *reinterpret_cast<const uint32_t*>(&wv);
                            }
                        }
                    }
                    if (it >= S_A && !mbar_wait_warp(&bars->empty_a[sa], ((it / S_A) - 1) & 1, &bars->abort_flag, a.err)) { ok = false; break; }
                    __syncwarp();
                    tc_fence_after();
                    tc_st16(tmem + (static_cast<uint32_t>(quad * 32) << 16) + a_col(sa, khalf), v);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->full_a[sa]);
                }
                if (last_of_slab) {
                    // every chunk of the slab that this warp needs has been read
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->empty_w[sw]);
                }
            }
            if (ok) pending_tile = tile;
        }
        if (pending_tile >= 0) epilogue(pending_tile, tile_i - 1);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace wide

// Activations -> fp16 in the staged order (0,4,1,5,2,6,3,7 inside every eight), eight elements per thread.
// bf16 values beyond the fp16 range are clamped to +-65504.
__device__ __forceinline__ void stage_x_part(const uint16_t* __restrict__ x, int is_bf16, long long x_stride, __half* __restrict__ out, long long T, int K,
                                             unsigned block, unsigned blocks) {
    const long long chunks = static_cast<long long>(K) / 8;
    const long long n = T * chunks;
    for (long long i = block * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(blocks) * blockDim.x) {
        const long long t = i / chunks, c = i - t * chunks;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + t * x_stride + c * 8));
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
        if (is_bf16) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float lo = fminf(fmaxf(__uint_as_float(w[j] << 16), -65504.0f), 65504.0f);
                const float hi = fminf(fmaxf(__uint_as_float(w[j] & 0xFFFF0000u), -65504.0f), 65504.0f);
                const __half2 h = __floats2half2_rn(lo, hi);
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        // w = (x0,x1) (x2,x3) (x4,x5) (x6,x7)  ->  (x0,x4) (x1,x5) (x2,x6) (x3,x7)
        const uint4 o = make_uint4(__byte_perm(w[0], w[2], 0x5410), __byte_perm(w[0], w[2], 0x7632),
                                   __byte_perm(w[1], w[3], 0x5410), __byte_perm(w[1], w[3], 0x7632));
        *reinterpret_cast<uint4*>(out + t * K + c * 8) = o;
    }
}

// Scales and biases -> the table the dequantising warps read: entry [(slab * 2 + khalf) * o_pad + row] holds, for the
// four K stages of weight slab `slab`, (fp16(scale * 2^20) | fp16(bias) << 16) of the group that the 32 codes
// (stage, khalf) of `row` belong to.  Scales of magnitude 0.0624 and above get SCALE_MARKER instead (the kernel
// then takes the scale from the layer's tensor).  Rows past O and stages past K hold zeros.
__device__ __forceinline__ void stage_scales_part(const void* __restrict__ s, const void* __restrict__ b, int s_dtype, int O, int o_pad, int gpr,
                                                  int gs_shift, int k_stages, int n_slabs, uint4* __restrict__ out, unsigned block, unsigned blocks) {
    const long long n = static_cast<long long>(n_slabs) * o_pad;
    for (long long i = block * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(blocks) * blockDim.x) {
        const int row = static_cast<int>(i % o_pad);
        const int slab = static_cast<int>(i / o_pad);
        uint32_t e[2][4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int ks = slab * W_SPAN + j;
            uint32_t prev = 0u;
            int prev_grp = -1;
#pragma unroll
            for (int khalf = 0; khalf < 2; khalf++) {
                uint32_t v = 0u;
                if (row < O && ks < k_stages) {
                    const int grp = min((ks * BK + khalf * 32) >> gs_shift, gpr - 1);
                    if (grp == prev_grp) {
                        v = prev;                   // groups of 64 and more: both K halves of a stage share one
                    } else {
                        const float sf = load_scalar(s, s_dtype, static_cast<size_t>(row) * gpr + grp);
                        const float bf = load_scalar(b, s_dtype, static_cast<size_t>(row) * gpr + grp);
                        const __half hs = __float2half_rn(sf * 1048576.0f), hb = __float2half_rn(bf);
                        const uint32_t lo = fabsf(sf) < 0.0624f ? static_cast<uint32_t>(__half_as_ushort(hs)) : SCALE_MARKER;
                        v = lo | (static_cast<uint32_t>(__half_as_ushort(hb)) << 16);
                    }
                    prev = v;
                    prev_grp = grp;
                }
                e[khalf][j] = v;
            }
        }
        out[static_cast<size_t>(slab) * 2 * o_pad + row] = make_uint4(e[0][0], e[0][1], e[0][2], e[0][3]);
        out[(static_cast<size_t>(slab) * 2 + 1) * o_pad + row] = make_uint4(e[1][0], e[1][1], e[1][2], e[1][3]);
    }
}

// Both pre-passes in one launch: the first `x_blocks` blocks rewrite the activations, the rest build the table.
struct StageArgs {
    const uint16_t* x; int is_bf16; long long x_stride; __half* xs; long long T; int K;
    const void* s; const void* b; int s_dtype; int O; int o_pad; int gpr; int gs_shift; int k_stages; int n_slabs; uint4* pairs;
    unsigned x_blocks;
};
__global__ void stage_inputs_kernel(const StageArgs g) {
    // the GEMM that follows is launched as a programmatic dependent: it may set up (barriers, tensor memory, first
    // weight slabs) while this grid runs, and waits for this grid before it touches what is written here
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (blockIdx.x < g.x_blocks) stage_x_part(g.x, g.is_bf16, g.x_stride, g.xs, g.T, g.K, blockIdx.x, g.x_blocks);
    else stage_scales_part(g.s, g.b, g.s_dtype, g.O, g.o_pad, g.gpr, g.gs_shift, g.k_stages, g.n_slabs, g.pairs,
                           blockIdx.x - g.x_blocks, gridDim.x - g.x_blocks);
}

// ---- host side --------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

bool make_map_2d(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer, uint64_t row_bytes,
                 uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    return fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count(int device) {
    static int cached[64] = {};
    if (device < 0 || device >= 64) return 148;
    if (!cached[device]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cached[device] = n;
    }
    return cached[device];
}

// One stream-ordered memory pool per device for the scratch copy of bf16 activations; freed blocks stay
// in the pool (release threshold = unlimited) so steady-state calls do not reach the driver's allocator.
cudaMemPool_t scratch_pool(int device) {
    static cudaMemPool_t pools[64] = {};
    static std::mutex mu;
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!pools[device]) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = device;
        cudaMemPool_t p = nullptr;
        if (cudaMemPoolCreate(&p, &props) != cudaSuccess) return nullptr;
        uint64_t keep = ~0ull;
        cudaMemPoolSetAttribute(p, cudaMemPoolAttrReleaseThreshold, &keep);
        pools[device] = p;
    }
    return pools[device];
}

}  // namespace

// Batches of more than 128 tokens take the wide tile (128 rows x 256 tokens), shorter ones the tall one (256 x 128).
static bool use_wide(long long T) { return T > 128; }

int qgemm_tile_tokens(const GemmLayer& L, int x_dtype, long long x_stride, const void* x, long long T) {
    if (L.bits != 4 || L.K % BK != 0 || L.K < 2 * S_A * BK || L.gs < 32 || (L.gs & (L.gs - 1)) != 0 || L.O < 1 || T < 1) return 0;
    if (x_dtype != DT_F16 && x_dtype != DT_BF16) return 0;
    if ((reinterpret_cast<uintptr_t>(L.w) & 15u) != 0) return 0;
    if (x != nullptr && ((reinterpret_cast<uintptr_t>(x) & 15u) != 0 || (x_stride * 2) % 16 != 0)) return 0;
    if (T > 0x7FFFFFFFLL) return 0;
    return use_wide(T) ? wide::BN : BN;
}

namespace {

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// Bytes of per-call scratch: the fp16 copy of the activations and the staged scale/bias table.
size_t x_bytes(const GemmLayer& L, long long T) { return align256(static_cast<size_t>(T) * L.K * 2); }
size_t table_bytes(const GemmLayer& L) {
    const size_t n_slabs = (static_cast<size_t>(L.K) / BK + W_SPAN - 1) / W_SPAN;
    const size_t o_pad = (static_cast<size_t>(L.O) + BM - 1) / BM * BM;
    return n_slabs * 2 * o_pad * sizeof(uint4);
}

// Opts the kernel into its shared-memory size, once per device (function attributes belong to a device's context;
// the caller has made `device` current).
cudaError_t gemm_attr(int device) {
    static std::mutex mu;
    static bool done[64] = {};
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lk(mu);
    if (!done[device]) {
        cudaError_t e = cudaFuncSetAttribute(qgemm4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(wide::qgemm4w_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wide::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        done[device] = true;
    }
    return cudaSuccess;
}

// The two pre-passes (activations -> fp16 in the staged order, scales/biases -> the dequantisers' table) and the
// GEMM, all on `st`; `xs` (x_bytes(L, T)) and `pairs` (table_bytes(L)) are their workspace, 256-byte aligned.
cudaError_t enqueue_gemm(const GemmLayer& L, const GemmCall& c, cudaStream_t st, __half* xs, uint4* pairs, const char** why) {
    GemmArgs a;
    a.s = L.s; a.b = L.b; a.bias = L.bias; a.y = c.y; a.err = c.err; a.y_stride = c.y_stride;
    a.s_dtype = L.s_dtype; a.bias_dtype = L.bias_dtype; a.y_dtype = c.y_dtype;
    a.O = L.O; a.K = L.K; a.gs = L.gs; a.T = static_cast<int>(c.T);
    a.gs_shift = 0;
    while ((1 << a.gs_shift) < L.gs) a.gs_shift++;
    const bool wide_tile = use_wide(c.T);
    const int bm = wide_tile ? wide::BM : BM, bn = wide_tile ? wide::BN : BN;
    a.m_tiles = (L.O + bm - 1) / bm;
    a.n_tiles = static_cast<int>((c.T + bn - 1) / bn);
    const bool have_table = c.table != nullptr;
    a.pairs = have_table ? static_cast<const uint4*>(c.table) : pairs;
    a.o_pad = (L.O + BM - 1) / BM * BM;          // the table is padded to the tall tile's 256 rows for both
    const int k_stages = L.K / BK, n_slabs = (k_stages + W_SPAN - 1) / W_SPAN;
    {
        const long long n = c.T * (L.K / 8);
        const long long ns = static_cast<long long>(n_slabs) * a.o_pad;
        StageArgs g;
        g.x = static_cast<const uint16_t*>(c.x); g.is_bf16 = c.x_dtype == DT_BF16 ? 1 : 0; g.x_stride = c.x_stride; g.xs = xs; g.T = c.T; g.K = L.K;
        g.s = L.s; g.b = L.b; g.s_dtype = L.s_dtype; g.O = L.O; g.o_pad = a.o_pad; g.gpr = L.K / L.gs; g.gs_shift = a.gs_shift;
        g.k_stages = k_stages; g.n_slabs = n_slabs; g.pairs = pairs;
        g.x_blocks = static_cast<unsigned>(n / 256 + 1 < 148LL * 6 ? n / 256 + 1 : 148LL * 6);
        // (the table part is left out when the layer's table was built ahead)
        const unsigned s_blocks = have_table ? 0u : static_cast<unsigned>(ns / 256 + 1 < 148LL * 4 ? ns / 256 + 1 : 148LL * 4);
        stage_inputs_kernel<<<g.x_blocks + s_blocks, 256, 0, st>>>(g);
    }
    CUtensorMap map_w, map_x;
    if (!make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, L.w, static_cast<uint64_t>(L.K) / 2, static_cast<uint64_t>(L.O),
                     static_cast<uint64_t>(L.K) / 2, 128, bm, CU_TENSOR_MAP_SWIZZLE_128B)) {
        *why = "tensor map of the packed weights";
        return cudaErrorInvalidValue;
    }
    if (!make_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT16, xs, static_cast<uint64_t>(L.K), static_cast<uint64_t>(c.T),
                     static_cast<uint64_t>(L.K) * 2, BK, bn, CU_TENSOR_MAP_SWIZZLE_128B)) {
        *why = "tensor map of the activations";
        return cudaErrorInvalidValue;
    }
    // instruction descriptor: fp32 accumulate (bit 4), A and B fp16 (format 0 at bits 7 and 10), both K-major,
    // N >> 3 at bit 17, M >> 4 at bit 24
    a.idesc = (1u << 4) | (0u << 7) | (0u << 10) | (static_cast<uint32_t>(128 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
    const long long tiles = static_cast<long long>(a.m_tiles) * a.n_tiles;
    const int sms = sm_count(L.device);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(tiles < sms ? tiles : sms));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = wide_tile ? wide::SMEM_BYTES : SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute la[1];
    la[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;       // a dependent of the pre-pass, see the kernels
    la[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = la;
    cfg.numAttrs = 1;
    if (wide_tile) return cudaLaunchKernelEx(&cfg, wide::qgemm4w_kernel, map_w, map_x, a);
    return cudaLaunchKernelEx(&cfg, qgemm4_kernel, map_w, map_x, a);
}

}  // namespace

cudaError_t qgemm_build_table(const GemmLayer& L, void* table, cudaStream_t st) {
    int gs_shift = 0;
    while ((1 << gs_shift) < L.gs) gs_shift++;
    const int k_stages = L.K / BK, n_slabs = (k_stages + W_SPAN - 1) / W_SPAN;
    StageArgs g = {};
    g.s = L.s; g.b = L.b; g.s_dtype = L.s_dtype; g.O = L.O; g.o_pad = (L.O + BM - 1) / BM * BM; g.gpr = L.K / L.gs; g.gs_shift = gs_shift;
    g.k_stages = k_stages; g.n_slabs = n_slabs; g.pairs = static_cast<uint4*>(table);
    g.x_blocks = 0;
    const long long ns = static_cast<long long>(n_slabs) * g.o_pad;
    stage_inputs_kernel<<<static_cast<unsigned>(ns / 256 + 1 < 148LL * 4 ? ns / 256 + 1 : 148LL * 4), 256, 0, st>>>(g);
    return cudaGetLastError();
}

cudaError_t launch_qgemm(const GemmLayer& L, const GemmCall& c, cudaStream_t st, const char** why) {
    *why = "";
    if (const cudaError_t ae = gemm_attr(L.device)) { *why = "shared-memory opt-in"; return ae; }
    // Workspace from the library's stream-ordered pool: allocated and released in stream order around the call.
    cudaMemPool_t pool = scratch_pool(L.device);
    if (!pool) { *why = "scratch pool"; return cudaErrorMemoryAllocation; }
    uint8_t* scratch = nullptr;
    cudaError_t e = cudaMallocFromPoolAsync(reinterpret_cast<void**>(&scratch), x_bytes(L, c.T) + (c.table ? 0 : table_bytes(L)), pool, st);
    if (e != cudaSuccess) { *why = "scratch allocation"; return e; }
    const cudaError_t launched = enqueue_gemm(L, c, st, reinterpret_cast<__half*>(scratch),
                                              reinterpret_cast<uint4*>(scratch + x_bytes(L, c.T)), why);
    cudaFreeAsync(scratch, st);                   // stream-ordered: released after the GEMM has read it
    return launched;
}

// ---- the GEMM without any allocation -------------------------------------------------------------------------
// Some hosts must not allocate device memory while they run: a serving loop that has handed every free byte
// to its KV cache, a host whose allocator is locked during its hot loop, a caller inside a region where
// cudaMalloc would synchronise the device.  For them the call's workspace -- the staged fp16 copy of the
// activations (up to 32 MiB) and the staged scale/bias table of the layer (up to 16 MiB) -- lives in this fixed
// array instead of pool memory.  The array is part of the library image: every GPU that loads the library holds
// its 48 MiB until the process exits.  Its contents are whatever the last call left; nothing in it needs to start
// at zero (each call rewrites the regions it later reads).  All calls on a device share it, so two calls that
// overlap on the GPU (different streams) race.
constexpr size_t STATIC_X_BYTES = 32u << 20;
constexpr size_t STATIC_TABLE_BYTES = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_X_BYTES + STATIC_TABLE_BYTES];

size_t qgemm_static_capacity() { return STATIC_X_BYTES; }
size_t qgemm_static_table_capacity() { return STATIC_TABLE_BYTES; }
size_t qgemm_table_bytes(const GemmLayer& L) { return table_bytes(L); }

cudaError_t launch_qgemm_static(const GemmLayer& L, const GemmCall& c, cudaStream_t st, const char** why) {
    *why = "";
    if (static_cast<unsigned long long>(c.T) * static_cast<unsigned long long>(L.K) * 2ull > STATIC_X_BYTES) {
        *why = "batch exceeds the static scratch";
        return cudaErrorInvalidValue;
    }
    if (!c.table && table_bytes(L) > STATIC_TABLE_BYTES) {
        *why = "the layer's scale table exceeds the static scratch";
        return cudaErrorInvalidValue;
    }
    // In host code the array's name is only a handle: the device address comes from cudaGetSymbolAddress, asked
    // once per device with that device current (the caller has selected L.device).  This first call per device
    // also opts the kernel into its shared-memory size; make it before any stream capture.
    static std::mutex mu;
    static unsigned char* base[64] = {};
    if (L.device < 0 || L.device >= 64) { *why = "device ordinal"; return cudaErrorInvalidDevice; }
    unsigned char* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!base[L.device]) {
            void* p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess) { *why = "address of the static scratch"; return e; }
            base[L.device] = static_cast<unsigned char*>(p);
        }
        scratch = base[L.device];
    }
    if (const cudaError_t ae = gemm_attr(L.device)) { *why = "shared-memory opt-in"; return ae; }
    return enqueue_gemm(L, c, st, reinterpret_cast<__half*>(scratch), reinterpret_cast<uint4*>(scratch + STATIC_X_BYTES), why);
}

}  // namespace mlxq
