/*
 * mlxq.h -- C ABI of libmlxq, a B200 (sm_100a) implementation of the MLX affine quantized-linear layer.
 *
 * The library replaces one class of the reference project (BackendStack21/mlx-runner): `Linear`
 * (Sources/MLXEngine/Transformer.swift:15-345) and the Metal kernels it dispatches
 * (Sources/MLXEngine/Kernels.swift:26-1023, 2752-2857).  Every entry point below names the reference
 * interface it stands in for.  All pointers to tensors are CUDA device pointers owned by the caller;
 * the library borrows them (as the reference borrows `Tensor` views, GPU.swift:145-154) and they must
 * outlive the handle.  Calls that take a stream only enqueue work and return; nothing throws or aborts
 * across this boundary: every call returns an `mlxq_status` and the text of the most recent failure on
 * the calling thread is available from mlxq_last_error().
 *
 * Format (normative): weight u32 [out_dim, in_dim*bits/32]; row r is one little-endian bit stream of
 * in_dim*bits/8 bytes; code k of the row is bits [k*bits, (k+1)*bits) of that stream.  scales and biases
 * [out_dim, in_dim/group_size] in f32, f16 or bf16 (same type).  w[r,k] = scale*q + bias, y = x . w^T.
 */
#ifndef MLXQ_H
#define MLXQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MLXQ_API __attribute__((visibility("default")))
#else
#define MLXQ_API
#endif

/* Status codes.  INVALID_FILE / UNSUPPORTED / MISSING_TENSOR / OUT_OF_MEMORY / GPU_FAILURE mirror the
 * cases of `EngineError` a Linear can raise (GPU.swift:4-33). */
typedef enum mlxq_status {
    MLXQ_OK = 0,
    MLXQ_INVALID_FILE = 1,    /* EngineError.invalidFile: shapes that do not describe a layer */
    MLXQ_UNSUPPORTED = 2,     /* EngineError.unsupported: bits / group size / dtype outside the format */
    MLXQ_MISSING_TENSOR = 3,  /* EngineError.missingTensor: scales without biases */
    MLXQ_OUT_OF_MEMORY = 4,   /* EngineError.outOfMemory */
    MLXQ_GPU_FAILURE = 5,     /* EngineError.gpuFailure: a CUDA call or an earlier kernel failed */
    MLXQ_INVALID_ARGUMENT = 6,/* a call the reference leaves undefined (null pointer, misaligned x, T < 1) */
    MLXQ_NCCL_FAILURE = 7,    /* the all-gather of output slices failed */
    MLXQ_TIMEOUT = 8          /* a bounded device-side wait ran out */
} mlxq_status;

/* Element types of scales/biases/bias, activations and outputs (DType, GPU.swift:121-142). */
typedef enum mlxq_dtype { MLXQ_F32 = 0, MLXQ_F16 = 1, MLXQ_BF16 = 2 } mlxq_dtype;

/* Gate activations of the gated epilogue (act_mul, Kernels.swift:124-130). */
typedef enum mlxq_act { MLXQ_ACT_SILU = 0, MLXQ_ACT_GELU_TANH = 1, MLXQ_ACT_GELU_ERF = 2 } mlxq_act;

typedef struct mlxq_linear* mlxq_linear_t;
typedef struct mlxq_comm* mlxq_comm_t;
typedef void* mlxq_stream_t; /* a cudaStream_t; NULL is the legacy default stream */

/* What `Linear.init(weight:scales:biases:bias:inDim:outDim:name:)` receives (Transformer.swift:48).
 * bits and group size are derived from the shapes exactly as Transformer.swift:68-70 does:
 * bits = weight_cols*32/in_dim, group_size = in_dim/scales_cols. */
typedef struct mlxq_linear_desc {
    const void* weight;      /* u32 [weight_rows, weight_cols]; dense layers: see `reserved` */
    const void* scales;      /* [scales_rows, scales_cols], may be NULL only together with biases == NULL (error) */
    const void* biases;      /* [biases_rows, biases_cols] */
    const void* bias;        /* optional per-output-row bias [bias_len]; NULL if absent */
    int64_t weight_rows, weight_cols;
    int64_t scales_rows, scales_cols;
    int64_t biases_rows, biases_cols;
    int64_t bias_len;        /* ignored when bias == NULL */
    int64_t in_dim;
    int64_t expect_out;      /* `outDim:` argument; 0 = do not check */
    int32_t scale_dtype;     /* mlxq_dtype of scales and biases */
    int32_t bias_dtype;      /* mlxq_dtype of bias */
    int32_t device;          /* CUDA device ordinal the pointers live on */
    int32_t reserved;        /* dense layers (scales == biases == NULL): 1 + mlxq_dtype of the weights, which are then
                              * [weight_rows, weight_cols = in_dim] elements of that type; 0 otherwise */
    const char* name;        /* used in error text only (the reference's `name prefix`); may be NULL */
} mlxq_linear_desc;

/* ---- library ----------------------------------------------------------------------------------------- */

/* Library version, major*10000 + minor*100 + patch.  No counterpart in the reference. */
MLXQ_API int mlxq_version(void);
/* Text of a status code (EngineError.errorDescription, GPU.swift:18-32). */
MLXQ_API const char* mlxq_status_string(int status);
/* Message of the most recent failing call on this thread ("" if none). */
MLXQ_API const char* mlxq_last_error(void);

/* ---- construction: Linear.init, Transformer.swift:48-111 ------------------------------------------- */

/* Validates the description (shape rules of Transformer.swift:52-60, format rules of :68-73) and returns
 * a handle.  Nothing is copied.  Errors: MLXQ_INVALID_FILE, MLXQ_UNSUPPORTED, MLXQ_MISSING_TENSOR.
 * A description without scales and biases is a dense layer (Transformer.swift:103-112: floating weights,
 * weight_cols == in_dim, in_dim a multiple of 4, the weights' type in `reserved`); mlxq_linear_forward serves it,
 * the other entry points return MLXQ_UNSUPPORTED for such a handle, and it cannot be sharded. */
MLXQ_API int mlxq_linear_create(const mlxq_linear_desc* desc, mlxq_linear_t* out);
/* The same layer restricted to output rows [rank*out_dim/nranks, (rank+1)*out_dim/nranks): the row
 * sharding of large projections across GPUs.  `desc` holds either the full tensors (desc_is_full != 0:
 * the library offsets the pointers, which must then be reachable from `desc->device`) or tensors the
 * caller already sliced.  out_dim must be divisible by 8*nranks.  No counterpart in the reference
 * (it is single-GPU); rows are independent there too (permuteRows, Transformer.swift:113-129). */
MLXQ_API int mlxq_linear_create_shard(const mlxq_linear_desc* desc, int rank, int nranks, int desc_is_full,
                                      mlxq_linear_t* out);
MLXQ_API void mlxq_linear_destroy(mlxq_linear_t h);
/* Load-time preparation (the place of `makePairs`, Transformer.swift:160-188, which repacks scales and biases once per
 * layer): builds the private table of scales and biases that the tensor-core GEMM reads (out_dim * in_dim / 8 bytes of
 * device memory owned by the handle) on `stream` and waits for it.  Optional: without it the first long batch builds
 * the table (and when that is not possible -- a stream being captured, no memory -- every such batch stages it in
 * scratch memory).  Results do not depend on it.  Layers the GEMM never takes are left untouched. */
MLXQ_API int mlxq_linear_prepare(mlxq_linear_t h, mlxq_stream_t stream);

/* Properties of `Linear` (Transformer.swift:16-23). */
MLXQ_API int64_t mlxq_linear_in_dim(mlxq_linear_t h);
MLXQ_API int64_t mlxq_linear_out_dim(mlxq_linear_t h);
MLXQ_API int mlxq_linear_bits(mlxq_linear_t h);
MLXQ_API int mlxq_linear_group_size(mlxq_linear_t h);
/* First global output row of a shard (0 for an unsharded layer). */
MLXQ_API int64_t mlxq_linear_row_offset(mlxq_linear_t h);
/* Rows of the whole layer: out_dim for an unsharded handle, the sum over the shards otherwise. */
MLXQ_API int64_t mlxq_linear_total_rows(mlxq_linear_t h);

/* ---- encode: Linear.encode, Transformer.swift:272-315 ---------------------------------------------- */

/* y[t, 0:out_dim] = x[t, 0:in_dim] . W^T (+ bias) for t in [0, T).  Strides are in elements.  Picks the
 * decode matvec for small T and the tensor-core GEMM for long batches, as the reference picks among
 * qmv/qmvt4/qmvx4/qgemms/qgemm by T.  x rows must start on 16-byte boundaries (the reference's kernels
 * load float4, Kernels.swift:93); a violation returns MLXQ_INVALID_ARGUMENT instead of faulting. */
MLXQ_API int mlxq_linear_forward(mlxq_linear_t h, mlxq_stream_t stream, const void* x, int x_dtype, int64_t x_stride,
                                 void* y, int y_dtype, int64_t y_stride, int64_t T);

/* mlxq_linear_forward for callers that cannot allocate device memory.  It has no counterpart in the reference.
 * The tensor-core GEMM of mlxq_linear_forward stages an fp16 copy of the activations (T * in_dim * 2 bytes)
 * and a table of the layer's scales and biases (out_dim * in_dim / 8 bytes) in pool memory it allocates on
 * the stream.  A host that has given all free device memory to its own caches, or that must not enter the
 * CUDA allocator while it runs (an allocator lock held by the host, a latency budget that cannot absorb the
 * allocator's device synchronisation), calls this entry point instead: both live in a fixed array inside the
 * library (32 MiB = MLXQ_STATIC_SCRATCH_BYTES for the activations, 16 MiB for the table), no cudaMalloc,
 * cudaFree or other allocating routine is called, and results are the same as mlxq_linear_forward's.
 *   - Batches with T * in_dim * 2 above 32 MiB, and layers with out_dim * in_dim / 8 above 16 MiB (rows
 *     rounded up to 256), are rejected with MLXQ_INVALID_ARGUMENT (split the batch; shard the layer).
 *   - Batches the GEMM does not take (T <= 16, fp32 activations, other bit widths) run on kernels that use no
 *     scratch memory, exactly as in mlxq_linear_forward.
 *   - Every call on a device shares the one array, which keeps whatever the last call wrote: calls that
 *     overlap on the GPU (different streams) race; order them on one stream or with events.
 *   - The first call on each device looks up the array's device address and sets the kernel's shared-memory
 *     attribute; make that first call before any stream capture begins. */
#define MLXQ_STATIC_SCRATCH_BYTES (32u << 20)
MLXQ_API int mlxq_linear_forward_static(mlxq_linear_t h, mlxq_stream_t stream, const void* x, int x_dtype,
                                        int64_t x_stride, void* y, int y_dtype, int64_t y_stride, int64_t T);

/* Linear.encodeFusedDecode, Transformer.swift:206-244: one launch computing the rows [A | B | C] of up
 * to three layers that satisfy mlxq_fusable(). */
MLXQ_API int mlxq_fused_forward(const mlxq_linear_t* parts, int n_parts, mlxq_stream_t stream, const void* x,
                                int x_dtype, int64_t x_stride, void* y, int y_dtype, int64_t y_stride, int64_t T);

/* Linear.encodeGated, Transformer.swift:247-261: y[o] = act(x . W^T + bias)[o] * e[o], one token.
 * e is fp32 [out_dim]. */
MLXQ_API int mlxq_linear_forward_gated(mlxq_linear_t h, mlxq_stream_t stream, const void* x, int x_dtype, void* y,
                                       int y_dtype, const float* e, int act);

/* Linear.encodeLookup (qembed, Kernels.swift:1002-1023): out[t, :] = dequantised row ids[t], fp32
 * [T, in_dim].  Ids outside [0, out_dim) produce a row of zeros and set the stream's error word
 * (see mlxq_stream_status) instead of reading out of bounds. */
MLXQ_API int mlxq_linear_lookup(mlxq_linear_t h, mlxq_stream_t stream, const int32_t* ids, float* out, int64_t T);

/* The row-list matvec of head_exact (Kernels.swift:2752-2787): y[list[i]] = W[list[i]] . x for
 * i < *count (count and list live on the device); rows outside [0, out_dim) are skipped. */
MLXQ_API int mlxq_linear_forward_rows(mlxq_linear_t h, mlxq_stream_t stream, const void* x, int x_dtype, float* y,
                                      const uint32_t* count, const int32_t* list, int64_t max_rows);

/* silu_mul / gelu_tanh_mul (Kernels.swift:2004-2030): out[t, i] = act(gu[t, i]) * gu[t, cols + i]; gu is fp32
 * [T, stride] (the [gate | up] buffer of a fused gate/up projection), out fp32 [T, cols]. */
MLXQ_API int mlxq_act_mul(mlxq_stream_t stream, int device, const float* gu, int64_t stride, int64_t cols, int64_t T, int act,
                          float* out);

/* The down projection reading the [gate | up] buffer itself (no counterpart in the reference, which runs silu_mul as a
 * kernel of its own between the two projections, Transformer.swift:1528-1535): y = Linear(act(gu[:, :in_dim]) *
 * gu[:, in_dim : 2 in_dim]), the product formed while the decode kernel stages its activations.  1 to 8 tokens, shapes
 * the persistent decode kernels serve; others return MLXQ_UNSUPPORTED (use mlxq_act_mul, then mlxq_linear_forward). */
MLXQ_API int mlxq_linear_forward_glu(mlxq_linear_t h, mlxq_stream_t stream, const float* gu, int64_t gu_stride, int act,
                                     void* y, int y_dtype, int64_t y_stride, int64_t T);

/* add_rms_norm (Kernels.swift:1141-1175): h += r; y = RMSNorm(h) * w, for `rows` rows of `dim` fp32 values `row_stride`
 * apart (dim a multiple of 4, rows 16-byte aligned); w is [dim] in w_dtype. */
MLXQ_API int mlxq_add_rms_norm(mlxq_stream_t stream, int device, float* h, const float* r, float* y, const void* w,
                               int w_dtype, int64_t dim, int64_t rows, int64_t row_stride, float eps);

/* First pass of the token selection (sample_blocks, Kernels.swift:2339-2377): for every token t and every block b of
 * 256 logits, the block's maximum and the lowest index that holds it.  logits is fp32 [T, stride] on `device`;
 * pairs receives the maxima as fp32 [T][nb] followed by the indices as int32 [T][nb], nb = ceil(V / 256)
 * (2 * T * nb 4-byte words).  index_base is added to every index (a shard's first row).  A NaN never wins; a block
 * with no value above -inf reports the index 0x7fffffff. */
MLXQ_API int mlxq_block_max(mlxq_stream_t stream, int device, const float* logits, int64_t stride, int64_t V, int64_t T,
                            int32_t index_base, uint32_t* pairs);

/* Greedy second pass (the argmax branch of sample_token, Kernels.swift:2379 ff.): token[t] = the lowest index holding
 * the maximum over n_seg segments of block maxima, each laid out as mlxq_block_max writes them (segment s starts
 * 2 * T * nb words after segment s - 1); value[t] (optional) = that maximum.  0x7fffffff when no block has one. */
MLXQ_API int mlxq_block_argmax(mlxq_stream_t stream, int device, const uint32_t* pairs, int n_seg, int64_t T, int64_t nb,
                               int32_t* token, float* value);

/* Writes the codes of every weight as one byte each, u8 [out_dim, in_dim].  The GPU half of the
 * bit-exact unpack check (unpack8, Kernels.swift:34-55). */
MLXQ_API int mlxq_unpack_codes(mlxq_linear_t h, mlxq_stream_t stream, uint8_t* out);

/* ---- host policy the reference's tests pin ---------------------------------------------------------- */

/* Linear.fusable, Transformer.swift:191-198. */
MLXQ_API int mlxq_fusable(const mlxq_linear_t* parts, int n_parts);
/* Linear.canFuse, Transformer.swift:201-203. */
MLXQ_API int mlxq_can_fuse(const mlxq_linear_t* parts, int n_parts, int64_t T);
/* Linear.useGemm64, Transformer.swift:266-269 (kept as the reference's tile policy; this library's GEMM
 * picks its own tile with mlxq_gemm_tile_tokens()). */
MLXQ_API int mlxq_use_gemm64(int64_t T, int64_t out_dim);
/* Token-tile width the tensor-core GEMM uses for a batch of T tokens (0 = the batch takes the matvec). */
MLXQ_API int mlxq_gemm_tile_tokens(mlxq_linear_t h, int64_t T);
/* Name of the kernel family mlxq_linear_forward would launch for T tokens with these dtypes
 * ("qmv", "qmm", "qgemm"); for tests of the selection table (Transformer.swift:272-315). */
MLXQ_API const char* mlxq_kernel_for(mlxq_linear_t h, int x_dtype, int y_dtype, int64_t T);

/* ---- errors raised on the device: cb.error -> EngineError.gpuFailure, Transformer.swift:1159-1163 --- */

/* Waits for `stream` and reports a failed launch/kernel or a device-side error word (bad lookup id,
 * a bounded wait that ran out) as a status.  Clears the error word. */
MLXQ_API int mlxq_stream_status(mlxq_stream_t stream, int device);

/* ---- output-row sharding across GPUs (no counterpart in the reference) ----------------------------- */

#define MLXQ_COMM_ID_BYTES 128
/* Fills `id` with a fresh rendezvous token; rank 0 calls it and hands the bytes to the other ranks. */
MLXQ_API int mlxq_comm_unique_id(uint8_t id[MLXQ_COMM_ID_BYTES]);
/* Joins the communicator of `nranks` GPUs (one process per GPU) on `device`. */
MLXQ_API int mlxq_comm_create(const uint8_t id[MLXQ_COMM_ID_BYTES], int rank, int nranks, int device,
                              mlxq_comm_t* out);
MLXQ_API void mlxq_comm_destroy(mlxq_comm_t c);
MLXQ_API int mlxq_comm_rank(mlxq_comm_t c);
MLXQ_API int mlxq_comm_size(mlxq_comm_t c);
/* Shard forward + all-gather: computes this rank's rows into y[t, row_offset : row_offset+rows] and
 * all-gathers the slices so every rank holds y[T, out_dim_total] (fp32, row stride y_stride).  `h` must
 * come from mlxq_linear_create_shard with the communicator's rank and size.  With one rank no
 * collective is issued. */
MLXQ_API int mlxq_linear_forward_gather(mlxq_linear_t h, mlxq_comm_t c, mlxq_stream_t stream, const void* x,
                                        int x_dtype, int64_t x_stride, float* y, int64_t y_stride, int64_t T);

/* Fused shard forward + gather (no counterpart in the reference, which runs on one GPU).  The decode kernel
 * itself stores every output row into the gather window of every rank (peer memory over NVLink); the rank's next
 * kernel on the communicator (the next fused call or mlxq_comm_wait) tells the peers that the rows are out, so no
 * collective kernel follows the call.
 *
 * mlxq_comm_window allocates the window: two buffers of `bytes` each (a positive multiple of 256; at least
 * T * total rows * 4), mapped into the other ranks through CUDA IPC.  It is a collective: every rank calls
 * it, once per communicator, with the same size, with no work pending on the device.
 *
 * mlxq_linear_forward_gather_fused enqueues the call and returns in *y_full the device address of the
 * gathered output, fp32 [T, total rows] (row stride = total rows).  The kernel does not wait for the other
 * ranks.  Their rows are complete for two readers only: the next fused call of the communicator when its x lies
 * inside the window (it waits for the peers itself before it reads its activations, while its weight copies are
 * already in flight), and anything enqueued after mlxq_comm_wait(c, stream), which enqueues that wait alone.
 * The rows may be read by work enqueued on `stream` before this rank's NEXT fused call on the communicator, and only
 * by such work: calls alternate between two buffers, and a peer that runs ahead starts storing its second-next
 * call's rows into this buffer as soon as this rank's next call has started.
 * A rank's rows are announced to the peers by the kernel that follows the call on the communicator (the rank's next
 * fused call or its mlxq_comm_wait), not by the call itself: a rank must enqueue one of those before it blocks on its
 * peers, or a peer whose next call reads these rows gives up after two seconds.
 * Every rank must issue the same sequence of fused calls.  The calls may be captured into a CUDA graph and replayed
 * (the call's number is kept on the device); a captured sequence must then hold an even number of fused calls of the
 * communicator, so that the two buffers keep alternating from one replay to the next.  Only shapes the persistent decode kernel serves
 * (T <= 16, the usual alignment) are accepted; others return MLXQ_UNSUPPORTED and leave the communicator
 * untouched -- use mlxq_linear_forward_gather for those.  A wait for a peer gives up after two seconds:
 * the result is then incomplete and mlxq_stream_status reports MLXQ_TIMEOUT. */
MLXQ_API int mlxq_comm_window(mlxq_comm_t c, size_t bytes);
MLXQ_API int mlxq_linear_forward_gather_fused(mlxq_linear_t h, mlxq_comm_t c, mlxq_stream_t stream, const void* x,
                                              int x_dtype, int64_t x_stride, int64_t T, float** y_full);
MLXQ_API int mlxq_comm_wait(mlxq_comm_t c, mlxq_stream_t stream);

/* Vocabulary head sharded by rows with the selection's first pass folded in (Transformer.swift:1574, 1588-1611 on
 * one GPU; no counterpart for the sharding): the shard's logits go to y_local (fp32 [T, shard rows], the caller's
 * scratch), their block maxima -- indices counted in the full vocabulary -- to this rank's segment of `pairs`
 * (n ranks x 2 * T * nb words, nb = ceil(shard rows / 256)), and only those segments are gathered (ncclAllGather):
 * 8 bytes per 256 logits cross NVLink instead of 1024.  Every rank's shard must have the same number of rows.
 * mlxq_block_argmax(pairs, n ranks, T, nb) then gives the greedy token on every rank. */
MLXQ_API int mlxq_linear_forward_blockmax_gather(mlxq_linear_t h, mlxq_comm_t c, mlxq_stream_t stream, const void* x,
                                                 int x_dtype, int64_t x_stride, int64_t T, float* y_local, uint32_t* pairs);

#ifdef __cplusplus
}
#endif
#endif /* MLXQ_H */
