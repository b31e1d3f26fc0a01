"""Host-side mirror of the reference's ``Linear`` class over the libmlxq C ABI.

Names, argument meaning and error behaviour follow ``Sources/MLXEngine/Transformer.swift:15-345`` so that
code (and tests) written against the reference's layer read the same here:

=========================================  ===============================================
reference (Swift)                          here
=========================================  ===============================================
``Linear(weight:scales:biases:bias:...)``  ``Linear(weight, scales, biases, bias, inDim=..)``
``encode(enc, x:, xStride:, y:, ...)``     ``encode(stream, x, xStride, y, yStride, T)``
``Linear.encodeFusedDecode(enc, parts..)`` ``Linear.encodeFusedDecode(stream, parts, ...)``
``encodeGated(enc, x:, y:, e:, act:)``     ``encodeGated(stream, x, y, e, act)``
``encodeLookup(enc, ids:, out:, T:)``      ``encodeLookup(stream, ids, out, T)``
``Linear.useGemm64 / fusable / canFuse``   same names
``permuteRows / concatRows / makePairs``   same names
``throws EngineError.invalidFile ...``     raises ``EngineError`` subclasses
=========================================  ===============================================

The Metal command encoder becomes a CUDA stream: every ``encode*`` call only enqueues work.  Tensors are
borrowed views of device memory (``TensorView`` or a CUDA ``torch.Tensor``), never copied, exactly like
the reference's ``Tensor`` (``GPU.swift:145-154``).  PyTorch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

from . import _lib as L

# ---- errors: EngineError, GPU.swift:4-33 -----------------------------------------------------------------


class EngineError(Exception):
    """Base of the errors a layer can raise; ``status`` is the C ABI's code."""
    status = -1

    def __init__(self, message: str = ""):
        super().__init__(message)
        self.message = message


class InvalidFile(EngineError):
    status = L.INVALID_FILE


class Unsupported(EngineError):
    status = L.UNSUPPORTED


class MissingTensor(EngineError):
    status = L.MISSING_TENSOR


class OutOfMemory(EngineError):
    status = L.OUT_OF_MEMORY


class GPUFailure(EngineError):
    status = L.GPU_FAILURE


class InvalidArgument(EngineError):
    status = L.INVALID_ARGUMENT


class CollectiveFailure(EngineError):
    status = L.NCCL_FAILURE


class DeviceTimeout(EngineError):
    status = L.TIMEOUT


class InvalidOutput(EngineError):
    """EngineError.invalidOutput (raised by permuteRows for a bad permutation)."""


_BY_STATUS = {c.status: c for c in (InvalidFile, Unsupported, MissingTensor, OutOfMemory, GPUFailure, InvalidArgument,
                                    CollectiveFailure, DeviceTimeout)}


def check(status: int) -> None:
    """Raise the EngineError that corresponds to a non-zero status."""
    if status != L.OK:
        text = L.last_error() or L.load().mlxq_status_string(status).decode()
        raise _BY_STATUS.get(status, EngineError)(text)


# ---- tensors: Tensor / DType, GPU.swift:121-154 -------------------------------------------------------------

_DTYPE_SIZE = {"f32": 4, "f16": 2, "bf16": 2, "u32": 4, "i32": 4, "u8": 1}
_DTYPE_CODE = {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}


@dataclass(frozen=True)
class TensorView:
    """A borrowed view of device memory: address, element type name and shape."""
    ptr: int
    dtype: str
    shape: tuple
    owner: object = None     # keeps the backing allocation alive

    @property
    def count(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        return self.count * _DTYPE_SIZE[self.dtype]


def _torch_dtype_name(t) -> str:
    import torch
    table = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16", torch.int32: "u32",
             torch.uint8: "u8"}
    if hasattr(torch, "uint32"):
        table[torch.uint32] = "u32"
    if t.dtype not in table:
        raise Unsupported(f"tensor dtype {t.dtype}")
    return table[t.dtype]


def view(t) -> Optional[TensorView]:
    """TensorView of a contiguous CUDA torch.Tensor (or pass a TensorView / None through)."""
    if t is None or isinstance(t, TensorView):
        return t
    if not t.is_contiguous():
        raise InvalidArgument("tensor must be contiguous")
    return TensorView(t.data_ptr(), _torch_dtype_name(t), tuple(t.shape), t)


def _stream_handle(stream) -> int:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _ptr(t) -> int:
    if t is None:
        return 0
    if isinstance(t, int):
        return t
    if isinstance(t, TensorView):
        return t.ptr
    return t.data_ptr()


def _act_dtype(t, default: Optional[int] = None) -> int:
    if isinstance(t, TensorView):
        return _DTYPE_CODE[t.dtype]
    if isinstance(t, int):
        if default is None:
            raise InvalidArgument("a raw pointer needs an explicit dtype")
        return default
    return _DTYPE_CODE[_torch_dtype_name(t)]


class Linear:
    """An MLX-quantized linear layer (``Transformer.swift:15``)."""

    def __init__(self, weight, scales, biases, bias=None, inDim: int = 0, outDim: Optional[int] = None,
                 name: str = "linear", device: Optional[int] = None, _shard: Optional[tuple] = None):
        w, s, b, rb = view(weight), view(scales), view(biases), view(bias)
        if w is None:
            raise MissingTensor(name + ".weight")
        if device is None:
            device = weight.device.index if hasattr(weight, "device") and weight.device.index is not None else 0
        d = L.LinearDesc()
        d.weight = w.ptr
        d.weight_rows, d.weight_cols = (w.shape + (0, 0))[:2] if len(w.shape) == 2 else (0, 0)
        if w.dtype != "u32" and len(w.shape) == 2:
            # the reference takes any integer storage and counts bytes (Transformer.swift:57, :68)
            d.weight_cols = w.shape[1] * _DTYPE_SIZE[w.dtype] // 4 if (w.shape[1] * _DTYPE_SIZE[w.dtype]) % 4 == 0 else 0
        if s is None and b is None and len(w.shape) == 2 and w.dtype in _DTYPE_CODE:
            # a dense layer (Transformer.swift:103-112): the weights' own type travels in the descriptor's spare field
            d.weight_cols = w.shape[1]
            d.reserved = 1 + _DTYPE_CODE[w.dtype]
        d.scales = s.ptr if s else None
        d.biases = b.ptr if b else None
        d.scales_rows, d.scales_cols = (s.shape if s is not None and len(s.shape) == 2 else (0, 0))
        d.biases_rows, d.biases_cols = (b.shape if b is not None and len(b.shape) == 2 else (0, 0))
        if s is not None and s.dtype not in _DTYPE_CODE:
            raise Unsupported(f"{name}: scales dtype {s.dtype}")
        if s is not None and b is not None and s.dtype != b.dtype:
            raise InvalidFile(f"{name}: inconsistent quantization tensors")
        d.scale_dtype = _DTYPE_CODE[s.dtype] if s is not None else 0
        d.bias = rb.ptr if rb else None
        d.bias_len = rb.shape[0] if rb is not None and len(rb.shape) == 1 else (-1 if rb is not None else 0)
        if rb is not None and rb.dtype not in _DTYPE_CODE:
            raise Unsupported(f"{name}: bias dtype {rb.dtype}")
        d.bias_dtype = _DTYPE_CODE[rb.dtype] if rb is not None else 0
        d.in_dim = inDim
        d.expect_out = outDim or 0
        d.device = device
        d.name = name.encode()
        self._desc = d
        self._keep = (w, s, b, rb)
        self.weight, self.scales, self.biases, self.bias = w, s, b, rb
        self.name = name
        self.device = device
        h = C.c_void_p()
        lib = L.load()
        if _shard is None:
            check(lib.mlxq_linear_create(C.byref(d), C.byref(h)))
        else:
            rank, nranks, full = _shard
            check(lib.mlxq_linear_create_shard(C.byref(d), rank, nranks, 1 if full else 0, C.byref(h)))
        self._h = h
        self.inDim = int(lib.mlxq_linear_in_dim(h))
        self.outDim = int(lib.mlxq_linear_out_dim(h))
        self.bits = int(lib.mlxq_linear_bits(h))
        self.groupSize = int(lib.mlxq_linear_group_size(h))
        self.rowOffset = int(lib.mlxq_linear_row_offset(h))
        self.totalOut = int(lib.mlxq_linear_total_rows(h))
        self.description = f"q{self.bits}g{self.groupSize}" if self.bits else w.dtype

    @classmethod
    def shard(cls, weight, scales, biases, bias=None, inDim: int = 0, rank: int = 0, nranks: int = 1, full: bool = True,
              name: str = "linear", device: Optional[int] = None) -> "Linear":
        """Rows [rank*O/nranks, (rank+1)*O/nranks) of the layer (``full``: the tensors hold all rows)."""
        return cls(weight, scales, biases, bias, inDim=inDim, name=name, device=device, _shard=(rank, nranks, full))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                L.load().mlxq_linear_destroy(h)
            except Exception:
                pass

    # ---- encode: Transformer.swift:272-315 ------------------------------------------------------------------
    def encode(self, stream, x, xStride: int, y, yStride: int, T: int, xDtype: Optional[int] = None,
               yDtype: Optional[int] = None) -> None:
        """y[t, :outDim] = x[t] . W^T (+ bias), enqueued on ``stream``.  Strides are in elements."""
        check(L.load().mlxq_linear_forward(self._h, _stream_handle(stream), _ptr(x), _act_dtype(x, xDtype), xStride,
                                           _ptr(y), _act_dtype(y, yDtype), yStride, T))

    def prepare(self, stream=None) -> None:
        """Load-time preparation (the place of ``makePairs``, ``Transformer.swift:160-188``): builds the GEMM's private
        table of scales and biases ahead of the first long batch.  Optional; results do not depend on it."""
        check(L.load().mlxq_linear_prepare(self._h, _stream_handle(stream)))

    def encodeStatic(self, stream, x, xStride: int, y, yStride: int, T: int, xDtype: Optional[int] = None,
                     yDtype: Optional[int] = None) -> None:
        """``encode`` for hosts that must not allocate device memory while they run: the GEMM's staged copy
        of the activations goes into the library's fixed 32 MiB array instead of pool memory.  Same results;
        batches with ``T * inDim * 2`` bytes above the array are refused (``InvalidArgument``); calls that
        overlap on the GPU share the array and race.  No counterpart in the reference."""
        check(L.load().mlxq_linear_forward_static(self._h, _stream_handle(stream), _ptr(x), _act_dtype(x, xDtype),
                                                  xStride, _ptr(y), _act_dtype(y, yDtype), yStride, T))

    @staticmethod
    def encodeFusedDecode(stream, parts: Sequence["Linear"], x, y, xStride: int = 0, yStride: int = 0, T: int = 1,
                          xDtype: Optional[int] = None, yDtype: Optional[int] = None) -> None:
        """One launch computing the rows [A | B | C] (``Transformer.swift:206-244``)."""
        arr = (C.c_void_p * len(parts))(*[p._h for p in parts])
        if T == 1:
            xStride = xStride or parts[0].inDim
            yStride = yStride or sum(p.outDim for p in parts)
        check(L.load().mlxq_fused_forward(arr, len(parts), _stream_handle(stream), _ptr(x), _act_dtype(x, xDtype),
                                          xStride, _ptr(y), _act_dtype(y, yDtype), yStride, T))

    def encodeGated(self, stream, x, y, e, act: int, xDtype: Optional[int] = None, yDtype: Optional[int] = None) -> None:
        """y[:outDim] = act(x . W^T + bias) * e[:outDim], one token (``Transformer.swift:247-261``)."""
        check(L.load().mlxq_linear_forward_gated(self._h, _stream_handle(stream), _ptr(x), _act_dtype(x, xDtype), _ptr(y),
                                                 _act_dtype(y, yDtype), _ptr(e), act))

    def encodeGLU(self, stream, gu, guStride: int, act: int, y, yStride: int, T: int, yDtype: Optional[int] = None) -> None:
        """y = self(act(gu[:, :inDim]) * gu[:, inDim:2 inDim]): the down projection reading the fp32 [gate | up] buffer
        itself, ``silu_mul`` (``Kernels.swift:2004-2013``) folded into the staging of its activations.  1-8 tokens."""
        check(L.load().mlxq_linear_forward_glu(self._h, _stream_handle(stream), _ptr(gu), guStride, act, _ptr(y),
                                               _act_dtype(y, yDtype), yStride, T))

    def encodeLookup(self, stream, ids, out, T: int) -> None:
        """out[t, :] = dequantised row ids[t] in fp32 (``Transformer.swift:318-344``)."""
        check(L.load().mlxq_linear_lookup(self._h, _stream_handle(stream), _ptr(ids), _ptr(out), T))

    def encodeRows(self, stream, x, y, count, rows, maxRows: int, xDtype: Optional[int] = None) -> None:
        """y[rows[i]] = W[rows[i]] . x for i < count[0] (``head_exact``, ``Kernels.swift:2752-2787``)."""
        check(L.load().mlxq_linear_forward_rows(self._h, _stream_handle(stream), _ptr(x), _act_dtype(x, xDtype), _ptr(y),
                                                _ptr(count), _ptr(rows), maxRows))

    def unpackCodes(self, stream, out) -> None:
        """out u8 [outDim, inDim] = the code of every weight (the bit-exact format check)."""
        check(L.load().mlxq_unpack_codes(self._h, _stream_handle(stream), _ptr(out)))

    def kernelFor(self, T: int, xDtype: int = L.F32, yDtype: int = L.F32) -> str:
        return L.load().mlxq_kernel_for(self._h, xDtype, yDtype, T).decode()

    def gemmTileTokens(self, T: int) -> int:
        return int(L.load().mlxq_gemm_tile_tokens(self._h, T))

    # ---- policy: Transformer.swift:191-203, 266-269 -------------------------------------------------------
    @staticmethod
    def useGemm64(T: int, outDim: int) -> bool:
        return bool(L.load().mlxq_use_gemm64(T, outDim))

    @staticmethod
    def fusable(parts: Sequence["Linear"]) -> bool:
        if not parts:
            return False
        arr = (C.c_void_p * len(parts))(*[p._h for p in parts])
        return bool(L.load().mlxq_fusable(arr, len(parts)))

    @staticmethod
    def canFuse(parts: Sequence["Linear"], T: int) -> bool:
        arr = (C.c_void_p * len(parts))(*[p._h for p in parts])
        return bool(L.load().mlxq_can_fuse(arr, len(parts), T))

    # ---- load-time transforms: Transformer.swift:113-188 --------------------------------------------------
    def permuteRows(self, perm: Sequence[int]) -> None:
        """Reorder the output rows in place: row r becomes the old row perm[r]."""
        import torch
        perm = list(perm)
        if len(perm) != self.outDim or sorted(perm) != list(range(self.outDim)):
            raise InvalidOutput("bad row permutation")
        for tv in (self.weight, self.scales, self.biases, self.bias):
            if tv is None:
                continue
            t = tv.owner
            if t is None:
                raise InvalidArgument("permuteRows needs torch-backed tensors")
            idx = torch.tensor(perm, device=t.device, dtype=torch.long)
            t.copy_(t.index_select(0, idx))

    @staticmethod
    def concatRows(a: "Linear", b: "Linear", name: str) -> Optional["Linear"]:
        """One layer computing [a | b] when both are stored alike; None otherwise (tensors are copied)."""
        import torch
        if (a.inDim != b.inDim or a.bias is not None or b.bias is not None or a.weight.dtype != b.weight.dtype
                or a.weight.shape[1] != b.weight.shape[1] or a.scales.dtype != b.scales.dtype
                or a.scales.shape[-1] != b.scales.shape[-1] or a.biases.dtype != b.biases.dtype):
            return None
        cat = lambda p, q: torch.cat([p.owner, q.owner], dim=0).contiguous()
        return Linear(cat(a.weight, b.weight), cat(a.scales, b.scales), cat(a.biases, b.biases), None, inDim=a.inDim,
                      outDim=a.outDim + b.outDim, name=name, device=a.device)

    def makePairs(self) -> None:
        """The reference interleaves (scale, bias) pairs for its K = 1024 decode kernel
        (``Transformer.swift:156-188``).  The CUDA kernels read the two arrays as they are stored, so
        this is a no-op kept for call-site compatibility; outputs do not change either way."""
        return None

    # ---- convenience for hosts that hold activations in host memory --------------------------------------
    def forwardHost(self, x_host, y_host, stream=None, staging=None):
        """x_host [T, inDim] pinned host tensor -> y_host [T, outDim] pinned host tensor, through device
        staging buffers (allocated once and returned for reuse): copy in, encode, copy out, wait."""
        import torch
        T = x_host.shape[0] if x_host.dim() == 2 else 1
        stream = stream or torch.cuda.current_stream()
        if staging is None:
            dev = torch.device("cuda", self.device)
            staging = (torch.empty((T, self.inDim), dtype=x_host.dtype, device=dev),
                       torch.empty((T, self.outDim), dtype=y_host.dtype, device=dev))
        xd, yd = staging
        with torch.cuda.stream(stream):
            xd.copy_(x_host.view(T, self.inDim), non_blocking=True)
            self.encode(stream, xd, self.inDim, yd, self.outDim, T)
            y_host.view(T, self.outDim).copy_(yd, non_blocking=True)
        stream.synchronize()
        return staging


SELECT_BLOCK = 256          # logits per block of the selection's first pass
SELECT_NONE = 0x7FFFFFFF    # index reported for a block (or token) with no value above -inf


def actMul(stream, gu, stride: int, cols: int, T: int, act: int, out, device: int = 0) -> None:
    """out[t, i] = act(gu[t, i]) * gu[t, cols + i] (``silu_mul`` / ``gelu_tanh_mul``, ``Kernels.swift:2004-2030``)."""
    check(L.load().mlxq_act_mul(_stream_handle(stream), device, _ptr(gu), stride, cols, T, act, _ptr(out)))


def addRMSNorm(stream, h, r, y, w, dim: int, rows: int, rowStride: int, eps: float, wDtype: Optional[int] = None,
               device: int = 0) -> None:
    """h += r; y = RMSNorm(h) * w (``add_rms_norm``, ``Kernels.swift:1141-1175``)."""
    check(L.load().mlxq_add_rms_norm(_stream_handle(stream), device, _ptr(h), _ptr(r), _ptr(y), _ptr(w), _act_dtype(w, wDtype),
                                     dim, rows, rowStride, eps))


def blockMax(stream, logits, V: int, T: int, stride: int, pairs, indexBase: int = 0, device: int = 0) -> None:
    """First pass of the token selection (``sample_blocks``, ``Kernels.swift:2339-2377``): per token and block of 256
    logits the maximum and the lowest index holding it.  ``pairs`` (int32 or uint32, 2 * T * nb words, nb =
    ceil(V / 256)) receives the maxima as fp32 bit patterns [T][nb], then the indices [T][nb]."""
    check(L.load().mlxq_block_max(_stream_handle(stream), device, _ptr(logits), stride, V, T, indexBase, _ptr(pairs)))


def blockArgmax(stream, pairs, nSeg: int, T: int, nb: int, token, value=None, device: int = 0) -> None:
    """Greedy second pass over ``nSeg`` segments of block maxima: token[t] = lowest index holding the maximum."""
    check(L.load().mlxq_block_argmax(_stream_handle(stream), device, _ptr(pairs), nSeg, T, nb, _ptr(token),
                                     _ptr(value) if value is not None else None))


def streamStatus(stream=None, device: int = 0) -> None:
    """Wait for ``stream`` and raise if a kernel failed or recorded an error (``cb.error`` in the reference)."""
    check(L.load().mlxq_stream_status(_stream_handle(stream), device))


class _DeviceArray:
    """An fp32 device buffer owned by the library, exposed through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape, device: int):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (ptr, False), "version": 3,
                                         "strides": None}
        self.device = device


class Comm:
    """The communicator behind row-sharded layers: one process per GPU, NCCL all-gather of output slices."""

    def __init__(self, rank: int, nranks: int, device: int, unique_id: Optional[bytes] = None):
        lib = L.load()
        idbuf = (C.c_uint8 * L.COMM_ID_BYTES)()
        if nranks > 1:
            if unique_id is None or len(unique_id) != L.COMM_ID_BYTES:
                raise InvalidArgument("a 128-byte rendezvous id from Comm.uniqueId() is required")
            C.memmove(idbuf, unique_id, L.COMM_ID_BYTES)
        h = C.c_void_p()
        check(lib.mlxq_comm_create(idbuf, rank, nranks, device, C.byref(h)))
        self._h, self.rank, self.size, self.device = h, rank, nranks, device
        self._views = {}

    @staticmethod
    def uniqueId() -> bytes:
        buf = (C.c_uint8 * L.COMM_ID_BYTES)()
        check(L.load().mlxq_comm_unique_id(buf))
        return bytes(buf)

    def forwardGather(self, layer: Linear, stream, x, xStride: int, y, yStride: int, T: int,
                      xDtype: Optional[int] = None) -> None:
        """Shard matvec into y's slice, then all-gather so every rank holds y[T, total rows] (fp32)."""
        check(L.load().mlxq_linear_forward_gather(layer._h, self._h, _stream_handle(stream), _ptr(x),
                                                  _act_dtype(x, xDtype), xStride, _ptr(y), yStride, T))

    def window(self, nbytes: int) -> None:
        """Collective: allocate this rank's gather window (two buffers of nbytes) and map the peers' windows."""
        check(L.load().mlxq_comm_window(self._h, nbytes))

    def forwardGatherFused(self, layer: Linear, stream, x, xStride: int, T: int, xDtype: Optional[int] = None,
                           wait: bool = True):
        """Shard matvec whose kernel stores its rows into every rank's window.  Returns the gathered output as
        an fp32 CUDA tensor [T, total rows] that aliases the window: readable by work enqueued on ``stream`` before this
        rank's next fused call, and only by such work (a peer that runs ahead reuses the buffer after that).
        ``wait=False`` leaves out the wait for the peers' rows: right when the next thing in the stream is
        another fused call (it waits itself) -- call ``wait(stream)`` before anything else reads the tensor."""
        out = C.c_void_p()
        check(L.load().mlxq_linear_forward_gather_fused(layer._h, self._h, _stream_handle(stream), _ptr(x),
                                                        _act_dtype(x, xDtype), xStride, T, C.byref(out)))
        if wait:
            self.wait(stream)
        key = (out.value, T, layer.totalOut)
        view = self._views.get(key)
        if view is None:                 # two addresses per shape: the views are made once
            import torch
            view = torch.as_tensor(_DeviceArray(out.value, (T, layer.totalOut), self.device), device=f"cuda:{self.device}")
            self._views[key] = view
        return view

    def forwardBlockMaxGather(self, layer: Linear, stream, x, xStride: int, T: int, yLocal, pairs,
                              xDtype: Optional[int] = None) -> None:
        """Row-sharded vocabulary head with the selection's first pass folded in: the shard's logits go to ``yLocal``
        (fp32 [T, shard rows]), their block maxima (indices in the full vocabulary) to this rank's segment of ``pairs``
        (nranks x 2 * T * nb words), and only the segments are gathered.  ``blockArgmax(pairs, nranks, T, nb)`` then
        yields the greedy token."""
        check(L.load().mlxq_linear_forward_blockmax_gather(layer._h, self._h, _stream_handle(stream), _ptr(x),
                                                           _act_dtype(x, xDtype), xStride, T, _ptr(yLocal), _ptr(pairs)))

    def wait(self, stream) -> None:
        """Enqueue the wait for every peer's rows of the last fused call."""
        check(L.load().mlxq_comm_wait(self._h, _stream_handle(stream)))

    def close(self) -> None:
        h, self._h = self._h, None
        self._views = {}
        if h:
            L.load().mlxq_comm_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
