"""ctypes front-end of the CPU oracle (``mlxq_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module.  It exists so that the tests, the smoke check and
the benchmark's CPU-baseline leg can compute what the reference project's own CPU code would compute
for the quantized-linear path:

* ``pack`` / ``unpack``            -- Tests/MLXEngineTests/KernelTests.swift:34-43,
                                      Sources/MLXEngine/SieveImport.swift:101-109
* ``dequantize``                   -- Sources/MLXEngine/SieveImport.swift:90-112
* ``matmul_dense`` / ``qmatmul``   -- Tests/MLXEngineTests/KernelTests.swift:102-113 (double accumulate)
* ``QuantFixture``                 -- Tests/MLXEngineTests/KernelTests.swift:48-114 (same xorshift stream)
* ``act_mul``                      -- Sources/MLXEngine/Kernels.swift:116-130
* ``quantize4``                    -- Sources/MLXEngine/SieveImport.swift:244-265
* ``use_gemm64``                   -- Sources/MLXEngine/Transformer.swift:266-269

Parity status: the reference stores no input/output vectors for this path and cannot be compiled on
Linux (Swift + Metal), so matvec outputs are pinned by algorithm; the literal known-answer material in
the reference's tests (f16 bit patterns, half round trip, quantize4 bound, useGemm64 table) is checked
in ``tests/test_oracle.py``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmlxq_oracle.so")

F32, F16, BF16 = 0, 1, 2
DTYPE_NAMES = {F32: "f32", F16: "f16", BF16: "bf16"}


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file; returns the library path."""
    src = os.path.join(_HERE, "mlxq_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"] + (["-B"] if force else []), check=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        u8p, f32p, u16p, u32p, vp = (C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_uint16),
                                     C.POINTER(C.c_uint32), C.c_void_p)
        sz = C.c_size_t
        L.mlxq_o_rng_next.restype = C.c_uint64
        L.mlxq_o_rng_next.argtypes = [C.POINTER(C.c_uint64)]
        L.mlxq_o_rng_float.restype = C.c_float
        L.mlxq_o_rng_float.argtypes = [C.POINTER(C.c_uint64), C.c_float, C.c_float]
        L.mlxq_o_rng_fill_codes.restype = None
        L.mlxq_o_rng_fill_codes.argtypes = [C.POINTER(C.c_uint64), sz, C.c_int, u8p]
        L.mlxq_o_rng_fill_floats.restype = None
        L.mlxq_o_rng_fill_floats.argtypes = [C.POINTER(C.c_uint64), sz, C.c_float, C.c_float, f32p]
        L.mlxq_o_rng_fill_pairs.restype = None
        L.mlxq_o_rng_fill_pairs.argtypes = [C.POINTER(C.c_uint64), sz, C.c_float, C.c_float, C.c_float, C.c_float, f32p, f32p]
        L.mlxq_o_half_to_float.restype = C.c_float
        L.mlxq_o_half_to_float.argtypes = [C.c_uint16]
        L.mlxq_o_float_to_half.restype = C.c_uint16
        L.mlxq_o_float_to_half.argtypes = [C.c_float]
        L.mlxq_o_float_to_bf16_trunc.restype = C.c_uint16
        L.mlxq_o_float_to_bf16_trunc.argtypes = [C.c_float]
        L.mlxq_o_float_to_bf16_rne.restype = C.c_uint16
        L.mlxq_o_float_to_bf16_rne.argtypes = [C.c_float]
        L.mlxq_o_bf16_to_float.restype = C.c_float
        L.mlxq_o_bf16_to_float.argtypes = [C.c_uint16]
        L.mlxq_o_to_float.restype = None
        L.mlxq_o_to_float.argtypes = [vp, C.c_int, sz, f32p]
        L.mlxq_o_pack.restype = None
        L.mlxq_o_pack.argtypes = [u8p, sz, C.c_int, u8p]
        L.mlxq_o_unpack.restype = None
        L.mlxq_o_unpack.argtypes = [u8p, sz, sz, C.c_int, u8p]
        L.mlxq_o_dequantize.restype = None
        L.mlxq_o_dequantize.argtypes = [u8p, vp, vp, C.c_int, sz, sz, C.c_int, sz, f32p]
        L.mlxq_o_matmul_dense.restype = None
        L.mlxq_o_matmul_dense.argtypes = [f32p, f32p, f32p, sz, sz, sz, f32p]
        L.mlxq_o_qmatmul.restype = None
        L.mlxq_o_qmatmul.argtypes = [u8p, vp, vp, C.c_int, f32p, f32p, sz, f32p, sz, sz, sz, sz, C.c_int, sz,
                                     C.c_int, C.c_int]
        L.mlxq_o_max_threads.restype = C.c_int
        L.mlxq_o_act_mul.restype = C.c_float
        L.mlxq_o_act_mul.argtypes = [C.c_int, C.c_float, C.c_float]
        L.mlxq_o_quantize4.restype = None
        L.mlxq_o_quantize4.argtypes = [f32p, sz, sz, u32p, u16p, u16p]
        L.mlxq_o_use_gemm64.restype = C.c_int
        L.mlxq_o_use_gemm64.argtypes = [C.c_int, C.c_int]
        L.mlxq_o_max_rel_err.restype = C.c_float
        L.mlxq_o_max_rel_err.argtypes = [f32p, f32p, sz]
        _lib = L
    return _lib


def _p(a: np.ndarray, ty):
    return a.ctypes.data_as(C.POINTER(ty))


def _vp(a: np.ndarray):
    return C.c_void_p(a.ctypes.data)


# ---- scalar helpers ------------------------------------------------------------------------------------

class RNG:
    """The reference tests' xorshift64 generator (KernelTests.swift:8-14)."""

    def __init__(self, seed: int):
        self._s = C.c_uint64(seed)

    def next(self) -> int:
        return int(lib().mlxq_o_rng_next(C.byref(self._s)))

    def float(self, lo: float = -1.0, hi: float = 1.0) -> float:
        return float(lib().mlxq_o_rng_float(C.byref(self._s), lo, hi))

    def floats(self, n: int, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().mlxq_o_rng_fill_floats(C.byref(self._s), n, lo, hi, _p(out, C.c_float))
        return out

    def codes(self, n: int, bits: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint8)
        lib().mlxq_o_rng_fill_codes(C.byref(self._s), n, bits, _p(out, C.c_uint8))
        return out

    def pairs(self, n: int, lo0: float, hi0: float, lo1: float, hi1: float):
        a, b = np.empty(n, dtype=np.float32), np.empty(n, dtype=np.float32)
        lib().mlxq_o_rng_fill_pairs(C.byref(self._s), n, lo0, hi0, lo1, hi1, _p(a, C.c_float), _p(b, C.c_float))
        return a, b


def half_to_float(bits: int) -> float:
    return float(lib().mlxq_o_half_to_float(bits))


def float_to_half(v: float) -> int:
    return int(lib().mlxq_o_float_to_half(v))


def store(values: np.ndarray, dtype: int, bf16_truncate: bool = False):
    """Round fp32 values to a storage dtype.  Returns (raw array as stored, the same values as fp32).

    f16 uses the reference's round-to-nearest-even; bf16 truncates when ``bf16_truncate`` (what the
    reference's test helper does, KernelTests.swift:45) and rounds to nearest even otherwise."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    if dtype == F32:
        return v.copy(), v.copy()
    if dtype == F16:
        raw = v.astype(np.float16)          # IEEE RNE, identical to halfBits (checked in tests)
        return raw.view(np.uint16).copy(), raw.astype(np.float32)
    u = v.view(np.uint32)
    if bf16_truncate:
        raw = (u >> 16).astype(np.uint16)
    else:
        nan = (u & 0x7F800000) == 0x7F800000
        nan &= (u & 0x7FFFFF) != 0
        r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
        raw = np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)
    back = (raw.astype(np.uint32) << 16).view(np.float32)
    return raw, back.copy()


def to_float(raw: np.ndarray, dtype: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw)
    out = np.empty(raw.size, dtype=np.float32)
    lib().mlxq_o_to_float(_vp(raw), dtype, raw.size, _p(out, C.c_float))
    return out.reshape(raw.shape)


# ---- format ----------------------------------------------------------------------------------------------

def pack(q: np.ndarray, bits: int) -> np.ndarray:
    """Pack codes [O, K] (uint8) row by row; returns uint8 [O, K*bits/8]."""
    q = np.ascontiguousarray(q, dtype=np.uint8)
    O, K = q.shape
    assert (K * bits) % 8 == 0
    out = np.empty((O, K * bits // 8), dtype=np.uint8)
    L = lib()
    for r in range(O):
        L.mlxq_o_pack(_p(q[r], C.c_uint8), K, bits, _p(out[r], C.c_uint8))
    return out


def pack_fast(q: np.ndarray, bits: int) -> np.ndarray:
    """numpy packer for large matrices (same stream as ``pack``; the tests check they agree)."""
    q = np.ascontiguousarray(q, dtype=np.uint8)
    O, K = q.shape
    bitsarr = ((q[:, :, None] >> np.arange(bits, dtype=np.uint8)) & 1).astype(np.uint8)   # [O, K, bits] LSB first
    return np.packbits(bitsarr.reshape(O, K * bits), axis=1, bitorder="little")


def unpack(packed: np.ndarray, K: int, bits: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed).view(np.uint8).reshape(packed.shape[0], -1)
    O = packed.shape[0]
    assert packed.shape[1] == K * bits // 8
    q = np.empty((O, K), dtype=np.uint8)
    lib().mlxq_o_unpack(_p(packed, C.c_uint8), O, K, bits, _p(q, C.c_uint8))
    return q


def dequantize(packed: np.ndarray, scales_raw: np.ndarray, biases_raw: np.ndarray, sdtype: int, K: int, bits: int,
               gs: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed).view(np.uint8).reshape(packed.shape[0], -1)
    O = packed.shape[0]
    out = np.empty((O, K), dtype=np.float32)
    s, b = np.ascontiguousarray(scales_raw), np.ascontiguousarray(biases_raw)
    lib().mlxq_o_dequantize(_p(packed, C.c_uint8), _vp(s), _vp(b), sdtype, O, K, bits, gs, _p(out, C.c_float))
    return out


def matmul_dense(dense: np.ndarray, x: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    dense = np.ascontiguousarray(dense, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    O, K = dense.shape
    T = x.size // K
    y = np.empty((T, O), dtype=np.float32)
    bp = _p(np.ascontiguousarray(bias, dtype=np.float32), C.c_float) if bias is not None else None
    lib().mlxq_o_matmul_dense(_p(dense, C.c_float), _p(x, C.c_float), bp, T, O, K, _p(y, C.c_float))
    return y


def qmatmul(packed: np.ndarray, scales_raw: np.ndarray, biases_raw: np.ndarray, sdtype: int, x: np.ndarray, K: int,
            bits: int, gs: int, bias: np.ndarray | None = None, accumulate_double: bool = True,
            threads: int = 0) -> np.ndarray:
    """y[T, O] from packed weights without building the dense table (OpenMP over rows)."""
    packed = np.ascontiguousarray(packed).view(np.uint8).reshape(packed.shape[0], -1)
    O = packed.shape[0]
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, K)
    T = x.shape[0]
    y = np.empty((T, O), dtype=np.float32)
    s, b = np.ascontiguousarray(scales_raw), np.ascontiguousarray(biases_raw)
    bias32 = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
    lib().mlxq_o_qmatmul(_p(packed, C.c_uint8), _vp(s), _vp(b), sdtype,
                         _p(bias32, C.c_float) if bias32 is not None else None,
                         _p(x, C.c_float), K, _p(y, C.c_float), O, T, O, K, bits, gs,
                         1 if accumulate_double else 0, threads)
    return y


def max_threads() -> int:
    return int(lib().mlxq_o_max_threads())


def act_mul(act: int, g: np.ndarray, u: np.ndarray) -> np.ndarray:
    L = lib()
    g = np.asarray(g, dtype=np.float32)
    u = np.asarray(u, dtype=np.float32)
    return np.array([L.mlxq_o_act_mul(act, float(a), float(b)) for a, b in zip(g.ravel(), u.ravel())],
                    dtype=np.float32).reshape(g.shape)


def quantize4(s: np.ndarray):
    """In-place 4-bit g64 quantisation of s [V, r]; returns (codes u32 [V, r/8], scales u16, biases u16)."""
    assert s.dtype == np.float32 and s.flags.c_contiguous
    V, r = s.shape
    codes = np.zeros((V, r // 8), dtype=np.uint32)
    scales = np.zeros((V, r // 64), dtype=np.uint16)
    biases = np.zeros((V, r // 64), dtype=np.uint16)
    lib().mlxq_o_quantize4(_p(s, C.c_float), V, r, _p(codes, C.c_uint32), _p(scales, C.c_uint16),
                           _p(biases, C.c_uint16))
    return codes, scales, biases


def use_gemm64(T: int, out_dim: int) -> bool:
    return bool(lib().mlxq_o_use_gemm64(T, out_dim))


def max_rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """assertClose's metric (KernelTests.swift:116-124): max |got-ref| / max(1, |ref|)."""
    a = np.ascontiguousarray(got, dtype=np.float32).ravel()
    b = np.ascontiguousarray(ref, dtype=np.float32).ravel()
    assert a.size == b.size
    return float(lib().mlxq_o_max_rel_err(_p(a, C.c_float), _p(b, C.c_float), a.size))


# ---- the reference's test fixture -----------------------------------------------------------------------

class QuantFixture:
    """QuantFixture of KernelTests.swift:48-114, drawing the same xorshift stream in the same order.

    Attributes: q [O,K] uint8, packed uint8 [O, K*bits/8], scales_raw / biases_raw (storage dtype),
    dense fp32 [O,K] (= sRef*Float(q)+bRef), bias_raw / bias (or None)."""

    def __init__(self, O: int, K: int, bits: int, gs: int, scale_type: int = F16, with_bias: bool = False,
                 seed: int = 7):
        rng = RNG(seed)
        groups = K // gs
        self.O, self.K, self.bits, self.gs, self.scale_type = O, K, bits, gs, scale_type
        self.q = rng.codes(O * K, bits).reshape(O, K)
        sc, bi = rng.pairs(O * groups, 0.001, 0.05, -0.2, 0.2)
        self.scales_raw, s_ref = store(sc.reshape(O, groups), scale_type, bf16_truncate=True)
        self.biases_raw, b_ref = store(bi.reshape(O, groups), scale_type, bf16_truncate=True)
        self.packed = pack_fast(self.q, bits)
        self.bias_raw = self.bias = None
        if with_bias:
            raw = rng.floats(O, -0.5, 0.5)
            self.bias_raw, self.bias = store(raw, scale_type, bf16_truncate=True)
        # dense[r][k] = sRef[g] * Float(q) + bRef[g] in fp32, two roundings (KernelTests.swift:93-96)
        qf = self.q.astype(np.float32)
        prod = (np.repeat(s_ref, gs, axis=1) * qf).astype(np.float32)
        self.dense = (prod + np.repeat(b_ref, gs, axis=1)).astype(np.float32)

    def reference(self, x: np.ndarray) -> np.ndarray:
        """y [T, O]: double accumulate, cast, then add the row bias (KernelTests.swift:102-113)."""
        return matmul_dense(self.dense, x, self.bias)


# ---- token selection, first pass and greedy second pass -----------------------------------------------------------
SELECT_BLOCK = 256
SELECT_NONE = 0x7FFFFFFF


def block_max(logits: np.ndarray, index_base: int = 0):
    """``sample_blocks`` / ``smp_block`` (Sources/MLXEngine/Kernels.swift:2339-2377): for every row of ``logits``
    [T, V] and every block of 256 values, the maximum and the lowest index holding it.  The scan is a strict ``>``
    from -inf in index order, so a NaN never wins and a block with nothing above -inf reports SELECT_NONE."""
    logits = np.asarray(logits, dtype=np.float32)
    T, V = logits.shape
    nb = (V + SELECT_BLOCK - 1) // SELECT_BLOCK
    bmax = np.full((T, nb), -np.inf, dtype=np.float32)
    barg = np.full((T, nb), SELECT_NONE, dtype=np.int64)
    for t in range(T):
        for b in range(nb):
            seg = logits[t, b * SELECT_BLOCK:(b + 1) * SELECT_BLOCK]
            best, bi = np.float32(-np.inf), SELECT_NONE
            for j, v in enumerate(seg):
                if v > best:
                    best, bi = v, b * SELECT_BLOCK + j + index_base
            bmax[t, b], barg[t, b] = best, bi
    return bmax, barg.astype(np.int32)


def block_argmax(bmax: np.ndarray, barg: np.ndarray):
    """The greedy branch of ``sample_token`` (Kernels.swift:2379 ff.) over block maxima [T, n]: the maximum and the
    lowest index that holds it (SELECT_NONE when no block has a value above -inf)."""
    T = bmax.shape[0]
    tok = np.full(T, SELECT_NONE, dtype=np.int32)
    val = np.full(T, -np.inf, dtype=np.float32)
    for t in range(T):
        best, bi = np.float32(-np.inf), SELECT_NONE
        for m, ix in zip(bmax[t], barg[t]):
            if m > best or (m == best and ix < bi):
                best, bi = m, int(ix)
        tok[t], val[t] = bi, best
    return tok, val


def add_rms_norm(h: np.ndarray, r: np.ndarray, w: np.ndarray, eps: float):
    """``add_rms_norm`` (Sources/MLXEngine/Kernels.swift:1141-1175): h += r; y = RMSNorm(h) * w, row by row.  Returns
    (h, y) in fp32; the sum of squares is accumulated in float64 here (the kernel's fp32 tree sits within 1e-6 of it)."""
    h = (np.asarray(h, dtype=np.float32) + np.asarray(r, dtype=np.float32)).astype(np.float32)
    ss = np.sum(h.astype(np.float64) ** 2, axis=-1, keepdims=True)
    inv = (1.0 / np.sqrt(ss / h.shape[-1] + eps)).astype(np.float32)
    return h, (h * inv * np.asarray(w, dtype=np.float32)).astype(np.float32)
