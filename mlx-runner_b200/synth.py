"""Seeded synthetic layers in the MLX affine format, with the shapes and value distributions of the
benchmark configurations (there are no model files to load: weights are random by design).

    codes  q ~ U{0 .. 2^bits - 1}
    scale  = |N(0,1)| * 0.002 + 1e-4          stored as f16 / bf16 / f32
    bias   = -2^(bits-1) * scale (+ N(0, 1e-4) when ``bias_noise``)
    x      ~ N(0,1)

numpy's ``default_rng(seed)`` is the generator; the same (shape, seed) always gives the same bytes.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

F32, F16, BF16 = 0, 1, 2


def pack_codes(q: np.ndarray, bits: int) -> np.ndarray:
    """Pack codes [O, K] into the row-wise little-endian bit stream; returns uint32 [O, K*bits/32]."""
    q = np.ascontiguousarray(q, dtype=np.uint8)
    O, K = q.shape
    if (K * bits) % 32:
        raise ValueError("K*bits must be a multiple of 32")
    out = np.empty((O, K * bits // 8), dtype=np.uint8)
    step = max(1, (1 << 24) // max(1, K * bits))          # bound the temporary bit array
    shifts = np.arange(bits, dtype=np.uint8)
    for r0 in range(0, O, step):
        blk = q[r0:r0 + step]
        bitarr = ((blk[:, :, None] >> shifts) & 1).reshape(blk.shape[0], K * bits)
        out[r0:r0 + step] = np.packbits(bitarr, axis=1, bitorder="little")
    return out.view(np.uint32)


def round_to(values: np.ndarray, dtype: int):
    """(raw storage array, the stored values as fp32) for f32 / f16 / bf16 (round to nearest even)."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    if dtype == F32:
        return v, v
    if dtype == F16:
        h = v.astype(np.float16)
        return h.view(np.uint16), h.astype(np.float32)
    u = v.view(np.uint32).astype(np.uint64)
    raw = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return raw, (raw.astype(np.uint32) << 16).view(np.float32)


@dataclass
class SynthLayer:
    q: np.ndarray            # uint8 [O, K]
    packed: np.ndarray       # uint32 [O, K*bits/32]
    scales_raw: np.ndarray   # storage dtype [O, K/gs]
    biases_raw: np.ndarray
    scales: np.ndarray       # fp32 values as stored
    biases: np.ndarray
    bits: int
    gs: int
    scale_dtype: int


def make_layer(O: int, K: int, bits: int, gs: int, scale_dtype: int = F16, seed: int = 0, bias_noise: bool = False,
               keep_codes: bool = True) -> SynthLayer:
    g = np.random.default_rng(seed)
    q = g.integers(0, 1 << bits, size=(O, K), dtype=np.uint8)
    scale = (np.abs(g.standard_normal((O, K // gs), dtype=np.float32)) * np.float32(0.002) + np.float32(1e-4))
    s_raw, s_val = round_to(scale, scale_dtype)
    bias = -np.float32(1 << (bits - 1)) * s_val
    if bias_noise:
        bias = bias + g.standard_normal((O, K // gs), dtype=np.float32) * np.float32(1e-4)
    b_raw, b_val = round_to(bias.astype(np.float32), scale_dtype)
    packed = pack_codes(q, bits)
    return SynthLayer(q if keep_codes else None, packed, s_raw, b_raw, s_val, b_val, bits, gs, scale_dtype)


def make_layer_fast(O: int, K: int, bits: int, gs: int, scale_dtype: int = F16, seed: int = 0) -> SynthLayer:
    """The same distribution for layers too large to draw code by code (a vocabulary-sized head): uniform codes are
    uniform bits, so the packed words are drawn directly.  ``q`` is not kept."""
    g = np.random.default_rng(seed)
    packed = g.integers(0, 1 << 32, size=(O, K * bits // 32), dtype=np.uint32)
    scale = (np.abs(g.standard_normal((O, K // gs), dtype=np.float32)) * np.float32(0.002) + np.float32(1e-4))
    s_raw, s_val = round_to(scale, scale_dtype)
    b_raw, b_val = round_to((-np.float32(1 << (bits - 1)) * s_val).astype(np.float32), scale_dtype)
    return SynthLayer(None, packed, s_raw, b_raw, s_val, b_val, bits, gs, scale_dtype)


def make_activations(T: int, K: int, dtype: int = F16, seed: int = 1):
    """(raw storage array [T, K], values as fp32)."""
    g = np.random.default_rng(seed)
    return round_to(g.standard_normal((T, K), dtype=np.float32), dtype)
