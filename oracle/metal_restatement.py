"""A second, independent CPU restatement of the quantized-linear arithmetic.  TEST INFRASTRUCTURE ONLY.

``oracle.py`` / ``mlxq_oracle.c`` follow the reference's *Swift test code* (KernelTests.swift, SieveImport.swift).
This file follows the *Metal kernel text* instead, in numpy only and without looking at the other restatement:

* ``unpack8``   -- Sources/MLXEngine/Kernels.swift:34-55: eight codes from BITS bytes; a u32 load for 4 bits, byte
                   loads for 8 bits, a u16 load for 2 bits, and for 3/5/6 bits a 64-bit value assembled from BITS
                   bytes and shifted by multiples of BITS.
* ``qmm``       -- Sources/MLXEngine/Kernels.swift:60-113: lane l of a 32-wide simdgroup walks the 8-code chunks
                   l, l + 32, ...; per chunk ``acc += s * (dot(qa, xa) + dot(qb, xb)) + b * dot(xa + xb, 1)`` in
                   fp32, then ``simd_sum`` over the lanes.

Two checkers written from different parts of the reference must agree (tests/test_oracle.py): bit for bit on the
codes, and to fp32 summation noise on the outputs.  Nothing in the product imports this module.
"""
from __future__ import annotations

import numpy as np


def _f32_to(raw: np.ndarray, dtype: int) -> np.ndarray:
    """Stored scales / biases -> fp32 (0 = f32, 1 = f16 bits, 2 = bf16 bits)."""
    if dtype == 0:
        return np.asarray(raw, dtype=np.float32)
    u = np.asarray(raw, dtype=np.uint16)
    if dtype == 1:
        return u.view(np.float16).astype(np.float32)
    return (u.astype(np.uint32) << 16).view(np.float32)


def unpack8(row_bytes: np.ndarray, bits: int) -> np.ndarray:
    """Codes of packed rows: ``row_bytes`` u8 [..., K*bits/8] -> u8 [..., K], chunk by chunk as Kernels.swift:34-55."""
    b = np.ascontiguousarray(row_bytes, dtype=np.uint8)
    lead, nbytes = b.shape[:-1], b.shape[-1]
    chunks = nbytes // bits
    c = b.reshape(lead + (chunks, bits))
    if bits == 4:
        w = c.astype(np.uint32)
        w = w[..., 0] | (w[..., 1] << 8) | (w[..., 2] << 16) | (w[..., 3] << 24)          # *(device const uint*)p
        q = np.stack([(w >> (4 * i)) & 0xF for i in range(8)], axis=-1)
    elif bits == 8:
        q = c                                                                           # uchar4 lo, hi
    elif bits == 2:
        w = c[..., 0].astype(np.uint32) | (c[..., 1].astype(np.uint32) << 8)            # *(device const ushort*)p
        q = np.stack([(w >> (2 * i)) & 3 for i in range(8)], axis=-1)
    else:
        v = np.zeros(lead + (chunks,), dtype=np.uint64)
        for i in range(bits):
            v |= c[..., i].astype(np.uint64) << np.uint64(8 * i)                          # v |= ulong(p[i]) << (8 * i)
        m = np.uint64((1 << bits) - 1)
        q = np.stack([(v >> np.uint64(i * bits)) & m for i in range(8)], axis=-1)
    return q.astype(np.uint8).reshape(lead + (chunks * 8,))


def qmm(packed: np.ndarray, scales_raw: np.ndarray, biases_raw: np.ndarray, sdtype: int, x: np.ndarray, K: int, bits: int,
        gs: int) -> np.ndarray:
    """y [T, O] fp32 with the kernel's own order of operations (fp32 throughout, 32 lanes, chunk stride 32)."""
    rows = np.ascontiguousarray(packed).view(np.uint8).reshape(packed.shape[0], -1)
    O = rows.shape[0]
    x = np.asarray(x, dtype=np.float32).reshape(-1, K)
    T = x.shape[0]
    chunks = K // 8
    q = unpack8(rows, bits).astype(np.float32).reshape(O, chunks, 8)
    s = _f32_to(scales_raw, sdtype).reshape(O, K // gs)
    b = _f32_to(biases_raw, sdtype).reshape(O, K // gs)
    grp = (np.arange(chunks) * 8) // gs                                                    # g = k / p.gs
    sc, bc = s[:, grp], b[:, grp]                                                          # [O, chunks]
    xc = x.reshape(T, chunks, 8)
    xs = ((xc[..., 0:4] + xc[..., 4:8]) * np.float32(1.0)).astype(np.float32)
    xs = ((xs[..., 0] + xs[..., 1]) + (xs[..., 2] + xs[..., 3])).astype(np.float32)        # dot(xa + xb, float4(1))
    y = np.zeros((T, O), dtype=np.float32)
    lanes = 32
    pad = (-chunks) % lanes
    for t in range(T):
        pa = q[..., 0:4] * xc[t][None, :, 0:4]
        pb = q[..., 4:8] * xc[t][None, :, 4:8]
        da = ((pa[..., 0] + pa[..., 1]) + (pa[..., 2] + pa[..., 3])).astype(np.float32)    # dot(qa, xa)
        db = ((pb[..., 0] + pb[..., 1]) + (pb[..., 2] + pb[..., 3])).astype(np.float32)    # dot(qb, xb)
        term = (sc * (da + db) + bc * xs[t][None, :]).astype(np.float32)                   # [O, chunks]
        if pad:
            term = np.concatenate([term, np.zeros((O, pad), dtype=np.float32)], axis=1)
        per_turn = term.reshape(O, -1, lanes)                                              # chunk c -> (turn c // 32, lane c % 32)
        acc = np.zeros((O, lanes), dtype=np.float32)
        for j in range(per_turn.shape[1]):
            acc = (acc + per_turn[:, j, :]).astype(np.float32)                             # acc[r][t] += ...
        # simd_sum: a butterfly over the 32 lanes
        v = acc
        w = lanes
        while w > 1:
            w //= 2
            v = (v[:, :w] + v[:, w:2 * w]).astype(np.float32)
        y[t] = v[:, 0]
    return y
