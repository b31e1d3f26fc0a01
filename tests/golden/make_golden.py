"""Writes tests/golden/qlinear_cases.npz: small known-answer cases of the quantized-linear path.

The reference engine is Swift + Metal and cannot run on the machines these tests run on, so the vectors come
from the CPU restatement of its algorithm (oracle/, pinned against the reference's own known-answer material in
tests/test_oracle.py) at the moment this file was generated.  They pin BOTH sides from then on: the oracle
must keep reproducing them bit for bit (tests/test_oracle.py) and the CUDA kernels must match them
(tests/test_parity_gpu.py).

Every case mirrors QuantFixture of the reference's KernelTests.swift:48-114 (same xorshift stream, same
packing, same two-rounding dense weights, double accumulation): for each bit width and group size,
    q       uint8  [O, K]          the codes
    packed  uint8  [O, K*bits/8]   MLX little-endian bit stream (3/5/6-bit codes straddle words)
    scales  uint16 [O, K/gs]       fp16 or bf16 storage bits
    biases  uint16 [O, K/gs]
    bias    uint16 [O]             row bias storage bits (cases with one)
    x       fp32   [T, K]
    y       fp32   [T, O]          reference output

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402

CASES = [  # bits, gs, O, K, T, scale type, row bias, seed
    (b, gs, 24, 256, 3, oracle.F16 if (b + gs) % 3 else oracle.BF16, b in (3, 6), 100 + b * 7 + gs)
    for b in (2, 3, 4, 5, 6, 8) for gs in (32, 64, 128)
]


def build():
    out = {}
    names = []
    for bits, gs, O, K, T, sdt, with_bias, seed in CASES:
        fx = oracle.QuantFixture(O=O, K=K, bits=bits, gs=gs, scale_type=sdt, with_bias=with_bias, seed=seed)
        x = oracle.RNG(seed + 1).floats(T * K).reshape(T, K).astype(np.float32)
        name = f"b{bits}_g{gs}"
        names.append(name)
        out[name + "_meta"] = np.array([bits, gs, O, K, T, sdt, int(with_bias), seed], dtype=np.int64)
        out[name + "_q"] = fx.q
        out[name + "_packed"] = fx.packed
        out[name + "_scales"] = fx.scales_raw
        out[name + "_biases"] = fx.biases_raw
        if with_bias:
            out[name + "_bias"] = fx.bias_raw
        out[name + "_x"] = x
        out[name + "_y"] = fx.reference(x)
    out["names"] = np.array(names)
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qlinear_cases.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
