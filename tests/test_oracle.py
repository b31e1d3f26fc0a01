"""Pins the CPU oracle against the literal known-answer material the reference's tests hold, and against
an independent restatement of the packer.  No GPU."""
import struct

import numpy as np
import pytest


def test_half_to_float_matches_ieee_patterns(oracle):
    # Tests/MLXEngineTests/EngineTests.swift:213 -- halfToFloat(bits) == Float(Float16(bitPattern: bits))
    for bits in [0x0000, 0x8000, 0x3C00, 0xBC00, 0x3555, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0xFBFF, 0x7C00, 0xFC00, 0x1234,
                 0xABCD]:
        want = np.array([bits], dtype=np.uint16).view(np.float16).astype(np.float32)[0]
        got = oracle.half_to_float(bits)
        assert struct.pack("<f", got) == struct.pack("<f", want), hex(bits)
    assert np.isnan(oracle.half_to_float(0x7E00))


def test_half_bits_round_trip(oracle):
    # Tests/MLXEngineTests/SieveTests.swift:113-126
    for v in [0.0, -0.0, 1.0, -1.0, 0.1, 65504.0, 1e-5, 6e-8, 1e9, -1e9, float("inf")]:
        h = oracle.half_to_float(oracle.float_to_half(v))
        if abs(v) > 65520:
            assert np.isinf(h) and (h > 0) == (v > 0)
        else:
            assert abs(h - np.float32(v)) <= max(abs(v) * 0.0005, 3e-8)
    rng = oracle.RNG(3)
    for _ in range(10000):
        bits = rng.next() & 0xFFFF
        f = oracle.half_to_float(bits)
        if np.isnan(f):
            continue
        assert oracle.float_to_half(f) == bits     # every half value survives float -> half exactly


def test_float_to_half_is_ieee_rne(oracle):
    # halfBits is round-to-nearest-even, so numpy's float16 cast must agree on arbitrary floats.
    g = np.random.default_rng(0)
    vals = np.concatenate([g.normal(size=4000), g.normal(size=2000) * 1e-5, g.normal(size=2000) * 3e4,
                           [65519.9, 65520.0, 5.96e-8, 2.98e-8, 2.99e-8]]).astype(np.float32)
    want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.float_to_half(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)


def test_xorshift_stream(oracle):
    # KernelTests.swift:8-14, written out independently in Python integers.
    s, mask = 7, (1 << 64) - 1
    rng = oracle.RNG(7)
    for _ in range(100):
        s ^= (s << 13) & mask
        s ^= s >> 7
        s ^= (s << 17) & mask
        assert rng.next() == s


def _pack_bitwise(q, bits):
    """KernelTests.swift:34-43 in pure Python: one bit at a time."""
    out = bytearray((len(q) * bits + 7) // 8)
    for i, v in enumerate(q):
        for b in range(bits):
            if (int(v) >> b) & 1:
                bit = i * bits + b
                out[bit // 8] |= 1 << (bit % 8)
    return bytes(out)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_pack_unpack_round_trip(oracle, bits):
    g = np.random.default_rng(bits)
    q = g.integers(0, 1 << bits, size=(5, 96), dtype=np.uint8)
    packed = oracle.pack(q, bits)
    assert packed.shape == (5, 96 * bits // 8)
    for r in range(5):
        assert packed[r].tobytes() == _pack_bitwise(q[r], bits)
    assert np.array_equal(oracle.pack_fast(q, bits), packed)
    assert np.array_equal(oracle.unpack(packed, 96, bits), q)
    # reading the stream as little-endian u32 words gives the same codes: code k = bits [k*b, (k+1)*b)
    words = packed.view(np.uint32)
    for r in range(5):
        big = int.from_bytes(words[r].tobytes(), "little")
        assert [(big >> (k * bits)) & ((1 << bits) - 1) for k in range(96)] == q[r].tolist()


def test_four_bit_word_layout(oracle):
    # word w holds codes 8w..8w+7 with code 8w in the low nibble
    q = np.arange(16, dtype=np.uint8).reshape(1, 16)
    words = oracle.pack(q, 4).view(np.uint32)[0]
    assert words[0] == 0x76543210 and words[1] == 0xFEDCBA98


def test_quantize4_dequantize_round_trip(oracle):
    # Tests/MLXEngineTests/SieveTests.swift:288-306
    V, r = 300, 128
    rng = oracle.RNG(9)
    orig = np.empty(V * r, dtype=np.float32)
    for i in range(V * r):
        # RNG.signed(): uniform in [-1, 1) from the same stream; the bound below does not depend on its exact form
        orig[i] = rng.float(-1.0, 1.0) * (1 + (i % 7))
    s = orig.reshape(V, r).copy()
    codes, scales, biases = oracle.quantize4(s)
    read = oracle.dequantize(codes.view(np.uint8).reshape(V, -1), scales, biases, oracle.F16, r, 4, 64)
    o2 = orig.reshape(V, r)
    assert np.all(np.abs(read - s) <= 1e-5 * np.maximum(1, np.abs(s)))
    for g in range(r // 64):
        blk = o2[:, g * 64:(g + 1) * 64]
        step = (blk.max(axis=1) - blk.min(axis=1)) / 15
        ok = np.abs(s[:, g * 64:(g + 1) * 64] - blk) <= step[:, None] * 0.51 + 0.002 * np.maximum(1, np.abs(blk))
        assert ok.all()


def test_use_gemm64_truth_table(oracle):
    # KernelTests.swift:153-156 and :179
    for T, O, big in [(64, 41, False), (128, 41, False), (517, 41, False), (96, 2050, False), (128, 2050, True),
                      (517, 520, True), (256, 2050, True)]:
        assert oracle.use_gemm64(T, O) == big, (T, O)


def test_dense_reference_matches_numpy(oracle):
    fx = oracle.QuantFixture(O=12, K=128, bits=5, gs=32, scale_type=oracle.BF16, with_bias=True, seed=11)
    x = oracle.RNG(5).floats(3 * 128).reshape(3, 128)
    ref = fx.reference(x)
    want = (fx.dense.astype(np.float64) @ x.astype(np.float64).T).T.astype(np.float32) + fx.bias[None, :]
    assert np.allclose(ref, want, rtol=0, atol=1e-6)
    # the fused unpack+dequant+dot path is the same numbers
    y2 = oracle.qmatmul(fx.packed, fx.scales_raw, fx.biases_raw, fx.scale_type, x, 128, 5, 32, bias=fx.bias)
    assert np.array_equal(y2, ref)
    # and dequantize() is the fixture's dense table
    d = oracle.dequantize(fx.packed, fx.scales_raw, fx.biases_raw, fx.scale_type, 128, 5, 32)
    assert np.array_equal(d, fx.dense)


def test_bf16_storage(oracle):
    v = np.array([1.0, 1.00390625, 0.1, -3.14159, 1e-3], dtype=np.float32)
    raw_t, back_t = oracle.store(v, oracle.BF16, bf16_truncate=True)
    assert np.array_equal(raw_t, (v.view(np.uint32) >> 16).astype(np.uint16))        # KernelTests.swift:45
    raw_r, back_r = oracle.store(v, oracle.BF16)
    import torch
    assert np.array_equal(raw_r.view(np.int16), torch.from_numpy(v).to(torch.bfloat16).view(torch.int16).numpy())


def test_act_mul_values(oracle):
    g = np.array([-3.0, -0.5, 0.0, 0.7, 2.5], dtype=np.float32)
    u = np.array([1.0, -2.0, 3.0, 0.5, 1.5], dtype=np.float32)
    silu = g / (1 + np.exp(-g.astype(np.float64))) * u
    assert np.allclose(oracle.act_mul(0, g, u), silu, atol=1e-6)
    gelu_t = 0.5 * g * (1 + np.tanh(0.7978845608 * (g + 0.044715 * g ** 3))) * u     # KernelTests.swift:210
    assert np.allclose(oracle.act_mul(1, g, u), gelu_t, atol=1e-6)
    from math import erf
    gelu_e = np.array([0.5 * a * (1 + erf(a / np.sqrt(2))) for a in g]) * u
    assert np.allclose(oracle.act_mul(2, g, u), gelu_e, atol=1e-6)


def test_oracle_reproduces_the_committed_golden_cases(oracle):
    # tests/golden/qlinear_cases.npz pins the oracle at the state that was checked against the reference's
    # known-answer material: packing, unpacking and the dense double-accumulate reference, bit for bit
    import golden_cases
    cases = golden_cases.load()
    assert len(cases) == 18
    for c in cases:
        assert np.array_equal(oracle.pack(c.q, c.bits), c.packed), c.name
        assert np.array_equal(oracle.unpack(c.packed, c.K, c.bits), c.q), c.name
        fx = oracle.QuantFixture(O=c.O, K=c.K, bits=c.bits, gs=c.gs, scale_type=c.sdt, with_bias=c.bias is not None, seed=c.seed)
        assert np.array_equal(fx.scales_raw, c.scales) and np.array_equal(fx.biases_raw, c.biases), c.name
        assert np.array_equal(fx.reference(c.x).view(np.uint32), c.y.view(np.uint32)), c.name
        # the fused form the kernels implement (scale * sum(q x) + bias * sum(x)) agrees with it to 1e-3
        y2 = oracle.qmatmul(c.packed, c.scales, c.biases, c.sdt, c.x, c.K, c.bits, c.gs,
                            bias=None if c.bias is None else fx.bias)
        assert oracle.max_rel_err(y2, c.y) < 1e-3, c.name


def test_two_independent_restatements_agree(oracle):
    # oracle/ follows the reference's Swift test code; oracle/metal_restatement.py was written from the Metal
    # kernel text (unpack8, Kernels.swift:34-55; qmm, Kernels.swift:60-113).  Codes must agree bit for bit; outputs
    # to fp32 summation noise (the kernel text accumulates in fp32 over 32 lanes, the Swift oracle in double):
    # max |a - b| / max(1, |b|) < 2e-5, fifty times inside the 1e-3 bar the kernels are held to.
    import importlib
    import golden_cases
    from oracle import metal_restatement as mr
    for c in golden_cases.load():
        rows = np.ascontiguousarray(c.packed).view(np.uint8).reshape(c.O, -1)
        codes = mr.unpack8(rows, c.bits)
        assert np.array_equal(codes, c.q), c.name
        assert np.array_equal(codes, oracle.unpack(c.packed, c.K, c.bits)), c.name
        y = mr.qmm(c.packed, c.scales, c.biases, c.sdt, c.x, c.K, c.bits, c.gs)
        ref = oracle.qmatmul(c.packed, c.scales, c.biases, c.sdt, c.x, c.K, c.bits, c.gs)
        assert oracle.max_rel_err(y, ref) < 2e-5, c.name
    # the benchmark's own generators (BASELINE distributions) at full K
    synth = importlib.import_module("mlx-runner_b200.synth")
    for bits, gs, sdt in [(4, 64, synth.F16), (6, 64, synth.F16), (8, 64, synth.F16), (3, 32, synth.BF16), (5, 128, synth.BF16),
                          (2, 64, synth.F16)]:
        lay = synth.make_layer(48, 4096, bits, gs, sdt, seed=bits)
        rows = np.ascontiguousarray(lay.packed).view(np.uint8).reshape(48, -1)
        assert np.array_equal(mr.unpack8(rows, bits), lay.q)
        _, x = synth.make_activations(3, 4096, synth.F16, seed=bits)
        y = mr.qmm(lay.packed, lay.scales_raw, lay.biases_raw, sdt, x, 4096, bits, gs)
        ref = oracle.qmatmul(lay.packed, lay.scales_raw, lay.biases_raw, sdt, x, 4096, bits, gs)
        assert oracle.max_rel_err(y, ref) < 2e-5, (bits, gs)


def test_block_maxima_and_greedy_token(oracle):
    # sample_blocks / the argmax branch of sample_token (Kernels.swift:2339-2377): against plain numpy on rows with a
    # ragged last block, equal maxima (the lowest index wins), NaNs (never win) and an all -inf block (reports none)
    g = np.random.default_rng(5)
    x = g.standard_normal((3, 256 * 3 + 77)).astype(np.float32)
    x[0, 10] = x[0, 700] = 50.0                     # equal maxima in two blocks
    x[1, 5] = np.nan
    x[1, 256:512] = -np.inf
    x[2, 800] = 7.5
    bmax, barg = oracle.block_max(x, index_base=1000)
    nb = bmax.shape[1]
    assert nb == 4
    for t in range(3):
        for b in range(nb):
            seg = x[t, b * 256:(b + 1) * 256]
            if np.all(np.isneginf(seg) | np.isnan(seg)):
                assert barg[t, b] == oracle.SELECT_NONE and np.isneginf(bmax[t, b])
            else:
                assert bmax[t, b] == np.nanmax(seg)
                assert barg[t, b] == 1000 + b * 256 + int(np.nanargmax(seg))
    tok, val = oracle.block_argmax(bmax, barg)
    assert tok.tolist() == [1000 + 10, 1000 + int(np.nanargmax(x[1])), 1000 + 800]
    assert val.tolist() == [50.0, float(np.nanmax(x[1])), 7.5]
