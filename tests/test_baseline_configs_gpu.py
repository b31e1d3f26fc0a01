"""The benchmark configurations at full size, through the C ABI, against the CPU oracle.

Shapes: the vocabulary-sized head (151936 x 4096, 6- and 8-bit), the projections of a 36-layer 4096-wide
transformer with a 12288-wide gated MLP (fused q|k|v 6144 x 4096, o 4096 x 4096, fused gate|up 24576 x 4096,
down 4096 x 12288), the transposed sweep shapes (K = 11008, K = 14336) and every bit width x group size at full K.
The oracle is evaluated on a sample of rows (always including the first and the last block); the device error word
must stay clear."""
import importlib

import numpy as np
import pytest
import torch

from helpers import DevLayer, as_dtype, dev, run

pytestmark = pytest.mark.gpu

synth = importlib.import_module("mlx-runner_b200.synth")


def sample_rows(O, n=96, seed=0):
    g = np.random.default_rng(seed + O)
    mid = g.choice(np.arange(16, O - 16), size=min(n, O - 32), replace=False)
    return np.sort(np.concatenate([np.arange(16), mid, np.arange(O - 16, O)]))


def check_rows(oracle, lay, got, x, rows, label, tol=1e-3):
    ref = oracle.qmatmul(lay.packed[rows], lay.scales_raw[rows], lay.biases_raw[rows], lay.scale_dtype, x, lay.packed.shape[1] * 32 // lay.bits,
                         lay.bits, lay.gs)
    err = oracle.max_rel_err(got[:, rows], ref)
    assert err < tol, f"{label}: max relative error {err}"


@pytest.mark.parametrize("bits", [6, 8])
def test_vocabulary_head(mlxq, oracle, bits):
    # config 5: 151936 x 4096, group 64, fp16 hidden states, batches 1 to 16, fp32 logits
    O, K = 151936, 4096
    lay = synth.make_layer_fast(O, K, bits, 64, synth.F16, seed=50 + bits)
    layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.F16, K)
    rows = sample_rows(O, seed=bits)
    for T in (1, 4, 16):
        _, x = synth.make_activations(T, K, synth.F16, seed=T)
        got = run(layer, x, T, x_dtype=1)
        mlxq.streamStatus(None, 0)
        assert np.isfinite(got).all()
        check_rows(oracle, lay, got, x, rows, f"head b{bits} T={T}")


@pytest.mark.parametrize("T", [1, 8])
def test_transformer_projections(mlxq, oracle, T):
    # config 4: 4-bit group-64 projections of one layer; q|k|v and gate|up run as one fused launch each
    H, KV, FF = 4096, 1024, 12288
    _, x = synth.make_activations(T, H, synth.F16, seed=10 + T)

    def fused(parts_rows, K, seed, xin):
        lays = [synth.make_layer(r, K, 4, 64, synth.F16, seed=seed + i, keep_codes=False) for i, r in enumerate(parts_rows)]
        devs = [DevLayer(mlxq, l.packed, l.scales_raw, l.biases_raw, synth.F16, K, name=f"p{i}") for i, l in enumerate(lays)]
        total = sum(parts_rows)
        xd = as_dtype(xin, 1)
        yd = torch.full((T, total), float("nan"), dtype=torch.float32, device="cuda")
        mlxq.Linear.encodeFusedDecode(None, [d.linear for d in devs], xd, yd, xStride=K, yStride=total, T=T)
        torch.cuda.synchronize()
        mlxq.streamStatus(None, 0)
        got = yd.cpu().numpy()
        r0 = 0
        for i, (l, r) in enumerate(zip(lays, parts_rows)):
            rows = sample_rows(r, n=48, seed=seed + i)
            check_rows(oracle, l, got[:, r0:r0 + r], xin, rows, f"fused part {i} of {parts_rows} T={T}")
            r0 += r

    fused([H, KV, KV], H, 100, x)                     # q | k | v : 6144 x 4096
    fused([FF, FF], H, 200, x)                        # gate | up : 24576 x 4096
    for O, K, seed in [(H, H, 300), (H, FF, 400)]:    # o : 4096 x 4096, down : 4096 x 12288
        lay = synth.make_layer(O, K, 4, 64, synth.F16, seed=seed, keep_codes=False)
        layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.F16, K)
        _, xin = synth.make_activations(T, K, synth.F16, seed=seed + T)
        got = run(layer, xin, T, x_dtype=1)
        mlxq.streamStatus(None, 0)
        check_rows(oracle, lay, got, xin, sample_rows(O, n=48, seed=seed), f"{O}x{K} T={T}")


@pytest.mark.parametrize("K", [11008, 14336])
def test_transposed_sweep_shapes(mlxq, oracle, K):
    # 4096 x 11008 (config 2's second orientation) and 4096 x 14336 (config 3's), decode batches
    O = 4096
    for bits in (4, 3, 8):
        lay = synth.make_layer(O, K, bits, 64, synth.F16, seed=K + bits, keep_codes=False)
        layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.F16, K)
        rows = sample_rows(O, n=32, seed=K)
        for T in (1, 2, 8):
            _, x = synth.make_activations(T, K, synth.F16, seed=T)
            got = run(layer, x, T, x_dtype=1)
            mlxq.streamStatus(None, 0)
            check_rows(oracle, lay, got, x, rows, f"{O}x{K} b{bits} T={T}")


def test_every_width_and_group_at_full_k(mlxq, oracle):
    # config 2: all eighteen (bits, group) pairs at K = 4096, batches 1, 2, 4, 8; 6- and 8-bit also at 12 and 16
    O, K = 688, 4096
    for bits in (2, 3, 4, 5, 6, 8):
        for gs in (32, 64, 128):
            lay = synth.make_layer(O, K, bits, gs, synth.F16, seed=bits * 7 + gs, keep_codes=False)
            layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.F16, K)
            batches = (1, 2, 4, 8) + ((12, 16) if bits in (6, 8) and gs == 64 else ())
            for T in batches:
                _, x = synth.make_activations(T, K, synth.F16, seed=T)
                ref = oracle.qmatmul(lay.packed, lay.scales_raw, lay.biases_raw, synth.F16, x, K, bits, gs)
                got = run(layer, x, T, x_dtype=1)
                err = oracle.max_rel_err(got, ref)
                assert err < 1e-3, f"bits {bits} gs {gs} T {T}: max relative error {err}"
    mlxq.streamStatus(None, 0)
