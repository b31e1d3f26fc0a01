"""GPU parity tests of the tensor-core dequant-GEMM (tcgen05 / TMEM path), through the C ABI.

The GEMM takes 16-bit activations (the benchmark's prefill configuration: bf16 in, fp32 accumulate) and
feeds the tensor cores fp16 weights: w = scale*q + bias rounded once to fp16, a relative error of at most
2^-12 per weight, random in sign.  The oracle sees the same rounded activations, so what is compared is
that weight rounding plus the fp32 accumulation order.  Bars:

* benchmark value distributions (|w| ~ 0.01, |y| < 1): max |got-ref| / max(1,|ref|) < 1e-3 and normwise
  ||got-ref|| / ||ref|| < 1e-3;
* the reference fixture's much larger magnitudes (|w| ~ 0.3, |y| ~ 5-20): normwise < 5e-4 (= 2 * 2^-12);
  the element-wise metric, which divides the absolute error by max(1,|ref|) even where |ref| is small
  next to the row's terms, must stay < 1.5e-2.  (fp32 activations never take this path: they use the
  fp32 CUDA-core kernel and meet 1e-3 element-wise, tests/test_parity_gpu.py.)"""
import importlib

import numpy as np
import pytest
import torch

from helpers import DevLayer, as_dtype, run

pytestmark = pytest.mark.gpu

synth = importlib.import_module("mlx-runner_b200.synth")


def _ref(oracle, lay_or_fx, x_rounded, K, bits, gs, sdt, bias=None):
    return oracle.qmatmul(lay_or_fx.packed, lay_or_fx.scales_raw, lay_or_fx.biases_raw, sdt, x_rounded, K, bits, gs, bias=bias)


@pytest.mark.parametrize("x_dtype", [1, 2])
def test_gemm_is_selected_and_matches_oracle(mlxq, oracle, x_dtype):
    # one full tile, bf16 scales: fp16 operands hold the weights almost exactly
    O, K, T = 256, 512, 128
    fx = oracle.QuantFixture(O=O, K=K, bits=4, gs=64, scale_type=oracle.BF16, seed=5)
    layer = DevLayer.from_fixture(mlxq, fx)
    assert layer.linear.kernelFor(T, x_dtype, 0) == "qgemm"
    assert layer.linear.gemmTileTokens(T) == 128 and layer.linear.gemmTileTokens(4) == 0
    assert layer.linear.gemmTileTokens(129) == 256          # longer batches take the 128-row x 256-token tile
    x = oracle.RNG(77).floats(T * K).reshape(T, K)
    xr = as_dtype(x, x_dtype).float().cpu().numpy()
    got = run(layer, x, T, x_dtype=x_dtype)
    mlxq.streamStatus(None, 0)
    ref = fx.reference(xr)
    nrm = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
    assert nrm < 5e-4 and oracle.max_rel_err(got, ref) < 1.5e-2, f"x dtype {x_dtype}: normwise {nrm}"


@pytest.mark.parametrize("T,O,K,gs", [(17, 40, 512, 32), (33, 41, 576, 64), (517, 520, 576, 32), (96, 2050, 1024, 128),
                                      (300, 777, 4096, 64)])
def test_gemm_ragged_shapes(mlxq, oracle, T, O, K, gs):
    # tokens and rows that do not fill a tile, strided x / y with NaN padding, row bias, bf16 output too
    fx = oracle.QuantFixture(O=O, K=K, bits=4, gs=gs, scale_type=oracle.BF16, with_bias=True, seed=T + O)
    layer = DevLayer.from_fixture(mlxq, fx)
    x = oracle.RNG(T * 7 + 4).floats(T * K).reshape(T, K)
    xr = as_dtype(x, 2).float().cpu().numpy()
    ref = _ref(oracle, fx, xr, K, 4, gs, oracle.BF16, bias=fx.bias)
    assert layer.linear.kernelFor(T, 2, 0) == "qgemm"
    got = run(layer, x, T, x_dtype=2, x_stride=K + 8, y_stride=O + 3)
    nrm = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
    assert nrm < 5e-4 and oracle.max_rel_err(got, ref) < 1.5e-2, f"normwise {nrm}"
    got16 = run(layer, x, T, x_dtype=2, y_dtype=2, y_stride=O + 5)
    assert float(np.linalg.norm(got16 - ref) / np.linalg.norm(ref)) < 4e-3        # bf16 output rounding, 2^-9 per element
    mlxq.streamStatus(None, 0)


def test_gemm_baseline_distribution_fp16_scales(mlxq, oracle):
    # the prefill configuration's value distribution at reduced O (oracle cost), fp16 and bf16 scales
    O, K, T = 512, 4096, 256
    for sdt in (synth.F16, synth.BF16):
        lay = synth.make_layer(O, K, 4, 64, sdt, seed=9, bias_noise=True)
        layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, sdt, K)
        _, x = synth.make_activations(T, K, synth.BF16, seed=2)
        ref = oracle.qmatmul(lay.packed, lay.scales_raw, lay.biases_raw, sdt, x, K, 4, 64)
        got = run(layer, x, T, x_dtype=2)
        err = oracle.max_rel_err(got, ref)
        nrm = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
        assert err < 1e-3 and nrm < 1e-3, f"scales {sdt}: max-rel {err}, normwise {nrm}"


def test_gemm_fp16_scales_reference_fixture_magnitudes(mlxq, oracle):
    O, K, T = 384, 1024, 160
    fx = oracle.QuantFixture(O=O, K=K, bits=4, gs=64, scale_type=oracle.F16, seed=12)
    layer = DevLayer.from_fixture(mlxq, fx)
    x = oracle.RNG(13).floats(T * K).reshape(T, K)
    xr = as_dtype(x, 1).float().cpu().numpy()
    ref = fx.reference(xr)
    got = run(layer, x, T, x_dtype=1)
    nrm = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
    assert nrm < 5e-4 and oracle.max_rel_err(got, ref) < 1.5e-2


def test_gemm_token_outputs_do_not_depend_on_the_batch(mlxq, oracle):
    # KernelTests.swift:168-184 for the GEMM family: bit-identical rows whatever batch they ride in
    O, K = 2050, 1024
    fx = oracle.QuantFixture(O=O, K=K, bits=4, gs=64, seed=3)
    layer = DevLayer.from_fixture(mlxq, fx)
    x = oracle.RNG(11).floats(256 * K).reshape(256, K)
    full = run(layer, x, 256, x_dtype=2).view(np.uint32)
    for T in (17, 33, 96, 131):
        assert np.array_equal(run(layer, x[:T], T, x_dtype=2).view(np.uint32), full[:T]), f"T {T} vs T 256"


def test_gemm_round_trip_property_at_full_size(mlxq, oracle):
    # full prefill size (14336 x 4096, M = 2048): linearity in x, checked without the oracle --
    # W.(x1 + x2) = W.x1 + W.x2 for activations whose sum is exact in bf16 -- plus an oracle check on a
    # random sample of output rows.
    O, K, T = 14336, 4096, 2048
    lay = synth.make_layer(O, K, 4, 64, synth.BF16, seed=21, keep_codes=False)
    layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.BF16, K)
    g = np.random.default_rng(5)
    x1 = g.integers(-8, 9, size=(T, K)).astype(np.float32) / 8       # small dyadic values: sums stay exact in bf16
    x2 = g.integers(-8, 9, size=(T, K)).astype(np.float32) / 8
    y1, y2, y12 = run(layer, x1, T, x_dtype=2), run(layer, x2, T, x_dtype=2), run(layer, x1 + x2, T, x_dtype=2)
    assert oracle.max_rel_err(y12, y1 + y2) < 1e-4
    rows = np.sort(g.choice(O, size=64, replace=False))
    sub = oracle.qmatmul(lay.packed[rows], lay.scales_raw[rows], lay.biases_raw[rows], synth.BF16, x1[:128], K, 4, 64)
    assert oracle.max_rel_err(y1[:128][:, rows], sub) < 1e-3
    mlxq.streamStatus(None, 0)


def test_gemm_repeats_bit_for_bit_at_full_size(mlxq):
    # 14336 x 4096, M = 2048, twelve calls on the same inputs: the pipeline's hand-offs (TMA rings, tensor-memory A
    # ring, deferred epilogue) leave no room for timing to change a single bit.  Tensor-memory stores issued after the
    # lanes of a warp had polled a barrier one by one showed up here as a few rows of one tile differing.
    O, K, T = 14336, 4096, 2048
    lay = synth.make_layer(O, K, 4, 64, synth.BF16, seed=31, keep_codes=False)
    layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.BF16, K)
    _, xv = synth.make_activations(T, K, synth.BF16, seed=100)
    x = torch.from_numpy(xv).to("cuda").to(torch.bfloat16)
    ys = [torch.empty((T, O), dtype=torch.float32, device="cuda") for _ in range(2)]
    layer.linear.encode(None, x, K, ys[0], O, T)
    for call in range(12):
        layer.linear.encode(None, x, K, ys[1], O, T)
        torch.cuda.synchronize()
        differing = int((ys[1].view(torch.int32) != ys[0].view(torch.int32)).sum())
        assert differing == 0, f"call {call}: {differing} outputs differ from the first call's"
    mlxq.streamStatus(None, 0)


def _bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.int64)


@pytest.mark.parametrize("O,K", [(14336, 4096), (4096, 14336)])
def test_gemm_prefill_sizes_against_oracle(mlxq, oracle, O, K):
    # the prefill configuration at its own sizes: M = 128, 512, 8192 on both orientations (M = 2048 is covered above);
    # the oracle on a sample of rows x tokens.  fp32 output: the 1e-3 bar.  bf16 output: within one bf16 ulp of the
    # oracle rounded to bf16 (outputs so close to zero that an ulp is below the fp32 bar are held to that bar instead).
    lay = synth.make_layer(O, K, 4, 64, synth.BF16, seed=O % 97, keep_codes=False)
    layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.BF16, K)
    g = np.random.default_rng(K)
    rows = np.sort(g.choice(O, size=48, replace=False))
    for T in (128, 512, 8192):
        _, x = synth.make_activations(T, K, synth.BF16, seed=T)
        toks = np.sort(np.concatenate([np.arange(8), g.choice(np.arange(8, T), size=24, replace=False)]))
        ref = oracle.qmatmul(lay.packed[rows], lay.scales_raw[rows], lay.biases_raw[rows], synth.BF16, x[toks], K, 4, 64)
        assert layer.linear.kernelFor(T, 2, 0) == "qgemm"
        got = run(layer, x, T, x_dtype=2)[toks][:, rows]
        err = oracle.max_rel_err(got, ref)
        assert err < 1e-3, f"{O}x{K} T={T}: max relative error {err}"
        got16 = run(layer, x, T, x_dtype=2, y_dtype=2)[toks][:, rows]
        ulps = np.abs(_bf16_bits(got16) - _bf16_bits(ref))
        near_zero = np.abs(got16 - ref) <= 1e-3 * np.maximum(1.0, np.abs(ref))
        assert np.all((ulps <= 1) | near_zero), f"{O}x{K} T={T}: bf16 output off by {int(ulps[~near_zero].max())} ulps"
    mlxq.streamStatus(None, 0)


def test_prepared_table_changes_nothing(mlxq, oracle):
    # mlxq_linear_prepare builds the GEMM's scale/bias table ahead; a batch encoded while its stream is being captured
    # cannot keep a table and stages it per call.  All routes must give the same bits.
    O, K, T = 768, 2048, 160
    lay = synth.make_layer(O, K, 4, 64, synth.BF16, seed=77, bias_noise=True)
    _, xv = synth.make_activations(T, K, synth.BF16, seed=5)
    x = torch.from_numpy(xv).to("cuda").to(torch.bfloat16)
    outs = []
    for route in ("prepared", "first call builds it", "captured"):
        layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.BF16, K, name=route)
        y = torch.full((T, O), float("nan"), dtype=torch.float32, device="cuda")
        if route == "prepared":
            layer.linear.prepare(None)
        if route == "captured":
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                layer.linear.encode(torch.cuda.current_stream(), x, K, y, O, T)
            g.replay()
        else:
            layer.linear.encode(None, x, K, y, O, T)
        torch.cuda.synchronize()
        mlxq.streamStatus(None, 0)
        outs.append(y.cpu().numpy())
    ref = oracle.qmatmul(lay.packed, lay.scales_raw, lay.biases_raw, synth.BF16, xv, K, 4, 64)
    assert oracle.max_rel_err(outs[0], ref) < 1e-3
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    assert np.array_equal(outs[0].view(np.uint32), outs[2].view(np.uint32))
