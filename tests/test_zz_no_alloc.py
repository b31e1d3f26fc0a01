"""The allocation-free forward (`mlxq_linear_forward_static`) against the ordinary one, through the C ABI.

Who needs it: a host that must not allocate device memory while it runs -- a serving loop that has handed
every free byte to its KV cache, or one that cannot afford to enter the CUDA allocator (and its possible
device synchronisation) inside its latency budget.  The ordinary GEMM stages an fp16 copy of the
activations in pool memory; this entry point stages it in a fixed 32 MiB array inside the library.

The file is named so that pytest collects it last: a run that stops at the first failure has already run
every other test.  It passes on its own in a fresh process and after the rest of the suite."""
import importlib

import numpy as np
import pytest
import torch

from helpers import DevLayer, TORCH_DT

pytestmark = pytest.mark.gpu

synth = importlib.import_module("mlx-runner_b200.synth")


def _forward(layer, x_dev, T, static):
    lin = layer.linear
    y = torch.full((T, lin.outDim), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    held = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    (lin.encodeStatic if static else lin.encode)(None, x_dev, lin.inDim, y, lin.outDim, T)
    torch.cuda.synchronize()
    if static:
        assert torch.cuda.memory_allocated() == held       # nothing of torch's was allocated by the call either
        # the device's free bytes see what torch's counter cannot: a cudaMalloc or a pool growing inside the library
        assert torch.cuda.mem_get_info()[0] == free_before
    return y.cpu().numpy()


def test_static_forward_matches_the_allocating_one_twice_in_a_row(mlxq, oracle):
    O, K, T = 512, 2048, 192
    lay = synth.make_layer(O, K, 4, 64, synth.BF16, seed=31, bias_noise=True)
    layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.BF16, K)
    assert layer.linear.kernelFor(T, mlxq.BF16, mlxq.F32) == "qgemm"       # the path that needs scratch memory
    for call in range(2):                                                   # the array keeps the last call's contents
        _, xv = synth.make_activations(T, K, synth.BF16, seed=100 + call)
        x_dev = torch.from_numpy(xv).to("cuda").to(TORCH_DT[2])
        want = _forward(layer, x_dev, T, static=False)
        got = _forward(layer, x_dev, T, static=True)
        mlxq.streamStatus(None, 0)
        assert np.isfinite(got).all()
        # same kernel, same staged values: the two entry points agree to the last bit, far inside the 1e-3 bar
        assert oracle.max_rel_err(got, want) < 1e-3
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        ref = oracle.qmatmul(lay.packed, lay.scales_raw, lay.biases_raw, synth.BF16, xv, K, 4, 64)
        assert oracle.max_rel_err(got, ref) < 1e-3


def test_static_forward_rejects_batches_beyond_the_array(mlxq):
    K = 4096
    lay = synth.make_layer(256, K, 4, 64, synth.BF16, seed=5, keep_codes=False)
    layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.BF16, K)
    T = mlxq._lib.STATIC_SCRATCH_BYTES // (2 * K) + 1                        # one token too many
    x = torch.zeros((T, K), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((T, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(mlxq.InvalidArgument, match="static scratch"):
        layer.linear.encodeStatic(None, x, K, y, 256, T)
    layer.linear.encodeStatic(None, x, K, y, 256, T - 1)                     # the largest batch that fits
    mlxq.streamStatus(None, 0)


def test_static_forward_rejects_layers_whose_table_exceeds_the_array(mlxq):
    # the staged scale/bias table takes out_dim * in_dim / 8 bytes: 36864 x 4096 needs 18 MiB, the array has 16
    O, K, T = 36864, 4096, 32
    w = torch.zeros((O, K // 8), dtype=torch.int32, device="cuda")
    s = torch.ones((O, K // 64), dtype=torch.bfloat16, device="cuda")
    lin = mlxq.Linear(w, s, s, None, inDim=K, name="too_tall")
    assert lin.kernelFor(T, mlxq.BF16, mlxq.F32) == "qgemm"
    x = torch.zeros((T, K), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((T, O), dtype=torch.float32, device="cuda")
    with pytest.raises(mlxq.InvalidArgument, match="scale table"):
        lin.encodeStatic(None, x, K, y, O, T)
    lin.encode(None, x, K, y, O, T)                                          # the allocating entry point takes it
    mlxq.streamStatus(None, 0)


def test_static_forward_small_batches_use_no_scratch(mlxq, oracle):
    fx = oracle.QuantFixture(O=64, K=512, bits=6, gs=64, seed=4)
    layer = DevLayer.from_fixture(mlxq, fx)
    x = oracle.RNG(2).floats(3 * 512).reshape(3, 512)
    x_dev = torch.from_numpy(x).to("cuda")
    got = _forward(layer, x_dev, 3, static=True)
    assert oracle.max_rel_err(got, fx.reference(x)) < 1e-3
