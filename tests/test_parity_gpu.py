"""GPU parity tests: the CUDA layer, called through the C ABI, against the CPU oracle on the same seeded
inputs.  The matrix mirrors the reference's kernel tests (Tests/MLXEngineTests/KernelTests.swift:126-297):
same shapes, same xorshift seeds, same error metric (max |got-ref| / max(1,|ref|)).

Tolerance: 1e-3 (the bar this build states; the reference's own bar is 2e-3), 5e-3 for the gated output
(as KernelTests.swift:211) and 1e-5 for the dequantising lookup (KernelTests.swift:295).  Unpacked codes
must be bit-exact."""
import importlib

import numpy as np
import pytest
import torch

from helpers import DevLayer, as_dtype, dev, run

synth = importlib.import_module("mlx-runner_b200.synth")

pytestmark = pytest.mark.gpu

TOL = 1e-3


def close(oracle, got, ref, label, tol=TOL):
    err = oracle.max_rel_err(got, ref)
    assert err < tol, f"{label}: max relative error {err}"


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_quantized_matches_reference(mlxq, oracle, bits):
    # KernelTests.swift:128-146
    K, O = 512, 40
    for gs in (32, 64, 128):
        for st in (oracle.F16, oracle.BF16):
            fx = oracle.QuantFixture(O=O, K=K, bits=bits, gs=gs, scale_type=st)
            layer = DevLayer.from_fixture(mlxq, fx)
            for T in (1, 2, 3, 4, 5, 8, 9, 15, 16, 17, 33):
                x = oracle.RNG(T * 31 + bits).floats(T * K).reshape(T, K)
                close(oracle, run(layer, x, T), fx.reference(x), f"bits {bits} gs {gs} st {st} T {T}")


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_unpacked_codes_are_bit_exact(mlxq, oracle, bits):
    fx = oracle.QuantFixture(O=37, K=544, bits=bits, gs=32, seed=bits + 100)
    layer = DevLayer.from_fixture(mlxq, fx)
    out = torch.zeros((37, 544), dtype=torch.uint8, device="cuda")
    layer.linear.unpackCodes(None, out)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.array_equal(got, fx.q)
    assert np.array_equal(got, oracle.unpack(fx.packed, 544, bits))


@pytest.mark.parametrize("bits", [3, 4, 8])
def test_prefill_tiles_match_reference(mlxq, oracle, bits):
    # KernelTests.swift:150-164: long batches, odd O, K % 64 != 0
    for T, O, K in [(64, 41, 1056), (128, 41, 544), (517, 41, 544), (96, 2050, 544), (128, 2050, 544), (517, 520, 544)]:
        fx = oracle.QuantFixture(O=O, K=K, bits=bits, gs=32, seed=T + O)
        layer = DevLayer.from_fixture(mlxq, fx)
        x = oracle.RNG(T * 7 + bits).floats(T * K).reshape(T, K)
        ref = oracle.qmatmul(fx.packed, fx.scales_raw, fx.biases_raw, fx.scale_type, x, K, bits, 32)
        close(oracle, run(layer, x, T), ref, f"bits {bits} T {T} O {O} K {K}")


def test_batches_agree_bitwise(mlxq, oracle):
    # KernelTests.swift:168-184: a token's output does not depend on the batch it was computed in
    # (checked within each kernel family: the matvec up to 16 tokens, the GEMM above).
    O, K = 2050, 1024
    fx = oracle.QuantFixture(O=O, K=K, bits=4, gs=64, seed=3)
    layer = DevLayer.from_fixture(mlxq, fx)
    x = oracle.RNG(11).floats(256 * K).reshape(256, K)
    full16 = run(layer, x[:16], 16).view(np.uint32)
    for T in (9, 12):
        assert np.array_equal(run(layer, x[:T], T).view(np.uint32), full16[:T]), f"T {T} vs T 16"
    # and a decode call is reproducible bit for bit (sums are formed in a fixed order)
    assert np.array_equal(run(layer, x[:1], 1).view(np.uint32), run(layer, x[:1], 1).view(np.uint32))
    full = run(layer, x, 256).view(np.uint32)
    for T in (33, 96, 131):
        assert np.array_equal(run(layer, x[:T], T).view(np.uint32), full[:T]), f"T {T} vs T 256"


@pytest.mark.parametrize("K", [1152, 1536, 2304, 2560, 896, 1664, 6912])
def test_four_bit_decode_with_partial_pass(mlxq, oracle, K):
    # KernelTests.swift:188-199
    O = 24
    for gs in (32, 64, 128):
        if K % gs:
            continue
        fx = oracle.QuantFixture(O=O, K=K, bits=4, gs=gs, seed=K)
        layer = DevLayer.from_fixture(mlxq, fx)
        x = oracle.RNG(K).floats(K).reshape(1, K)
        close(oracle, run(layer, x, 1), fx.reference(x), f"K {K} gs {gs}")


def test_gated_output_matches_reference(mlxq, oracle):
    # KernelTests.swift:202-212: y = act(x . W^T) * e, tanh-GELU, e read at an offset
    O, K = 40, 1536
    fx = oracle.QuantFixture(O=O, K=K, bits=4, gs=64, seed=21)
    layer = DevLayer.from_fixture(mlxq, fx)
    rng = oracle.RNG(6)
    x = rng.floats(K) * np.float32(4)
    e = rng.floats(2 * O)
    xd, ed = as_dtype(x, 0), as_dtype(e, 0)
    for act in (0, 1, 2):
        yd = torch.zeros(O, dtype=torch.float32, device="cuda")
        layer.linear.encodeGated(None, xd, yd, ed[O:], act)
        torch.cuda.synchronize()
        g = fx.reference(x.reshape(1, K))[0]
        if act == 1:
            ref = 0.5 * g * (1 + np.tanh(np.float32(0.7978845608) * (g + np.float32(0.044715) * g * g * g))) * e[O:]
            close(oracle, yd.cpu().numpy(), ref.astype(np.float32), "gated output (formula of the reference test)", 5e-3)
        close(oracle, yd.cpu().numpy(), oracle.act_mul(act, g, e[O:]), f"gated output act {act}", 5e-3)


def _fused_parts(mlxq, oracle, K):
    fxs = [oracle.QuantFixture(O=o, K=K, bits=4, gs=64, with_bias=True, seed=s) for o, s in [(64, 1), (16, 2), (16, 3)]]
    return fxs, [DevLayer.from_fixture(mlxq, f, name=f"p{i}") for i, f in enumerate(fxs)]


def test_fused_decode_with_bias_matches_separate(mlxq, oracle):
    # KernelTests.swift:214-227
    K = 256
    fxs, layers = _fused_parts(mlxq, oracle, K)
    lins = [l.linear for l in layers]
    assert mlxq.Linear.fusable(lins)
    x = oracle.RNG(99).floats(K)
    yd = torch.zeros(96, dtype=torch.float32, device="cuda")
    mlxq.Linear.encodeFusedDecode(None, lins, as_dtype(x, 0), yd)
    torch.cuda.synchronize()
    ref = np.concatenate([f.reference(x.reshape(1, K))[0] for f in fxs])
    close(oracle, yd.cpu().numpy(), ref, "fused q/k/v")


@pytest.mark.parametrize("K", [512, 1152, 544, 1056])
def test_small_batch_four_bit_matches_reference(mlxq, oracle, K):
    # KernelTests.swift:232-252: strided x / y, NaN padding that must not be read, rows that end inside a warp
    for O, gs in [(40, 64), (44, 32), (40, 128)]:
        if K % gs:
            continue
        for st in (oracle.F16, oracle.BF16):
            fx = oracle.QuantFixture(O=O, K=K, bits=4, gs=gs, scale_type=st, seed=K + O)
            layer = DevLayer.from_fixture(mlxq, fx)
            for T in (2, 3, 4, 5, 8):
                assert mlxq.Linear.canFuse([layer.linear], T)
                x = oracle.RNG(T * 131 + K).floats(T * K).reshape(T, K)
                got = run(layer, x, T, x_stride=K + 4, y_stride=O + 3)
                close(oracle, got, fx.reference(x), f"K {K} O {O} gs {gs} st {st} T {T}")


def test_small_batch_fused_with_bias_matches_separate(mlxq, oracle):
    # KernelTests.swift:255-269
    K = 1152
    fxs, layers = _fused_parts(mlxq, oracle, K)
    lins = [l.linear for l in layers]
    for T in (2, 7, 8):
        x = oracle.RNG(T).floats(T * K).reshape(T, K)
        yd = torch.zeros((T, 96), dtype=torch.float32, device="cuda")
        mlxq.Linear.encodeFusedDecode(None, lins, as_dtype(x, 0), yd, xStride=K, yStride=96, T=T)
        torch.cuda.synchronize()
        ref = np.concatenate([f.reference(x) for f in fxs], axis=1)
        close(oracle, yd.cpu().numpy(), ref, f"fused q/k/v T {T}")


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_small_batches_every_width_and_group(mlxq, oracle, bits):
    # Two to sixteen tokens take the decode kernel whose accumulator columns are tokens (where it serves the width and
    # group size; the others fall to the general kernels): both 16-bit scale types, fp16 and fp32 activations, a row
    # count that ends inside a block, group counts that leave windows of eight groups partly empty.  The bar is the
    # fp32 reassociation noise of a K-long sum, far below the 1e-3 of the reference's own tests.
    K, O = 1536, 72
    for gs in (32, 64, 128):
        for st in (oracle.F16, oracle.BF16):
            fx = oracle.QuantFixture(O=O, K=K, bits=bits, gs=gs, scale_type=st, with_bias=(gs == 64), seed=bits * 7 + gs)
            layer = DevLayer.from_fixture(mlxq, fx)
            for T, x_dtype in ((2, 1), (5, 1), (8, 1), (9, 1), (16, 1), (3, 0), (8, 0), (4, 2)):
                x = oracle.RNG(T * 17 + gs + bits).floats(T * K).reshape(T, K)
                xr = as_dtype(x, x_dtype).float().cpu().numpy()
                got = run(layer, x, T, x_dtype=x_dtype, x_stride=K + 8, y_stride=O + 5)
                # (fp32 activations ride as two fp16 columns: the split leaves 2^-22 of every product)
                close(oracle, got, fx.reference(xr), f"bits {bits} gs {gs} st {st} T {T} x {x_dtype}", 1e-4 if x_dtype == 0 else 3e-5)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_quantized_embedding_lookup(mlxq, oracle, bits):
    # KernelTests.swift:287-296 (4-bit there; every width here)
    K, V = 128, 16
    fx = oracle.QuantFixture(O=V, K=K, bits=bits, gs=64)
    layer = DevLayer.from_fixture(mlxq, fx)
    ids = torch.tensor([3, 0, 15, 7], dtype=torch.int32, device="cuda")
    out = torch.zeros((4, K), dtype=torch.float32, device="cuda")
    layer.linear.encodeLookup(None, ids, out, 4)
    mlxq.streamStatus(None, 0)
    ref = fx.dense[[3, 0, 15, 7]]
    close(oracle, out.cpu().numpy(), ref, "embedding", 1e-5)
    assert np.array_equal(out.cpu().numpy(), ref)          # two roundings, as the CPU code evaluates it


def test_lookup_rejects_ids_outside_the_table(mlxq, oracle):
    fx = oracle.QuantFixture(O=16, K=128, bits=4, gs=64)
    layer = DevLayer.from_fixture(mlxq, fx)
    ids = torch.tensor([3, 16, -1, 7], dtype=torch.int32, device="cuda")
    out = torch.full((4, 128), 5.0, dtype=torch.float32, device="cuda")
    layer.linear.encodeLookup(None, ids, out, 4)
    with pytest.raises(mlxq.GPUFailure, match="lookup id"):
        mlxq.streamStatus(None, 0)
    o = out.cpu().numpy()
    assert np.all(o[1] == 0) and np.all(o[2] == 0) and np.array_equal(o[0], fx.dense[3])
    mlxq.streamStatus(None, 0)                              # the error word is cleared after it is reported


def test_row_list_matvec(mlxq, oracle):
    # head_exact, Kernels.swift:2752-2787: only the listed rows are written
    O, K = 300, 512
    fx = oracle.QuantFixture(O=O, K=K, bits=6, gs=64, seed=5)
    layer = DevLayer.from_fixture(mlxq, fx)
    x = oracle.RNG(8).floats(K)
    rows = [5, 299, 0, 17, -3, 300, 123]
    lst = torch.tensor(rows + [1, 2], dtype=torch.int32, device="cuda")
    cnt = torch.tensor([len(rows)], dtype=torch.int32, device="cuda")
    y = torch.full((O,), -7.0, dtype=torch.float32, device="cuda")
    layer.linear.encodeRows(None, as_dtype(x, 0), y, cnt, lst, len(rows) + 2)
    torch.cuda.synchronize()
    got, ref = y.cpu().numpy(), fx.reference(x.reshape(1, K))[0]
    valid = [r for r in rows if 0 <= r < O]
    close(oracle, got[valid], ref[valid], "row list")
    untouched = np.ones(O, dtype=bool)
    untouched[valid] = False
    assert np.all(got[untouched] == -7.0)


@pytest.mark.parametrize("x_dtype,y_dtype", [(1, 0), (2, 0), (1, 1), (2, 2), (0, 2)])
def test_activation_and_output_dtypes(mlxq, oracle, x_dtype, y_dtype):
    # the benchmark configurations feed f16 / bf16 activations; outputs may be 16-bit too
    O, K = 72, 1024
    for bits in (4, 6):
        fx = oracle.QuantFixture(O=O, K=K, bits=bits, gs=64, with_bias=True, seed=bits)
        layer = DevLayer.from_fixture(mlxq, fx)
        for T in (1, 4, 7):
            x = oracle.RNG(T + 50).floats(T * K).reshape(T, K)
            xr = as_dtype(x, x_dtype).float().cpu().numpy()            # what the kernel actually sees
            ref = fx.reference(xr)
            got = run(layer, x, T, x_dtype=x_dtype, y_dtype=y_dtype)
            tol = TOL if y_dtype == 0 else (2e-3 if y_dtype == 1 else 1e-2)   # output rounding: f16 2^-11, bf16 2^-8
            close(oracle, got, ref, f"bits {bits} x {x_dtype} y {y_dtype} T {T}", tol)


def test_unaligned_rows_and_odd_groups(mlxq, oracle):
    # rows that are not 16-byte multiples (K*bits/8 % 16 != 0) and group sizes that are only multiples of 8
    for bits, K, gs in [(3, 64, 8), (5, 96, 24), (6, 80, 8), (4, 72, 24), (2, 208, 16), (8, 24, 8), (4, 40, 40)]:
        fx = oracle.QuantFixture(O=19, K=K, bits=bits, gs=gs, seed=K)
        layer = DevLayer.from_fixture(mlxq, fx)
        for T in (1, 3):
            x = oracle.RNG(K + T).floats(T * K).reshape(T, K)
            close(oracle, run(layer, x, T, x_stride=K + (4 - K % 4) % 4 + 4), fx.reference(x), f"bits {bits} K {K} gs {gs} T {T}")


def test_misaligned_x_is_rejected(mlxq, oracle):
    fx = oracle.QuantFixture(O=8, K=64, bits=4, gs=32)
    layer = DevLayer.from_fixture(mlxq, fx)
    xb = torch.zeros(2 * 70, dtype=torch.float32, device="cuda")
    yb = torch.zeros(2 * 8, dtype=torch.float32, device="cuda")
    with pytest.raises(mlxq.InvalidArgument, match="16-byte"):
        layer.linear.encode(None, xb[1:], 64, yb, 8, 1)
    with pytest.raises(mlxq.InvalidArgument, match="16-byte"):
        layer.linear.encode(None, xb, 66, yb, 8, 2)
    with pytest.raises(mlxq.InvalidArgument):
        layer.linear.encode(None, xb, 64, yb, 8, 0)


def test_row_permutation_and_concat(mlxq, oracle):
    # permuteRows / concatRows, Transformer.swift:113-151
    K = 256
    a = oracle.QuantFixture(O=24, K=K, bits=4, gs=64, seed=1)
    b = oracle.QuantFixture(O=16, K=K, bits=4, gs=64, seed=2)
    la, lb = DevLayer.from_fixture(mlxq, a), DevLayer.from_fixture(mlxq, b)
    x = oracle.RNG(4).floats(K).reshape(1, K)
    cat = mlxq.Linear.concatRows(la.linear, lb.linear, "ab")
    assert cat is not None and cat.outDim == 40
    close(oracle, run(cat, x, 1), np.concatenate([a.reference(x), b.reference(x)], axis=1), "concatRows")
    perm = list(np.random.default_rng(0).permutation(24))
    la.linear.permuteRows(perm)
    close(oracle, run(la, x, 1), a.reference(x)[:, perm], "permuteRows")
    with pytest.raises(mlxq.InvalidOutput):
        la.linear.permuteRows([0] * 24)


def test_baseline_shapes_against_oracle(mlxq, oracle):
    # config 1 of the benchmark (4096 x 4096, 4-bit g64, fp32 x) and a slice of the config-2 sweep at full K
    synth = __import__("importlib").import_module("mlx-runner_b200.synth")
    lay = synth.make_layer(4096, 4096, 4, 64, synth.F16, seed=0, bias_noise=True)
    assert np.array_equal(lay.packed.view(np.uint8), oracle.pack_fast(lay.q, 4))
    layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, lay.scale_dtype, 4096)
    _, x = synth.make_activations(1, 4096, synth.F32, seed=1)
    ref = oracle.qmatmul(lay.packed, lay.scales_raw, lay.biases_raw, lay.scale_dtype, x, 4096, 4, 64)
    close(oracle, run(layer, x, 1), ref, "config 1")
    for bits, gs in [(2, 32), (3, 64), (5, 128), (6, 64), (8, 32)]:
        lay = synth.make_layer(688, 4096, bits, gs, synth.F16, seed=bits)
        layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, lay.scale_dtype, 4096)
        for M in (1, 2, 4, 8):
            _, x = synth.make_activations(M, 4096, synth.F16, seed=M)
            ref = oracle.qmatmul(lay.packed, lay.scales_raw, lay.biases_raw, lay.scale_dtype, x, 4096, bits, gs)
            close(oracle, run(layer, x, M, x_dtype=1), ref, f"config 2 bits {bits} gs {gs} M {M}")


def test_committed_golden_cases(mlxq, oracle):
    # every bit width x group size of tests/golden/qlinear_cases.npz: codes bit-exact, outputs within 1e-3
    import golden_cases
    for c in golden_cases.load():
        layer = DevLayer(mlxq, c.packed, c.scales, c.biases, c.sdt, c.K, bias_raw=c.bias, name=c.name)
        codes = torch.full((c.O, c.K), 255, dtype=torch.uint8, device="cuda")
        layer.linear.unpackCodes(None, codes)
        torch.cuda.synchronize()
        assert np.array_equal(codes.cpu().numpy(), c.q), c.name
        for T in (1, c.T):
            got = run(layer, c.x[:T], T)
            assert oracle.max_rel_err(got, c.y[:T]) < 1e-3, f"{c.name} T={T}"
    mlxq.streamStatus(None, 0)


@pytest.mark.parametrize("bits,T,O", [(5, 1, 11008), (4, 8, 11008), (4, 1, 40000), (8, 2, 11008)])
def test_tall_layers_and_larger_batches_run_clean(mlxq, oracle, bits, T, O):
    # benchmark-sized layers whose CTAs hold more 16-row blocks than the shared-memory ring: outputs against the
    # oracle on a sample of rows, and the stream's error word stays clear (a bounded wait that ran out would set it)
    K = 4096
    lay = synth.make_layer(O, K, bits, 64, synth.F16, seed=bits + T, keep_codes=False)
    layer = DevLayer(mlxq, lay.packed, lay.scales_raw, lay.biases_raw, synth.F16, K)
    _, x = synth.make_activations(T, K, synth.F16, seed=3)
    got = run(layer, x, T, x_dtype=1)
    mlxq.streamStatus(None, 0)
    rows = np.sort(np.random.default_rng(O).choice(O, size=96, replace=False))
    ref = oracle.qmatmul(lay.packed[rows], lay.scales_raw[rows], lay.biases_raw[rows], synth.F16, x, K, bits, 64)
    assert oracle.max_rel_err(got[:, rows], ref) < 1e-3


def test_block_maxima_and_greedy_token_are_exact(mlxq, oracle):
    # first pass of the token selection and the greedy pass over it, bit for bit against the oracle: vocabulary-sized
    # rows, a ragged last block, a row stride that breaks 16-byte alignment (scalar path), equal maxima, NaN, -inf
    g = np.random.default_rng(9)
    for V, T, stride in ((151936, 3, 151936), (1000, 4, 1003), (256, 1, 256), (37, 2, 40)):
        x = g.standard_normal((T, stride)).astype(np.float32)
        x[0, V // 3] = x[0, V // 3 + (300 if V > 600 else 1)] = 40.0
        if T > 1:
            x[1, : min(V, 256)] = np.where(np.arange(min(V, 256)) == 1, np.nan, -np.inf)
        ref_m, ref_i = oracle.block_max(x[:, :V], index_base=77)
        nb = ref_m.shape[1]
        xd = torch.from_numpy(x).cuda()
        pairs = torch.zeros((2, T, nb), dtype=torch.int32, device="cuda")
        mlxq.blockMax(None, xd, V, T, stride, pairs, indexBase=77)
        token = torch.zeros(T, dtype=torch.int32, device="cuda")
        value = torch.zeros(T, dtype=torch.float32, device="cuda")
        mlxq.blockArgmax(None, pairs, 1, T, nb, token, value)
        torch.cuda.synchronize()
        got = pairs.cpu().numpy()
        assert np.array_equal(got[0].view(np.float32), ref_m), f"V {V}: block maxima"
        assert np.array_equal(got[1], ref_i), f"V {V}: block indices"
        tok, val = oracle.block_argmax(ref_m, ref_i)
        assert np.array_equal(token.cpu().numpy(), tok) and np.array_equal(value.cpu().numpy(), val), f"V {V}: greedy token"


def test_layers_built_from_safetensors_shards(mlxq, oracle, tmp_path):
    # a model directory written the way MLX writes it (nested names of a multimodal export, 2-byte tensors that leave
    # the following ones off 16-byte boundaries) -> WeightStore on the GPU -> Linear by prefix -> matvec against the oracle
    import json
    import struct
    weights = importlib.import_module("mlx-runner_b200.weights")
    fxs = {"model.layers.0.self_attn.o_proj": oracle.QuantFixture(O=72, K=512, bits=4, gs=64, with_bias=True, seed=3),
           "model.layers.0.mlp.down_proj": oracle.QuantFixture(O=48, K=1024, bits=6, gs=64, scale_type=oracle.BF16, seed=4)}
    header, blobs, off = {}, [], 0

    def put(name, dt, arr):
        nonlocal off
        b = np.ascontiguousarray(arr).tobytes()
        header["language_model." + name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    put("model.layer_scalar", "F16", np.array([0.5], dtype=np.float16))                 # shifts everything after it
    for prefix, fx in fxs.items():
        sdt = "F16" if fx.scale_type == oracle.F16 else "BF16"
        put(prefix + ".weight", "U32", fx.packed.view(np.uint32).reshape(fx.O, -1))
        put(prefix + ".scales", sdt, fx.scales_raw)
        put(prefix + ".biases", sdt, fx.biases_raw)
        if fx.bias_raw is not None:
            put(prefix + ".bias", sdt, fx.bias_raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    d = tmp_path / "model"
    d.mkdir()
    with open(d / "model.safetensors", "wb") as fh:
        fh.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))
    store = weights.WeightStore(str(d), device=0)
    assert store.totalBytes == off
    for prefix, fx in fxs.items():
        lin = store.linear(prefix, inDim=fx.K, outDim=fx.O)
        assert (lin.bits, lin.groupSize, lin.outDim) == (fx.bits, fx.gs, fx.O)
        for T in (1, 5):
            x = oracle.RNG(T + fx.O).floats(T * fx.K).reshape(T, fx.K)
            y = torch.zeros((T, fx.O), dtype=torch.float32, device="cuda")
            lin.encode(None, as_dtype(x, 0), fx.K, y, fx.O, T)
            torch.cuda.synchronize()
            close(oracle, y.cpu().numpy(), fx.reference(x), f"{prefix} T {T}")
    with pytest.raises(mlxq.InvalidFile):
        store.linear("model.layers.0.mlp.down_proj", inDim=fxs["model.layers.0.mlp.down_proj"].K, outDim=41)
    # a rank's row shard built from its slice alone (the store stays in host memory, only the slice goes to the GPU)
    host = weights.WeightStore(str(d))
    prefix, fx = "model.layers.0.mlp.down_proj", fxs["model.layers.0.mlp.down_proj"]
    x = oracle.RNG(77).floats(3 * fx.K).reshape(3, fx.K)
    y = torch.zeros((3, fx.O), dtype=torch.float32, device="cuda")
    for r in range(2):
        shard = host.linearShard(prefix, fx.K, r, 2, device=0)
        assert (shard.outDim, shard.totalOut, shard.rowOffset) == (fx.O // 2, fx.O, r * (fx.O // 2))
        shard.encode(None, as_dtype(x, 0), fx.K, y[:, shard.rowOffset:], fx.O, 3)
    torch.cuda.synchronize()
    close(oracle, y.cpu().numpy(), fx.reference(x), "row shards from slices")


def test_gate_up_product_folded_into_the_down_projection(mlxq, oracle):
    # silu_mul / gelu_tanh_mul (Kernels.swift:2004-2030) as a kernel of its own, and folded into the staging of the down
    # projection's activations: both against the oracle's act_mul followed by the layer's reference product
    g = np.random.default_rng(21)
    for bits, K, O in ((4, 1024, 72), (6, 512, 40), (8, 1536, 48)):
        fx = oracle.QuantFixture(O=O, K=K, bits=bits, gs=64, seed=bits)
        layer = DevLayer.from_fixture(mlxq, fx)
        for T, act in ((1, 0), (4, 1), (8, 0)):
            stride = 2 * K + 8
            gu = (g.standard_normal((T, stride)) * 1.5).astype(np.float32)
            gud = torch.from_numpy(gu).cuda()
            xref = oracle.act_mul(act, gu[:, :K], gu[:, K:2 * K])
            out = torch.zeros((T, K), dtype=torch.float32, device="cuda")
            mlxq.actMul(None, gud, stride, K, T, act, out)
            y = torch.full((T, O + 3), float("nan"), dtype=torch.float32, device="cuda")
            layer.linear.encodeGLU(None, gud, stride, act, y, O + 3, T)
            torch.cuda.synchronize()
            mlxq.streamStatus(None, 0)
            close(oracle, out.cpu().numpy(), xref, f"act_mul bits {bits} T {T} act {act}", 1e-5)
            close(oracle, y.cpu().numpy()[:, :O], fx.reference(xref), f"gated input bits {bits} T {T} act {act}")
            assert torch.isnan(y[:, O:]).all()
    with pytest.raises(mlxq.Unsupported):
        layer.linear.encodeGLU(None, gud, stride, 0, y, O + 3, 9)


def test_residual_add_fused_with_the_next_norm(mlxq, oracle):
    # add_rms_norm (Kernels.swift:1141-1175): h += r; y = RMSNorm(h) * w
    g = np.random.default_rng(22)
    for dim, rows, wdt in ((4096, 5, torch.bfloat16), (1000, 1, torch.float32), (64, 3, torch.float16)):
        stride = dim + 4
        h = g.standard_normal((rows, stride)).astype(np.float32)
        r = g.standard_normal((rows, stride)).astype(np.float32)
        w = torch.from_numpy(g.standard_normal(dim).astype(np.float32)).to(wdt)
        hd, rd = torch.from_numpy(h).cuda(), torch.from_numpy(r).cuda()
        yd = torch.zeros((rows, stride), dtype=torch.float32, device="cuda")
        mlxq.addRMSNorm(None, hd, rd, yd, w.cuda(), dim, rows, stride, 1e-6)
        torch.cuda.synchronize()
        href, yref = oracle.add_rms_norm(h[:, :dim], r[:, :dim], w.float().numpy(), 1e-6)
        assert np.array_equal(hd.cpu().numpy()[:, :dim], href)
        assert np.array_equal(hd.cpu().numpy()[:, dim:], h[:, dim:])                    # the padding is not touched
        close(oracle, yd.cpu().numpy()[:, :dim], yref, f"add_rms_norm dim {dim}", 1e-5)


@pytest.mark.parametrize("wdt", [torch.float16, torch.bfloat16, torch.float32])
def test_dense_layers_through_the_same_handle(mlxq, oracle, wdt):
    # dmm (Kernels.swift:938-999): y = x . W^T + bias with W in f32 / f16 / bf16, fp32 accumulation; vector and scalar
    # paths (a K that is not a multiple of 8, strided activations), batches beyond one pass of eight tokens
    g = np.random.default_rng(31)
    for O, K, T, xdt in ((72, 1024, 1, 1), (40, 1000, 5, 0), (33, 36, 20, 2), (16, 4096, 9, 1)):
        w = torch.from_numpy((g.standard_normal((O, K)) * 0.05).astype(np.float32)).to(wdt).cuda()
        bias = torch.from_numpy(g.standard_normal(O).astype(np.float32)).to(wdt).cuda() if O % 2 == 0 else None
        lin = mlxq.Linear(w, None, None, bias, inDim=K, name="dense")
        assert lin.bits == 0
        x = g.standard_normal((T, K)).astype(np.float32)
        xd = as_dtype(x, xdt)
        pad = 8 if K % 8 == 0 else 4                                   # (activation rows stay 16-byte aligned)
        xs = torch.zeros((T, K + pad), dtype=xd.dtype, device="cuda")
        xs[:, :K] = xd
        y = torch.full((T, O + 1), float("nan"), dtype=torch.float32, device="cuda")
        lin.encode(None, xs, K + pad, y, O + 1, T)
        torch.cuda.synchronize()
        ref = oracle.matmul_dense(w.float().cpu().numpy(), xd.float().cpu().numpy(), None if bias is None else bias.float().cpu().numpy())
        close(oracle, y.cpu().numpy()[:, :O], ref, f"dense {wdt} {O}x{K} T {T}", 2e-5)
        assert torch.isnan(y[:, O]).all()
        with pytest.raises(mlxq.Unsupported):
            lin.unpackCodes(None, torch.zeros((O, K), dtype=torch.uint8, device="cuda"))
