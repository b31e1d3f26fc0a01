"""The C-ABI boundary without a GPU: every symbol include/mlxq.h declares is exported, and construction
validates exactly as the reference's Linear.init does (Transformer.swift:48-111).  No compute calls."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "mlxq.h")).read()
    return sorted(set(re.findall(r"MLXQ_API\s+[\w\s\*]+?\b(mlxq_\w+)\s*\(", text)))


def test_header_symbols_are_exported(mlxq):
    names = _declared_symbols()
    assert len(names) >= 25
    lib = C.CDLL(mlxq._lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in mlxq.h but not exported"
    # and the Python binding covers exactly the declared set
    assert sorted(mlxq._lib.SIGNATURES) == names


def test_no_torch_types_in_the_abi():
    text = open(os.path.join(ROOT, "include", "mlxq.h")).read()
    assert "torch" not in text and "at::" not in text and "#include <cuda" not in text


def _views(mlxq, O=40, K=512, bits=4, gs=64, sdt="f16"):
    tv = mlxq.TensorView
    return (tv(0x100000, "u32", (O, K * bits // 32)), tv(0x200000, sdt, (O, K // gs)), tv(0x300000, sdt, (O, K // gs)))


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_bits_and_group_size_are_derived_from_shapes(mlxq, bits, gs):
    w, s, b = _views(mlxq, bits=bits, gs=gs)
    lin = mlxq.Linear(w, s, b, None, inDim=512)
    assert (lin.bits, lin.groupSize, lin.inDim, lin.outDim) == (bits, gs, 512, 40)
    assert lin.description == f"q{bits}g{gs}"


def test_construction_errors_mirror_linear_init(mlxq):
    tv = mlxq.TensorView
    w, s, b = _views(mlxq)
    with pytest.raises(mlxq.MissingTensor):                       # Transformer.swift:43
        mlxq.Linear(w, s, None, None, inDim=512)
    with pytest.raises(mlxq.InvalidFile, match="2-D"):            # :52
        mlxq.Linear(tv(0x1000, "u32", (40,)), s, b, None, inDim=512)
    with pytest.raises(mlxq.InvalidFile, match="2-D"):
        mlxq.Linear(w, s, b, None, inDim=0)
    with pytest.raises(mlxq.InvalidFile, match="expected 48 output rows"):   # :53
        mlxq.Linear(w, s, b, None, inDim=512, outDim=48)
    with pytest.raises(mlxq.InvalidFile, match="bias shape"):     # :54
        mlxq.Linear(w, s, b, tv(0x4000, "f16", (39,)), inDim=512)
    with pytest.raises(mlxq.InvalidFile, match="inconsistent"):   # :56-57 scales rows
        mlxq.Linear(w, tv(0x2000, "f16", (39, 8)), tv(0x3000, "f16", (39, 8)), None, inDim=512)
    with pytest.raises(mlxq.InvalidFile, match="inconsistent"):   # biases shape != scales shape
        mlxq.Linear(w, s, tv(0x3000, "f16", (40, 4)), None, inDim=512)
    with pytest.raises(mlxq.InvalidFile, match="inconsistent"):   # inDim % groups != 0
        mlxq.Linear(w, tv(0x2000, "f16", (40, 7)), tv(0x3000, "f16", (40, 7)), None, inDim=512)
    with pytest.raises(mlxq.InvalidFile, match="inconsistent"):   # packed bits not a multiple of inDim
        mlxq.Linear(tv(0x1000, "u32", (40, 63)), s, b, None, inDim=520)
    with pytest.raises(mlxq.Unsupported, match="7-bit"):          # :71-73
        mlxq.Linear(tv(0x1000, "u32", (40, 7 * 512 // 32)), s, b, None, inDim=512)
    with pytest.raises(mlxq.Unsupported, match="group 4"):        # group size not a multiple of 8
        mlxq.Linear(w, tv(0x2000, "f16", (40, 128)), tv(0x3000, "f16", (40, 128)), None, inDim=512)
    # dense layers (Transformer.swift:103-112): a floating weight with as many columns as inputs, inDim % 4 == 0
    dense = mlxq.Linear(tv(0x1000, "f16", (40, 512)), None, None, None, inDim=512)
    assert (dense.bits, dense.outDim, dense.inDim, dense.description, dense.kernelFor(1)) == (0, 40, 512, "f16", "dmm")
    with pytest.raises(mlxq.InvalidFile, match="expected 520 input columns"):
        mlxq.Linear(tv(0x1000, "f16", (40, 512)), None, None, None, inDim=520)
    with pytest.raises(mlxq.Unsupported, match="input dim"):
        mlxq.Linear(tv(0x1000, "bf16", (40, 510)), None, None, None, inDim=510)
    with pytest.raises(mlxq.Unsupported):                          # an integer tensor without scales is not a layer
        mlxq.Linear(tv(0x1000, "u32", (40, 512)), None, None, None, inDim=512)
    with pytest.raises(mlxq.Unsupported, match="not sharded"):
        mlxq.Linear.shard(tv(0x1000, "f16", (40, 512)), None, None, None, inDim=512, rank=0, nranks=2)
    ok = mlxq.Linear(w, s, b, tv(0x4000, "f16", (40,)), inDim=512, outDim=40)
    assert ok.outDim == 40


def test_policy_functions(mlxq, oracle):
    # useGemm64 truth table (KernelTests.swift:153-156, :179) through the C ABI, and against the oracle
    for T, O, big in [(64, 41, False), (128, 41, False), (517, 41, False), (96, 2050, False), (128, 2050, True),
                      (517, 520, True), (256, 2050, True)]:
        assert mlxq.Linear.useGemm64(T, O) == big
    for T in range(1, 700, 7):
        for O in (8, 41, 520, 2050, 4096, 151936):
            assert mlxq.Linear.useGemm64(T, O) == oracle.use_gemm64(T, O)
    tv = mlxq.TensorView
    mk = lambda O, bits=4, gs=64, K=256, bias=False, sdt="f16": mlxq.Linear(
        tv(0x1000, "u32", (O, K * bits // 32)), tv(0x2000, sdt, (O, K // gs)), tv(0x3000, sdt, (O, K // gs)),
        tv(0x4000, sdt, (O,)) if bias else None, inDim=K)
    parts = [mk(64, bias=True), mk(16, bias=True), mk(16, bias=True)]
    assert mlxq.Linear.fusable(parts)                               # KernelTests.swift:219
    assert not mlxq.Linear.fusable([mk(64), mk(16, bias=True)])     # same bias presence
    assert not mlxq.Linear.fusable([mk(64), mk(12)])                # rows % 8
    assert not mlxq.Linear.fusable([mk(64), mk(16, gs=32)])         # same group size
    assert not mlxq.Linear.fusable([mk(64), mk(16, bits=8)])        # same bits
    assert not mlxq.Linear.fusable([mk(64), mk(16, sdt="bf16")])    # same scale dtype
    assert not mlxq.Linear.fusable([mk(8)] * 4)                     # at most three
    one = [mk(40, K=512)]
    for T in (1, 2, 3, 4, 5, 8):
        assert mlxq.Linear.canFuse(one, T)                          # KernelTests.swift:238
    assert not mlxq.Linear.canFuse(one, 9)
    assert mlxq.Linear.canFuse([mk(40, bits=6, K=512)], 1) and not mlxq.Linear.canFuse([mk(40, bits=6, K=512)], 2)
    # 4-bit needs K % 32 and gs % 32 for the fused decode kernel (Transformer.swift:76-77)
    assert not mlxq.Linear.canFuse([mk(40, K=528, gs=24)], 1)


def test_shard_construction(mlxq):
    tv = mlxq.TensorView
    O, K = 4096, 512
    w, s, b = tv(0x100000, "u32", (O, K // 8)), tv(0x800000, "f16", (O, K // 64)), tv(0xA00000, "f16", (O, K // 64))
    for n in (1, 2, 4, 8):
        offs = []
        for r in range(n):
            sh = mlxq.Linear.shard(w, s, b, None, inDim=K, rank=r, nranks=n)
            assert sh.outDim == O // n and sh.inDim == K
            offs.append(sh.rowOffset)
        assert offs == [r * (O // n) for r in range(n)]
    with pytest.raises(mlxq.Unsupported):
        mlxq.Linear.shard(tv(0x1000, "u32", (40, K // 8)), tv(0x2000, "f16", (40, 8)), tv(0x3000, "f16", (40, 8)), None,
                          inDim=K, rank=0, nranks=2)
    with pytest.raises(mlxq.InvalidArgument):
        mlxq.Linear.shard(w, s, b, None, inDim=K, rank=2, nranks=2)
    pre = mlxq.Linear.shard(tv(0x1000, "u32", (512, K // 8)), tv(0x2000, "f16", (512, 8)), tv(0x3000, "f16", (512, 8)),
                            None, inDim=K, rank=3, nranks=8, full=False)
    assert pre.outDim == 512 and pre.rowOffset == 1536


def test_status_strings(mlxq):
    lib = mlxq._lib.load()
    assert lib.mlxq_version() >= 100
    assert lib.mlxq_status_string(0) == b"ok"
    assert b"Unsupported" in lib.mlxq_status_string(2)
