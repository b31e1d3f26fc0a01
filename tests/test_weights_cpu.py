"""The safetensors reader and the weight store on the CPU: header validation of untrusted files, shard selection,
aliases, unused tensors, and the (weight, scales, biases, bias) collection of a layer -- the behaviours of
SafeTensorFile / WeightStore (Sources/MLXEngine/GPU.swift:195-365) and Linear's convenience initialiser
(Transformer.swift:40-46).  Files are written here, byte by byte, the way MLX writes them (header padded to 8 bytes)."""
import importlib
import json
import os
import struct

import numpy as np
import pytest

weights = importlib.import_module("mlx-runner_b200.weights")
mlxq = importlib.import_module("mlx-runner_b200")

NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "U32": np.uint32, "I32": np.int32, "U8": np.uint8, "I64": np.int64}


def write_safetensors(path, tensors, pad=8, metadata=None, raw_header=None):
    """tensors: name -> (dtype string, numpy array).  Returns the header dict that was written."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, (dt, arr) in tensors.items():
        b = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    text = (raw_header if raw_header is not None else json.dumps(header)).encode()
    text += b" " * (-len(text) % pad)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))
    return header


def quant_layer(g, O, K, bits=4, gs=64):
    return {"weight": ("U32", g.integers(0, 2 ** 32, size=(O, K * bits // 32), dtype=np.uint32)),
            "scales": ("F16", g.random((O, K // gs)).astype(np.float16)),
            "biases": ("F16", g.random((O, K // gs)).astype(np.float16))}


def test_reads_tensors_of_every_used_type_and_skips_unknown_ones(tmp_path):
    g = np.random.default_rng(1)
    t = {"a.weight": ("U32", g.integers(0, 2 ** 32, size=(8, 16), dtype=np.uint32)),
         "a.scales": ("BF16", g.integers(0, 2 ** 16, size=(8, 2), dtype=np.uint16)),
         "norm.weight": ("F32", g.standard_normal(7).astype(np.float32)),
         "scalar": ("F16", np.array(1.5, dtype=np.float16)),                   # a 0-d, 2-byte tensor (shifts what follows)
         "ids": ("I64", np.arange(5, dtype=np.int64))}
    write_safetensors(tmp_path / "m.safetensors", t, metadata={"format": "mlx"})
    # an entry of a type the engine does not know is skipped, not an error
    hdr = json.loads(open(tmp_path / "m.safetensors", "rb").read()[8:8 + struct.unpack("<Q", open(tmp_path / "m.safetensors", "rb").read(8))[0]])
    f = weights.SafeTensorFile(str(tmp_path / "m.safetensors"))
    assert set(f.infos) == set(t)
    import torch
    assert f.tensor("a.weight").dtype == torch.int32 and np.array_equal(f.tensor("a.weight").numpy().view(np.uint32), t["a.weight"][1])
    assert f.tensor("a.scales").dtype == torch.bfloat16 and np.array_equal(f.tensor("a.scales").view(torch.int16).numpy().view(np.uint16), t["a.scales"][1])
    assert np.array_equal(f.tensor("norm.weight").numpy(), t["norm.weight"][1])
    assert f.tensor("scalar").shape == () and float(f.tensor("scalar")) == 1.5
    assert f.byteCount == sum(a.nbytes for _, a in t.values()) and f.tensor("nope") is None
    hdr["odd"] = {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}
    write_safetensors(tmp_path / "n.safetensors", t, raw_header=json.dumps(hdr))
    assert "odd" not in weights.SafeTensorFile(str(tmp_path / "n.safetensors")).infos


@pytest.mark.parametrize("case", ["truncated", "header_length", "json", "entry", "dims", "negative", "offsets", "size", "float_shape"])
def test_untrusted_headers_are_rejected(tmp_path, case):
    g = np.random.default_rng(2)
    p = tmp_path / "bad.safetensors"
    arr = g.standard_normal((4, 4)).astype(np.float32)
    good = {"w": {"dtype": "F32", "shape": [4, 4], "data_offsets": [0, 64]}}
    if case == "truncated":
        open(p, "wb").write(b"\x01\x02\x03")
    elif case == "header_length":
        open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}" + arr.tobytes())
    elif case == "json":
        write_safetensors(p, {"w": ("F32", arr)}, raw_header="{not json")
    else:
        bad = json.loads(json.dumps(good))
        if case == "entry":
            bad["w"] = {"shape": [4, 4], "data_offsets": [0, 64]}                     # no dtype
        elif case == "dims":
            bad["w"]["shape"] = [1] * 9
        elif case == "negative":
            bad["w"]["shape"] = [-4, -4]
        elif case == "offsets":
            bad["w"]["data_offsets"] = [0, 1 << 30]
        elif case == "size":
            bad["w"]["shape"] = [4, 5]
        elif case == "float_shape":
            bad["w"]["shape"] = [4.0, 4]
        write_safetensors(p, {"w": ("F32", arr)}, raw_header=json.dumps(bad))
    with pytest.raises(mlxq.InvalidFile):
        weights.SafeTensorFile(str(p))
    with pytest.raises(mlxq.InvalidFile):
        weights.SafeTensorFile(str(tmp_path / "absent.safetensors"))


def test_store_uses_the_index_aliases_and_leaves_unused_tensors_on_disk(tmp_path):
    g = np.random.default_rng(3)
    d = tmp_path / "model"
    d.mkdir()
    a = {f"language_model.model.layers.0.mlp.down_proj.{k}": v for k, v in quant_layer(g, 16, 128).items()}
    a["language_model.lm_head.weight"] = ("U32", g.integers(0, 2 ** 32, size=(32, 16), dtype=np.uint32))
    a["vision_tower.patch.weight"] = ("F32", g.standard_normal((64, 64)).astype(np.float32))
    b = {f"language_model.model.layers.1.mlp.down_proj.{k}": v for k, v in quant_layer(g, 16, 128).items()}
    del b["language_model.model.layers.1.mlp.down_proj.biases"]
    write_safetensors(d / "model-00001-of-00002.safetensors", a)
    write_safetensors(d / "model-00002-of-00002.safetensors", b)
    write_safetensors(d / "sidecar_vision.safetensors", {"huge": ("F32", np.zeros((256, 256), dtype=np.float32))})
    wm = {k: "model-00001-of-00002.safetensors" for k in a}
    wm.update({k: "model-00002-of-00002.safetensors" for k in b})
    json.dump({"weight_map": wm}, open(d / "model.safetensors.index.json", "w"))
    assert weights.WeightStore.shardFiles(str(d)) == ["model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"]
    store = weights.WeightStore(str(d))
    assert not store.has("huge") and not store.has("vision_tower.patch.weight")
    assert store.totalBytes == sum(v[1].nbytes for k, v in {**a, **b}.items() if not k.startswith("vision_tower."))
    # the nested names answer to the engine's names
    assert store.has("model.layers.0.mlp.down_proj.weight") and store.has("lm_head.weight")
    w, s, bq, bias = store.parts("model.layers.0.mlp.down_proj")
    assert tuple(w.shape) == (16, 16) and tuple(s.shape) == (16, 2) and tuple(bq.shape) == (16, 2) and bias is None
    with pytest.raises(mlxq.MissingTensor) as e:
        store.parts("model.layers.1.mlp.down_proj")                                   # scales without biases
    assert "biases" in str(e.value)
    with pytest.raises(mlxq.MissingTensor):
        store.require("model.layers.7.mlp.down_proj.weight")
    # without an index every shard is read, and a directory without shards is an error
    os.remove(d / "model.safetensors.index.json")
    assert "sidecar_vision.safetensors" in weights.WeightStore.shardFiles(str(d))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(mlxq.InvalidFile):
        weights.WeightStore(str(empty))


def _write_raw(tmp_path, header: str, payload: bytes, header_len=None):
    d = tmp_path / "m"
    d.mkdir(exist_ok=True)
    text = header.encode()
    with open(d / "model.safetensors", "wb") as fh:
        fh.write(struct.pack("<Q", len(text) if header_len is None else header_len) + text + payload)
    return str(d)


def test_reference_case_misaligned_tensor_is_realigned(tmp_path):
    # Tests/MLXEngineTests/EngineTests.swift:126-152: a = 3 x f16 (6 bytes) so b starts misaligned; b = 4 x f32
    a = np.array([1, 2, 3], dtype=np.float16)
    b = np.array([0.5, -1, 2.25, 8], dtype=np.float32)
    header = '{"a":{"dtype":"F16","shape":[3],"data_offsets":[0,6]},"b":{"dtype":"F32","shape":[4],"data_offsets":[6,22]}}'
    while (len(header) + 8) % 8 != 0:
        header += " "
    store = weights.WeightStore(_write_raw(tmp_path, header, a.tobytes() + b.tobytes()))
    tb = store.require("b")
    assert tuple(tb.shape) == (4,) and str(tb.dtype) == "torch.float32"
    assert tb.data_ptr() % 16 == 0
    assert tb.numpy().tolist() == b.tolist()
    assert store.get("missing") is None


@pytest.mark.parametrize("header", [
    '{"a":{"dtype":"F32","shape":[4],"data_offsets":[0,1000]}}',                    # past end of file
    '{"a":{"dtype":"F32","shape":[4],"data_offsets":[8,0]}}',                       # start > end
    '{"a":{"dtype":"F32","shape":[4],"data_offsets":[-16,0]}}',                     # negative
    '{"a":{"dtype":"F32","shape":[5],"data_offsets":[0,16]}}',                      # shape / bytes mismatch
    '{"a":{"dtype":"F32","shape":[4611686018427387904,4],"data_offsets":[0,16]}}',  # overflow
    '{"a":{"dtype":"F32","shape":[-4],"data_offsets":[0,16]}}',                     # negative dim
    "not json",
])
def test_reference_cases_malformed_headers(tmp_path, header):
    # EngineTests.swift:166-179, the reference's own malformed headers, 16 bytes of payload
    with pytest.raises(mlxq.EngineError):
        weights.WeightStore(_write_raw(tmp_path, header, bytes(16)))


def test_reference_case_huge_header_length(tmp_path):
    # EngineTests.swift:181-190
    with pytest.raises(mlxq.EngineError):
        weights.WeightStore(_write_raw(tmp_path, "", bytes(64), header_len=2 ** 64 - 5))


def test_a_rank_takes_only_its_rows(tmp_path):
    g = np.random.default_rng(4)
    d = tmp_path / "model"
    d.mkdir()
    layer = {f"model.layers.0.mlp.up_proj.{k}": v for k, v in quant_layer(g, 24, 128).items()}
    layer["model.layers.0.mlp.up_proj.bias"] = ("F16", g.random(24).astype(np.float16))
    write_safetensors(d / "model.safetensors", layer)
    store = weights.WeightStore(str(d))                                   # host-resident
    whole = store.parts("model.layers.0.mlp.up_proj")
    got = [store.shardParts("model.layers.0.mlp.up_proj", r, 3) for r in range(3)]
    import torch
    for i, t in enumerate(whole):
        assert torch.equal(torch.cat([p[i] for p in got]), t)
        assert all(p[i].shape[0] == 8 and p[i].is_contiguous() for p in got)
    with pytest.raises(mlxq.InvalidFile):
        store.shardParts("model.layers.0.mlp.up_proj", 0, 5)              # 24 rows over 5 ranks
