"""Safetensors shards of a model directory as tensors in device memory, and quantized layers built from them.

Mirrors ``SafeTensorFile`` / ``WeightStore`` (``Sources/MLXEngine/GPU.swift:195-365``) and ``Linear``'s convenience
initialiser (``Sources/MLXEngine/Transformer.swift:40-46``): the header of every shard is validated as untrusted
input (sizes, offsets, shapes) before any byte of a tensor is touched, entries of element types the engine does not use
are skipped, names resolve through the nesting aliases of multimodal exports, and a missing tensor raises
``MissingTensor`` with its name.

What differs on this hardware: the reference wraps a file whose tensors are all 16-byte aligned in place (unified
memory) and copies the others tensor by tensor; a B200 reads its weights from HBM, so every tensor the text model uses
is copied once, in file order, into an allocation of its own (device allocations are 256-byte aligned, which the
kernels' 16-byte vector loads need), the mapping is released, and the tensors of vision towers and multi-token-prediction
heads stay on disk.  ``device=None`` keeps the tensors in host memory (for hosts that place weights themselves and for
tests without a GPU)."""
import json
import mmap
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np

from .linear import InvalidFile, Linear, MissingTensor, OutOfMemory

# element types of the safetensors format the reference knows (GPU.swift:121-131): name, bytes, numpy type, torch name
_DTYPES = {     # (the numpy type is the one the bytes are read as: same width, a type torch converts; the torch type is the view)
    "F32": ("f32", 4, np.float32, "float32"), "F16": ("f16", 2, np.float16, "float16"), "BF16": ("bf16", 2, np.int16, "bfloat16"),
    "U32": ("u32", 4, np.int32, "int32"), "I32": ("i32", 4, np.int32, "int32"), "U8": ("u8", 1, np.uint8, "uint8"),
    "I8": ("i8", 1, np.int8, "int8"), "I64": ("i64", 8, np.int64, "int64"), "U16": ("u16", 2, np.int16, "int16"),
    "I16": ("i16", 2, np.int16, "int16"), "F64": ("f64", 8, np.float64, "float64"), "BOOL": ("bool", 1, np.uint8, "uint8"),
}
MAX_HEADER_BYTES = 100 << 20
INT32_MAX = 2 ** 31 - 1
INT64_MAX = 2 ** 63 - 1
# tensors of a multimodal export that the text model never reads (GPU.swift:297)
UNUSED_PREFIXES = ("vision_tower.", "model.visual.", "visual.", "mtp.", "model.mtp.", "language_model.mtp.")


class TensorInfo(tuple):
    """(dtype name, shape, first byte, end byte) of a tensor inside its file."""
    __slots__ = ()
    dtype = property(lambda self: self[0])
    shape = property(lambda self: self[1])
    start = property(lambda self: self[2])
    end = property(lambda self: self[3])


def parse_header(path: str, size: int, head: bytes, read) -> Tuple[Dict[str, TensorInfo], int]:
    """The validated table of a shard: name -> TensorInfo with absolute byte positions, and the header's end.
    ``head`` holds the file's first eight bytes, ``read(offset, n)`` returns n bytes of the file."""
    file = os.path.basename(path)
    if size < 8:
        raise InvalidFile(f"{file} is truncated")
    (header_len,) = struct.unpack("<Q", head[:8])
    if header_len > min(MAX_HEADER_BYTES, size - 8):
        raise InvalidFile(f"bad header length in {file}")
    try:
        header = json.loads(read(8, header_len).decode("utf-8"))
    except (UnicodeDecodeError, ValueError):
        header = None
    if not isinstance(header, dict):
        raise InvalidFile(f"bad header JSON in {file}")
    data_start = 8 + header_len
    data_size = size - data_start
    infos: Dict[str, TensorInfo] = {}
    for name, value in header.items():
        if name == "__metadata__":
            continue
        if not isinstance(value, dict) or not isinstance(value.get("dtype"), str):
            raise InvalidFile(f"bad entry '{name}' in {file}")
        if value["dtype"] not in _DTYPES:
            continue                                    # element types the engine never reads
        dname, esize, _, _ = _DTYPES[value["dtype"]]
        shape, offs = value.get("shape"), value.get("data_offsets")

        def whole(v):
            return isinstance(v, int) and not isinstance(v, bool)
        if (not isinstance(shape, list) or len(shape) > 8 or not all(whole(d) for d in shape)
                or not isinstance(offs, list) or len(offs) != 2 or not all(whole(o) for o in offs)):
            raise InvalidFile(f"bad entry '{name}' in {file}")
        if not (all(0 <= d <= INT32_MAX for d in shape) and 0 <= offs[0] <= offs[1] <= data_size):
            raise InvalidFile(f"tensor '{name}' is out of bounds in {file}")
        count = 1
        for d in shape:
            count *= d
            if count > INT64_MAX:
                raise InvalidFile(f"tensor '{name}' is too large in {file}")
        if count * esize > INT64_MAX or count * esize != offs[1] - offs[0]:
            raise InvalidFile(f"tensor '{name}' size does not match its shape in {file}")
        infos[name] = TensorInfo((dname, tuple(shape), data_start + offs[0], data_start + offs[1]))
    return infos, data_start


class SafeTensorFile:
    """One safetensors shard, its used tensors copied to ``device`` (``GPU.swift:205-304``)."""

    def __init__(self, path: str, device=None):
        self.path = path
        self.infos: Dict[str, TensorInfo] = {}
        self.byteCount = 0
        self._tensors: Dict[str, object] = {}
        try:
            fd = os.open(path, os.O_RDONLY)
        except OSError:
            raise InvalidFile(f"cannot open {os.path.basename(path)}") from None
        try:
            size = os.fstat(fd).st_size
            if size < 8:
                raise InvalidFile(f"{os.path.basename(path)} is truncated")
            with mmap.mmap(fd, 0, access=mmap.ACCESS_READ) as mm:
                infos, _ = parse_header(path, size, mm[:8], lambda off, n: mm[off:off + n])
                self._load(mm, infos, device)
        finally:
            os.close(fd)

    def _load(self, mm, infos: Dict[str, TensorInfo], device) -> None:
        import torch
        target = None if device is None else (torch.device("cuda", device) if isinstance(device, int) else torch.device(device))
        # in file order (a sequential read), one allocation per tensor
        for name, info in sorted(infos.items(), key=lambda kv: kv[1].start):
            if name.startswith(UNUSED_PREFIXES):
                continue
            nbytes = info.end - info.start
            np_type = next(v[2] for v in _DTYPES.values() if v[0] == info.dtype)
            torch_type = getattr(torch, next(v[3] for v in _DTYPES.values() if v[0] == info.dtype))
            host = np.frombuffer(mm, dtype=np_type, count=nbytes // np.dtype(np_type).itemsize, offset=info.start)
            t = torch.from_numpy(host.copy()).view(torch_type).reshape(info.shape)          # (the copy leaves the mapping)
            if target is not None:
                try:
                    t = t.to(target)
                except RuntimeError as e:       # allocation failure
                    raise OutOfMemory(f"could not allocate {nbytes} bytes for {name} in {os.path.basename(self.path)}: {str(e)[:80]}") from None
            self._tensors[name] = t
            self.byteCount += nbytes
            self.infos[name] = TensorInfo((info.dtype, info.shape, 0, nbytes))

    def tensor(self, name: str):
        """The tensor as a torch.Tensor (bf16 / f16 / f32 as such, u32 and i32 as int32 bit patterns), or None."""
        return self._tensors.get(name)


class WeightStore:
    """All safetensors shards of a model directory (``GPU.swift:306-365``)."""

    def __init__(self, directory: str, device=None):
        self.directory = directory
        names = self.shardFiles(directory)
        if not names:
            raise InvalidFile(f"no .safetensors files in {os.path.basename(os.path.normpath(directory))}")
        self.files: List[SafeTensorFile] = []
        self._index: Dict[str, int] = {}
        self._alias: Dict[str, str] = {}
        for i, n in enumerate(names):
            f = SafeTensorFile(os.path.join(directory, n), device)
            self.files.append(f)
            for k in f.infos:
                self._index[k] = i
        # multimodal exports nest the language model (GPU.swift:341-348)
        if "model.embed_tokens.weight" not in self._index:
            for src, dst in (("language_model.model.", "model."), ("language_model.lm_head.", "lm_head."), ("model.language_model.", "model.")):
                for k in list(self._index):
                    if k.startswith(src):
                        name = dst + k[len(src):]
                        if name not in self._index and name not in self._alias:
                            self._alias[name] = k

    @staticmethod
    def shardFiles(directory: str) -> List[str]:
        """The shards that hold the model: those ``model.safetensors.index.json`` maps weights to, or every
        ``.safetensors`` file when there is no usable index -- unrelated sidecars stay out of memory."""
        every = sorted(n for n in os.listdir(directory) if n.endswith(".safetensors"))
        try:
            with open(os.path.join(directory, "model.safetensors.index.json"), "rb") as fh:
                obj = json.loads(fh.read().decode("utf-8"))
            wmap = obj.get("weight_map") if isinstance(obj, dict) else None
            if isinstance(wmap, dict) and all(isinstance(k, str) and isinstance(v, str) for k, v in wmap.items()):
                listed = [n for n in every if n in set(wmap.values())]
                if listed:
                    return listed
        except (OSError, UnicodeDecodeError, ValueError):
            pass
        return every

    @property
    def names(self):
        return self._index.keys()

    def has(self, name: str) -> bool:
        return self._alias.get(name, name) in self._index

    def get(self, name: str):
        n = self._alias.get(name, name)
        i = self._index.get(n)
        return None if i is None else self.files[i].tensor(n)

    def require(self, name: str):
        t = self.get(name)
        if t is None:
            raise MissingTensor(name)
        return t

    @property
    def totalBytes(self) -> int:
        return sum(f.byteCount for f in self.files)

    def parts(self, prefix: str) -> Tuple[object, Optional[object], Optional[object], Optional[object]]:
        """(weight, scales, biases, bias) of a layer as the reference's convenience initialiser collects them: the
        weight is required, scales without biases is an error."""
        s, b = self.get(prefix + ".scales"), self.get(prefix + ".biases")
        if s is not None and b is None:
            raise MissingTensor(prefix + ".biases")
        return self.require(prefix + ".weight"), s, b, self.get(prefix + ".bias")

    def shardParts(self, prefix: str, rank: int, nranks: int, device=None):
        """Rows [rank * O / nranks, (rank + 1) * O / nranks) of a layer's tensors, each slice copied to ``device`` on its
        own -- with the store kept in host memory (``device=None`` at construction) a rank then holds 1 / nranks of the
        layer in HBM instead of all of it.  The row count must divide evenly."""
        import torch
        w, s, b, bias = self.parts(prefix)
        rows = int(w.shape[0])
        if nranks < 1 or not 0 <= rank < nranks or rows % nranks != 0:
            raise InvalidFile(f"{prefix}: {rows} rows do not split over {nranks} ranks")
        r0, r1 = rank * (rows // nranks), (rank + 1) * (rows // nranks)
        target = None if device is None else (torch.device("cuda", device) if isinstance(device, int) else torch.device(device))

        def cut(t):
            if t is None:
                return None
            if int(t.shape[0]) != rows:
                raise InvalidFile(f"{prefix}: inconsistent quantization tensors")
            piece = t[r0:r1].contiguous()
            return piece if target is None else piece.to(target)
        return cut(w), cut(s), cut(b), cut(bias)

    def linearShard(self, prefix: str, inDim: int, rank: int, nranks: int, device: int) -> Linear:
        """This rank's row shard of a layer, built from its slice alone (``Linear.shard(..., full=False)``)."""
        w, s, b, bias = self.shardParts(prefix, rank, nranks, device)
        return Linear.shard(w, s, b, bias, inDim=inDim, rank=rank, nranks=nranks, full=False, name=prefix, device=device)

    def linear(self, prefix: str, inDim: int, outDim: Optional[int] = None, device: Optional[int] = None) -> Linear:
        """``Linear(store, prefix, inDim:, outDim:)`` (``Transformer.swift:40-46``); the tensors must be on a GPU."""
        w, s, b, bias = self.parts(prefix)
        return Linear(w, s, b, bias, inDim=inDim, outDim=outDim, name=prefix, device=device)
