"""Shared helpers of the GPU parity tests: move oracle fixtures to the device, run the layer through
the C ABI, bring results back."""
from __future__ import annotations

import numpy as np
import torch

TORCH_DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def dev(raw: np.ndarray, dtype_code=None, device="cuda"):
    """Raw storage array -> device tensor (uint16 storage is reinterpreted as f16 / bf16)."""
    t = torch.from_numpy(np.ascontiguousarray(raw))
    if raw.dtype == np.uint16:
        t = t.view(torch.int16).to(device).view(TORCH_DT[dtype_code])
    elif raw.dtype == np.uint32:
        t = t.view(torch.int32).to(device)
    else:
        t = t.to(device)
    return t


def as_dtype(x: np.ndarray, dtype_code: int, device="cuda"):
    """fp32 values -> device tensor of the activation dtype (round to nearest even)."""
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device).to(TORCH_DT[dtype_code])


class DevLayer:
    """A fixture's tensors on the device plus the Linear built over them."""

    def __init__(self, mlxq, packed, scales_raw, biases_raw, sdtype, K, bias_raw=None, name="test", device="cuda"):
        packed32 = np.ascontiguousarray(packed).view(np.uint32).reshape(packed.shape[0], -1)
        self.w = dev(packed32, device=device)
        self.s = dev(scales_raw, sdtype, device)
        self.b = dev(biases_raw, sdtype, device)
        self.bias = dev(bias_raw, sdtype, device) if bias_raw is not None else None
        self.linear = mlxq.Linear(self.w, self.s, self.b, self.bias, inDim=K, name=name)

    @classmethod
    def from_fixture(cls, mlxq, fx, name="test"):
        return cls(mlxq, fx.packed, fx.scales_raw, fx.biases_raw, fx.scale_type, fx.K, fx.bias_raw, name)


def run(layer, x: np.ndarray, T: int, x_dtype=0, y_dtype=0, x_stride=None, y_stride=None, pad=float("nan")):
    """Encode one forward through the C ABI.  x fp32 [T, K] is converted to x_dtype; strides in elements
    (padding is filled with NaN so a kernel that reads it poisons the result).  Returns fp32 [T, O]."""
    lin = layer.linear if hasattr(layer, "linear") else layer
    K, O = lin.inDim, lin.outDim
    xs, ys = x_stride or K, y_stride or O
    xb = torch.full((T, xs), pad, dtype=TORCH_DT[x_dtype], device="cuda")
    xb[:, :K] = as_dtype(np.asarray(x, dtype=np.float32).reshape(T, K), x_dtype)
    yb = torch.full((T, ys), float("nan"), dtype=TORCH_DT[y_dtype], device="cuda")
    lin.encode(None, xb, xs, yb, ys, T)
    torch.cuda.synchronize()
    out = yb[:, :O].float().cpu().numpy()
    if ys > O:
        assert torch.isnan(yb[:, O:].float()).all(), "the kernel wrote into y's row padding"
    return out
