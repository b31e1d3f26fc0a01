"""mlx-runner_b200 -- the MLX affine quantized-linear layer on NVIDIA B200 (sm_100a).

The package is a thin host layer over ``lib/libmlxq.so`` (C ABI in ``include/mlxq.h``): ``Linear`` mirrors the
reference's layer class, ``Comm`` adds output-row sharding across GPUs.  The directory name carries a
hyphen, so import it with ``importlib.import_module("mlx-runner_b200")``.

Importing the package loads the CUDA library and fails if it has not been built: there is no CPU or
PyTorch fallback for the layer.
"""
from . import _lib
from ._lib import ACT_GELU_ERF, ACT_GELU_TANH, ACT_SILU, BF16, F16, F32
from .linear import (CollectiveFailure, Comm, DeviceTimeout, EngineError, GPUFailure, InvalidArgument, InvalidFile,
                     InvalidOutput, Linear, MissingTensor, OutOfMemory, SELECT_BLOCK, SELECT_NONE, TensorView, Unsupported,
                     actMul, addRMSNorm, blockArgmax, blockMax, check, streamStatus)

_lib.load()

__all__ = ["Linear", "Comm", "TensorView", "EngineError", "InvalidFile", "Unsupported", "MissingTensor", "OutOfMemory",
           "GPUFailure", "InvalidArgument", "InvalidOutput", "CollectiveFailure", "DeviceTimeout", "check",
           "streamStatus", "blockMax", "blockArgmax", "actMul", "addRMSNorm", "SELECT_BLOCK", "SELECT_NONE", "F32", "F16", "BF16", "ACT_SILU", "ACT_GELU_TANH", "ACT_GELU_ERF"]
