"""ctypes binding of libmlxq.so: exactly the entry points ``include/mlxq.h`` declares.

The library is loaded from ``lib/libmlxq.so`` beside this file.  There is no fallback: when the library
is missing or fails to load, importing the package raises, so a host can never silently compute the
layer some other way.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmlxq.so")

# status codes (mlxq_status)
OK, INVALID_FILE, UNSUPPORTED, MISSING_TENSOR, OUT_OF_MEMORY, GPU_FAILURE, INVALID_ARGUMENT, NCCL_FAILURE, TIMEOUT = range(9)
# element types (mlxq_dtype)
F32, F16, BF16 = 0, 1, 2
# gate activations (mlxq_act)
ACT_SILU, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
COMM_ID_BYTES = 128
STATIC_SCRATCH_BYTES = 32 << 20     # MLXQ_STATIC_SCRATCH_BYTES


class LinearDesc(C.Structure):
    """struct mlxq_linear_desc."""
    _fields_ = [
        ("weight", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("bias", C.c_void_p),
        ("weight_rows", C.c_int64), ("weight_cols", C.c_int64),
        ("scales_rows", C.c_int64), ("scales_cols", C.c_int64),
        ("biases_rows", C.c_int64), ("biases_cols", C.c_int64),
        ("bias_len", C.c_int64), ("in_dim", C.c_int64), ("expect_out", C.c_int64),
        ("scale_dtype", C.c_int32), ("bias_dtype", C.c_int32), ("device", C.c_int32), ("reserved", C.c_int32),
        ("name", C.c_char_p),
    ]


# name -> (restype, argtypes); the list the symbol-export test walks.
SIGNATURES = {
    "mlxq_version": (C.c_int, []),
    "mlxq_status_string": (C.c_char_p, [C.c_int]),
    "mlxq_last_error": (C.c_char_p, []),
    "mlxq_linear_create": (C.c_int, [C.POINTER(LinearDesc), C.POINTER(C.c_void_p)]),
    "mlxq_linear_create_shard": (C.c_int, [C.POINTER(LinearDesc), C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "mlxq_linear_destroy": (None, [C.c_void_p]),
    "mlxq_linear_prepare": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mlxq_linear_in_dim": (C.c_int64, [C.c_void_p]),
    "mlxq_linear_out_dim": (C.c_int64, [C.c_void_p]),
    "mlxq_linear_bits": (C.c_int, [C.c_void_p]),
    "mlxq_linear_group_size": (C.c_int, [C.c_void_p]),
    "mlxq_linear_row_offset": (C.c_int64, [C.c_void_p]),
    "mlxq_linear_total_rows": (C.c_int64, [C.c_void_p]),
    "mlxq_linear_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_int,
                                      C.c_int64, C.c_int64]),
    "mlxq_linear_forward_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_void_p,
                                             C.c_int, C.c_int64, C.c_int64]),
    "mlxq_fused_forward": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int64,
                                     C.c_void_p, C.c_int, C.c_int64, C.c_int64]),
    "mlxq_linear_forward_gated": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                            C.c_void_p, C.c_int]),
    "mlxq_linear_lookup": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]),
    "mlxq_linear_forward_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.c_int64]),
    "mlxq_unpack_codes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "mlxq_act_mul": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "mlxq_linear_forward_glu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_int, C.c_int64,
                                          C.c_int64]),
    "mlxq_add_rms_norm": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64,
                                    C.c_int64, C.c_int64, C.c_float]),
    "mlxq_block_max": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "mlxq_block_argmax": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "mlxq_fusable": (C.c_int, [C.POINTER(C.c_void_p), C.c_int]),
    "mlxq_can_fuse": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int64]),
    "mlxq_use_gemm64": (C.c_int, [C.c_int64, C.c_int64]),
    "mlxq_gemm_tile_tokens": (C.c_int, [C.c_void_p, C.c_int64]),
    "mlxq_kernel_for": (C.c_char_p, [C.c_void_p, C.c_int, C.c_int, C.c_int64]),
    "mlxq_stream_status": (C.c_int, [C.c_void_p, C.c_int]),
    "mlxq_comm_unique_id": (C.c_int, [C.POINTER(C.c_uint8)]),
    "mlxq_comm_create": (C.c_int, [C.POINTER(C.c_uint8), C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "mlxq_comm_destroy": (None, [C.c_void_p]),
    "mlxq_comm_rank": (C.c_int, [C.c_void_p]),
    "mlxq_comm_size": (C.c_int, [C.c_void_p]),
    "mlxq_linear_forward_gather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64,
                                             C.c_void_p, C.c_int64, C.c_int64]),
    "mlxq_comm_window": (C.c_int, [C.c_void_p, C.c_size_t]),
    "mlxq_comm_wait": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mlxq_linear_forward_blockmax_gather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64,
                                                      C.c_int64, C.c_void_p, C.c_void_p]),
    "mlxq_linear_forward_gather_fused": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64,
                                                   C.c_int64, C.POINTER(C.c_void_p)]),
}

_lib = None


def load() -> C.CDLL:
    """Load libmlxq.so once and attach the prototypes.  Raises OSError if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} is missing: build it with `python mlx-runner_b200/build.py` "
                          "(there is no CPU or PyTorch fallback for this layer)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)       # AttributeError here means the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return load().mlxq_last_error().decode("utf-8", "replace")
