"""ctypes binding of the C-ABI library ``libaila_nf4.so`` (include/aila_nf4.h).

The library is the product; there is no Python or CPU fallback. Importing this module with the
library missing raises ImportError with the build command.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libaila_nf4.so")

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_UNSUPPORTED = 2
ERR_CUDA = 3
ERR_OUT_OF_MEMORY = 4
NOT_APPLICABLE = 5
ERR_KERNEL_TIMEOUT = 6

SHARD_ROWS = 0
SHARD_COLS = 1
IPC_HANDLE_BYTES = 64


class WeightDesc(ctypes.Structure):
    """AilaNf4WeightDesc."""
    _fields_ = [
        ("out_features", ctypes.c_int64),
        ("in_features", ctypes.c_int64),
        ("blocksize", ctypes.c_int32),
        ("nested", ctypes.c_int32),
        ("nested_blocksize", ctypes.c_int32),
        ("nested_offset", ctypes.c_float),
        ("packed_weight", ctypes.c_void_p),
        ("absmax", ctypes.c_void_p),
        ("quant_map", ctypes.c_void_p),
        ("nested_absmax", ctypes.c_void_p),
        ("nested_quant_map", ctypes.c_void_p),
        ("nested_absmax_count", ctypes.c_int64),
        ("pointers_on_device", ctypes.c_int32),
        ("device", ctypes.c_int32),
    ]


class StTensorView(ctypes.Structure):
    """AilaStTensorView."""
    _fields_ = [("dtype", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("shape", ctypes.c_int64 * 8), ("data", ctypes.c_void_p),
                ("nbytes", ctypes.c_int64)]


ST_DTYPES = ("unknown", "U8", "I8", "F16", "BF16", "F32", "F64", "I32", "I64", "BOOL")

class RmsNorm(ctypes.Structure):
    """AilaNf4RmsNorm."""
    _fields_ = [("add_bf16", ctypes.c_void_p), ("weight_bf16", ctypes.c_void_p),
                ("eps", ctypes.c_float), ("hidden_out_bf16", ctypes.c_void_p)]


class ChainOp(ctypes.Structure):
    """AilaNf4ChainOp."""
    _fields_ = [("linear", ctypes.c_void_p), ("ff_dim", ctypes.c_int64), ("x_bf16", ctypes.c_void_p),
                ("y_bf16", ctypes.c_void_p), ("residual_bf16", ctypes.c_void_p),
                ("norm", ctypes.POINTER(RmsNorm))]


# name -> (restype, argtypes); every symbol include/aila_nf4.h declares
_VP = ctypes.c_void_p
_SIGNATURES = {
    "aila_nf4_last_error": (ctypes.c_char_p, []),
    "aila_nf4_version": (ctypes.c_int, []),
    "aila_nf4_linear_create": (ctypes.c_int, [ctypes.POINTER(WeightDesc), ctypes.POINTER(_VP)]),
    "aila_nf4_linear_create_shard": (ctypes.c_int, [ctypes.POINTER(WeightDesc), ctypes.c_int,
                                                    ctypes.c_int, ctypes.c_int,
                                                    ctypes.POINTER(_VP)]),
    "aila_nf4_linear_create_fused_rows": (ctypes.c_int, [ctypes.POINTER(_VP), ctypes.c_int,
                                                         ctypes.POINTER(_VP)]),
    "aila_nf4_linear_destroy": (None, [_VP]),
    "aila_nf4_linear_in_features": (ctypes.c_int64, [_VP]),
    "aila_nf4_linear_out_features": (ctypes.c_int64, [_VP]),
    "aila_nf4_linear_device_bytes": (ctypes.c_int64, [_VP]),
    "aila_nf4_linear_device": (ctypes.c_int, [_VP]),
    "aila_nf4_scratch_create": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(_VP)]),
    "aila_nf4_scratch_destroy": (None, [_VP]),
    "aila_nf4_scratch_reserve": (ctypes.c_int, [_VP, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_int]),
    "aila_nf4_scratch_check": (ctypes.c_int, [_VP, _VP]),
    "aila_nf4_forward": (ctypes.c_int, [_VP, _VP, _VP, _VP, ctypes.c_int, _VP, _VP]),
    "aila_nf4_forward_gate_up_swiglu": (ctypes.c_int, [_VP, _VP, _VP, _VP, ctypes.c_int,
                                                       ctypes.c_int64, _VP]),
    "aila_nf4_forward_host": (ctypes.c_int, [_VP, _VP, _VP, _VP, ctypes.c_int, _VP]),
    "aila_nf4_forward_gate_up_swiglu_host": (ctypes.c_int, [_VP, _VP, _VP, _VP, ctypes.c_int,
                                                            ctypes.c_int64, _VP]),
    "aila_nf4_forward_decode_static": (ctypes.c_int, [_VP, _VP, _VP, _VP, _VP]),
    "aila_nf4_static_check": (ctypes.c_int, [ctypes.c_int, _VP]),
    "aila_nf4_peerbuf_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                               ctypes.c_int64, ctypes.POINTER(_VP)]),
    "aila_nf4_peerbuf_export": (ctypes.c_int, [_VP, _VP]),
    "aila_nf4_peerbuf_import": (ctypes.c_int, [_VP, ctypes.c_int, _VP]),
    "aila_embedding_lookup": (ctypes.c_int, [_VP, ctypes.c_int64, _VP, ctypes.c_int, ctypes.c_int, _VP, ctypes.c_int, _VP]),
    "aila_decode_prepare_qkv": (ctypes.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, ctypes.c_int, ctypes.c_int, _VP,
                                                ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int,
                                                _VP]),
    "aila_attention_decode": (ctypes.c_int, [_VP, _VP, _VP, _VP, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              _VP, ctypes.c_int, ctypes.c_int, _VP]),
    "aila_nf4_peerbuf_import_local": (ctypes.c_int, [_VP, ctypes.c_int, _VP]),
    "aila_nf4_peerbuf_destroy": (None, [_VP]),
    "aila_nf4_forward_decode_allreduce": (ctypes.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    "aila_nf4_forward_rmsnorm": (ctypes.c_int, [_VP, _VP, _VP, ctypes.POINTER(RmsNorm), _VP, _VP, _VP]),
    "aila_nf4_forward_gate_up_swiglu_rmsnorm": (ctypes.c_int, [_VP, _VP, _VP, ctypes.POINTER(RmsNorm),
                                                               _VP, ctypes.c_int64, _VP]),
    "aila_add_rms_norm": (ctypes.c_int, [_VP, _VP, _VP, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                         _VP, _VP, ctypes.c_int, _VP]),
    "aila_dense_linear_create": (ctypes.c_int, [_VP, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                                ctypes.c_int, ctypes.POINTER(_VP)]),
    "aila_dense_linear_destroy": (None, [_VP]),
    "aila_dense_linear_in_features": (ctypes.c_int64, [_VP]),
    "aila_dense_linear_out_features": (ctypes.c_int64, [_VP]),
    "aila_dense_linear_forward": (ctypes.c_int, [_VP, _VP, _VP, _VP, ctypes.c_int, _VP, _VP]),
    "aila_argmax_bf16": (ctypes.c_int, [_VP, ctypes.c_int64, _VP, ctypes.c_int, _VP]),
    "aila_argmax_bf16_shard": (ctypes.c_int, [_VP, ctypes.c_int64, ctypes.c_int64, _VP, ctypes.c_int, _VP]),
    "aila_st_open": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(_VP)]),
    "aila_st_close": (None, [_VP]),
    "aila_st_tensor_count": (ctypes.c_int64, [_VP]),
    "aila_st_tensor_name": (ctypes.c_char_p, [_VP, ctypes.c_int64]),
    "aila_st_find": (ctypes.c_int, [_VP, ctypes.c_char_p, ctypes.POINTER(StTensorView)]),
    "aila_st_dir_open": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(_VP)]),
    "aila_st_dir_close": (None, [_VP]),
    "aila_st_dir_shard_count": (ctypes.c_int64, [_VP]),
    "aila_st_dir_shard": (_VP, [_VP, ctypes.c_int64]),
    "aila_st_dir_find": (ctypes.c_int, [_VP, ctypes.c_char_p, ctypes.POINTER(StTensorView)]),
    "aila_st_dir_load_bnb4_weight": (ctypes.c_int, [_VP, ctypes.c_char_p, ctypes.c_int,
                                                     ctypes.POINTER(WeightDesc)]),
    "aila_st_load_bnb4_weight": (ctypes.c_int, [_VP, ctypes.c_char_p, ctypes.c_int,
                                                ctypes.POINTER(WeightDesc)]),
    "aila_nf4_dequantize": (ctypes.c_int, [_VP, _VP, _VP]),
    "aila_nf4_dequantize_rowmajor": (ctypes.c_int, [_VP, _VP, _VP]),
    "aila_nf4_expand_absmax": (ctypes.c_int, [_VP, _VP, _VP]),
    "aila_nf4_set_gemv_kernel": (ctypes.c_int, [ctypes.c_int]),
    "aila_nf4_chain_create": (ctypes.c_int, [_VP, ctypes.POINTER(ChainOp), ctypes.c_int,
                                             ctypes.POINTER(_VP)]),
    "aila_nf4_chain_create_allreduce": (ctypes.c_int, [_VP, ctypes.POINTER(ChainOp), ctypes.c_int, _VP,
                                                        ctypes.POINTER(_VP)]),
    "aila_nf4_chain_destroy": (None, [_VP]),
    "aila_nf4_chain_length": (ctypes.c_int, [_VP]),
    "aila_nf4_chain_run": (ctypes.c_int, [_VP, _VP]),
    "aila_nf4_chain_run_host": (ctypes.c_int, [_VP, _VP, _VP, _VP]),
    "aila_nf4_scratch_set_wait_limit": (ctypes.c_int, [_VP, ctypes.c_int64]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def load() -> ctypes.CDLL:
    """Loads the library (once) and declares every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C aila_b200/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). "
            "There is no fallback implementation.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class Nf4Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"aila_nf4 status {status}: {message}")
        self.status = status


def check(status: int) -> None:
    if status != OK:
        raise Nf4Error(status, load().aila_nf4_last_error().decode("utf-8", "replace"))
