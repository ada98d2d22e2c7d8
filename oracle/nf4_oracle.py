"""ctypes front-end of the CPU oracle (oracle/nf4_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of bench.py, never by the shipped package.

All tensors are numpy arrays; bf16 travels as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libnf4_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile; returns the library path."""
    src = os.path.join(_HERE, "nf4_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.nf4o_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().nf4o_num_threads())


def set_num_threads(n: int) -> None:
    lib().nf4o_set_num_threads(ctypes.c_int(n))


def f32_to_bf16(a) -> np.ndarray:
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    lib().nf4o_f32_to_bf16(_p(a), ctypes.c_int64(a.size), _p(out))
    return out


def bf16_to_f32(a) -> np.ndarray:
    a = _c(a, np.uint16)
    out = np.empty(a.shape, np.float32)
    lib().nf4o_bf16_to_f32(_p(a), ctypes.c_int64(a.size), _p(out))
    return out


def expand_absmax(codes, nested_map, nested_absmax, nested_blocksize, nested_offset,
                  flat_base: int = 0, fused: bool = False) -> np.ndarray:
    codes = _c(codes, np.uint8).reshape(-1)
    nested_map = _c(nested_map, np.float32)
    nested_absmax = _c(nested_absmax, np.float32)
    out = np.empty(codes.size, np.float32)
    fn = lib().nf4o_expand_absmax_fused if fused else lib().nf4o_expand_absmax
    fn(_p(codes), ctypes.c_int64(codes.size), _p(nested_map), _p(nested_absmax),
       ctypes.c_int(nested_blocksize), ctypes.c_float(nested_offset),
       ctypes.c_int64(flat_base), _p(out))
    return out


def dequantize_kn(packed, qmap, absmax, N, K, blocksize) -> np.ndarray:
    """bf16 bits of the transposed weight, shape [K, N] (the reference's layout)."""
    packed = _c(packed, np.uint8).reshape(-1)
    out = np.empty((K, N), np.uint16)
    lib().nf4o_dequantize_kn(_p(packed), _p(_c(qmap, np.float32)), _p(_c(absmax, np.float32)),
                             ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(blocksize),
                             _p(out))
    return out


def dequantize_nk(packed, qmap, absmax, N, K, blocksize) -> np.ndarray:
    packed = _c(packed, np.uint8).reshape(-1)
    out = np.empty((N, K), np.uint16)
    lib().nf4o_dequantize_nk(_p(packed), _p(_c(qmap, np.float32)), _p(_c(absmax, np.float32)),
                             ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(blocksize),
                             _p(out))
    return out


def gemv(packed, qmap, absmax, x_bf16, N, K, blocksize, residual=None) -> np.ndarray:
    packed = _c(packed, np.uint8).reshape(-1)
    x = _c(x_bf16, np.uint16).reshape(-1)
    assert x.size == K
    y = np.empty(N, np.uint16)
    res = None
    if residual is not None:
        res = _c(residual, np.uint16).reshape(-1)
        assert res.size == N
    lib().nf4o_gemv(_p(packed), _p(_c(qmap, np.float32)), _p(_c(absmax, np.float32)), _p(x),
                    ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(blocksize),
                    _p(res) if res is not None else None, _p(y))
    return y


def gemv_f32(packed, qmap, absmax, x_bf16, N, K, blocksize) -> np.ndarray:
    packed = _c(packed, np.uint8).reshape(-1)
    x = _c(x_bf16, np.uint16).reshape(-1)
    y = np.empty(N, np.float32)
    lib().nf4o_gemv_f32(_p(packed), _p(_c(qmap, np.float32)), _p(_c(absmax, np.float32)),
                        _p(x), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(blocksize),
                        _p(y))
    return y


def gemv_gate_up_swiglu(packed, qmap, absmax, x_bf16, ff, K, blocksize) -> np.ndarray:
    packed = _c(packed, np.uint8).reshape(-1)
    x = _c(x_bf16, np.uint16).reshape(-1)
    out = np.empty(ff, np.uint16)
    lib().nf4o_gemv_gate_up_swiglu(_p(packed), _p(_c(qmap, np.float32)),
                                   _p(_c(absmax, np.float32)), _p(x), ctypes.c_int64(ff),
                                   ctypes.c_int64(K), ctypes.c_int(blocksize), _p(out))
    return out


def gemm_bf16w(w_nk_bf16, x_mk_bf16, M, N, K) -> np.ndarray:
    w = _c(w_nk_bf16, np.uint16).reshape(N, K)
    x = _c(x_mk_bf16, np.uint16).reshape(M, K)
    y = np.empty((M, N), np.uint16)
    lib().nf4o_gemm_bf16w(_p(w), _p(x), ctypes.c_int64(M), ctypes.c_int64(N),
                          ctypes.c_int64(K), _p(y))
    return y


def swiglu_rows(gate_up_bf16, M, ff) -> np.ndarray:
    gu = _c(gate_up_bf16, np.uint16).reshape(M, 2 * ff)
    out = np.empty((M, ff), np.uint16)
    lib().nf4o_swiglu_rows(_p(gu), ctypes.c_int64(M), ctypes.c_int64(ff), _p(out))
    return out


def add_rms_norm(x_bf16, residual_bf16, weight_bf16, eps, M, H):
    """(hidden_out, normed) of ops::fused_add_rms_norm (NormOps.cpp:141-260); residual may be None."""
    x = _c(x_bf16, np.uint16).reshape(M, H)
    r = _c(residual_bf16, np.uint16).reshape(M, H) if residual_bf16 is not None else None
    w = _c(weight_bf16, np.uint16).reshape(H)
    hidden = np.empty((M, H), np.uint16)
    normed = np.empty((M, H), np.uint16)
    lib().nf4o_add_rms_norm(_p(x), _p(r) if r is not None else None, _p(w), ctypes.c_float(eps),
                            ctypes.c_int64(M), ctypes.c_int64(H), _p(hidden), _p(normed))
    return hidden, normed


def forward(packed, qmap, absmax, x_bf16, M, N, K, blocksize) -> np.ndarray:
    """What Bnb4BitLinear::forward (Bnb4BitLinear.cpp:799-949) returns for [M,K] input:
    the decode GEMV for M == 1 (:813-818), otherwise bf16-rounded weights followed by a
    bf16 GEMM with fp32 accumulation (:839-948)."""
    if M == 1:
        return gemv(packed, qmap, absmax, x_bf16, N, K, blocksize).reshape(1, N)
    w = dequantize_nk(packed, qmap, absmax, N, K, blocksize)
    return gemm_bf16w(w, x_bf16, M, N, K)
