"""ctypes front-end of the reference's own NF4 operator built for the host (oracle/ref_harness.cpp
around src/ops/Bnb4BitLinear.cpp, against the stand-in runtime headers in oracle/ref_shim/).

TEST INFRASTRUCTURE ONLY: the tests use it to check the CPU oracle's restatement against the code
it restates. The library exists only where the reference's sources were present at build time;
``available()`` says whether it does, and the tests skip otherwise.

All tensors are numpy arrays; bf16 travels as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libaila_ref.so")


class _Weight(ctypes.Structure):
    _fields_ = [("packed", ctypes.c_void_p), ("absmax", ctypes.c_void_p), ("quant_map", ctypes.c_void_p),
                ("nested_absmax", ctypes.c_void_p), ("nested_quant_map", ctypes.c_void_p),
                ("nested_absmax_count", ctypes.c_int64), ("out_features", ctypes.c_int64),
                ("in_features", ctypes.c_int64), ("blocksize", ctypes.c_int32), ("nested", ctypes.c_int32),
                ("nested_blocksize", ctypes.c_int32), ("nested_offset", ctypes.c_float)]


class RefError(RuntimeError):
    pass


_lib = None


def available() -> bool:
    return os.path.exists(_SO)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_SO)
        for name in ("aila_ref_forward", "aila_ref_gate_up_swiglu", "aila_ref_expand_absmax", "aila_ref_dequantize"):
            getattr(_lib, name).restype = ctypes.c_int
    return _lib


def _desc(w, keep):
    """C descriptor of a synthetic weight (aila_b200.synth.Nf4Tensors); `keep` holds the arrays alive."""
    def hold(a, dtype):
        a = np.ascontiguousarray(a, dtype=dtype)
        keep.append(a)
        return a.ctypes.data
    d = _Weight()
    d.packed = hold(np.asarray(w.packed).reshape(-1), np.uint8)
    d.quant_map = hold(w.quant_map, np.float32)
    d.out_features, d.in_features, d.blocksize = w.out_features, w.in_features, w.blocksize
    d.nested = 1 if w.nested else 0
    if w.nested:
        d.absmax = hold(w.absmax_codes, np.uint8)
        d.nested_absmax = hold(w.nested_absmax, np.float32)
        d.nested_absmax_count = int(np.asarray(w.nested_absmax).size)
        d.nested_quant_map = hold(w.nested_quant_map, np.float32)
        d.nested_blocksize = w.nested_blocksize
        d.nested_offset = float(w.nested_offset)
    else:
        d.absmax = hold(w.absmax_f32, np.float32)
    return d


def _check(rc, err):
    if rc < 0:
        raise RefError(err.value.decode("utf-8", "replace"))
    return rc


def forward(weights, x_bf16, M, residual=None) -> np.ndarray:
    """Bnb4BitLinear::forward on one weight, or on init_fused_rows of a list of 2..4 weights."""
    ws = list(weights) if isinstance(weights, (list, tuple)) else [weights]
    keep = []
    arr = (_Weight * len(ws))(*[_desc(w, keep) for w in ws])
    K = ws[0].in_features
    N = sum(w.out_features for w in ws)
    x = np.ascontiguousarray(x_bf16, np.uint16).reshape(M, K)
    y = np.zeros((M, N), np.uint16)
    res = None
    if residual is not None:
        res = np.ascontiguousarray(residual, np.uint16).reshape(M, N)
    err = ctypes.create_string_buffer(512)
    _check(lib().aila_ref_forward(arr, ctypes.c_int(len(ws)), x.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(M),
                                  y.ctypes.data_as(ctypes.c_void_p),
                                  res.ctypes.data_as(ctypes.c_void_p) if res is not None else None, err,
                                  ctypes.c_int(512)), err)
    return y


def gate_up_swiglu(gate, up, x_bf16, ff):
    """try_forward_decode_gate_up_swiglu on init_fused_rows(gate, up): the output, or None when the
    reference declined the fused route."""
    keep = []
    g, u = _desc(gate, keep), _desc(up, keep)
    x = np.ascontiguousarray(x_bf16, np.uint16).reshape(-1)
    out = np.zeros(ff, np.uint16)
    err = ctypes.create_string_buffer(512)
    rc = _check(lib().aila_ref_gate_up_swiglu(ctypes.byref(g), ctypes.byref(u), x.ctypes.data_as(ctypes.c_void_p),
                                              ctypes.c_int(ff), out.ctypes.data_as(ctypes.c_void_p), err,
                                              ctypes.c_int(512)), err)
    return out if rc == 1 else None


def expand_absmax(w) -> np.ndarray:
    keep = []
    d = _desc(w, keep)
    blocks = (w.out_features * w.in_features + w.blocksize - 1) // w.blocksize
    out = np.zeros(blocks, np.float32)
    err = ctypes.create_string_buffer(512)
    _check(lib().aila_ref_expand_absmax(ctypes.byref(d), out.ctypes.data_as(ctypes.c_void_p), err, ctypes.c_int(512)),
           err)
    return out


def dequantize_kn(w) -> np.ndarray:
    keep = []
    d = _desc(w, keep)
    out = np.zeros((w.in_features, w.out_features), np.uint16)
    err = ctypes.create_string_buffer(512)
    _check(lib().aila_ref_dequantize(ctypes.byref(d), out.ctypes.data_as(ctypes.c_void_p), err, ctypes.c_int(512)),
           err)
    return out


# ---------------------------------------------------------------- operators around the linears
def _u16(a):
    return np.ascontiguousarray(a, np.uint16)


def _vp(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _run(name, *args):
    err = ctypes.create_string_buffer(512)
    fn = getattr(lib(), name)
    fn.restype = ctypes.c_int
    _check(fn(*args, err, ctypes.c_int(512)), err)


def rms_norm(x_bf16, weight_bf16, eps, M, H) -> np.ndarray:
    x, w = _u16(x_bf16).reshape(M, H).copy(), _u16(weight_bf16).reshape(H).copy()
    out = np.zeros((M, H), np.uint16)
    _run("aila_ref_rms_norm", _vp(x), _vp(w), ctypes.c_float(eps), _vp(out), ctypes.c_int(M), ctypes.c_int(H))
    return out


def fused_add_rms_norm(x_bf16, residual_bf16, weight_bf16, eps, M, H):
    """(hidden, normed): the reference updates its input in place; here the input is copied first."""
    x, r = _u16(x_bf16).reshape(M, H).copy(), _u16(residual_bf16).reshape(M, H).copy()
    w = _u16(weight_bf16).reshape(H).copy()
    out = np.zeros((M, H), np.uint16)
    _run("aila_ref_fused_add_rms_norm", _vp(x), _vp(r), _vp(w), ctypes.c_float(eps), _vp(out), ctypes.c_int(M),
         ctypes.c_int(H))
    return x, out


def embedding_lookup(table_bf16, token_ids) -> np.ndarray:
    t = _u16(table_bf16).copy()
    ids = np.ascontiguousarray(token_ids, np.int32)
    out = np.zeros((ids.size, t.shape[1]), np.uint16)
    _run("aila_ref_embedding_lookup", _vp(t), ctypes.c_int(t.shape[0]), _vp(ids), ctypes.c_int(ids.size), _vp(out),
         ctypes.c_int(t.shape[1]))
    return out


def decode_prepare_qkv(q_bf16, k_bf16, v_bf16, freq, q_norm_w, k_norm_w, k_cache, v_cache, pos, n_heads, n_kv,
                       head_dim, eps, theta=1e6) -> np.ndarray:
    """Returns the rotated q; k_cache / v_cache ([n_kv, max_len, head_dim] uint16) are updated in place."""
    q, k, v = _u16(q_bf16).reshape(-1).copy(), _u16(k_bf16).reshape(-1).copy(), _u16(v_bf16).reshape(-1).copy()
    f = np.ascontiguousarray(freq, np.float32).copy()
    qn, kn = _u16(q_norm_w).copy(), _u16(k_norm_w).copy()
    assert k_cache.dtype == np.uint16 and k_cache.flags.c_contiguous and v_cache.flags.c_contiguous
    _run("aila_ref_decode_prepare_qkv", _vp(q), _vp(k), _vp(v), _vp(f), _vp(qn), _vp(kn), _vp(k_cache), _vp(v_cache),
         ctypes.c_int(k_cache.shape[1]), ctypes.c_int(pos), ctypes.c_int(n_heads), ctypes.c_int(n_kv),
         ctypes.c_int(head_dim), ctypes.c_float(eps), ctypes.c_float(theta))
    return q


def swiglu(gate_bf16, up_bf16) -> np.ndarray:
    g, u = _u16(gate_bf16).reshape(-1).copy(), _u16(up_bf16).reshape(-1).copy()
    out = np.zeros(g.size, np.uint16)
    _run("aila_ref_swiglu", _vp(g), _vp(u), _vp(out), ctypes.c_int(g.size))
    return out


def fused_gate_up_swiglu(gate_up_bf16, ff) -> np.ndarray:
    gu = _u16(gate_up_bf16).reshape(-1).copy()
    out = np.zeros(ff, np.uint16)
    _run("aila_ref_fused_gate_up_swiglu", _vp(gu), _vp(out), ctypes.c_int(ff))
    return out


def argmax(logits_bf16) -> int:
    l = _u16(logits_bf16).reshape(-1).copy()
    out = np.zeros(1, np.int32)
    _run("aila_ref_argmax", _vp(l), ctypes.c_int(l.size), _vp(out))
    return int(out[0])


def attention_decode(q_bf16, k_cache, v_cache, n_heads, n_kv, head_dim, cached_len) -> np.ndarray:
    q = _u16(q_bf16).reshape(-1).copy()
    kc, vc = _u16(k_cache).copy(), _u16(v_cache).copy()
    out = np.zeros(n_heads * head_dim, np.uint16)
    _run("aila_ref_attention_decode", _vp(q), _vp(kc), _vp(vc), _vp(out), ctypes.c_int(kc.shape[1]),
         ctypes.c_int(n_heads), ctypes.c_int(n_kv), ctypes.c_int(head_dim), ctypes.c_int(cached_len))
    return out
