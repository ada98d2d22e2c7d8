"""CPU checks of the C-ABI boundary: the library loads without a GPU, exports every symbol
include/aila_nf4.h declares, and rejects bad descriptors on the host before touching CUDA."""
import ctypes
import os
import re

import numpy as np
import pytest

from aila_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    return _lib.load()


def test_header_and_binding_agree(lib):
    text = open(os.path.join(ROOT, "include", "aila_nf4.h")).read()
    declared = set(re.findall(r"\b(aila_(?:nf4|st|dense|argmax|add|embedding|decode|attention)_[a-z0-9_]+)\s*\(", text))
    assert declared == set(_lib.EXPORTED_SYMBOLS), declared ^ set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_version(lib):
    assert lib.aila_nf4_version() >= 100


def _desc(**kw):
    d = _lib.WeightDesc()
    keep = [np.zeros(64 * 64 // 2, np.uint8), np.zeros(64, np.uint8), np.zeros(16, np.float32),
            np.zeros(1, np.float32), np.zeros(256, np.float32)]
    d.out_features, d.in_features, d.blocksize = 64, 64, 64
    d.nested, d.nested_blocksize, d.nested_offset = 1, 256, 0.0
    d.packed_weight, d.absmax, d.quant_map = keep[0].ctypes.data, keep[1].ctypes.data, keep[2].ctypes.data
    d.nested_absmax, d.nested_quant_map = keep[3].ctypes.data, keep[4].ctypes.data
    d.nested_absmax_count, d.pointers_on_device, d.device = 1, 0, 0
    for k, v in kw.items():
        setattr(d, k, v)
    return d, keep


@pytest.mark.parametrize("kw,status,needle", [
    (dict(out_features=0), _lib.ERR_INVALID_ARGUMENT, "shape"),
    (dict(packed_weight=None), _lib.ERR_INVALID_ARGUMENT, "side tensors"),
    (dict(blocksize=0), _lib.ERR_INVALID_ARGUMENT, "blocksize"),
    (dict(blocksize=32), _lib.ERR_UNSUPPORTED, "blocksize"),
    (dict(in_features=96), _lib.ERR_UNSUPPORTED, "multiple of blocksize"),
    (dict(nested_absmax=None), _lib.ERR_INVALID_ARGUMENT, "nested"),
    (dict(nested_blocksize=0), _lib.ERR_INVALID_ARGUMENT, "nested blocksize"),
    (dict(nested_absmax_count=7), _lib.ERR_INVALID_ARGUMENT, "nested_absmax length"),
])
def test_descriptor_validation_on_host(lib, kw, status, needle):
    d, keep = _desc(**kw)
    h = ctypes.c_void_p()
    st = lib.aila_nf4_linear_create(ctypes.byref(d), ctypes.byref(h))
    assert st == status
    assert needle in lib.aila_nf4_last_error().decode()
    assert not h.value


def test_shard_argument_validation(lib):
    d, keep = _desc()
    h = ctypes.c_void_p()
    assert lib.aila_nf4_linear_create_shard(ctypes.byref(d), 0, 3, 2, ctypes.byref(h)) == \
        _lib.ERR_INVALID_ARGUMENT
    assert lib.aila_nf4_linear_create_shard(ctypes.byref(d), 1, 0, 2, ctypes.byref(h)) == \
        _lib.ERR_INVALID_ARGUMENT  # 64 / 2 is not a multiple of blocksize
    assert lib.aila_nf4_linear_create_shard(ctypes.byref(d), 0, 0, 3, ctypes.byref(h)) == \
        _lib.ERR_INVALID_ARGUMENT  # 64 rows not divisible by 3


def test_null_handles_are_rejected(lib):
    assert lib.aila_nf4_forward(None, None, None, None, 1, None, None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.aila_nf4_linear_in_features(None) == 0
    assert lib.aila_nf4_linear_out_features(None) == 0
    lib.aila_nf4_linear_destroy(None)
    lib.aila_nf4_scratch_destroy(None)
    assert lib.aila_nf4_set_gemv_kernel(7) == _lib.ERR_INVALID_ARGUMENT
    assert lib.aila_nf4_set_gemv_kernel(0) == _lib.OK


def test_no_cpu_fallback_without_a_gpu(lib):
    """On a machine without a CUDA device creation fails loudly with a CUDA error."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA device present")
    d, keep = _desc()
    h = ctypes.c_void_p()
    st = lib.aila_nf4_linear_create(ctypes.byref(d), ctypes.byref(h))
    assert st in (_lib.ERR_CUDA, _lib.ERR_INVALID_ARGUMENT) and not h.value
    s = ctypes.c_void_p()
    assert lib.aila_nf4_scratch_create(0, ctypes.byref(s)) != _lib.OK
