"""Checkpoint front-end: memory-mapped safetensors files and bitsandbytes 4-bit weight views.

Python face of ``aila_st_*`` (include/aila_nf4.h). ``SafetensorsFile.load_bnb4_weight_ref`` plays
the role of the reference's ``LoadBnb4BitWeightRef`` (src/utils/SafeTensors.cpp:370-489): it
collects ``<w>.absmax``, ``<w>.quant_map``, ``<w>.nested_absmax``, ``<w>.nested_quant_map`` and
``<w>.quant_state.bitsandbytes__nf4``, applies the same dtype and size rules and returns a
descriptor whose pointers lie inside the mapping, so ``Bnb4BitLinear.init_from_desc`` uploads the
weight straight into its device layout. Parsing is native code; there is no Python fallback.

``write_safetensors`` writes the same file format from numpy arrays (for fixtures and exports).
"""
from __future__ import annotations

import ctypes
import json
import struct

import numpy as np

from . import _lib
from .synth import Nf4Tensors

_NP_TO_ST = {np.dtype(np.uint8): "U8", np.dtype(np.int8): "I8", np.dtype(np.float16): "F16",
             np.dtype(np.float32): "F32", np.dtype(np.float64): "F64", np.dtype(np.int32): "I32",
             np.dtype(np.int64): "I64", np.dtype(np.bool_): "BOOL"}
_ST_TO_NP = {v: k for k, v in _NP_TO_ST.items()}
_ST_TO_NP["BF16"] = np.dtype(np.uint16)  # raw bits


class SafetensorsFile:
    """One memory-mapped ``.safetensors`` file. Tensor data stays valid until ``close``."""

    def __init__(self, path: str):
        self._h = ctypes.c_void_p()
        self.path = str(path)
        _lib.check(_lib.load().aila_st_open(self.path.encode(), ctypes.byref(self._h)))

    def close(self) -> None:
        if self._h:
            _lib.load().aila_st_close(self._h)
            self._h = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def names(self) -> list[str]:
        lib = _lib.load()
        return [lib.aila_st_tensor_name(self._h, i).decode() for i in
                range(lib.aila_st_tensor_count(self._h))]

    def has(self, name: str) -> bool:
        view = _lib.StTensorView()
        st = _lib.load().aila_st_find(self._h, name.encode(), ctypes.byref(view))
        if st == _lib.NOT_APPLICABLE:
            return False
        _lib.check(st)
        return True

    def get(self, name: str) -> np.ndarray:
        """A copy of the tensor as a numpy array (bf16 comes back as raw uint16 bits)."""
        view = _lib.StTensorView()
        _lib.check(_lib.load().aila_st_find(self._h, name.encode(), ctypes.byref(view)))
        dt = _ST_TO_NP[_lib.ST_DTYPES[view.dtype]]
        shape = tuple(view.shape[i] for i in range(view.rank))
        raw = ctypes.string_at(view.data, view.nbytes) if view.nbytes else b""
        return np.frombuffer(raw, dtype=dt).reshape(shape).copy()

    def load_bnb4_weight_ref(self, name: str, device: int = 0) -> _lib.WeightDesc:
        """The checked descriptor of weight ``name``; raises ``Nf4Error`` with the violated rule."""
        desc = _lib.WeightDesc()
        _lib.check(_lib.load().aila_st_load_bnb4_weight(self._h, name.encode(), int(device),
                                                        ctypes.byref(desc)))
        return desc


class ModelDir:
    """A model directory: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` names (reference LoadModelWeightsFromDir,
    src/utils/SafeTensors.cpp:491-535). Tensor data stays valid until ``close``."""

    def __init__(self, path: str):
        self._h = ctypes.c_void_p()
        self.path = str(path)
        _lib.check(_lib.load().aila_st_dir_open(self.path.encode(), ctypes.byref(self._h)))

    def close(self) -> None:
        if self._h:
            _lib.load().aila_st_dir_close(self._h)
            self._h = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def shard_count(self) -> int:
        return int(_lib.load().aila_st_dir_shard_count(self._h))

    def names(self) -> list[str]:
        lib = _lib.load()
        seen: dict[str, None] = {}
        for i in range(self.shard_count()):
            f = lib.aila_st_dir_shard(self._h, i)
            for j in range(lib.aila_st_tensor_count(f)):
                seen[lib.aila_st_tensor_name(f, j).decode()] = None
        return list(seen)

    def has(self, name: str) -> bool:
        view = _lib.StTensorView()
        st = _lib.load().aila_st_dir_find(self._h, name.encode(), ctypes.byref(view))
        if st == _lib.NOT_APPLICABLE:
            return False
        _lib.check(st)
        return True

    def get(self, name: str) -> np.ndarray:
        view = _lib.StTensorView()
        _lib.check(_lib.load().aila_st_dir_find(self._h, name.encode(), ctypes.byref(view)))
        dt = _ST_TO_NP[_lib.ST_DTYPES[view.dtype]]
        shape = tuple(view.shape[i] for i in range(view.rank))
        raw = ctypes.string_at(view.data, view.nbytes) if view.nbytes else b""
        return np.frombuffer(raw, dtype=dt).reshape(shape).copy()

    def load_bnb4_weight_ref(self, name: str, device: int = 0) -> _lib.WeightDesc:
        desc = _lib.WeightDesc()
        _lib.check(_lib.load().aila_st_dir_load_bnb4_weight(self._h, name.encode(), int(device),
                                                            ctypes.byref(desc)))
        return desc


def write_safetensors(path: str, tensors: dict[str, np.ndarray],
                      metadata: dict[str, str] | None = None) -> None:
    """Writes ``tensors`` in safetensors layout: u64 header length, JSON header, tensor bytes."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    blobs = []
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        blob = arr.tobytes()
        header[name] = {"dtype": _NP_TO_ST[arr.dtype], "shape": list(arr.shape),
                        "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)  # the data section starts on an 8-byte boundary
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for blob in blobs:
            f.write(blob)


def bnb4_checkpoint_tensors(name: str, w: Nf4Tensors) -> dict[str, np.ndarray]:
    """The tensors a bitsandbytes NF4 export holds for one weight (names and dtypes as the
    reference's loader expects them, src/utils/SafeTensors.cpp:383-387)."""
    state = {"quant_type": "nf4", "blocksize": int(w.blocksize), "dtype": "bfloat16",
             "shape": [int(w.out_features), int(w.in_features)]}
    out = {name: np.asarray(w.packed, dtype=np.uint8).reshape(-1, 1),
           name + ".quant_map": np.asarray(w.quant_map, dtype=np.float32)}
    if w.nested:
        state.update(nested_blocksize=int(w.nested_blocksize), nested_dtype="float32",
                     nested_offset=float(w.nested_offset))
        out[name + ".absmax"] = np.asarray(w.absmax_codes, dtype=np.uint8)
        out[name + ".nested_absmax"] = np.asarray(w.nested_absmax, dtype=np.float32)
        out[name + ".nested_quant_map"] = np.asarray(w.nested_quant_map, dtype=np.float32)
    else:
        out[name + ".absmax"] = np.asarray(w.absmax_f32, dtype=np.float32)
    out[name + ".quant_state.bitsandbytes__nf4"] = np.frombuffer(
        json.dumps(state).encode(), dtype=np.uint8).copy()
    return out
