"""Checkpoint front-end (aila_st_*): safetensors parsing and the bitsandbytes weight view.

CPU-only: these calls do no GPU work. The rules mirror the reference's LoadBnb4BitWeightRef
(src/utils/SafeTensors.cpp:370-489): side-tensor names, dtype rules, size invariants and the
quant_state JSON keys; every violated rule must be reported, never patched over.
"""
import ctypes
import json
import struct

import numpy as np
import pytest

from aila_b200 import _lib, checkpoint
from tests.helpers import make_weight


def _write(tmp_path, tensors, name="model.safetensors"):
    path = tmp_path / name
    checkpoint.write_safetensors(str(path), tensors, metadata={"format": "pt"})
    return str(path)


def _array_at(ptr, dtype, count):
    raw = ctypes.string_at(ptr, count * np.dtype(dtype).itemsize)
    return np.frombuffer(raw, dtype=dtype)


@pytest.mark.parametrize("nested", [True, False])
def test_weight_view_matches_the_tensors(tmp_path, nested):
    w = make_weight(7, 48, 256, 64, nested)
    other = make_weight(8, 16, 128, 64, True)
    tensors = {"embed.weight": np.arange(12, dtype=np.float32).reshape(3, 4)}
    tensors.update(checkpoint.bnb4_checkpoint_tensors("model.layers.0.mlp.down_proj.weight", w))
    tensors.update(checkpoint.bnb4_checkpoint_tensors("model.layers.0.mlp.up_proj.weight", other))
    with checkpoint.SafetensorsFile(_write(tmp_path, tensors)) as f:
        assert f.names() == list(tensors)
        assert f.has("embed.weight") and not f.has("nope")
        assert np.array_equal(f.get("embed.weight"), tensors["embed.weight"])
        d = f.load_bnb4_weight_ref("model.layers.0.mlp.down_proj.weight", device=3)
        assert (d.out_features, d.in_features, d.blocksize) == (48, 256, 64)
        assert d.nested == (1 if nested else 0) and d.pointers_on_device == 0 and d.device == 3
        assert np.array_equal(_array_at(d.packed_weight, np.uint8, 48 * 256 // 2), w.packed)
        assert np.array_equal(_array_at(d.quant_map, np.float32, 16), w.quant_map)
        blocks = 48 * 256 // 64
        if nested:
            assert d.nested_blocksize == w.nested_blocksize
            assert d.nested_offset == np.float32(w.nested_offset)
            assert np.array_equal(_array_at(d.absmax, np.uint8, blocks), w.absmax_codes)
            assert d.nested_absmax_count == w.nested_absmax.size
            assert np.array_equal(_array_at(d.nested_absmax, np.float32, w.nested_absmax.size),
                                  w.nested_absmax)
            assert np.array_equal(_array_at(d.nested_quant_map, np.float32, 256), w.nested_quant_map)
        else:
            assert np.array_equal(_array_at(d.absmax, np.float32, blocks), w.absmax_f32)
            assert not d.nested_absmax and not d.nested_quant_map


def _broken(tmp_path, mutate, nested=True):
    w = make_weight(9, 32, 128, 64, nested)
    tensors = checkpoint.bnb4_checkpoint_tensors("w", w)
    mutate(tensors)
    f = checkpoint.SafetensorsFile(_write(tmp_path, tensors))
    try:
        with pytest.raises(_lib.Nf4Error) as e:
            f.load_bnb4_weight_ref("w")
        return str(e.value)
    finally:
        f.close()


def _set_state(tensors, **changes):
    key = "w.quant_state.bitsandbytes__nf4"
    state = json.loads(bytes(tensors[key]).decode())
    for k, v in changes.items():
        if v is None:
            state.pop(k, None)
        else:
            state[k] = v
    tensors[key] = np.frombuffer(json.dumps(state).encode(), dtype=np.uint8).copy()


def test_rules_of_the_weight_view(tmp_path):
    assert "Missing bitsandbytes packed weight" in _broken(tmp_path, lambda t: t.pop("w"))
    assert "Missing required bitsandbytes side tensors" in _broken(tmp_path, lambda t: t.pop("w.absmax"))
    assert "side tensors" in _broken(tmp_path, lambda t: t.pop("w.quant_map"))
    assert "side tensors" in _broken(tmp_path, lambda t: t.pop("w.quant_state.bitsandbytes__nf4"))
    assert "packed weight must be uint8" in _broken(
        tmp_path, lambda t: t.__setitem__("w", t["w"].astype(np.int8)))
    assert "quant_map must be float32" in _broken(
        tmp_path, lambda t: t.__setitem__("w.quant_map", t["w.quant_map"].astype(np.float64)))
    assert "absmax must be uint8 or float32" in _broken(
        tmp_path, lambda t: t.__setitem__("w.absmax", t["w.absmax"].astype(np.int32)))
    assert "missing blocksize" in _broken(tmp_path, lambda t: _set_state(t, blocksize=None))
    assert "missing shape" in _broken(tmp_path, lambda t: _set_state(t, shape=None))
    assert "non-integer" in _broken(tmp_path, lambda t: _set_state(t, shape=[32, 128.5]))
    assert "Invalid bitsandbytes weight view" in _broken(tmp_path, lambda t: _set_state(t, shape=[4096]))
    assert "Only NF4" in _broken(tmp_path, lambda t: _set_state(t, quant_type="fp4"))
    assert "blocksize must be positive" in _broken(tmp_path, lambda t: _set_state(t, blocksize=0))
    assert "does not match logical shape" in _broken(tmp_path, lambda t: _set_state(t, shape=[32, 256]))
    assert "absmax length" in _broken(tmp_path, lambda t: _set_state(t, blocksize=128))
    assert "at least 16" in _broken(
        tmp_path, lambda t: t.__setitem__("w.quant_map", t["w.quant_map"][:8].copy()))
    assert "nested quantization tensors are missing" in _broken(
        tmp_path, lambda t: t.pop("w.nested_absmax"))
    assert "nested tensors must be float32" in _broken(
        tmp_path, lambda t: t.__setitem__("w.nested_quant_map", t["w.nested_quant_map"].astype(np.float64)))
    assert "nested blocksize must be positive" in _broken(tmp_path, lambda t: _set_state(t, nested_blocksize=0))
    assert "nested_absmax length" in _broken(tmp_path, lambda t: _set_state(t, nested_blocksize=16))
    assert "Non-nested bitsandbytes absmax must be float32" in _broken(
        tmp_path, lambda t: t.__setitem__("w.absmax", (t["w.absmax"] * 0).astype(np.uint8)), nested=False)
    assert "parse bitsandbytes quant_state failed" in _broken(
        tmp_path, lambda t: t.__setitem__("w.quant_state.bitsandbytes__nf4",
                                          np.frombuffer(b'{"quant_type": "nf4", ', dtype=np.uint8).copy()))


def test_malformed_files_are_rejected(tmp_path):
    def expect(blob, text):
        p = tmp_path / "bad.safetensors"
        p.write_bytes(blob)
        with pytest.raises(_lib.Nf4Error) as e:
            checkpoint.SafetensorsFile(str(p))
        assert text in str(e.value)

    with pytest.raises(_lib.Nf4Error):
        checkpoint.SafetensorsFile(str(tmp_path / "missing.safetensors"))
    expect(b"\x01\x02", "shorter than")
    expect(struct.pack("<Q", 1 << 40) + b"{}", "header length")
    expect(struct.pack("<Q", 2) + b"[]", "not a JSON object")
    expect(struct.pack("<Q", 5) + b"{\"a\":", "not valid JSON")
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    expect(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8, "outside the file")
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}).encode()
    expect(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16, "do not match")
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4]}}).encode()
    expect(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16, "lacks dtype, shape or data_offsets")
    # a shape whose product wraps around 2^64 to the byte range's size must not pass
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [1 << 62, 4, 1 << 60, 16],
                            "data_offsets": [0, 16]}}).encode()
    expect(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16, "shape overflows")


def test_header_escapes_and_empty_tensors(tmp_path):
    tensors = {'odd "name"\\with\tescapes \u00e9': np.zeros((0, 4), dtype=np.float32),
               "b": np.array([1, 2, 3], dtype=np.int64)}
    with checkpoint.SafetensorsFile(_write(tmp_path, tensors)) as f:
        assert f.names() == list(tensors)
        assert f.get('odd "name"\\with\tescapes \u00e9').shape == (0, 4)
        assert np.array_equal(f.get("b"), tensors["b"])


def _index(tmp_path, weight_map, **extra):
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map, **extra}))


def test_model_directory_single_file_and_shards(tmp_path):
    """LoadModelWeightsFromDir (SafeTensors.cpp:491-535): model.safetensors wins; otherwise the
    shards of the index, sorted; a weight's side tensors may sit in another shard than its bytes; a
    tensor held by two shards comes from the last one."""
    wa, wb = make_weight(11, 32, 128), make_weight(12, 48, 64, nested=False)
    ta, tb = checkpoint.bnb4_checkpoint_tensors("a.weight", wa), checkpoint.bnb4_checkpoint_tensors("b.weight", wb)
    single = tmp_path / "single"
    single.mkdir()
    checkpoint.write_safetensors(str(single / "model.safetensors"), {**ta, **tb})
    with checkpoint.ModelDir(str(single)) as d:
        assert d.shard_count() == 1 and d.has("a.weight") and not d.has("c.weight")
        assert d.load_bnb4_weight_ref("b.weight").out_features == 48
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    # shard 1: a's packed bytes and b; shard 2: a's side tensors and a second copy of "dup"
    first = {"a.weight": ta["a.weight"], **tb, "dup": np.full(4, 1.0, np.float32)}
    second = {k: v for k, v in ta.items() if k != "a.weight"}
    second["dup"] = np.full(4, 2.0, np.float32)
    checkpoint.write_safetensors(str(sharded / "model-00001-of-00002.safetensors"), first)
    checkpoint.write_safetensors(str(sharded / "model-00002-of-00002.safetensors"), second)
    wm = {k: "model-00001-of-00002.safetensors" for k in first}
    wm.update({k: "model-00002-of-00002.safetensors" for k in second})
    _index(sharded, wm)
    with checkpoint.ModelDir(str(sharded)) as d:
        assert d.shard_count() == 2
        assert set(d.names()) == set(first) | set(second)
        desc = d.load_bnb4_weight_ref("a.weight")
        assert (desc.out_features, desc.in_features, desc.nested) == (32, 128, 1)
        assert np.array_equal(_array_at(desc.packed_weight, np.uint8, 32 * 128 // 2), np.asarray(wa.packed))
        assert np.array_equal(_array_at(desc.absmax, np.uint8, 32 * 2), np.asarray(wa.absmax_codes))
        assert np.array_equal(_array_at(desc.nested_absmax, np.float32, desc.nested_absmax_count),
                              np.asarray(wa.nested_absmax))
        assert d.load_bnb4_weight_ref("b.weight").nested == 0
        assert np.array_equal(d.get("dup"), np.full(4, 2.0, np.float32))
        with pytest.raises(_lib.Nf4Error, match="Missing bitsandbytes packed weight tensor"):
            d.load_bnb4_weight_ref("c.weight")


def test_model_directory_errors(tmp_path):
    def expect(text):
        with pytest.raises(_lib.Nf4Error) as e:
            checkpoint.ModelDir(str(tmp_path))
        assert text in str(e.value)

    expect("No model.safetensors or model.safetensors.index.json found in")
    (tmp_path / "model.safetensors.index.json").write_text("")
    expect("Empty or unreadable safetensors index")
    (tmp_path / "model.safetensors.index.json").write_text("[1, 2]")
    expect("Invalid safetensors index")
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}}))
    expect("missing weight_map")
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": [1]}))
    expect("weight_map is not an object")
    _index(tmp_path, {})
    expect("No shard entries found in")
    _index(tmp_path, {"t": "model-00001-of-00001.safetensors"})
    expect("Missing safetensors shard")
    _index(tmp_path, {"t": "../elsewhere.safetensors"})
    expect("Missing safetensors shard")
    checkpoint.write_safetensors(str(tmp_path / "model-00001-of-00001.safetensors"), {"t": np.zeros(3, np.float32)})
    _index(tmp_path, {"t": "model-00001-of-00001.safetensors"})
    with checkpoint.ModelDir(str(tmp_path)) as d:
        assert d.names() == ["t"]
