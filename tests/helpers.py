"""Shared builders for the parity tests: seeded synthetic NF4 weights plus their oracle views."""
from __future__ import annotations

import numpy as np
import torch

from aila_b200 import synth


def make_weight(seed, N, K, blocksize=64, nested=True):
    return synth.synth_linear(seed, N, K, blocksize, nested)


def oracle_absmax(O, w):
    """fp32 absmax as Bnb4BitLinear::init computes it (Bnb4BitLinear.cpp:472-488)."""
    if w.nested:
        return O.expand_absmax(w.absmax_codes, w.nested_quant_map, w.nested_absmax,
                               w.nested_blocksize, w.nested_offset)
    return np.asarray(w.absmax_f32, np.float32)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint16).numpy()


def from_bits(a: np.ndarray, device=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a, np.uint16)).view(torch.bfloat16)
    return t.to(device) if device is not None else t


def bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, np.uint16).astype(np.uint32) << 16).view(np.float32)


def assert_close_norm(got_bits, want_bits, rel=2e-2, what=""):
    """max |err| <= rel * ||want||_inf : the acceptance bound for GEMV/GEMM outputs."""
    g, w = bits_to_f32(got_bits).astype(np.float64), bits_to_f32(want_bits).astype(np.float64)
    assert g.shape == w.shape, (g.shape, w.shape)
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    err = np.abs(g - w).max() if g.size else 0.0
    bound = rel * (np.abs(w).max() if w.size else 0.0)
    assert err <= bound + 1e-30, f"{what}: max err {err:.4g} > {rel} * |y|inf = {bound:.4g}"
    return err, bound


def concat_rows(ws):
    """Row concatenation of quantised weights with fp32 absmax, as init_fused_rows does
    (Bnb4BitLinear.cpp:604-615). Returns (packed, absmax_f32_list_placeholder)."""
    return np.concatenate([np.asarray(w.packed, np.uint8).reshape(-1) for w in ws])
