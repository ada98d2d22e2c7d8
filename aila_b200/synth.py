"""Seeded synthetic bitsandbytes-NF4 weights (stand-in for real checkpoints).

The reference consumes tensors written by the third-party ``bitsandbytes`` exporter
(export_bnb_nf4.py:33,114-121): packed nibbles, absmax codes, ``quant_map``,
``nested_absmax``, ``nested_quant_map`` and a JSON quant_state
(src/utils/SafeTensors.cpp:383-387). bitsandbytes is not available offline, so this module
produces tensors of the same format from seeded Gaussian weights.

Both codebooks are CONSTRUCTED HERE from the published recipes (normal-quantile NF4 code;
dynamic-exponent 8-bit map for the second level). Their identity with the tables that
bitsandbytes ships has not been verified. Nothing downstream depends on it: the kernels
take both tables as runtime inputs, exactly like the reference (SafeTensors.cpp:384,397).
"""
from __future__ import annotations

import dataclasses
import json

import numpy as np
import torch


def nf4_codebook() -> np.ndarray:
    """16-entry NormalFloat4 code: 8 positive and 7 negative normal quantiles plus an exact
    zero, sorted, scaled to [-1, 1]."""
    from scipy.stats import norm

    offset = 0.9677083
    pos = norm.ppf(np.linspace(offset, 0.5, 9)[:-1])
    neg = -norm.ppf(np.linspace(offset, 0.5, 8)[:-1])
    vals = np.sort(np.concatenate([pos, [0.0], neg]))
    vals = vals / np.abs(vals).max()
    return vals.astype(np.float32)


def dynamic_map_256() -> np.ndarray:
    """256-entry signed dynamic-exponent map in [-1, 1] (monotone, contains 0 and 1): seven
    decades, each filled with a growing number of linearly spaced fraction means."""
    exponent_bits, non_sign_bits = 7, 7
    data: list[float] = []
    for i in range(exponent_bits):
        n_items = 2 ** (i + non_sign_bits - exponent_bits) + 1
        edges = np.linspace(0.1, 1.0, n_items)
        means = (edges[:-1] + edges[1:]) / 2.0
        scale = 10.0 ** (-(exponent_bits - 1) + i)
        data += (scale * means).tolist()
        data += (-scale * means).tolist()
    data += [0.0, 1.0]
    data += [0.0] * (256 - len(data))
    out = np.sort(np.asarray(data, dtype=np.float64)).astype(np.float32)
    assert out.size == 256
    return out


@dataclasses.dataclass
class Nf4Tensors:
    """One quantised weight in checkpoint form (all numpy, host)."""
    out_features: int
    in_features: int
    blocksize: int
    packed: np.ndarray            # u8 [N*K/2], high nibble = even k
    absmax_codes: np.ndarray | None  # u8 [N*K/bs] when nested
    absmax_f32: np.ndarray | None    # f32 [N*K/bs] when not nested
    quant_map: np.ndarray         # f32 [16]
    nested_absmax: np.ndarray | None     # f32 [ceil(blocks/nbs)]
    nested_quant_map: np.ndarray | None  # f32 [256]
    nested_blocksize: int = 256
    nested_offset: float = 0.0

    @property
    def nested(self) -> bool:
        return self.absmax_codes is not None

    def quant_state_json(self) -> str:
        """The JSON blob the reference parses (SafeTensors.cpp:281-334)."""
        d = {"quant_type": "nf4", "blocksize": self.blocksize, "dtype": "float16",
             "shape": [self.out_features, self.in_features]}
        if self.nested:
            d.update({"nested_blocksize": self.nested_blocksize, "nested_dtype": "float32",
                      "nested_offset": float(self.nested_offset)})
        return json.dumps(d)


def _nearest_code(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Index of the table entry nearest to each x (table sorted ascending)."""
    mids = (table[1:] + table[:-1]) / 2
    return torch.bucketize(x, mids)


def quantize_nf4(w: torch.Tensor, blocksize: int = 64, nested: bool = True,
                 nested_blocksize: int = 256, quant_map: np.ndarray | None = None,
                 nested_quant_map: np.ndarray | None = None) -> Nf4Tensors:
    """Blockwise NF4 quantisation of a float32 [N, K] matrix, bitsandbytes-style: per-block
    absmax, nearest code, two codes per byte with the first (even-k) code in the high nibble;
    optional double quantisation of the absmax (mean offset, per-256 absmax, 8-bit codes)."""
    assert w.dtype == torch.float32 and w.dim() == 2
    N, K = w.shape
    assert (N * K) % blocksize == 0 and blocksize % 2 == 0
    qm = torch.from_numpy(nf4_codebook() if quant_map is None else
                          np.asarray(quant_map, np.float32))
    flat = w.reshape(-1, blocksize)
    absmax = flat.abs().amax(dim=1)
    scaled = flat / absmax.clamp_min(1e-30).unsqueeze(1)
    codes = _nearest_code(scaled, qm).to(torch.uint8).reshape(-1)
    packed = ((codes[0::2] << 4) | codes[1::2]).contiguous()

    if not nested:
        return Nf4Tensors(N, K, blocksize, packed.numpy(), None, absmax.numpy().copy(),
                          qm.numpy().copy(), None, None)

    nqm = torch.from_numpy(dynamic_map_256() if nested_quant_map is None else
                           np.asarray(nested_quant_map, np.float32))
    offset = absmax.mean()
    centred = absmax - offset
    n_blocks = centred.numel()
    pad = (-n_blocks) % nested_blocksize
    cpad = torch.cat([centred, centred.new_zeros(pad)]).reshape(-1, nested_blocksize)
    nabs = cpad.abs().amax(dim=1)
    nscaled = cpad / nabs.clamp_min(1e-30).unsqueeze(1)
    ncodes = _nearest_code(nscaled, nqm).to(torch.uint8).reshape(-1)[:n_blocks]
    return Nf4Tensors(N, K, blocksize, packed.numpy(), ncodes.numpy().copy(), None,
                      qm.numpy().copy(), nabs.numpy().copy(), nqm.numpy().copy(),
                      nested_blocksize, float(offset))


def gaussian_weight(seed: int, out_features: int, in_features: int,
                    std: float = 0.02) -> torch.Tensor:
    """fp32 N(0, std) weight from a CPU generator (CPU so fixtures do not depend on the GPU)."""
    g = torch.Generator().manual_seed(int(seed))
    return torch.randn(out_features, in_features, generator=g, dtype=torch.float32) * std


def gaussian_activation(seed: int, *shape: int) -> torch.Tensor:
    """bf16 N(0, 1) activations from a CPU generator."""
    g = torch.Generator().manual_seed(int(seed))
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(torch.bfloat16)


def synth_linear(seed: int, out_features: int, in_features: int, blocksize: int = 64,
                 nested: bool = True) -> Nf4Tensors:
    return quantize_nf4(gaussian_weight(seed, out_features, in_features), blocksize, nested)


# Seed scheme for the benchmark configurations: 1000*cfg + 10*layer + projection.
PROJ = {"q": 0, "k": 1, "v": 2, "o": 3, "gate": 4, "up": 5, "down": 6, "lm_head": 7}


def seed_for(cfg: int, layer: int, proj: str) -> int:
    return 1000 * cfg + 10 * layer + PROJ[proj]
