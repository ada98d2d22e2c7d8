"""Writes tests/golden/nf4_small.npz: one small seeded NF4 weight with every oracle output.

The reference project holds no golden vectors for this path and cannot be run offline, so
these vectors come from oracle/nf4_oracle.c; they pin the oracle (and through it the CUDA
library) against accidental change, not against the reference.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from aila_b200 import synth  # noqa: E402
from oracle import nf4_oracle as O  # noqa: E402


def main():
    N, K, bs, M = 96, 512, 64, 3
    w = synth.synth_linear(424242, N, K, bs, nested=True)
    am = O.expand_absmax(w.absmax_codes, w.nested_quant_map, w.nested_absmax, w.nested_blocksize,
                         w.nested_offset)
    x = synth.gaussian_activation(424243, K).view(torch.uint16).numpy()
    xm = synth.gaussian_activation(424244, M, K).view(torch.uint16).numpy()
    out = dict(
        N=N, K=K, blocksize=bs, M=M, packed=w.packed, absmax_codes=w.absmax_codes,
        quant_map=w.quant_map, nested_absmax=w.nested_absmax, nested_quant_map=w.nested_quant_map,
        nested_blocksize=w.nested_blocksize, nested_offset=np.float32(w.nested_offset),
        absmax_f32=am, x=x, xm=xm,
        dequant_kn=O.dequantize_kn(w.packed, w.quant_map, am, N, K, bs),
        y_gemv=O.gemv(w.packed, w.quant_map, am, x, N, K, bs),
        y_swiglu=O.gemv_gate_up_swiglu(w.packed, w.quant_map, am, x, N // 2, K, bs),
        y_prefill=O.forward(w.packed, w.quant_map, am, xm, M, N, K, bs),
    )
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nf4_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
