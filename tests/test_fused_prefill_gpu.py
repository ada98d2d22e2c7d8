"""The fused prefill kernel (AILA_NF4_FUSED_PREFILL=1: sixteen more warps rebuild every w tile from
the NF4 units inside the tcgen05 GEMM, no bf16 copy of W in HBM) against the two-phase route
(dequantisation pass, then the same GEMM): the rebuilt weights are bit-equal to dequantize_weight and
the tensor-core schedule is the same, so the outputs must be IDENTICAL. The choice is read once per
process, hence two child processes writing their outputs to a scratch directory.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, numpy as np, torch
from aila_b200 import linear as nf4, synth
from tests.helpers import make_weight
scratch = nf4.Bnb4BitLinearScratch(0)
def lin_of(w):
    l = nf4.Bnb4BitLinear()
    assert l.init(w, 0), l.last_error
    return l
outs = {}
# (N, K, nested, M): one and several tiles of x, N that is not a multiple of the tile width, plain
# fp32 absmax, K of one and of many 64-column steps, 256-row and 128-row tiles
for N, K, nested, M in [(272, 512, True, 64), (1600, 512, False, 33), (2560, 9728, True, 300),
                        (6144, 2560, True, 2048), (4112, 1024, True, 129), (48, 64, True, 40)]:
    w = make_weight(9100 + N + M, N, K, 64, nested)
    lin = lin_of(w)
    x = synth.gaussian_activation(9200 + N, M, K).cuda()
    res = synth.gaussian_activation(9300 + N, M, N).cuda()
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):
        lin.forward(scratch, x, y, M, add_residual=res)
    torch.cuda.synchronize()
    scratch.check()
    outs[f"plain_{N}_{K}_{M}"] = y.cpu().view(torch.uint16).numpy()
for H, FF, M in [(512, 1040, 64), (2560, 9728, 2048), (2560, 9728, 100)]:
    g, u = make_weight(9601, FF, H), make_weight(9602, FF, H)
    lg, lu, f = lin_of(g), lin_of(u), nf4.Bnb4BitLinear()
    assert f.init_fused_rows(lg, lu)
    x = synth.gaussian_activation(9603 + M, M, H).cuda()
    out = torch.empty(M, FF, dtype=torch.bfloat16, device="cuda")
    assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x, out, FF, seq_len=M)
    torch.cuda.synchronize()
    scratch.check()
    outs[f"swiglu_{H}_{FF}_{M}"] = out.cpu().view(torch.uint16).numpy()
np.savez(sys.argv[1], **outs)
print("prefill outputs written")
"""


def test_fused_prefill_is_bit_identical_to_the_two_phase_route(oracle):
    with tempfile.TemporaryDirectory() as tmp:
        got = {}
        for mode in ("0", "1"):
            path = os.path.join(tmp, f"out_{mode}.npz")
            env = dict(os.environ, AILA_NF4_FUSED_PREFILL=mode, PYTHONPATH=ROOT)
            r = subprocess.run([sys.executable, "-c", CHILD, path], cwd=ROOT, env=env, capture_output=True, text=True,
                               timeout=600)
            assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
            got[mode] = dict(np.load(path))
        assert got["0"].keys() == got["1"].keys()
        for k in got["0"]:
            assert np.array_equal(got["0"][k], got["1"][k]), k
        # and the route itself against the oracle on one case (sampled rows)
        from tests.helpers import bits_to_f32, make_weight, oracle_absmax
        from aila_b200 import synth
        import torch
        N, K, M = 272, 512, 64
        w = make_weight(9100 + N + M, N, K, 64, True)
        x = synth.gaussian_activation(9200 + N, M, K)
        res = synth.gaussian_activation(9300 + N, M, N)
        want = bits_to_f32(oracle.forward(w.packed, w.quant_map, oracle_absmax(oracle, w),
                                          x.view(torch.uint16).numpy(), M, N, K, 64)) + \
            bits_to_f32(res.view(torch.uint16).numpy())
        have = bits_to_f32(got["1"][f"plain_{N}_{K}_{M}"])
        assert np.abs(have - want).max() <= 2e-2 * np.abs(want).max()
