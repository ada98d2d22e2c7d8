"""The two small-batch decode kernels behind aila_nf4_forward / aila_nf4_forward_gate_up_swiglu with
2..32 rows, each forced over the whole row range in a child process (the choice is read once per
process): AILA_NF4_ROWS_KERNEL=1 sends every batch to the K-sliced kernel (x slice in shared memory,
accumulation tiles in global memory), =0 to the streaming kernel's batched form (1, 2 or 4 blocks of
eight rows). Every row is compared with the single-row kernel on the same row and with the oracle.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import numpy as np, torch
from aila_b200 import linear as nf4
from oracle import nf4_oracle as O
from tests.helpers import make_weight, oracle_absmax, bf16_bits, bits_to_f32
from aila_b200 import synth
O.build()
scratch = nf4.Bnb4BitLinearScratch(0)
def lin_of(w):
    l = nf4.Bnb4BitLinear()
    assert l.init(w, 0), l.last_error
    return l
# (N, K, nested, rows): ragged N, K with a ragged last slice (448 = 7 units, 2560 = 40 units), outputs
# long enough that a CTA's range spans two slices, plain-absmax weights
cases = [(16, 64, True, 2), (100, 448, False, 3), (2560, 9728, True, 8), (33, 128, True, 7), (6144, 2560, True, 5),
         (2560, 9728, True, 16), (6144, 2560, True, 32), (100, 448, False, 13), (5120, 5120, False, 27),
         (33, 128, True, 32), (19456, 2560, True, 24), (272, 512, True, 9),
         # absmax blocks of 128 and 256 weights (two and four units share one absmax entry)
         (512, 1024, True, 20, 128), (272, 1024, True, 6, 256), (512, 2048, False, 31, 128)]
for case in cases:
    N, K, nested, M = case[:4]
    bs = case[4] if len(case) > 4 else 64
    w = make_weight(8400 + N + M, N, K, bs, nested)
    lin = lin_of(w)
    x = synth.gaussian_activation(8500 + N, M, K).cuda()
    res = synth.gaussian_activation(8600 + N, M, N).cuda()
    yb = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    for rep in range(2):  # twice: the second launch finds the work space as the first left it
        lin.forward(scratch, x, yb, M, add_residual=res)
    ys = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    for m in range(M):
        lin.forward(scratch, x[m:m + 1].contiguous(), ys[m:m + 1], 1, add_residual=res[m:m + 1].contiguous())
    torch.cuda.synchronize()
    scratch.check()
    a, b = yb.float().cpu().numpy(), ys.float().cpu().numpy()
    assert np.abs(a - b).max() <= 1e-2 * np.abs(b).max() + 1e-6, (N, K, M, np.abs(a - b).max())
    am = oracle_absmax(O, w)
    want = bits_to_f32(O.gemv(w.packed, w.quant_map, am, bf16_bits(x[M - 1:M]), N, K, bs)) + \
        bits_to_f32(bf16_bits(res[M - 1]))
    assert np.abs(a[M - 1] - want).max() <= 2e-2 * np.abs(want).max(), (N, K, M)
# gate|up + SiLU
for H, FF, M in [(512, 1040, 2), (512, 1040, 8), (2560, 9728, 11), (512, 1040, 16), (2560, 9728, 32)]:
    g, u = make_weight(8601, FF, H), make_weight(8602, FF, H)
    lg, lu, f = lin_of(g), lin_of(u), nf4.Bnb4BitLinear()
    assert f.init_fused_rows(lg, lu)
    x = synth.gaussian_activation(8603 + M, M, H)
    out = torch.empty(M, FF, dtype=torch.bfloat16, device="cuda")
    for rep in range(2):
        assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x.cuda(), out, FF, seq_len=M)
    torch.cuda.synchronize()
    scratch.check()
    packed = np.concatenate([g.packed, u.packed])
    am = np.concatenate([oracle_absmax(O, g), oracle_absmax(O, u)])
    xb = bf16_bits(x)
    got = out.float().cpu().numpy()
    for m in (0, M - 1):
        want = bits_to_f32(O.gemv_gate_up_swiglu(packed, g.quant_map, am, xb[m], FF, H, 64))
        assert np.abs(got[m] - want).max() <= 2e-2 * np.abs(want).max(), (H, FF, M, m)
print("small batches ok")
"""


@pytest.mark.parametrize("mode", ["0", "1"])
def test_small_batch_kernel_forced(mode):
    env = dict(os.environ, AILA_NF4_ROWS_KERNEL=mode, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "small batches ok" in r.stdout
