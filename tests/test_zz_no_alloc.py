"""The allocation-free decode entry point (aila_nf4_forward_decode_static) against the regular
one. Kept in a file pytest collects last so that a run stopping at the first failure has
already exercised everything else.

Hosts that must not touch the CUDA allocator on their token loop (all memory handed to their
own pool, or no tolerance for the device-wide sync of cudaMalloc/cudaFree) call this entry
point; it works on a fixed array inside the library. The test calls it twice in a row through
the C ABI - the array keeps the previous call's contents - and wants the same bf16 output as
aila_nf4_forward (same kernel and split, so the tolerance of the other GEMV tests is met with
room to spare), for a shape whose row tiles are cut by CTA boundaries (split-K fix-up in use).
"""
import numpy as np
import pytest
import torch

from aila_b200 import synth
from tests.helpers import assert_close_norm, bf16_bits, make_weight, oracle_absmax

pytestmark = pytest.mark.gpu

REL = 2e-2


@pytest.mark.parametrize("N,K", [(2560, 9728), (1000, 512)])
def test_static_scratch_entry_matches_regular_entry(oracle, N, K):
    from aila_b200 import linear as nf4
    w = make_weight(9000 + N, N, K)
    lin = nf4.Bnb4BitLinear()
    assert lin.init(w, 0), lin.last_error
    scratch = nf4.Bnb4BitLinearScratch(0)
    res = synth.gaussian_activation(9003, 1, N).cuda()
    want_oracle = None
    for call in range(2):
        x = synth.gaussian_activation(9001 + call, 1, K).cuda()
        y_ref = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
        lin.forward(scratch, x, y_ref, 1, add_residual=res)
        y = torch.full((1, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        lin.forward_decode_static(x, y, add_residual=res)
        torch.cuda.synchronize()
        if call == 1:  # (the first call may load the kernel's code)
            assert torch.cuda.mem_get_info()[0] == free_before, "the entry point allocated device memory"
        assert_close_norm(bf16_bits(y).reshape(-1), bf16_bits(y_ref).reshape(-1), REL,
                          f"static vs regular, call {call}")
        assert np.array_equal(bf16_bits(y), bf16_bits(y_ref)), f"call {call}: not bit-identical"
        want_oracle = oracle.gemv(w.packed, w.quant_map, oracle_absmax(oracle, w),
                                  bf16_bits(x).reshape(-1), N, K, 64,
                                  residual=bf16_bits(res).reshape(-1))
        assert_close_norm(bf16_bits(y).reshape(-1), want_oracle, REL, f"static vs oracle, call {call}")
    scratch.check()
    nf4.static_check(0)  # the status word of the built-in work space: no wait ran out


def test_static_scratch_entry_rejects_oversize():
    """Beyond the fixed work space the call fails with a clear message, it does not fall back."""
    from aila_b200 import _lib, linear as nf4
    N, K = 262144 + 16, 64
    packed = np.zeros(N * K // 2, np.uint8)
    absmax = np.ones(N * K // 64, np.float32)
    w = synth.Nf4Tensors(N, K, 64, packed, None, absmax, synth.nf4_codebook(), None, None)
    lin = nf4.Bnb4BitLinear()
    assert lin.init(w, 0), lin.last_error
    x = torch.zeros(1, K, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(1, N, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.Nf4Error) as e:
        lin.forward_decode_static(x, y)
    assert e.value.status == _lib.ERR_UNSUPPORTED and "exceeds the fixed work space" in str(e.value)
