"""Bounded device waits that run out: the kernel returns, the status word says
AILA_NF4_ERR_KERNEL_TIMEOUT, the context stays usable. The failures are built on the host (a peer
that never publishes, a wait limit of a few cycles); nothing here faults, traps or waits without
a bound.
"""
import pytest
import torch

from aila_b200 import _lib, synth
from tests.helpers import assert_close_norm, bf16_bits, make_weight, oracle_absmax

pytestmark = pytest.mark.gpu

MS = 2_000_000  # SM cycles in about a millisecond


@pytest.fixture(scope="module")
def nf4():
    from aila_b200 import linear
    assert torch.cuda.is_available()
    return linear


def _lin(nf4, w):
    l = nf4.Bnb4BitLinear()
    assert l.init(w, 0), l.last_error
    return l


def _oracle_gemv(oracle, w, x_bits):
    return oracle.gemv(w.packed, w.quant_map, oracle_absmax(oracle, w), x_bits.reshape(-1), w.out_features,
                       w.in_features, 64)


def test_peer_that_never_publishes_times_out(nf4, oracle):
    """Rank 0 of a group of two runs the row-parallel decode; rank 1's buffer lives in the same
    process and nobody ever writes rank 1's words. The call returns after the wait limit, y is
    untouched, the scratch reports the timeout, and a plain call afterwards works."""
    n, k = 512, 1024
    w = make_weight(101, n, k)
    shard = nf4.Bnb4BitLinear()
    assert shard.init_shard(w, _lib.SHARD_COLS, 0, 2, 0), shard.last_error
    sc = nf4.Bnb4BitLinearScratch(0)
    sc.set_wait_limit(5 * MS)
    mine = nf4.PeerBuffer(0, 0, 2, n)
    other = nf4.PeerBuffer(0, 1, 2, n)
    mine.import_local(1, other)
    other.import_local(0, mine)
    x = synth.gaussian_activation(7, 1, k // 2).cuda()
    y = torch.full((1, n), 3.0, dtype=torch.bfloat16, device="cuda")
    shard.forward_decode_allreduce(sc, mine, x, y, None)
    torch.cuda.synchronize()  # returns: the wait is bounded
    with pytest.raises(_lib.Nf4Error) as err:
        sc.check()
    assert err.value.status == _lib.ERR_KERNEL_TIMEOUT
    assert bool((y == 3.0).all()), "a launch whose wait ran out must not write y"
    sc.check()  # the status word was cleared by the failed check
    # the context is usable: a plain linear on fresh buffers gives the oracle's numbers
    full = _lin(nf4, w)
    xf = synth.gaussian_activation(8, 1, k).cuda()
    yf = torch.empty(1, n, dtype=torch.bfloat16, device="cuda")
    sc.set_wait_limit(2_000_000_000)
    full.forward(sc, xf, yf, 1)
    torch.cuda.synchronize()
    sc.check()
    assert_close_norm(bf16_bits(yf).reshape(-1), _oracle_gemv(oracle, w, bf16_bits(xf)), 2e-2, "after the timeout")
    for o in (mine, other, shard, full, sc):
        o.close()


def test_chained_kernel_gives_up_and_recovers(nf4, oracle):
    """A chain whose waits may take a single cycle: the first wait that is not satisfied at once
    gives up, every CTA drains, the launch ends and reports the timeout. With the default limit the
    same scratch then runs a fresh chain correctly."""
    k, n = 2560, 4864
    w1, w2 = make_weight(201, n, k), make_weight(202, k, n)
    l1, l2 = _lin(nf4, w1), _lin(nf4, w2)
    sc = nf4.Bnb4BitLinearScratch(0)
    x = synth.gaussian_activation(9, 1, k).cuda()
    y = torch.empty(1, k, dtype=torch.bfloat16, device="cuda")
    sc.set_wait_limit(1)
    bad = nf4.DecodeChain(sc, [dict(linear=l1, x=x), dict(linear=l2, y=y)] * 4)
    bad.run()
    torch.cuda.synchronize()
    with pytest.raises(_lib.Nf4Error) as err:
        sc.check()
    assert err.value.status == _lib.ERR_KERNEL_TIMEOUT
    bad.close()
    sc.set_wait_limit(2_000_000_000)
    good = nf4.DecodeChain(sc, [dict(linear=l1, x=x), dict(linear=l2, y=y)])
    for _ in range(2):
        good.run()
    torch.cuda.synchronize()
    sc.check()
    want = _oracle_gemv(oracle, w2, _oracle_gemv(oracle, w1, bf16_bits(x)))
    assert_close_norm(bf16_bits(y).reshape(-1), want, 2e-2, "chain after the timeout")
    for o in (good, l1, l2, sc):
        o.close()


def test_static_entry_reports_its_status(nf4):
    """The allocation-free entry point has a status word of its own; aila_nf4_static_check reads
    and clears it."""
    w = make_weight(301, 512, 1024)
    l = _lin(nf4, w)
    x = synth.gaussian_activation(11, 1, 1024).cuda()
    y = torch.empty(1, 512, dtype=torch.bfloat16, device="cuda")
    l.forward_decode_static(x, y)
    torch.cuda.synchronize()
    nf4.static_check(0)
    l.close()
