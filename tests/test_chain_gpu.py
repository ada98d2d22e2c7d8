"""The chained decode kernel (aila_nf4_chain_*): a run of seq_len == 1 linears in one launch,
against the CPU oracle and against the same linears called one by one. Through the C ABI.
"""
import numpy as np
import pytest
import torch

from aila_b200 import _lib, synth
from tests.helpers import assert_close_norm, bf16_bits, bits_to_f32, make_weight, oracle_absmax

pytestmark = pytest.mark.gpu

REL = 2e-2  # max |err| <= REL * ||y||_inf


@pytest.fixture(scope="module")
def nf4():
    from aila_b200 import linear
    assert torch.cuda.is_available()
    return linear


@pytest.fixture(autouse=True)
def chained_kernel_for_single_calls(nf4):
    """Single forward calls in this file run the chained kernel too (as one-operation launches), so
    that "the same linears called one by one" can be compared bit for bit."""
    nf4.set_gemv_kernel(3)
    yield
    nf4.set_gemv_kernel(0)


@pytest.fixture(scope="module")
def scratch(nf4):
    s = nf4.Bnb4BitLinearScratch(0)
    yield s
    torch.cuda.synchronize()
    s.check()
    s.close()


def _lin(nf4, w):
    l = nf4.Bnb4BitLinear()
    assert l.init(w, 0), l.last_error
    return l


def _fused(nf4, ws):
    ls = [_lin(nf4, w) for w in ws]
    f = nf4.Bnb4BitLinear()
    assert f.init_fused_rows(*ls), f.last_error
    return f


def _act(seed, *shape):
    return synth.gaussian_activation(seed, *shape)


def _empty(n):
    return torch.full((1, n), float("nan"), dtype=torch.bfloat16, device="cuda")


def _gemv_want(oracle, w, x_bits, residual=None):
    return oracle.gemv(w.packed, w.quant_map, oracle_absmax(oracle, w), x_bits.reshape(-1),
                       w.out_features, w.in_features, 64, residual=residual)


def _gate_up_want(oracle, g, u, x_bits):
    packed = np.concatenate([g.packed, u.packed])
    am = np.concatenate([oracle_absmax(oracle, g), oracle_absmax(oracle, u)])
    return oracle.gemv_gate_up_swiglu(packed, g.quant_map, am, x_bits.reshape(-1), g.out_features,
                                      g.in_features, 64)


@pytest.mark.parametrize("N,K,nested", [(16, 64, True), (40, 128, True), (48, 448, False),
                                        (100, 512, True), (2560, 9728, True), (6144, 2560, True)])
def test_one_operation_chain_equals_forward(nf4, oracle, scratch, N, K, nested):
    w = make_weight(7000 + N + K, N, K, 64, nested)
    lin = _lin(nf4, w)
    x = _act(7001 + N, 1, K).cuda()
    res = _act(7002 + N, 1, N).cuda()
    y_chain, y_fwd = _empty(N), _empty(N)
    chain = nf4.DecodeChain(scratch, [dict(linear=lin, x=x, y=y_chain, residual=res)])
    assert len(chain) == 1
    chain.run()
    lin.forward(scratch, x, y_fwd, 1, add_residual=res)
    torch.cuda.synchronize()
    scratch.check()
    assert torch.equal(y_chain.view(torch.uint16), y_fwd.view(torch.uint16))
    am = oracle_absmax(oracle, w)
    want = oracle.gemv(w.packed, w.quant_map, am, bf16_bits(x).reshape(-1), N, K, 64,
                       residual=bf16_bits(res).reshape(-1))
    assert_close_norm(bf16_bits(y_chain).reshape(-1), want, REL, f"chain of one {N}x{K}")


@pytest.mark.parametrize("H,FF", [(128, 256), (1024, 2048), (2560, 9728)])
def test_linked_mlp(nf4, oracle, scratch, H, FF):
    """gate|up + SwiGLU -> down (+ residual) as two linked operations: the intermediate vector
    never leaves the launch unless asked for."""
    g, u, d = make_weight(7100 + H, FF, H), make_weight(7101 + H, FF, H), make_weight(7102 + H, H, FF)
    gu, dn = _fused(nf4, [g, u]), _lin(nf4, d)
    x = _act(7103, 1, H).cuda()
    res = _act(7104, 1, H).cuda()
    mid, y_a, y_b = _empty(FF), _empty(H), _empty(H)
    with_mid = nf4.DecodeChain(scratch, [dict(linear=gu, ff_dim=FF, x=x, y=mid),
                                         dict(linear=dn, y=y_a, residual=res)])
    without = nf4.DecodeChain(scratch, [dict(linear=gu, ff_dim=FF, x=x),
                                        dict(linear=dn, y=y_b, residual=res)])
    with_mid.run()
    without.run()
    torch.cuda.synchronize()
    scratch.check()
    assert torch.equal(y_a.view(torch.uint16), y_b.view(torch.uint16))
    assert_close_norm(bf16_bits(mid).reshape(-1), _gate_up_want(oracle, g, u, bf16_bits(x)), REL, "mid")
    want = _gemv_want(oracle, d, bf16_bits(mid), residual=bf16_bits(res).reshape(-1))
    assert_close_norm(bf16_bits(y_a).reshape(-1), want, REL, "down of the linked pair")
    # the same two linears called one by one give the same bits
    mid2, y2 = _empty(FF), _empty(H)
    assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(gu, scratch, x, mid2, FF)
    dn.forward(scratch, mid2, y2, 1, add_residual=res)
    torch.cuda.synchronize()
    assert torch.equal(mid2.view(torch.uint16), mid.view(torch.uint16))
    assert torch.equal(y2.view(torch.uint16), y_a.view(torch.uint16))
    # x named by pointer (the previous output) is the same link
    y_c = _empty(H)
    by_ptr = nf4.DecodeChain(scratch, [dict(linear=gu, ff_dim=FF, x=x, y=mid),
                                       dict(linear=dn, x=mid, y=y_c, residual=res)])
    by_ptr.run()
    torch.cuda.synchronize()
    assert torch.equal(y_c.view(torch.uint16), y_a.view(torch.uint16))


def test_layer_chain_with_norms(nf4, oracle, scratch):
    """o_proj (+ residual) -> RMSNorm -> gate|up + SwiGLU -> down (+ residual) -> RMSNorm -> qkv:
    the linears of one decoder layer behind the attention, as one launch. Each stage is checked
    against the oracle applied to the previous stage's actual output."""
    H, Q, KV, FF = 1024, 1536, 256, 2048
    wo = make_weight(7201, H, Q)
    g, u, d = make_weight(7202, FF, H), make_weight(7203, FF, H), make_weight(7204, H, FF)
    wq, wk, wv = make_weight(7205, Q, H), make_weight(7206, KV, H), make_weight(7207, KV, H)
    o, gu, dn, qkv = _lin(nf4, wo), _fused(nf4, [g, u]), _lin(nf4, d), _fused(nf4, [wq, wk, wv])
    gen = torch.Generator().manual_seed(7208)
    nw1 = (1.0 + 0.1 * torch.randn(H, generator=gen)).to(torch.bfloat16).cuda()
    nw2 = (1.0 + 0.1 * torch.randn(H, generator=gen)).to(torch.bfloat16).cuda()
    attn, h0, r2 = _act(7209, 1, Q).cuda(), _act(7210, 1, H).cuda(), _act(7211, 1, H).cuda()
    h1, mid, h2, h2n, y_qkv = _empty(H), _empty(FF), _empty(H), _empty(H), _empty(Q + 2 * KV)
    chain = nf4.DecodeChain(scratch, [
        dict(linear=o, x=attn, y=h1, residual=h0),
        dict(linear=gu, ff_dim=FF, y=mid, norm=dict(weight=nw1, eps=1e-6)),
        dict(linear=dn, y=h2, residual=r2),
        dict(linear=qkv, y=y_qkv, norm=dict(weight=nw2, eps=1e-6, hidden_out=h2n)),
    ])
    for _ in range(2):  # a second launch reuses the exchange buffers
        chain.run()
    torch.cuda.synchronize()
    scratch.check()
    want_h1 = _gemv_want(oracle, wo, bf16_bits(attn), residual=bf16_bits(h0).reshape(-1))
    assert_close_norm(bf16_bits(h1).reshape(-1), want_h1, REL, "o_proj")
    _, n1 = oracle.add_rms_norm(bf16_bits(h1), None, bf16_bits(nw1), 1e-6, 1, H)
    assert_close_norm(bf16_bits(mid).reshape(-1), _gate_up_want(oracle, g, u, n1), REL, "gate_up")
    want_h2 = _gemv_want(oracle, d, bf16_bits(mid), residual=bf16_bits(r2).reshape(-1))
    assert_close_norm(bf16_bits(h2).reshape(-1), want_h2, REL, "down")
    assert torch.equal(h2n.view(torch.uint16), h2.view(torch.uint16))  # no add: hidden_out = input
    _, n2 = oracle.add_rms_norm(bf16_bits(h2), None, bf16_bits(nw2), 1e-6, 1, H)
    packed = np.concatenate([wq.packed, wk.packed, wv.packed])
    am = np.concatenate([oracle_absmax(oracle, w) for w in (wq, wk, wv)])
    want_qkv = oracle.gemv(packed, wq.quant_map, am, n2.reshape(-1), Q + 2 * KV, H, 64)
    assert_close_norm(bf16_bits(y_qkv).reshape(-1), want_qkv, REL, "qkv")


def test_operations_with_their_own_inputs(nf4, scratch):
    """Operations that bring their own x still run in list order; every result equals the
    stand-alone call bit for bit. Shapes from one unit to ragged row counts."""
    shapes = [(16, 64), (2560, 4096), (40, 128), (100, 512), (6144, 2560), (33, 2560)]
    lins = [_lin(nf4, make_weight(7300 + i, n, k)) for i, (n, k) in enumerate(shapes)]
    xs = [_act(7310 + i, 1, k).cuda() for i, (n, k) in enumerate(shapes)]
    ys = [_empty(n) for n, _ in shapes]
    chain = nf4.DecodeChain(scratch, [dict(linear=l, x=x, y=y) for l, x, y in zip(lins, xs, ys)])
    chain.run()
    torch.cuda.synchronize()
    scratch.check()
    for l, x, y, (n, _) in zip(lins, xs, ys, shapes):
        alone = _empty(n)
        l.forward(scratch, x, alone, 1)
        torch.cuda.synchronize()
        assert torch.equal(alone.view(torch.uint16), y.view(torch.uint16))


def test_chain_in_cuda_graph(nf4, scratch):
    H, FF = 1024, 2048
    g, u, d = make_weight(7401, FF, H), make_weight(7402, FF, H), make_weight(7403, H, FF)
    gu, dn = _fused(nf4, [g, u]), _lin(nf4, d)
    x, y = _act(7404, 1, H).cuda(), _empty(H)
    chain = nf4.DecodeChain(scratch, [dict(linear=gu, ff_dim=FF, x=x), dict(linear=dn, y=y, residual=x)])
    chain.run()
    torch.cuda.synchronize()
    y0 = y.clone()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            chain.run()
            chain.run()
        for _ in range(3):
            y.fill_(float("nan"))
            gr.replay()
            st.synchronize()
            assert torch.equal(y.view(torch.uint16), y0.view(torch.uint16))
        x.copy_(_act(7405, 1, H))  # new input, same graph
        gr.replay()
        st.synchronize()
    y1 = y.clone()
    chain.run()
    torch.cuda.synchronize()
    scratch.check()
    assert torch.equal(y.view(torch.uint16), y1.view(torch.uint16))
    assert not torch.equal(y1.view(torch.uint16), y0.view(torch.uint16))


def test_chain_host_buffers(nf4, scratch):
    H, FF = 512, 1024
    g, u, d = make_weight(7501, FF, H), make_weight(7502, FF, H), make_weight(7503, H, FF)
    gu, dn = _fused(nf4, [g, u]), _lin(nf4, d)
    x_dev, y_dev = torch.zeros(1, H, dtype=torch.bfloat16, device="cuda"), _empty(H)
    chain = nf4.DecodeChain(scratch, [dict(linear=gu, ff_dim=FF, x=x_dev), dict(linear=dn, y=y_dev)])
    xh = _act(7504, 1, H).pin_memory()
    yh = torch.empty(1, H, dtype=torch.bfloat16).pin_memory()
    chain.run_host(xh, yh)
    x_dev.copy_(xh)
    want = _empty(H)
    mid = _empty(FF)
    assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(gu, scratch, x_dev, mid, FF)
    dn.forward(scratch, mid, want, 1)
    torch.cuda.synchronize()
    assert torch.equal(yh.view(torch.uint16), want.cpu().view(torch.uint16))


def test_chain_rejects_bad_lists(nf4, scratch):
    a, b = _lin(nf4, make_weight(7601, 128, 64)), _lin(nf4, make_weight(7602, 64, 256))
    x, y = _act(7603, 1, 64).cuda(), _empty(64)
    with pytest.raises(_lib.Nf4Error, match="first operation needs an input"):
        nf4.DecodeChain(scratch, [dict(linear=a, y=y)])
    with pytest.raises(_lib.Nf4Error, match="differs from the previous"):
        nf4.DecodeChain(scratch, [dict(linear=a, x=x), dict(linear=b, y=y)])
    with pytest.raises(_lib.Nf4Error, match="needs an output"):
        nf4.DecodeChain(scratch, [dict(linear=a, x=x)])
    with pytest.raises(_lib.Nf4Error):
        nf4.DecodeChain(scratch, [])


def test_chain_with_exchange_on_one_rank(nf4, oracle, scratch):
    """gate|up -> down as one launch whose last operation goes through the row-parallel exchange,
    in a group of ONE rank: the sum over the ranks is this rank's sum, so the result must equal the
    plain chain bit for bit - eagerly (both halves of the exchange buffer) and replayed from a CUDA
    graph. The multi-rank case runs with the sharded tests."""
    H, FF = 1024, 2048
    g, u, d = make_weight(7600, FF, H), make_weight(7601, FF, H), make_weight(7602, H, FF)
    gu, dn = _fused(nf4, [g, u]), _lin(nf4, d)
    x, res = _act(7603, 1, H).cuda(), _act(7604, 1, H).cuda()
    y_plain, y_peer = _empty(H), _empty(H)
    plain = nf4.DecodeChain(scratch, [dict(linear=gu, ff_dim=FF, x=x), dict(linear=dn, y=y_plain, residual=res)])
    peers = nf4.PeerBuffer(0, 0, 1, H)
    shared = nf4.DecodeChain(scratch, [dict(linear=gu, ff_dim=FF, x=x), dict(linear=dn, y=y_peer, residual=res)],
                             peers=peers)
    plain.run()
    torch.cuda.synchronize()
    for _ in range(3):
        y_peer.fill_(float("nan"))
        shared.run()
        torch.cuda.synchronize()
        scratch.check()
        assert torch.equal(y_peer.view(torch.uint16), y_plain.view(torch.uint16))
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            shared.run()
        y_peer.fill_(float("nan"))
        for _ in range(3):
            graph.replay()
        st.synchronize()
    scratch.check()
    assert torch.equal(y_peer.view(torch.uint16), y_plain.view(torch.uint16))
    mid = _gate_up_want(oracle, g, u, bf16_bits(x))
    want = _gemv_want(oracle, d, mid, residual=bf16_bits(res).reshape(-1))
    assert_close_norm(bf16_bits(y_peer).reshape(-1), want, REL, "exchange chain on one rank")
    with pytest.raises(_lib.Nf4Error):  # a gate|up operation cannot be the row-parallel one
        nf4.DecodeChain(scratch, [dict(linear=gu, ff_dim=FF, x=x, y=_empty(FF))], peers=peers)
    shared.close()
    plain.close()
    peers.close()
