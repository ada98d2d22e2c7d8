"""Parity of the CUDA library with the CPU oracle, through the C ABI (ctypes), on a B200.

Bars: dequantised weights and absmax bit-exact; GEMV / fused gate+up+SiLU / prefill GEMM
outputs within max|err| <= 2e-2 * ||y||_inf at bf16 output (the bound this hot path is held to).
"""
import numpy as np
import pytest
import torch

from aila_b200 import synth
from tests.helpers import (assert_close_norm, bf16_bits, bits_to_f32, make_weight, oracle_absmax)

pytestmark = pytest.mark.gpu

REL = 2e-2  # max |err| <= REL * ||y||_inf


@pytest.fixture(scope="module")
def nf4():
    from aila_b200 import linear
    assert torch.cuda.is_available()
    return linear


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


def _act(seed, *shape):
    return synth.gaussian_activation(seed, *shape)


# ---------------------------------------------------------------- dequantisation (bit-exact)
@pytest.mark.parametrize("N,K,nested", [(16, 64, True), (64, 64, False), (48, 448, True),
                                        (100, 512, True), (33, 128, False), (512, 2560, True),
                                        (1024, 9728, True)])
def test_dequant_bit_exact(nf4, oracle, N, K, nested):
    w = make_weight(100 + N + K, N, K, 64, nested)
    am = oracle_absmax(oracle, w)
    l = _lin(nf4, w)
    assert (l.in_features(), l.out_features()) == (K, N)
    got_am = l.expand_absmax(64).cpu().numpy().reshape(-1)
    assert np.array_equal(got_am.view(np.uint32), am.view(np.uint32)), "absmax not bit-exact"
    want = oracle.dequantize_kn(w.packed, w.quant_map, am, N, K, 64)
    assert np.array_equal(bf16_bits(l.dequantize_weight()), want), "Wt[K,N] not bit-exact"
    assert np.array_equal(bf16_bits(l.dequantize_rowmajor()), want.T), "W[N,K] not bit-exact"


def test_dequant_every_byte_value(nf4, oracle):
    """All 256 packed byte values against sampled fp32 absmax, bitwise."""
    N, K = 64, 512
    rng = np.random.default_rng(5)
    packed = np.tile(np.arange(256, dtype=np.uint8), N * K // 2 // 256)
    rng.shuffle(packed)
    absmax = np.exp(rng.uniform(-12, 4, N * K // 64)).astype(np.float32)
    w = synth.Nf4Tensors(N, K, 64, packed, None, absmax, synth.nf4_codebook(), None, None)
    l = _lin(nf4, w)
    want = oracle.dequantize_kn(packed, w.quant_map, absmax, N, K, 64)
    assert np.array_equal(bf16_bits(l.dequantize_weight()), want)


@pytest.mark.parametrize("bs", [128, 256])
def test_dequant_larger_blocksize(nf4, oracle, bs):
    N, K = 32, 1024
    w = make_weight(77, N, K, bs, True)
    am = oracle_absmax(oracle, w)
    l = _lin(nf4, w)
    want = oracle.dequantize_kn(w.packed, w.quant_map, am, N, K, bs)
    assert np.array_equal(bf16_bits(l.dequantize_weight()), want)
    assert np.array_equal(l.expand_absmax(bs).cpu().numpy().reshape(-1).view(np.uint32),
                          am.view(np.uint32))


# ---------------------------------------------------------------- decode GEMV
GEMV_SHAPES = [(16, 64), (40, 128), (48, 448), (100, 512), (256, 2560), (2560, 9728),
               (9728, 2560), (6144, 2560), (2560, 4096)]


@pytest.mark.parametrize("kernel", [1, 2, 3])
@pytest.mark.parametrize("N,K", GEMV_SHAPES)
def test_gemv(nf4, oracle, scratch, kernel, N, K):
    w = make_weight(1000 + N + K, N, K)
    am = oracle_absmax(oracle, w)
    l = _lin(nf4, w)
    x = _act(1009 + N, 1, K)
    y = torch.full((1, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    nf4.set_gemv_kernel(kernel)
    try:
        l.forward(scratch, x.cuda(), y, 1)
        torch.cuda.synchronize()
    finally:
        nf4.set_gemv_kernel(0)
    scratch.check()
    want = oracle.gemv(w.packed, w.quant_map, am, bf16_bits(x).reshape(-1), N, K, 64)
    assert_close_norm(bf16_bits(y).reshape(-1), want, REL, f"gemv k{kernel} {N}x{K}")


@pytest.mark.parametrize("N,K", [(8192, 5120), (5120, 8192), (5120, 25600)])
def test_gemv_large_model_shapes(nf4, oracle, scratch, N, K):
    """The attention and MLP-down linears of the 32B-class configuration, unsharded on one GPU
    (the default kernel choice; 25600 input columns are beyond the chained kernel's reach)."""
    w = make_weight(1500 + N + K, N, K)
    l = _lin(nf4, w)
    x = _act(1509 + N, 1, K)
    y = torch.full((1, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    l.forward(scratch, x.cuda(), y, 1)
    torch.cuda.synchronize()
    scratch.check()
    want = oracle.gemv(w.packed, w.quant_map, oracle_absmax(oracle, w), bf16_bits(x).reshape(-1), N, K, 64)
    assert_close_norm(bf16_bits(y).reshape(-1), want, REL, f"gemv {N}x{K}")
    if K <= 16384:
        y3 = torch.full((1, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        nf4.set_gemv_kernel(3)
        try:
            l.forward(scratch, x.cuda(), y3, 1)
            torch.cuda.synchronize()
        finally:
            nf4.set_gemv_kernel(0)
        scratch.check()
        assert_close_norm(bf16_bits(y3).reshape(-1), want, REL, f"chained gemv {N}x{K}")
    l.close()


def test_gate_up_swiglu_large_model_shape(nf4, oracle, scratch):
    ff, K = 25600, 5120
    ws = [make_weight(1600, ff, K), make_weight(1601, ff, K)]
    f, _ = _fused(nf4, ws)
    packed = np.concatenate([w.packed for w in ws])
    am = np.concatenate([oracle_absmax(oracle, w) for w in ws])
    x = _act(1609, 1, K)
    want = oracle.gemv_gate_up_swiglu(packed, ws[0].quant_map, am, bf16_bits(x).reshape(-1), ff, K, 64)
    for kernel in (0, 3):
        out = torch.full((1, ff), float("nan"), dtype=torch.bfloat16, device="cuda")
        nf4.set_gemv_kernel(kernel)
        try:
            assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x.cuda(), out, ff)
            torch.cuda.synchronize()
        finally:
            nf4.set_gemv_kernel(0)
        scratch.check()
        assert_close_norm(bf16_bits(out).reshape(-1), want, REL, f"gate_up 2x{ff}x{K} kernel {kernel}")
    f.close()


def test_gemv_repeatable_and_residual(nf4, oracle, scratch):
    N, K = 2560, 9728
    w = make_weight(31, N, K)
    am = oracle_absmax(oracle, w)
    l = _lin(nf4, w)
    x = _act(32, 1, K).cuda()
    res = _act(33, 1, N)
    ys = []
    for _ in range(3):  # the split-K counters must return to zero after every launch
        y = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
        l.forward(scratch, x, y, 1, add_residual=res.cuda())
        ys.append(bf16_bits(y))
    assert np.array_equal(ys[0], ys[1]) and np.array_equal(ys[1], ys[2]), "not deterministic"
    want = oracle.gemv(w.packed, w.quant_map, am, bf16_bits(x).reshape(-1), N, K, 64,
                       residual=bf16_bits(res).reshape(-1))
    assert_close_norm(ys[0].reshape(-1), want, REL, "gemv+residual")


def test_gemv_non_nested(nf4, oracle, scratch):
    N, K = 512, 2560
    w = make_weight(41, N, K, 64, nested=False)
    l = _lin(nf4, w)
    x = _act(42, 1, K)
    for kernel in (1, 2, 3):
        y = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
        nf4.set_gemv_kernel(kernel)
        try:
            l.forward(scratch, x.cuda(), y, 1)
        finally:
            nf4.set_gemv_kernel(0)
        want = oracle.gemv(w.packed, w.quant_map, w.absmax_f32, bf16_bits(x).reshape(-1), N, K, 64)
        assert_close_norm(bf16_bits(y).reshape(-1), want, REL, f"gemv f32-absmax k{kernel}")


# ---------------------------------------------------------------- fused rows, gate+up+SiLU
def _fused(nf4, ws):
    ls = [_lin(nf4, w) for w in ws]
    f = nf4.Bnb4BitLinear()
    assert f.init_fused_rows(*ls), f.last_error
    return f, ls


def test_fused_rows_qkv(nf4, oracle, scratch):
    K = 2560
    ws = [make_weight(51, 4096, K), make_weight(52, 1024, K), make_weight(53, 1024, K)]
    f, _ = _fused(nf4, ws)
    assert f.out_features() == 6144
    packed = np.concatenate([w.packed for w in ws])
    am = np.concatenate([oracle_absmax(oracle, w) for w in ws])
    assert np.array_equal(f.expand_absmax(64).cpu().numpy().reshape(-1).view(np.uint32),
                          am.view(np.uint32))
    want = oracle.dequantize_kn(packed, ws[0].quant_map, am, 6144, K, 64)
    assert np.array_equal(bf16_bits(f.dequantize_weight()), want)
    x = _act(54, 1, K)
    y = torch.empty(1, 6144, dtype=torch.bfloat16, device="cuda")
    f.forward(scratch, x.cuda(), y, 1)
    wanty = oracle.gemv(packed, ws[0].quant_map, am, bf16_bits(x).reshape(-1), 6144, K, 64)
    assert_close_norm(bf16_bits(y).reshape(-1), wanty, REL, "qkv gemv")


def test_fused_rows_ragged_sources(nf4, oracle):
    """Sources whose row counts are not multiples of the 16-row tile."""
    K = 256
    ws = [make_weight(61, 40, K), make_weight(62, 7, K), make_weight(63, 33, K),
          make_weight(64, 16, K)]
    f, _ = _fused(nf4, ws)
    packed = np.concatenate([w.packed for w in ws])
    am = np.concatenate([oracle_absmax(oracle, w) for w in ws])
    want = oracle.dequantize_kn(packed, ws[0].quant_map, am, 96, K, 64)
    assert np.array_equal(bf16_bits(f.dequantize_weight()), want)


def test_fused_rows_rejects_mismatch(nf4):
    a, b = _lin(nf4, make_weight(1, 32, 128)), _lin(nf4, make_weight(2, 32, 256))
    f = nf4.Bnb4BitLinear()
    assert not f.init_fused_rows(a, b)
    assert "incompatible" in f.last_error
    assert not f.init_fused_rows(a)
    assert "2 to 4" in f.last_error


@pytest.mark.parametrize("kernel", [1, 2, 3])
@pytest.mark.parametrize("ff,K", [(64, 512), (1216, 2560), (9728, 2560)])
def test_gate_up_swiglu_decode(nf4, oracle, scratch, kernel, ff, K):
    ws = [make_weight(2000 + ff, ff, K), make_weight(2001 + ff, ff, K)]
    f, _ = _fused(nf4, ws)
    packed = np.concatenate([w.packed for w in ws])
    am = np.concatenate([oracle_absmax(oracle, w) for w in ws])
    x = _act(2009, 1, K)
    out = torch.full((1, ff), float("nan"), dtype=torch.bfloat16, device="cuda")
    nf4.set_gemv_kernel(kernel)
    try:
        assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x.cuda(), out, ff)
        torch.cuda.synchronize()
    finally:
        nf4.set_gemv_kernel(0)
    scratch.check()
    want = oracle.gemv_gate_up_swiglu(packed, ws[0].quant_map, am, bf16_bits(x).reshape(-1), ff, K, 64)
    assert_close_norm(bf16_bits(out).reshape(-1), want, REL, f"gate_up k{kernel}")


def test_gate_up_not_applicable(nf4, scratch):
    f, _ = _fused(nf4, [make_weight(1, 64, 128), make_weight(2, 64, 128)])
    x = _act(3, 1, 128).cuda()
    out = torch.empty(1, 64, dtype=torch.bfloat16, device="cuda")
    assert not nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x, out, 48)
    assert not nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x.float(), out, 64)


# ---------------------------------------------------------------- prefill GEMM (tcgen05)
@pytest.mark.parametrize("M,N,K", [(2, 32, 64), (7, 48, 128), (128, 256, 512), (200, 272, 448),
                                   (333, 1000, 1024), (512, 2560, 2560), (2048, 1024, 2560)])
def test_prefill_gemm(nf4, oracle, scratch, M, N, K):
    w = make_weight(3000 + M + N, N, K)
    am = oracle_absmax(oracle, w)
    l = _lin(nf4, w)
    x = _act(3009 + M, M, K)
    y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    l.forward(scratch, x.cuda(), y, M)
    torch.cuda.synchronize()
    scratch.check()
    want = oracle.forward(w.packed, w.quant_map, am, bf16_bits(x), M, N, K, 64)
    assert_close_norm(bf16_bits(y), want, REL, f"prefill {M}x{N}x{K}")


def test_prefill_residual(nf4, oracle, scratch):
    M, N, K = 130, 264, 256
    w = make_weight(3100, N, K)
    am = oracle_absmax(oracle, w)
    l = _lin(nf4, w)
    x, res = _act(3101, M, K), _act(3102, M, N)
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    l.forward(scratch, x.cuda(), y, M, add_residual=res.cuda())
    wb = bits_to_f32(oracle.dequantize_nk(w.packed, w.quant_map, am, N, K, 64)).astype(np.float64)
    want = bits_to_f32(bf16_bits(x)).astype(np.float64) @ wb.T + bits_to_f32(bf16_bits(res))
    got = bits_to_f32(bf16_bits(y)).astype(np.float64)
    assert np.abs(got - want).max() <= REL * np.abs(want).max()


@pytest.mark.parametrize("M,ff,K", [(5, 64, 128), (130, 1216, 512), (2048, 1216, 2560)])
def test_prefill_gate_up_swiglu(nf4, oracle, scratch, M, ff, K):
    ws = [make_weight(3200 + ff, ff, K), make_weight(3201 + ff, ff, K)]
    f, _ = _fused(nf4, ws)
    packed = np.concatenate([w.packed for w in ws])
    am = np.concatenate([oracle_absmax(oracle, w) for w in ws])
    x = _act(3209, M, K)
    out = torch.full((M, ff), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x.cuda(), out, ff,
                                                              seq_len=M)
    torch.cuda.synchronize()
    scratch.check()
    gu = oracle.forward(packed, ws[0].quant_map, am, bf16_bits(x), M, 2 * ff, K, 64)
    want = oracle.swiglu_rows(gu, M, ff)
    assert_close_norm(bf16_bits(out), want, REL, f"prefill swiglu {M}x{ff}x{K}")


def test_prefill_pair_full_size_properties(nf4, oracle, scratch):
    """cfg3 at full size (M = 2048, gate_up 2560 -> 2*9728, down 9728 -> 2560): linearity in
    x and a row-sample check against the oracle (the full CPU product would take minutes)."""
    M, H, FF = 2048, 2560, 9728
    gate, up = make_weight(3004, FF, H), make_weight(3005, FF, H)
    f, _ = _fused(nf4, [gate, up])
    down = _lin(nf4, make_weight(3006, H, FF))
    x = _act(3009, M, H).cuda()
    mid = torch.empty(M, FF, dtype=torch.bfloat16, device="cuda")
    assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x, mid, FF, seq_len=M)
    y = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    down.forward(scratch, mid, y, M)
    torch.cuda.synchronize()
    scratch.check()
    assert torch.isfinite(y.float()).all()
    # sampled rows against the oracle, gate_up + SwiGLU then down
    rows = [0, 1, 127, 128, 1029, 2047]
    packed = np.concatenate([gate.packed, up.packed])
    am = np.concatenate([oracle_absmax(oracle, gate), oracle_absmax(oracle, up)])
    xs = bf16_bits(x)[rows]
    gu = oracle.forward(packed, gate.quant_map, am, xs, len(rows), 2 * FF, H, 64)
    mid_want = oracle.swiglu_rows(gu, len(rows), FF)
    assert_close_norm(bf16_bits(mid)[rows], mid_want, REL, "cfg3 gate_up+swiglu rows")
    dw = make_weight(3006, H, FF)
    y_want = oracle.forward(dw.packed, dw.quant_map, oracle_absmax(oracle, dw),
                            bf16_bits(mid)[rows], len(rows), H, FF, 64)
    assert_close_norm(bf16_bits(y)[rows], y_want, REL, "cfg3 down rows")
    # linearity: W(2x) == 2 W(x) exactly in bf16 (power-of-two scaling)
    y2 = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    down.forward(scratch, mid * 2, y2, M)
    assert torch.equal(y2.float(), y.float() * 2)


# ---------------------------------------------------------------- shards
@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_shards_bit_equal_slices(nf4, oracle, world):
    N, K = 1024, 2560
    w = make_weight(4000, N, K)
    am = oracle_absmax(oracle, w)
    full = oracle.dequantize_kn(w.packed, w.quant_map, am, N, K, 64)  # [K, N]
    for r in range(world):
        l = nf4.Bnb4BitLinear()
        assert l.init_shard(w, 0, r, world, 0), l.last_error
        rows = N // world
        assert np.array_equal(bf16_bits(l.dequantize_weight()), full[:, r * rows:(r + 1) * rows])


@pytest.mark.parametrize("world", [2, 4, 8])
def test_col_shards_sum_to_full(nf4, oracle, scratch, world):
    N, K = 512, 4096
    w = make_weight(4100, N, K)
    am = oracle_absmax(oracle, w)
    full = oracle.dequantize_kn(w.packed, w.quant_map, am, N, K, 64)
    x = _act(4101, 1, K)
    acc = np.zeros(N, np.float64)
    cols = K // world
    for r in range(world):
        l = nf4.Bnb4BitLinear()
        assert l.init_shard(w, 1, r, world, 0), l.last_error
        assert np.array_equal(bf16_bits(l.dequantize_weight()), full[r * cols:(r + 1) * cols, :])
        y = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
        l.forward(scratch, x[:, r * cols:(r + 1) * cols].contiguous().cuda(), y, 1)
        acc += bits_to_f32(bf16_bits(y).reshape(-1))
    want = bits_to_f32(oracle.gemv(w.packed, w.quant_map, am, bf16_bits(x).reshape(-1), N, K, 64))
    assert np.abs(acc - want).max() <= REL * np.abs(want).max()


# ---------------------------------------------------------------- host-buffer entry points
def test_host_entry_points(nf4, oracle, scratch):
    ff, K = 256, 512
    ws = [make_weight(5000, ff, K), make_weight(5001, ff, K)]
    f, _ = _fused(nf4, ws)
    packed = np.concatenate([w.packed for w in ws])
    am = np.concatenate([oracle_absmax(oracle, w) for w in ws])
    x = _act(5002, 1, K).pin_memory()
    y = torch.empty(1, 2 * ff, dtype=torch.bfloat16).pin_memory()
    f.forward_host(scratch, x, y, 1)
    want = oracle.gemv(packed, ws[0].quant_map, am, bf16_bits(x).reshape(-1), 2 * ff, K, 64)
    assert_close_norm(bf16_bits(y).reshape(-1), want, REL, "forward_host")
    out = torch.empty(1, ff, dtype=torch.bfloat16).pin_memory()
    f.gate_up_swiglu_host(scratch, x, out, 1, ff)
    want = oracle.gemv_gate_up_swiglu(packed, ws[0].quant_map, am, bf16_bits(x).reshape(-1), ff, K, 64)
    assert_close_norm(bf16_bits(out).reshape(-1), want, REL, "gate_up_swiglu_host")


def test_forward_error_behaviour(nf4, scratch):
    l = _lin(nf4, make_weight(1, 32, 128))
    x = torch.zeros(1, 128, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(1, 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="bf16"):
        l.forward(scratch, x.float(), y, 1)
    with pytest.raises(RuntimeError, match="seq_len"):
        l.forward(scratch, x, y, 0)


def test_cache_dequant_env_mode(oracle, tmp_path):
    """AILA_BNB4_CACHE_DEQUANT=1 (the reference's flag, Bnb4BitLinear.cpp:642-650): the bf16
    weight cache gives the same prefill result as the per-call dequantisation route. The flag is
    read once per process, so the check runs in a child process."""
    import os
    import subprocess
    import sys
    script = tmp_path / "cache_mode.py"
    script.write_text(
        "import sys, torch, numpy as np\n"
        f"sys.path.insert(0, {os.path.dirname(os.path.dirname(os.path.abspath(__file__)))!r})\n"
        "from aila_b200 import synth\n"
        "from aila_b200.linear import Bnb4BitLinear, Bnb4BitLinearScratch\n"
        "w = synth.synth_linear(77, 272, 448)\n"
        "l = Bnb4BitLinear(); assert l.init(w, 0), l.last_error\n"
        "assert l.device_bytes() > 272 * 448 * 2\n"
        "s = Bnb4BitLinearScratch(0)\n"
        "x = synth.gaussian_activation(78, 200, 448).cuda()\n"
        "y = torch.empty(200, 272, dtype=torch.bfloat16, device='cuda')\n"
        "l.forward(s, x, y, 200); torch.cuda.synchronize(); s.check()\n"
        "np.save(sys.argv[1], y.cpu().view(torch.uint16).numpy())\n")
    out = tmp_path / "y.npy"
    env = dict(os.environ, AILA_BNB4_CACHE_DEQUANT="1")
    subprocess.run([sys.executable, str(script), str(out)], check=True, env=env, timeout=300)
    got = np.load(out)
    w = make_weight(77, 272, 448)
    x = _act(78, 200, 448)
    want = oracle.forward(w.packed, w.quant_map, oracle_absmax(oracle, w), bf16_bits(x), 200, 272,
                          448, 64)
    assert_close_norm(got, want, REL, "prefill with bf16 weight cache")


def test_dependent_decode_launches_in_cuda_graph(nf4):
    """A chain of decode launches where each consumes the previous one's output, captured in a
    CUDA graph and replayed: with programmatic dependent launch the consumer kernel is already
    resident while its input is being written, so its loads of x must not come from a
    non-coherent cache. Every replay (the first included) must reproduce the eager results."""
    H, FF = 1024, 2048
    g, u, d = make_weight(1, FF, H), make_weight(2, FF, H), make_weight(3, H, FF)
    Bnb4BitLinear = nf4.Bnb4BitLinear
    lg, lu, gu, ld = Bnb4BitLinear(), Bnb4BitLinear(), Bnb4BitLinear(), Bnb4BitLinear()
    assert lg.init(g, 0) and lu.init(u, 0) and gu.init_fused_rows(lg, lu) and ld.init(d, 0)
    sc = nf4.Bnb4BitLinearScratch(0)
    x = synth.gaussian_activation(11, 1, H).cuda()

    def mlp(inp):
        mid = torch.empty(1, FF, dtype=torch.bfloat16, device="cuda")
        assert Bnb4BitLinear.try_forward_decode_gate_up_swiglu(gu, sc, inp, mid, FF)
        y = torch.empty(1, H, dtype=torch.bfloat16, device="cuda")
        ld.forward(sc, mid, y, 1, add_residual=inp)
        return y

    y0 = mlp(x)
    torch.cuda.synchronize()
    y1 = mlp(y0)
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            ya = mlp(x)
            yb = mlp(ya)
        for _ in range(3):
            gr.replay()
            st.synchronize()
            assert torch.equal(ya, y0) and torch.equal(yb, y1)
    sc.check()


def test_linear_from_checkpoint_file(nf4, oracle, tmp_path):
    """safetensors file -> aila_st_load_bnb4_weight -> aila_nf4_linear_create: the weight goes from
    the mapped file straight into the device layout; dequantised values are bit-equal to the
    oracle's and to a linear created from the same tensors in memory."""
    from aila_b200 import checkpoint
    N, K = 80, 384
    w = make_weight(91, N, K, 64, True)
    path = tmp_path / "m.safetensors"
    tensors = {"pad": np.zeros(3, dtype=np.uint8)}  # odd-sized neighbour: unaligned tensor data
    tensors.update(checkpoint.bnb4_checkpoint_tensors("model.layers.3.self_attn.o_proj.weight", w))
    checkpoint.write_safetensors(str(path), tensors)
    with checkpoint.SafetensorsFile(str(path)) as f:
        lin = nf4.Bnb4BitLinear()
        assert lin.init_from_desc(f.load_bnb4_weight_ref("model.layers.3.self_attn.o_proj.weight", 0)), \
            lin.last_error
    direct = _lin(nf4, w)
    got = lin.dequantize_weight().cpu().view(torch.uint16).numpy()
    assert np.array_equal(got, direct.dequantize_weight().cpu().view(torch.uint16).numpy())
    want = oracle.dequantize_kn(w.packed, w.quant_map, oracle_absmax(oracle, w), N, K, 64)
    assert np.array_equal(got, want.reshape(K, N))


# ---------------------------------------------------------------- dense bf16 linear (lm_head)
def _dense_weight(seed, N, K):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)


@pytest.mark.parametrize("N,K", [(32, 64), (1000, 2560), (37, 264), (130, 100), (5, 8), (4099, 4096)])
def test_dense_linear_decode(nf4, oracle, scratch, N, K):
    """seq_len == 1 of the dense linear against the CPU oracle (bf16 weights, fp32 accumulation,
    one bf16 rounding); (130, 100) has K % 8 != 0 and takes the scalar kernel."""
    w = _dense_weight(7000 + N + K, N, K)
    lin = nf4.Linear()
    lin.init(w, K, N, 0)
    assert (lin.in_features(), lin.out_features()) == (K, N)
    x = _act(7100 + N, 1, K)
    y = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
    lin.forward(scratch, x.cuda(), y, 1)
    want = oracle.gemm_bf16w(bf16_bits(w), bf16_bits(x), 1, N, K)
    assert_close_norm(bf16_bits(y.cpu()), want, REL)
    # fp32 products of bf16 values are exact and both sides accumulate in fp32: the results may
    # differ by summation order only
    assert np.abs(bits_to_f32(bf16_bits(y.cpu())) - bits_to_f32(want)).max() <= \
        4e-3 * np.abs(bits_to_f32(want)).max() + 1e-6
    res = _act(7200 + N, 1, N)
    lin.forward(scratch, x.cuda(), y, 1, add_residual=res.cuda())
    want_r = bits_to_f32(want) + bits_to_f32(bf16_bits(res))
    assert np.abs(bits_to_f32(bf16_bits(y.cpu())) - want_r).max() <= 2e-2 * np.abs(want_r).max()


def test_dense_lm_head_full_size(nf4, oracle, scratch):
    """The whole 151936 x 2560 bf16 output head at seq_len == 1, and its argmax, against the CPU
    oracle."""
    N, K = 151936, 2560
    g = torch.Generator().manual_seed(7300)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    lin = nf4.Linear()
    lin.init(w, K, N, 0)
    x = _act(7301, 1, K)
    y = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
    lin.forward(scratch, x.cuda(), y, 1)
    torch.cuda.synchronize()
    want = oracle.gemm_bf16w(bf16_bits(w), bf16_bits(x), 1, N, K)
    got = bf16_bits(y.cpu())
    assert np.abs(bits_to_f32(got) - bits_to_f32(want)).max() <= 4e-3 * np.abs(bits_to_f32(want)).max() + 1e-6
    assert int(np.argmax(bits_to_f32(got))) == int(np.argmax(bits_to_f32(want)))


def test_dense_linear_prefill(nf4, oracle, scratch):
    N, K, M = 640, 512, 96
    w = _dense_weight(7301, N, K)
    lin = nf4.Linear()
    lin.init(w.cuda(), K, N, 0)  # device-resident weight
    x = _act(7302, M, K)
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    lin.forward(scratch, x.cuda(), y, M)
    want = oracle.gemm_bf16w(bf16_bits(w), bf16_bits(x), M, N, K)
    assert_close_norm(bf16_bits(y.cpu()), want, REL)


def test_dense_linear_errors(nf4, scratch):
    lin = nf4.Linear()
    with pytest.raises(RuntimeError):
        lin.init(torch.zeros(4, 8), 8, 4, 0)  # not bf16
    lin.init(_dense_weight(1, 16, 40), 40, 16, 0)
    x = torch.zeros(2, 40, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(2, 16, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        lin.forward(scratch, x.float(), y, 1)
    from aila_b200 import _lib
    with pytest.raises(_lib.Nf4Error):
        lin.forward(scratch, x, y, 2)  # in_features % 64 != 0: the GEMM does not take it


def test_argmax_bf16(nf4):
    """The greedy choice against the oracle's restatement of ops::argmax (itself held against the
    reference's kernel): random logits, crafted ties (the reference's tree keeps the left candidate,
    so equal maxima resolve by bit-reversed index % 256, not by index), nothing above the start value,
    and vocabulary shards whose local result must be the global one."""
    from oracle import backend_numpy as B
    g = torch.Generator().manual_seed(5)
    out = torch.full((1,), -1, dtype=torch.int32, device="cuda")

    def run(logits, offset=0):
        nf4.argmax(logits.cuda(), logits.numel(), out, offset)
        return int(out.item())

    for n in (1, 7, 1024, 151936):
        logits = torch.randn(n, generator=g).to(torch.bfloat16)
        if n > 100:
            logits[n // 3] = 9.0
            logits[n // 2] = 9.0
        assert run(logits) == B.argmax(bf16_bits(logits))
    for tied in ([2, 257], [1, 2], [128, 1], [255, 510], [3, 5, 9, 17], [700, 701, 702, 703], [40, 300]):
        logits = (torch.randn(1024, generator=g) * 0.1).to(torch.bfloat16)
        logits[tied] = 9.0
        want = B.argmax(bf16_bits(logits))
        assert run(logits) == want and want in tied
    logits = (torch.randn(1024, generator=g) * 0.1).to(torch.bfloat16)
    logits[[1, 2]] = 9.0
    assert run(logits) == 2                      # not the smallest index
    assert run(torch.full((300,), -3e38).to(torch.bfloat16)) == 0
    assert run(torch.full((300,), float("nan")).to(torch.bfloat16)) == 0
    # shards of 18992 entries (151936 / 8): offsets that are no multiple of 256
    logits = torch.randn(4 * 18992, generator=g).to(torch.bfloat16)
    logits[[18992 + 5, 18992 + 6, 18992 + 700]] = 9.0
    for r in range(4):
        part = logits[r * 18992:(r + 1) * 18992].contiguous()
        assert run(part, r * 18992) == B.argmax(bf16_bits(part), r * 18992)
    whole = B.argmax(bf16_bits(logits))
    assert whole == run(logits) and whole == 18992 + run(logits[18992:2 * 18992].contiguous(), 18992)


@pytest.mark.parametrize("M", [2, 5, 8, 9, 17, 32, 33, 41, 48, 49, 65])
def test_small_batch_routes_agree(nf4, oracle, scratch, M):
    """2..48 rows take the small-batch decode kernels (launches of up to 32 rows, one weight pass
    each), more rows the dequantise + GEMM route: both must meet the bound against the oracle's
    forward."""
    N, K = 272, 512
    w = make_weight(8100 + M, N, K)
    lin = _lin(nf4, w)
    x = _act(8200 + M, M, K)
    res = _act(8300 + M, M, N)
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    lin.forward(scratch, x.cuda(), y, M, add_residual=res.cuda())
    want = bits_to_f32(oracle.forward(w.packed, w.quant_map, oracle_absmax(oracle, w), bf16_bits(x),
                                      M, N, K, 64)) + bits_to_f32(bf16_bits(res))
    got = bits_to_f32(bf16_bits(y.cpu()))
    assert np.abs(got - want).max() <= REL * np.abs(want).max()


@pytest.mark.parametrize("N,K,nested,M", [(16, 64, True, 2), (100, 448, False, 3), (2560, 9728, True, 8),
                                          (6144, 2560, True, 5), (33, 128, True, 7),
                                          # two and four row blocks in one launch; ragged row counts;
                                          # outputs long enough that row tiles are shared between CTAs
                                          (2560, 9728, True, 16), (6144, 2560, True, 32), (100, 448, False, 13),
                                          (5120, 5120, False, 27), (33, 128, True, 32), (19456, 2560, True, 24)])
def test_batched_decode_rows_match_single_rows(nf4, scratch, N, K, nested, M):
    """Every row of a batched decode launch against the single-row kernel on the same row: the
    same dequantised operands and fp32 accumulation, different summation order across warps."""
    w = make_weight(8400 + N + M, N, K, 64, nested)
    lin = _lin(nf4, w)
    x = _act(8500 + N, M, K).cuda()
    yb = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    lin.forward(scratch, x, yb, M)
    ys = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    for m in range(M):
        lin.forward(scratch, x[m:m + 1].contiguous(), ys[m:m + 1], 1)
    torch.cuda.synchronize()
    a, b = yb.float().cpu().numpy(), ys.float().cpu().numpy()
    assert np.abs(a - b).max() <= 1e-2 * np.abs(b).max() + 1e-6


@pytest.mark.parametrize("M", [2, 8, 11, 16, 32])
def test_batched_gate_up_swiglu(nf4, oracle, scratch, M):
    H, FF = 512, 1040
    g, u = make_weight(8601, FF, H), make_weight(8602, FF, H)
    lg, lu, f = _lin(nf4, g), _lin(nf4, u), nf4.Bnb4BitLinear()
    assert f.init_fused_rows(lg, lu)
    x = _act(8603 + M, M, H)
    out = torch.empty(M, FF, dtype=torch.bfloat16, device="cuda")
    assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x.cuda(), out, FF, seq_len=M)
    packed = np.concatenate([g.packed, u.packed])
    am = np.concatenate([oracle_absmax(oracle, g), oracle_absmax(oracle, u)])
    xb = bf16_bits(x)
    want = np.stack([oracle.gemv_gate_up_swiglu(packed, g.quant_map, am, xb[m], FF, H, 64) for m in range(M)])
    assert_close_norm(bf16_bits(out.cpu()), want, REL)


# ---------------------------------------------------------------- RMSNorm around the linears
def _bf16_ulp_close(got_bits, want_bits, max_ulp=1):
    """bf16 results that differ by at most `max_ulp` units in the last place (same sign)."""
    g, w = got_bits.astype(np.int32), want_bits.astype(np.int32)
    return np.abs(g - w).max() <= max_ulp


@pytest.mark.parametrize("rows,H,with_add", [(1, 2560, True), (3, 1024, True), (2, 100, False), (1, 5120, True)])
def test_add_rms_norm(nf4, oracle, rows, H, with_add):
    x, add = _act(9001 + H, rows, H), (_act(9002 + H, rows, H) if with_add else None)
    g = torch.Generator().manual_seed(9003)
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    xc = x.cuda()
    hidden = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    normed = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    nf4.add_rms_norm(xc, add.cuda() if with_add else None, w.cuda(), 1e-6, hidden, normed)
    want_h, want_n = oracle.add_rms_norm(bf16_bits(x), bf16_bits(add) if with_add else None, bf16_bits(w),
                                         1e-6, rows, H)
    assert np.array_equal(bf16_bits(hidden.cpu()), want_h)           # one exact fp32 add, one rounding
    assert _bf16_ulp_close(bf16_bits(normed.cpu()), want_n)            # reduction order, rsqrt: 1 ulp
    nf4.add_rms_norm(xc, add.cuda() if with_add else None, w.cuda(), 1e-6, xc, normed)  # in place
    assert np.array_equal(bf16_bits(xc.cpu()), want_h)


@pytest.mark.parametrize("N,K", [(272, 512), (6144, 2560), (2560, 9728)])
def test_forward_with_folded_rms_norm(nf4, oracle, scratch, N, K):
    """aila_nf4_forward_rmsnorm against (stand-alone RMSNorm kernel -> plain forward): the linear
    must see the same normalised input up to one bf16 ulp, and hidden_out the same residual
    stream; and against the oracle chain within the output bound."""
    w = make_weight(9100 + N, N, K)
    lin = _lin(nf4, w)
    x, add = _act(9101 + N, 1, K), _act(9102 + N, 1, K)
    g = torch.Generator().manual_seed(9103)
    nw = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16)
    res = _act(9104 + N, 1, N)
    y = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
    hidden = torch.empty(1, K, dtype=torch.bfloat16, device="cuda")
    assert lin.forward_rmsnorm(scratch, x.cuda(), nw.cuda(), 1e-6, y, add=add.cuda(), hidden_out=hidden,
                               add_residual=res.cuda())
    want_h, want_n = oracle.add_rms_norm(bf16_bits(x), bf16_bits(add), bf16_bits(nw), 1e-6, 1, K)
    assert np.array_equal(bf16_bits(hidden.cpu()), want_h)
    want = bits_to_f32(oracle.gemv(w.packed, w.quant_map, oracle_absmax(oracle, w), want_n.reshape(-1),
                                   N, K, 64)) + bits_to_f32(bf16_bits(res)).reshape(-1)
    got = bits_to_f32(bf16_bits(y.cpu())).reshape(-1)
    assert np.abs(got - want).max() <= REL * np.abs(want).max()
    # the unfused pair of launches gives (nearly) the same output
    normed = torch.empty(1, K, dtype=torch.bfloat16, device="cuda")
    nf4.add_rms_norm(x.cuda(), add.cuda(), nw.cuda(), 1e-6, None, normed)
    y2 = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
    lin.forward(scratch, normed, y2, 1, add_residual=res.cuda())
    assert np.abs(got - y2.float().cpu().numpy().reshape(-1)).max() <= 5e-3 * np.abs(want).max()
    with pytest.raises(Exception):
        lin.forward_rmsnorm(scratch, hidden, nw.cuda(), 1e-6, y, hidden_out=hidden)  # aliasing


def test_gate_up_swiglu_with_folded_rms_norm(nf4, oracle, scratch):
    H, FF = 1024, 2048
    g, u = make_weight(9201, FF, H), make_weight(9202, FF, H)
    lg, lu, f = _lin(nf4, g), _lin(nf4, u), nf4.Bnb4BitLinear()
    assert f.init_fused_rows(lg, lu)
    x = _act(9203, 1, H)
    gen = torch.Generator().manual_seed(9204)
    nw = (1.0 + 0.1 * torch.randn(H, generator=gen)).to(torch.bfloat16)
    out = torch.empty(1, FF, dtype=torch.bfloat16, device="cuda")
    assert nf4.Bnb4BitLinear.try_forward_decode_gate_up_swiglu_rmsnorm(f, scratch, x.cuda(), nw.cuda(),
                                                                       1e-6, out, FF)
    _, want_n = oracle.add_rms_norm(bf16_bits(x), None, bf16_bits(nw), 1e-6, 1, H)
    packed = np.concatenate([g.packed, u.packed])
    am = np.concatenate([oracle_absmax(oracle, g), oracle_absmax(oracle, u)])
    want = oracle.gemv_gate_up_swiglu(packed, g.quant_map, am, want_n.reshape(-1), FF, H, 64)
    assert_close_norm(bf16_bits(out.cpu()).reshape(-1), want, REL)
