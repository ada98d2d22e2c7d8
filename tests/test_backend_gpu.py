"""The decode-step operators between the linears (embedding, per-head norm + RoPE + cache append,
single-token attention) and the Qwen3 NF4 backend skeleton built on the library, against the numpy /
C oracle. Through the C ABI.
"""
import numpy as np
import pytest
import torch

from oracle import backend_numpy as ref
from tests.helpers import bf16_bits, make_weight

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from aila_b200 import backend
    assert torch.cuda.is_available()
    return backend



def _rand_bf16(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16)


def _close(got_bits, want_bits, rel, what):
    got, want = ref.to_f32(got_bits).astype(np.float64), ref.to_f32(want_bits).astype(np.float64)
    err = np.abs(got - want).max()
    assert err <= rel * max(np.abs(want).max(), 1e-6), f"{what}: max err {err} vs {np.abs(want).max()}"


def test_embedding_lookup(be):
    gen = torch.Generator().manual_seed(1)
    table = _rand_bf16(gen, 1000, 256)
    ids = torch.tensor([0, 999, 17, 17, 512], dtype=torch.int32)
    out = torch.empty(5, 256, dtype=torch.bfloat16, device="cuda")
    be.embedding_lookup(table.cuda(), ids.cuda(), out)
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(out), ref.embedding_lookup(bf16_bits(table), ids.numpy()))


@pytest.mark.parametrize("heads,kv,hd,pos", [(4, 2, 64, 0), (32, 8, 128, 37), (16, 16, 128, 1000), (8, 1, 256, 5)])
def test_decode_prepare_qkv(be, heads, kv, hd, pos):
    gen = torch.Generator().manual_seed(100 + heads + pos)
    max_len = 1024
    qkv = _rand_bf16(gen, 1, (heads + 2 * kv) * hd)
    qw, kw = (1 + 0.1 * torch.randn(hd, generator=gen)).to(torch.bfloat16), \
        (1 + 0.1 * torch.randn(hd, generator=gen)).to(torch.bfloat16)
    freq = ref.rope_freq(hd, 1e6)
    kc = torch.zeros(kv, max_len, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    dq = qkv.cuda()
    q, k, v = dq[:, :heads * hd], dq[:, heads * hd:(heads + kv) * hd], dq[:, (heads + kv) * hd:]
    be.decode_prepare_qkv(q, k, v, torch.from_numpy(freq).cuda(), qw.cuda(), kw.cuda(), kc, vc, pos, heads, kv, hd,
                          1e-6)
    torch.cuda.synchronize()
    bits = bf16_bits(qkv).reshape(-1)
    kc_w = np.zeros((kv, max_len, hd), np.uint16)
    vc_w = np.zeros_like(kc_w)
    q_w = ref.decode_prepare_qkv(bits[:heads * hd], bits[heads * hd:(heads + kv) * hd], bits[(heads + kv) * hd:], freq,
                                 bf16_bits(qw), bf16_bits(kw), kc_w, vc_w, pos, heads, kv, hd, 1e-6)
    # cos/sin of angles up to 1000 rad differ in the last bits between libraries: one bf16 ulp
    _close(bf16_bits(dq).reshape(-1)[:heads * hd], q_w, 1e-2, "q")
    _close(bf16_bits(kc)[:, pos].reshape(-1), kc_w[:, pos].reshape(-1), 1e-2, "k cache")
    assert np.array_equal(bf16_bits(vc)[:, pos], vc_w[:, pos])
    assert not bf16_bits(kc)[:, pos + 1:].any() and not bf16_bits(kc)[:, :pos].any()


@pytest.mark.parametrize("heads,kv,hd,length", [(4, 2, 64, 1), (32, 8, 128, 300), (16, 16, 128, 2047), (8, 1, 256, 33)])
def test_attention_decode(be, heads, kv, hd, length):
    gen = torch.Generator().manual_seed(200 + heads + length)
    max_len = 2048
    q = _rand_bf16(gen, 1, heads * hd)
    kc = _rand_bf16(gen, kv, max_len, hd)
    vc = _rand_bf16(gen, kv, max_len, hd)
    out = torch.empty(1, heads * hd, dtype=torch.bfloat16, device="cuda")
    be.attention_decode(q.cuda(), kc.cuda(), vc.cuda(), out, heads, kv, hd, length)
    torch.cuda.synchronize()
    want = ref.attention_decode(bf16_bits(q), bf16_bits(kc), bf16_bits(vc), heads, kv, hd, length)
    _close(bf16_bits(out).reshape(-1), want, 1e-2, "attention")


def test_backend_rejects_bad_arguments(be):
    from aila_b200 import _lib
    q = torch.zeros(1, 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(1, 16, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.Nf4Error):
        be.attention_decode(q, kc, kc, q, 2, 1, 64, 17)      # beyond the cache
    with pytest.raises(_lib.Nf4Error):
        be.attention_decode(q, kc, kc, q, 3, 2, 64, 4)       # heads not a multiple of kv heads
    f = torch.zeros(32, dtype=torch.float32, device="cuda")
    w = torch.ones(64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.Nf4Error):
        be.decode_prepare_qkv(q, q, q, f, w, w, kc, kc, 16, 2, 1, 64, 1e-6)   # context window exceeded


def test_qwen3_backend_decodes_like_the_oracle(be, oracle):
    """A two-layer model with grouped-query attention: six tokens through forward(), the logits of
    every step against the oracle's decode step, the greedy token where the oracle's margin is clear,
    and the reference's error for a full context."""
    cfg = be.Qwen3Config(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=64, vocab_size=640, rms_norm_eps=1e-6, rope_theta=1e6)
    H, QD, KVD, FF = 256, 256, 128, 512
    gen = torch.Generator().manual_seed(4242)
    embed = _rand_bf16(gen, cfg.vocab_size, H)
    lm_head = _rand_bf16(gen, cfg.vocab_size, H, scale=0.05)
    final_norm = (1 + 0.1 * torch.randn(H, generator=gen)).to(torch.bfloat16)
    layers, ref_layers = [], []
    for i in range(cfg.num_hidden_layers):
        w = dict(q=make_weight(900 + 10 * i, QD, H), k=make_weight(901 + 10 * i, KVD, H),
                 v=make_weight(902 + 10 * i, KVD, H), o=make_weight(903 + 10 * i, H, QD),
                 gate=make_weight(904 + 10 * i, FF, H), up=make_weight(905 + 10 * i, FF, H),
                 down=make_weight(906 + 10 * i, H, FF))
        norms = {k: (1 + 0.1 * torch.randn(n, generator=gen)).to(torch.bfloat16)
                 for k, n in (("input_ln", H), ("post_attn_ln", H), ("q_norm", 64), ("k_norm", 64))}
        layers.append(be.Qwen3LayerWeights(**w, **norms))
        ref_layers.append({**w, **{k: bf16_bits(v) for k, v in norms.items()}})
    model = be.Qwen3Bnb4Backend(cfg, 0, max_seq_len=8)
    model.load(embed, layers, final_norm, lm_head)
    golden = ref.Qwen3Reference(oracle, cfg, bf16_bits(embed), ref_layers, bf16_bits(final_norm), bf16_bits(lm_head), 8)
    tokens = [3, 600, 17, 17, 255, 1]
    # a prompt of three tokens in one call, then one token per call
    logits = model.forward(torch.tensor(tokens[:3], dtype=torch.int32))
    torch.cuda.synchronize()
    model.scratch.check()
    want = [golden.step(t) for t in tokens[:3]][-1]
    _close(bf16_bits(logits).reshape(-1), want, 3e-2, "logits after the prompt")
    for t in tokens[3:]:
        logits = model.forward(torch.tensor([t], dtype=torch.int32))
        tok = int(model.greedy_token().cpu()[0])
        model.scratch.check()
        want = golden.step(t)
        _close(bf16_bits(logits).reshape(-1), want, 3e-2, f"logits of token {t}")
        w32 = ref.to_f32(want)
        top2 = np.sort(w32)[-2:]
        if top2[1] - top2[0] > 0.05 * np.abs(w32).max():
            assert tok == int(np.argmax(w32))
    assert model.current_length == 6
    with pytest.raises(RuntimeError, match="context window exceeded"):
        model.forward(torch.tensor([1, 2, 3], dtype=torch.int32))
    # greedy generation replayed from one captured step must choose what step-by-step calls choose
    prompt = torch.tensor(tokens[:3], dtype=torch.int32)
    model.reset()
    model.forward(prompt)
    by_hand = []
    for _ in range(4):
        tok = model.greedy_token().clone()
        by_hand.append(int(tok.cpu()[0]))
        model.forward(tok)
    last_by_hand = bf16_bits(model.logits).copy()
    model.reset()
    model.forward(prompt)
    replayed = model.generate(2).cpu().tolist() + model.generate(2).cpu().tolist()
    torch.cuda.synchronize()
    model.scratch.check()
    assert replayed == by_hand
    assert np.array_equal(bf16_bits(model.logits), last_by_hand)
    assert model.current_length == 7
    with pytest.raises(RuntimeError, match="context window exceeded"):
        model.generate(2)
    model.close()
