"""The numpy restatement of the decode-step operators against an independent float64 computation
(CPU): it pins conventions (which halves RoPE pairs up, cache layout, grouped heads), not bits."""
import numpy as np
import torch

from oracle import backend_numpy as ref


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).numpy()


def test_rounding_helpers_match_torch():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(10000, generator=g) * 37.0
    assert np.array_equal(ref.to_bf16(x.numpy()), _bits(x.to(torch.bfloat16)))
    assert np.array_equal(ref.to_f32(_bits(x.to(torch.bfloat16))), x.to(torch.bfloat16).float().numpy())


def test_attention_decode_against_float64():
    g = torch.Generator().manual_seed(2)
    heads, kv, hd, n, max_len = 8, 2, 64, 50, 64
    q = torch.randn(heads * hd, generator=g).to(torch.bfloat16)
    kc = torch.randn(kv, max_len, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(kv, max_len, hd, generator=g).to(torch.bfloat16)
    got = ref.to_f32(ref.attention_decode(_bits(q), _bits(kc), _bits(vc), heads, kv, hd, n)).reshape(heads, hd)
    qd = q.double().reshape(heads, hd)
    for h in range(heads):
        k, v = kc[h // 4, :n].double(), vc[h // 4, :n].double()
        p = torch.softmax((k @ qd[h]) / np.sqrt(hd), dim=0)
        want = (p[:, None] * v).sum(0).numpy()
        assert np.abs(got[h] - want).max() <= 1e-2 * np.abs(want).max()


def test_prepare_qkv_against_float64():
    g = torch.Generator().manual_seed(3)
    heads, kv, hd, pos, max_len = 4, 2, 32, 11, 16
    q = torch.randn(heads * hd, generator=g).to(torch.bfloat16)
    k = torch.randn(kv * hd, generator=g).to(torch.bfloat16)
    v = torch.randn(kv * hd, generator=g).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(hd, generator=g)).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(hd, generator=g)).to(torch.bfloat16)
    freq = ref.rope_freq(hd, 10000.0)
    assert np.allclose(freq, 10000.0 ** (-2.0 * np.arange(hd // 2) / hd), rtol=1e-6)
    kc, vc = np.zeros((kv, max_len, hd), np.uint16), np.zeros((kv, max_len, hd), np.uint16)
    got = ref.to_f32(ref.decode_prepare_qkv(_bits(q), _bits(k), _bits(v), freq, _bits(qw), _bits(kw), kc, vc, pos,
                                            heads, kv, hd, 1e-6)).reshape(heads, hd)

    def want(x, w):
        x = x.double()
        y = x / torch.sqrt((x * x).mean() + 1e-6) * w.double()
        ang = torch.tensor(pos * freq.astype(np.float64))
        a, b = y[:hd // 2], y[hd // 2:]
        return torch.cat([a * torch.cos(ang) - b * torch.sin(ang), b * torch.cos(ang) + a * torch.sin(ang)]).numpy()

    for h in range(heads):
        w = want(q[h * hd:(h + 1) * hd], qw)
        assert np.abs(got[h] - w).max() <= 2e-2 * np.abs(w).max()
    for h in range(kv):
        w = want(k[h * hd:(h + 1) * hd], kw)
        assert np.abs(ref.to_f32(kc[h, pos]) - w).max() <= 2e-2 * np.abs(w).max()
        assert np.array_equal(vc[h, pos], _bits(v)[h * hd:(h + 1) * hd])
    assert not kc[:, :pos].any() and not kc[:, pos + 1:].any()


def test_reference_tie_key_orders_like_the_reduction():
    """sharded.reference_tie_key (the order the vocabulary-parallel head uses between ranks) picks,
    among tied logits, the index the oracle's restatement of ops::argmax picks."""
    import torch

    from aila_b200 import sharded
    rng = np.random.default_rng(11)
    for _ in range(50):
        n = int(rng.integers(300, 3000))
        tied = rng.choice(n, size=int(rng.integers(2, 7)), replace=False)
        logits = ref.to_bf16((rng.standard_normal(n) * 0.1).astype(np.float32))
        logits[tied] = ref.to_bf16(np.float32([7.0]))[0]
        keys = sharded.reference_tie_key(torch.from_numpy(tied.astype(np.int64)))
        assert int(tied[int(torch.argmin(keys))]) == ref.argmax(logits)
