"""TEST INFRASTRUCTURE ONLY: numpy restatement of the reference operators that sit between the NF4
linears in a Qwen3 decode step, and of the decode step itself. Every function cites the lines it
follows; embedding_lookup, decode_prepare_qkv, attention_decode and argmax are held against the
reference's own sources compiled for the host (tests/test_reference_pin.py); how the decode step
strings them together is restated from reading (the reference has no golden vectors for it).

  embedding_lookup     src/ops/ElementwiseOps.cpp:14-27
  decode_prepare_qkv   src/ops/ElementwiseOps.cpp:105-215
  attention_decode     src/ops/AttentionOps.cpp:73-166 (baseline, whole window)
  argmax               src/ops/SamplingOps.cpp:321-358
  decode_step          src/models/Qwen3Bnb4Backend.cpp:298-439 (seq_len == 1)

bf16 tensors travel as uint16 bit patterns; arithmetic is fp32 with the reference's roundings.
"""
from __future__ import annotations

import numpy as np


def to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, as a float -> bf16 conversion does."""
    u = np.asarray(x, np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) >> 16
    return r.astype(np.uint16)


def embedding_lookup(table_bits: np.ndarray, token_ids) -> np.ndarray:
    return np.asarray(table_bits, np.uint16)[np.asarray(token_ids, np.int64)]


def rope_freq(head_dim: int, theta: float) -> np.ndarray:
    """Qwen3Bnb4Backend.cpp:283-288."""
    d = np.arange(head_dim // 2, dtype=np.float32)
    return (np.float32(1.0) / np.power(np.float32(theta), (np.float32(2.0) * d) / np.float32(head_dim))).astype(np.float32)


def _head_norm_rotate(x_bits, w_bits, freq, pos, eps):
    x = to_f32(x_bits)
    head_dim = x.shape[-1]
    half = head_dim // 2
    rms = np.sqrt(np.float32((x.astype(np.float32) ** 2).sum(dtype=np.float32) / np.float32(head_dim) + np.float32(eps)))
    y = to_f32(to_bf16((x / rms) * to_f32(w_bits)))      # normalised values are stored as bf16
    angle = (np.float32(pos) * freq).astype(np.float32)
    c, s = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    a, b = y[:half], y[half:]
    return np.concatenate([to_bf16(a * c - b * s), to_bf16(b * c + a * s)])


def decode_prepare_qkv(q_bits, k_bits, v_bits, freq, q_norm_w, k_norm_w, k_cache, v_cache, pos, n_heads, n_kv,
                       head_dim, eps):
    """Returns the rotated q [n_heads*head_dim]; appends k, v to the caches [n_kv, max_len, head_dim]
    (uint16 arrays, modified in place)."""
    q = np.asarray(q_bits, np.uint16).reshape(n_heads, head_dim)
    k = np.asarray(k_bits, np.uint16).reshape(n_kv, head_dim)
    v = np.asarray(v_bits, np.uint16).reshape(n_kv, head_dim)
    q_out = np.stack([_head_norm_rotate(q[h], q_norm_w, freq, pos, eps) for h in range(n_heads)])
    for h in range(n_kv):
        k_cache[h, pos] = _head_norm_rotate(k[h], k_norm_w, freq, pos, eps)
        v_cache[h, pos] = v[h]
    return q_out.reshape(-1)


def _tree_reduce(part: np.ndarray, op) -> np.float32:
    """Balanced tree t[i] = op(t[i], t[i + w]), w = n/2 .. 1: the work-group reduction order the C
    oracle assumes as well (SYCL leaves it open)."""
    t = part.astype(np.float32).copy()
    w = t.size // 2
    while w >= 1:
        t[:w] = op(t[:w], t[w:2 * w])
        w //= 2
    return t[0]


def attention_decode(q_bits, k_cache, v_cache, n_heads, n_kv, head_dim, cached_len, wg_size: int = 512) -> np.ndarray:
    """ops::attention_decode on its baseline route (AttentionOps.cpp:73-166, the whole window, the
    default work-group of 512): per head, score[t] = (sum over d in order of q[d] * k[t][d]) * scale
    with every product and sum rounded to fp32; the maximum; e[t] = exp(score[t] - max); their sum
    as work-item partial sums (item l adds t = l, l + 512, ...) reduced by a balanced tree;
    p[t] = e[t] / sum; out[d] = the sum over t in order of p[t] * v[t][d], rounded to bf16."""
    q = to_f32(np.asarray(q_bits, np.uint16).reshape(n_heads, head_dim))
    per = n_heads // n_kv
    scale = np.float32(1.0) / np.sqrt(np.float32(head_dim))
    out = np.empty((n_heads, head_dim), np.uint16)
    T = cached_len
    J = (T + wg_size - 1) // wg_size
    for h in range(n_heads):
        kv = h // per
        kk = to_f32(k_cache[kv, :T])
        vv = to_f32(v_cache[kv, :T])
        s = np.zeros(T, np.float32)
        for d in range(head_dim):
            s = s + q[h, d] * kk[:, d]
        s = (s * scale).astype(np.float32)
        mx = np.float32(max(np.float32(-1e30), s.max()))
        e = np.exp((s - mx).astype(np.float32)).astype(np.float32)
        lanes = np.zeros((J, wg_size), np.float32)
        lanes.reshape(-1)[:T] = e
        part = np.zeros(wg_size, np.float32)
        for j in range(J):
            part = part + lanes[j]
        total = _tree_reduce(part, np.add)
        p = (e / total).astype(np.float32)
        acc = np.zeros(head_dim, np.float32)
        for t in range(T):
            acc = acc + p[t] * vv[t]
        out[h] = to_bf16(acc)
    return out.reshape(-1)


def argmax(logits_bits, index_offset: int = 0) -> int:
    """ops::argmax as the reference's one work-group of 256 items computes it: item l scans
    l, l + 256, ... and keeps the first strict maximum above -1e30 (index 0 if none), then a tree with
    strides 128 .. 1 in which position l takes position l + stride only if that value is strictly
    greater. With ``index_offset`` the logits are a shard starting at that global index; the scan
    is over global indices and the local index is returned."""
    v = to_f32(np.asarray(logits_bits, np.uint16).reshape(-1)).astype(np.float32)
    n = v.size
    vals = np.full(256, np.float32(-1e30), np.float32)
    idx = np.zeros(256, np.int64)
    g = np.arange(n, dtype=np.int64) + index_offset
    for lid in range(256):
        sel = np.nonzero((g & 255) == lid)[0]
        for i in sel:                       # strict '>' keeps the first maximum; NaN never wins
            if v[i] > vals[lid]:
                vals[lid], idx[lid] = v[i], g[i]
    stride = 128
    while stride > 0:
        for lid in range(stride):
            if vals[lid + stride] > vals[lid]:
                vals[lid], idx[lid] = vals[lid + stride], idx[lid + stride]
        stride >>= 1
    won = vals[0] > np.float32(-1e30)
    return int(idx[0] - index_offset) if won else 0


class Qwen3Reference:
    """The decode step with the C oracle for the linears (oracle.nf4_oracle): same buffers, same
    order, same roundings as Qwen3Bnb4Backend::forward for seq_len == 1."""

    def __init__(self, O, cfg, embed_bits, layers, final_norm_bits, lm_head_bits, max_seq_len):
        self.O, self.cfg = O, cfg
        self.embed, self.final_norm, self.lm_head = embed_bits, final_norm_bits, lm_head_bits
        self.layers = layers  # dicts: q, k, v, o, gate, up, down (Nf4Tensors) + norm bit arrays
        self.freq = rope_freq(cfg.head_dim, cfg.rope_theta)
        self.k_cache = [np.zeros((cfg.num_key_value_heads, max_seq_len, cfg.head_dim), np.uint16)
                        for _ in layers]
        self.v_cache = [np.zeros_like(c) for c in self.k_cache]
        self.pos = 0

    def _am(self, w):
        return self.O.expand_absmax(w.absmax_codes, w.nested_quant_map, w.nested_absmax, w.nested_blocksize,
                                    w.nested_offset)

    def _gemv(self, ws, x_bits):
        packed = np.concatenate([w.packed for w in ws])
        am = np.concatenate([self._am(w) for w in ws])
        n = sum(w.out_features for w in ws)
        return self.O.gemv(packed, ws[0].quant_map, am, x_bits.reshape(-1), n, ws[0].in_features, 64)

    def step(self, token: int) -> np.ndarray:
        O, c = self.O, self.cfg
        H, QD, KVD = c.hidden_size, c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        hidden = embedding_lookup(self.embed, [token]).reshape(1, H)
        _, normed = O.add_rms_norm(hidden, None, self.layers[0]["input_ln"], c.rms_norm_eps, 1, H)
        for i, L in enumerate(self.layers):
            qkv = self._gemv([L["q"], L["k"], L["v"]], normed)
            q = decode_prepare_qkv(qkv[:QD], qkv[QD:QD + KVD], qkv[QD + KVD:], self.freq, L["q_norm"], L["k_norm"],
                                   self.k_cache[i], self.v_cache[i], self.pos, c.num_attention_heads,
                                   c.num_key_value_heads, c.head_dim, c.rms_norm_eps)
            attn = attention_decode(q, self.k_cache[i], self.v_cache[i], c.num_attention_heads,
                                    c.num_key_value_heads, c.head_dim, self.pos + 1)
            o = self._gemv([L["o"]], attn)
            hidden, normed = O.add_rms_norm(hidden, o.reshape(1, H), L["post_attn_ln"], c.rms_norm_eps, 1, H)
            packed = np.concatenate([L["gate"].packed, L["up"].packed])
            am = np.concatenate([self._am(L["gate"]), self._am(L["up"])])
            mid = O.gemv_gate_up_swiglu(packed, L["gate"].quant_map, am, normed.reshape(-1), c.intermediate_size,
                                        H, 64)
            down = self._gemv([L["down"]], mid)
            nxt = self.layers[i + 1]["input_ln"] if i + 1 < len(self.layers) else self.final_norm
            hidden, normed = O.add_rms_norm(hidden, down.reshape(1, H), nxt, c.rms_norm_eps, 1, H)
        self.pos += 1
        return O.gemm_bf16w(self.lm_head, normed, 1, c.vocab_size, H).reshape(-1)
