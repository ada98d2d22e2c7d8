"""Qwen3 NF4 decode backend on top of the library: the callers of the NF4 linears
(reference Qwen3Bnb4Backend::forward, src/models/Qwen3Bnb4Backend.cpp:298-439) as a skeleton that
runs end to end on one GPU. Per layer and token: one chained launch (o_proj -> residual add +
RMSNorm -> gate|up + SwiGLU -> down), the next layer's qkv with its residual add + RMSNorm folded
in, one launch that normalises, rotates and caches q/k/v, one attention launch. A prompt is fed token by token through
the same path (the reference's separate prefill kernels are not built).

Buffers follow the reference's names (buf_.hidden, normed, qkv, attn_out, logits; KVCache with
k_cache(i) / v_cache(i) of shape [kv_heads, max_seq_len, head_dim]).
"""
from __future__ import annotations

import dataclasses

import torch

from . import _lib
from .linear import (Bnb4BitLinear, Bnb4BitLinearScratch, DecodeChain, Linear, _stream_ptr, add_rms_norm,
                     argmax)
from .synth import Nf4Tensors


@dataclasses.dataclass
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6


@dataclasses.dataclass
class Qwen3LayerWeights:
    """Host tensors of one layer: NF4 projections as checkpoint tensors, norms as bf16."""
    q: Nf4Tensors
    k: Nf4Tensors
    v: Nf4Tensors
    o: Nf4Tensors
    gate: Nf4Tensors
    up: Nf4Tensors
    down: Nf4Tensors
    input_ln: torch.Tensor
    post_attn_ln: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor


def embedding_lookup(table: torch.Tensor, token_ids: torch.Tensor, out: torch.Tensor) -> None:
    """ops::embedding_lookup (src/ops/ElementwiseOps.cpp:14-27)."""
    _lib.check(_lib.load().aila_embedding_lookup(table.data_ptr(), table.shape[0], token_ids.data_ptr(),
                                                 token_ids.numel(), table.shape[1], out.data_ptr(),
                                                 table.device.index, _stream_ptr(table.device)))


def decode_prepare_qkv(q, k, v, rope_freq, q_norm_w, k_norm_w, k_cache, v_cache, start_pos, num_heads,
                       num_kv_heads, head_dim, eps, position: torch.Tensor | None = None) -> None:
    """ops::decode_prepare_qkv (src/ops/ElementwiseOps.cpp:105-215); q, k, v may be views into one
    qkv buffer. ``position`` (int32 device tensor of one element) overrides start_pos on the device."""
    _lib.check(_lib.load().aila_decode_prepare_qkv(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), rope_freq.data_ptr(), q_norm_w.data_ptr(), k_norm_w.data_ptr(),
        k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[1], int(start_pos),
        position.data_ptr() if position is not None else None, num_heads, num_kv_heads,
        head_dim, float(eps), q.device.index, _stream_ptr(q.device)))


def attention_decode(q, k_cache, v_cache, out, num_heads, num_kv_heads, head_dim, cached_len,
                     position: torch.Tensor | None = None) -> None:
    """ops::attention_decode (src/ops/AttentionOps.cpp:73-166, whole window). With ``position`` the
    kernel attends to position + 1 cached tokens (read on the device); cached_len is then the most
    the launch can hold."""
    _lib.check(_lib.load().aila_attention_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                 out.data_ptr(), num_heads, num_kv_heads, head_dim,
                                                 int(cached_len), position.data_ptr() if position is not None else None,
                                                 k_cache.shape[1], q.device.index, _stream_ptr(q.device)))


class Qwen3Bnb4Backend:
    """load() once, then forward(token_ids) per step; returns the logits of the last token."""

    def __init__(self, cfg: Qwen3Config, device: int = 0, max_seq_len: int = 2048):
        self.cfg, self.device, self.max_seq_len = cfg, device, max_seq_len
        self.dev = torch.device("cuda", device)
        self.scratch = Bnb4BitLinearScratch(device)
        self.current_length = 0
        self._keep = []

    # -- load ---------------------------------------------------------------------------------
    def load(self, embed: torch.Tensor, layers: list, final_norm: torch.Tensor, lm_head) -> None:
        """layers: Qwen3LayerWeights (host checkpoint tensors), or dicts of device linears
        {qkv, o, gate_up, down} plus the four norm weights; lm_head: a [vocab, hidden] tensor or a
        ready Linear."""
        c, dev = self.cfg, self.dev
        H, QD, KVD = c.hidden_size, c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        self.QD, self.KVD = QD, KVD
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.embed = embed.to(**bf).contiguous()
        self.final_norm = final_norm.to(**bf).contiguous()
        if isinstance(lm_head, Linear):
            self.lm_head = lm_head
        else:
            self.lm_head = Linear()
            self.lm_head.init(lm_head.to(torch.bfloat16), H, c.vocab_size, self.device)
        self.hidden = torch.zeros(1, H, **bf)     # residual stream (ping)
        self.hidden2 = torch.zeros(1, H, **bf)    # residual stream (pong)
        self.normed = torch.zeros(1, H, **bf)
        self.qkv = torch.zeros(1, QD + 2 * KVD, **bf)
        self.attn_out = torch.zeros(1, QD, **bf)
        self.down_out = torch.zeros(1, H, **bf)
        self.logits = torch.zeros(1, c.vocab_size, **bf)
        self.token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.next_token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.position = torch.zeros(1, dtype=torch.int32, device=dev)   # device copy of current_length
        self._graph = None
        self.rope_freq = (1.0 / torch.pow(torch.tensor(float(c.rope_theta)),
                                          2.0 * torch.arange(c.head_dim // 2, dtype=torch.float32) / c.head_dim)
                          ).to(dev)
        self.k_cache = [torch.zeros(c.num_key_value_heads, self.max_seq_len, c.head_dim, **bf)
                        for _ in range(c.num_hidden_layers)]
        self.v_cache = [torch.zeros_like(t) for t in self.k_cache]
        self.lin, self.norms = [], []

        def lin(w):
            l = Bnb4BitLinear()
            if not l.init(w, self.device):
                raise RuntimeError(l.last_error)
            return l

        def fuse(*ls):
            f = Bnb4BitLinear()
            if not f.init_fused_rows(*ls):
                raise RuntimeError(f.last_error)
            for l in ls:
                l.close()
            return f

        for lw in layers:
            if isinstance(lw, dict):  # linears already on the device: qkv, o, gate_up, down + the four norms
                self.lin.append({k: lw[k] for k in ("qkv", "o", "gate_up", "down")})
                self.norms.append({k: lw[k].to(**bf).contiguous()
                                   for k in ("input_ln", "post_attn_ln", "q_norm", "k_norm")})
                continue
            self.lin.append(dict(qkv=fuse(lin(lw.q), lin(lw.k), lin(lw.v)), o=lin(lw.o),
                                 gate_up=fuse(lin(lw.gate), lin(lw.up)), down=lin(lw.down)))
            self.norms.append({k: getattr(lw, k).to(**bf).contiguous()
                               for k in ("input_ln", "post_attn_ln", "q_norm", "k_norm")})
        # one chain per layer: o_proj -> (+hidden, post-attention norm) gate|up + SwiGLU -> down.
        # (The next layer's qkv reads hidden2 and the MLP output through pointers, so it is a launch
        # of its own: operations of one chain exchange data through their links only.)
        self.chains = []
        for i in range(c.num_hidden_layers):
            L = self.lin[i]
            self.chains.append(DecodeChain(self.scratch, [
                dict(linear=L["o"], x=self.attn_out),
                dict(linear=L["gate_up"], ff_dim=c.intermediate_size,
                     norm=dict(weight=self.norms[i]["post_attn_ln"], eps=c.rms_norm_eps, add=self.hidden,
                               hidden_out=self.hidden2)),
                dict(linear=L["down"], y=self.down_out)]))

    # -- one token ------------------------------------------------------------------------------
    def _decode_one(self, on_device: bool = False) -> None:
        """One token through the model. on_device: the position comes from self.position (for a
        captured step that is replayed), and the attention launch is sized for the whole window."""
        c = self.cfg
        pos = self.current_length
        if pos + 1 > self.max_seq_len:
            raise RuntimeError(f"Qwen3Bnb4Backend::forward: context window exceeded (cached_len={pos + 1}, "
                               f"max_seq_len={self.max_seq_len})")
        where = self.position if on_device else None
        length = self.max_seq_len if on_device else pos + 1
        embedding_lookup(self.embed, self.token, self.hidden)
        add_rms_norm(self.hidden, None, self.norms[0]["input_ln"], c.rms_norm_eps, None, self.normed)
        self.lin[0]["qkv"].forward(self.scratch, self.normed, self.qkv, 1)
        q = self.qkv[:, :self.QD]
        k = self.qkv[:, self.QD:self.QD + self.KVD]
        v = self.qkv[:, self.QD + self.KVD:]
        n = c.num_hidden_layers
        for i in range(n):
            decode_prepare_qkv(q, k, v, self.rope_freq, self.norms[i]["q_norm"], self.norms[i]["k_norm"],
                               self.k_cache[i], self.v_cache[i], pos, c.num_attention_heads,
                               c.num_key_value_heads, c.head_dim, c.rms_norm_eps, where)
            attention_decode(q, self.k_cache[i], self.v_cache[i], self.attn_out, c.num_attention_heads,
                             c.num_key_value_heads, c.head_dim, length, where)
            self.chains[i].run()  # hidden2 = hidden + o_proj(attn); down_out = MLP(norm(hidden2))
            if i + 1 < n:
                # hidden = hidden2 + down_out; qkv of the next layer from its input norm, one launch
                nxt = self.lin[i + 1]["qkv"]
                if not nxt.forward_rmsnorm(self.scratch, self.down_out, self.norms[i + 1]["input_ln"],
                                           c.rms_norm_eps, self.qkv, add=self.hidden2, hidden_out=self.hidden):
                    add_rms_norm(self.down_out, self.hidden2, self.norms[i + 1]["input_ln"], c.rms_norm_eps,
                                 self.hidden, self.normed)
                    nxt.forward(self.scratch, self.normed, self.qkv, 1)
        # after the last layer: hidden2 holds hidden + o, down_out the MLP output
        add_rms_norm(self.hidden2, self.down_out, self.final_norm, c.rms_norm_eps, None, self.normed)
        self.lm_head.forward(self.scratch, self.normed, self.logits, 1)
        if not on_device:
            self.current_length = pos + 1

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """token_ids: int32 device tensor [seq_len]; appends them to the context and returns the
        bf16 logits [1, vocab] of the last one (reference forward(ctx, token_ids_device, seq_len))."""
        if token_ids.numel() <= 0:
            raise RuntimeError("Qwen3Bnb4Backend::forward: seq_len must be positive")
        ids = token_ids.to(device=self.dev, dtype=torch.int32).reshape(-1)
        for s in range(ids.numel()):
            self.token.copy_(ids[s:s + 1])
            self._decode_one()
        return self.logits

    def greedy_token(self) -> torch.Tensor:
        """ops::argmax over the current logits (device int32 tensor of one element)."""
        argmax(self.logits, self.cfg.vocab_size, self.next_token)
        return self.next_token

    def generate(self, n_tokens: int) -> torch.Tensor:
        """Greedy decoding of n_tokens after the context so far, starting from the token that the
        last forward() chose. One whole step (embedding ... lm_head, argmax, feeding the choice back
        and advancing the position) is captured in a CUDA graph once and replayed per token: the
        host issues one launch per token and never waits. Returns the int32 tokens [n_tokens]."""
        if self.current_length == 0:
            raise RuntimeError("generate() continues a context: call forward() with a prompt first")
        if self.current_length + n_tokens > self.max_seq_len:
            raise RuntimeError(f"Qwen3Bnb4Backend::generate: context window exceeded (cached_len="
                               f"{self.current_length + n_tokens}, max_seq_len={self.max_seq_len})")
        out = torch.empty(n_tokens, dtype=torch.int32, device=self.dev)
        stream = torch.cuda.current_stream(self.dev)
        self.position.fill_(self.current_length)
        argmax(self.logits, self.cfg.vocab_size, self.token)    # the choice after the context so far
        if self._graph is None:
            side = torch.cuda.Stream(self.dev)
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                self._decode_one(on_device=True)               # warm-up outside the capture (same state)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    self._decode_one(on_device=True)
                    argmax(self.logits, self.cfg.vocab_size, self.token)
                    self.position.add_(1)
            stream.wait_stream(side)
            self._graph = graph
        for i in range(n_tokens):
            out[i:i + 1].copy_(self.token)
            self._graph.replay()
        self.current_length += n_tokens
        return out

    def reset(self) -> None:
        self.current_length = 0

    def close(self) -> None:
        for ch in getattr(self, "chains", []):
            ch.close()
        self.chains = []
