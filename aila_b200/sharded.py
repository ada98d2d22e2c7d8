"""Multi-GPU layer for the NF4 linears: one process per GPU, torch.distributed for the exchange.

Net-new relative to the reference (single device, no collectives). A weight shards naturally:
  * rows (out_features)  -> column-parallel linear, no exchange inside the op: q/k/v, gate, up;
  * columns (in_features) -> row-parallel linear, exactly one sum exchange: o_proj, down.
The MLP is chained Megatron-style: gate|up row-sharded with the SwiGLU kept local (each rank
holds gate_r and up_r), down column-sharded on the same ranks, so the only collective per MLP is
one all-reduce of the [M, hidden] partial sums.

Shards are cut from the whole-weight descriptor by ``aila_nf4_linear_create_shard`` and keep the
original second-level absmax numbering, so their dequantised values are bit-equal to the same
slice of the unsharded weight.

The compute object is injectable so that the host logic (slicing rules, collectives, result
assembly) can be exercised on CPU ranks with the gloo backend; the default is the CUDA library
and it has no fallback.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from .synth import Nf4Tensors

ROWS, COLS = _lib.SHARD_ROWS, _lib.SHARD_COLS


def check_shardable(w: Nf4Tensors, mode: int, world: int) -> None:
    """The divisibility rules of aila_nf4_linear_create_shard, raised early on the host."""
    if world <= 0:
        raise ValueError("world must be positive")
    if mode == ROWS:
        if w.out_features % world:
            raise ValueError(f"out_features {w.out_features} is not divisible by {world} shards")
    elif mode == COLS:
        if w.in_features % world or (w.in_features // world) % w.blocksize:
            raise ValueError(f"in_features {w.in_features} / {world} shards must be a multiple of "
                             f"blocksize {w.blocksize}")
    else:
        raise ValueError("unknown shard mode")


def shard_bounds(w: Nf4Tensors, mode: int, rank: int, world: int) -> tuple[int, int, int, int]:
    """(row0, rows, col0, cols) kept by ``rank``."""
    check_shardable(w, mode, world)
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    if mode == ROWS:
        rows = w.out_features // world
        return rank * rows, rows, 0, w.in_features
    cols = w.in_features // world
    return 0, w.out_features, rank * cols, cols


def exchange_handles(group, mine: bytes, device: torch.device | None = None) -> list[bytes]:
    """Every rank's fixed-size handle, in rank order (one all-gather through the process group;
    ``device`` is where the group's backend wants its tensors: None = host memory). A rank that
    never arrives makes the collective raise after the group's timeout, on every other rank."""
    world = dist.get_world_size(group)
    t = torch.frombuffer(bytearray(mine), dtype=torch.uint8)
    if device is not None:
        t = t.to(device)
    got = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(got, t, group=group)
    return [bytes(h.cpu().numpy().tobytes()) for h in got]


class CudaBackend:
    """Compute through libaila_nf4.so on this rank's GPU."""

    def __init__(self, device: int):
        from .linear import Bnb4BitLinear, Bnb4BitLinearScratch
        self._L = Bnb4BitLinear
        self.device = device
        self.scratch = Bnb4BitLinearScratch(device)

    def make_shard(self, w: Nf4Tensors, mode: int, rank: int, world: int):
        lin = self._L()
        if not lin.init_shard(w, mode, rank, world, self.device):
            raise RuntimeError(lin.last_error)
        return lin

    def fuse(self, *handles):
        f = self._L()
        if not f.init_fused_rows(*handles):
            raise RuntimeError(f.last_error)
        return f

    def empty(self, *shape, dtype=torch.bfloat16):
        return torch.empty(*shape, dtype=dtype, device=torch.device("cuda", self.device))

    def forward(self, handle, x: torch.Tensor, out: torch.Tensor, seq_len: int) -> None:
        handle.forward(self.scratch, x, out, seq_len)

    def gate_up_swiglu(self, handle, x: torch.Tensor, out: torch.Tensor, seq_len: int,
                       ff: int) -> bool:
        return self._L.try_forward_decode_gate_up_swiglu(handle, self.scratch, x, out, ff,
                                                         seq_len=seq_len)

    # -- fused decode exchange over NVLink peer memory -----------------------------------
    def make_peer_buffer(self, group, max_rows: int):
        """Creates this rank's exchange buffer and maps every other rank's (CUDA IPC handles
        travel through the process group). Collective: every rank of ``group`` must call it."""
        from .linear import PeerBuffer
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        buf = PeerBuffer(self.device, rank, world, max_rows)
        handles = exchange_handles(group, buf.export_handle(), torch.device("cuda", self.device))
        for r, h in enumerate(handles):
            if r != rank:
                buf.import_handle(r, h)
        dist.barrier(group=group)
        return buf

    def make_dense(self, weight: torch.Tensor):
        from .linear import Linear
        lin = Linear()
        lin.init(weight.to(torch.bfloat16), weight.shape[1], weight.shape[0], self.device)
        return lin

    def dense_forward(self, handle, x: torch.Tensor, out: torch.Tensor, seq_len: int) -> None:
        handle.forward(self.scratch, x, out, seq_len)

    def argmax(self, logits: torch.Tensor, n: int, result: torch.Tensor, index_offset: int = 0) -> None:
        from .linear import argmax
        argmax(logits, n, result, index_offset)

    def make_chain(self, ops: list[dict], peers=None):
        from .linear import DecodeChain
        return DecodeChain(self.scratch, ops, peers)

    def forward_allreduce(self, handle, peers, x: torch.Tensor, out: torch.Tensor,
                          residual: torch.Tensor | None = None) -> None:
        handle.forward_decode_allreduce(self.scratch, peers, x, out, residual)


def _group_info(group):
    return dist.get_rank(group), dist.get_world_size(group)


class ColumnParallelNf4Linear:
    """y[:, rank's rows] = x W_r^T; optional all-gather of the row slices."""

    def __init__(self, w: Nf4Tensors, backend, group=None):
        self.rank, self.world = _group_info(group)
        self.group, self.backend = group, backend
        self.out_features, self.in_features = w.out_features, w.in_features
        self.local_out = w.out_features // self.world
        self.handle = backend.make_shard(w, ROWS, self.rank, self.world)

    def forward(self, x: torch.Tensor, gather: bool = False) -> torch.Tensor:
        m = x.shape[0]
        y = self.backend.empty(m, self.local_out)
        self.backend.forward(self.handle, x, y, m)
        if not gather:
            return y
        parts = [torch.empty_like(y) for _ in range(self.world)]
        dist.all_gather(parts, y, group=self.group)
        return torch.cat(parts, dim=1)


class RowParallelNf4Linear:
    """y = sum_r x[:, rank's columns] W_r^T with one all-reduce (fp32 for small M).

    With ``peers`` (a buffer from ``backend.make_peer_buffer``) a single-row input takes the
    fused route: the GEMV stores its fp32 row sums into every rank's exchange buffer and a small
    kernel adds them up, with no library collective."""

    def __init__(self, w: Nf4Tensors, backend, group=None, peers=None):
        self.rank, self.world = _group_info(group)
        self.group, self.backend = group, backend
        self.out_features, self.in_features = w.out_features, w.in_features
        self.local_in = w.in_features // self.world
        self.handle = backend.make_shard(w, COLS, self.rank, self.world)
        self.peers = peers

    def forward(self, x_local: torch.Tensor, fp32_reduce: bool | None = None) -> torch.Tensor:
        """x_local: this rank's column slice [M, in/world]."""
        m = x_local.shape[0]
        if m == 1 and self.peers is not None:
            y = self.backend.empty(1, self.out_features)
            self.backend.forward_allreduce(self.handle, self.peers, x_local, y)
            return y
        part = self.backend.empty(m, self.out_features)
        self.backend.forward(self.handle, x_local, part, m)
        return reduce_partials(part, self.group, m <= 64 if fp32_reduce is None else fp32_reduce)


def reduce_partials(part: torch.Tensor, group, fp32: bool) -> torch.Tensor:
    """Sum of the ranks' partial outputs. fp32 exchange for decode-sized messages (tens of KB,
    latency-bound either way), bf16 for prefill-sized ones (halves the NVLink bytes)."""
    if dist.get_world_size(group) == 1:
        return part
    if fp32:
        acc = part.float()
        dist.all_reduce(acc, group=group)
        return acc.to(torch.bfloat16)
    dist.all_reduce(part, group=group)
    return part


def reference_tie_key(index: torch.Tensor) -> torch.Tensor:
    """Order in which ops::argmax (src/ops/SamplingOps.cpp:321-358) prefers equal logits: its tree over
    256 work-items keeps the left candidate at every level, so the smallest bit-reversed
    (index % 256) wins, then the smallest index. Smaller key = preferred. int64 in, int64 out."""
    low = index & 255
    rev = torch.zeros_like(low)
    for bit in range(8):
        rev = rev | (((low >> bit) & 1) << (7 - bit))
    return (rev << 32) | index


class VocabParallelHead:
    """The bf16 output head with its vocabulary rows split over the ranks, and the greedy token
    choice on top (reference: lm_head_.forward + ops::argmax, src/models/Qwen3Bnb4Backend.cpp:432-439,
    src/ops/SamplingOps.cpp:321-365; sharding is net-new). Each rank runs the dense GEMV on its row
    slice and the argmax over its slice of the logits; the ranks exchange one (value, index) pair
    each instead of the logits, and every rank picks the same winner: the largest value and, among
    equal values, the index the reference's single reduction over the whole vocabulary would keep
    (``reference_tie_key``)."""

    def __init__(self, weight: torch.Tensor, backend, group=None):
        self.rank, self.world = _group_info(group)
        self.group, self.backend = group, backend
        self.vocab, self.hidden = weight.shape
        if self.vocab % self.world:
            raise ValueError(f"vocabulary {self.vocab} is not divisible by {self.world} shards")
        if self.vocab >= 1 << 24:
            raise ValueError("vocabulary too large for the packed (value, index) exchange")
        self.local = self.vocab // self.world
        self.handle = backend.make_dense(weight[self.rank * self.local:(self.rank + 1) * self.local].contiguous())
        self.logits = backend.empty(1, self.local)
        self._idx = backend.empty(1, dtype=torch.int32)

    def greedy(self, x: torch.Tensor) -> torch.Tensor:
        """x: [1, hidden] bf16 (replicated). Returns the chosen token as an int64 tensor of one
        element, the same on every rank."""
        self.backend.dense_forward(self.handle, x, self.logits, 1)
        self.backend.argmax(self.logits, self.local, self._idx, self.rank * self.local)
        idx = self._idx.to(torch.int64)
        val = self.logits.reshape(-1)[idx].float()
        if self.world == 1:
            return idx
        # (a token index below 2^24 is exact in fp32, so the pair travels as one tensor)
        pair = torch.stack([val.reshape(()), (idx.reshape(()) + self.rank * self.local).float()])
        got = [torch.empty_like(pair) for _ in range(self.world)]
        dist.all_gather(got, pair, group=self.group)
        allp = torch.stack(got)                      # [world, 2]: each rank's (value, global index)
        keys = reference_tie_key(allp[:, 1].to(torch.int64))
        keys = torch.where(allp[:, 0] == allp[:, 0].max(), keys, torch.full_like(keys, 1 << 62))
        return allp[torch.argmin(keys), 1].to(torch.int64).reshape(1)


class ShardedNf4Mlp:
    """SwiGLU MLP: gate|up row-sharded (SwiGLU local) -> down column-sharded -> one all-reduce."""

    def __init__(self, gate: Nf4Tensors, up: Nf4Tensors, down: Nf4Tensors, backend, group=None,
                 peers=None):
        self.rank, self.world = _group_info(group)
        self.peers = peers  # exchange buffer: single-row inputs skip the library all-reduce
        self.group, self.backend = group, backend
        if gate.out_features != up.out_features or gate.in_features != up.in_features:
            raise ValueError("gate and up must have the same shape")
        if down.in_features != gate.out_features or down.out_features != gate.in_features:
            raise ValueError("down must map ff back to hidden")
        check_shardable(gate, ROWS, self.world)
        check_shardable(down, COLS, self.world)
        self.hidden, self.ff = gate.in_features, gate.out_features
        self.local_ff = self.ff // self.world
        g = backend.make_shard(gate, ROWS, self.rank, self.world)
        u = backend.make_shard(up, ROWS, self.rank, self.world)
        self.gate_up = backend.fuse(g, u)  # gate_r rows then up_r rows: SwiGLU stays local
        self.down = backend.make_shard(down, COLS, self.rank, self.world)
        self._chains = {}

    def forward_chained(self, x: torch.Tensor) -> torch.Tensor:
        """Single-row input, exchange buffer given: gate|up + SwiGLU -> down -> sum over the ranks as
        ONE launch per rank (aila_nf4_chain_create_allreduce). The chain is built once per input
        tensor and writes into a buffer of its own, which is returned (overwritten by the next
        call with the same input tensor)."""
        if x.shape[0] != 1 or self.peers is None:
            raise ValueError("forward_chained takes one row and needs the exchange buffer")
        key = x.data_ptr()
        hit = self._chains.get(key)
        if hit is None:
            out = self.backend.empty(1, self.hidden)
            chain = self.backend.make_chain([dict(linear=self.gate_up, ff_dim=self.local_ff, x=x),
                                             dict(linear=self.down, y=out)], self.peers)
            hit = self._chains[key] = (chain, out, x)
        hit[0].run()
        return hit[1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = x.shape[0]
        mid = self.backend.empty(m, self.local_ff)
        if not self.backend.gate_up_swiglu(self.gate_up, x, mid, m, self.local_ff):
            raise RuntimeError("fused gate+up+SiLU path not applicable to this shard "
                               "(ff / world must be a multiple of 16)")
        part = self.backend.empty(m, self.hidden)
        if m == 1 and self.peers is not None:
            self.backend.forward_allreduce(self.down, self.peers, mid, part)
            return part
        self.backend.forward(self.down, mid, part, m)
        return reduce_partials(part, self.group, m <= 64)
