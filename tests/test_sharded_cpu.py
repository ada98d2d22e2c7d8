"""Host logic of the multi-GPU layer on CPU: two gloo ranks, compute supplied by an
oracle-backed stand-in for the CUDA library (tests only). Checks the slicing rules, the
Megatron-style MLP chain and the collectives against the unsharded oracle result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aila_b200 import sharded, synth
from tests.helpers import bits_to_f32, make_weight, oracle_absmax


class OracleBackend:
    """Implements the backend interface of aila_b200.sharded with the CPU oracle. A handle is
    (packed, absmax_f32, quant_map, N, K) of the kept slice; slicing the EXPANDED absmax of the
    whole weight mirrors what the library's shards must reproduce."""

    def __init__(self):
        from oracle import nf4_oracle
        self.O = nf4_oracle

    def make_shard(self, w, mode, rank, world):
        r0, rows, c0, cols = sharded.shard_bounds(w, mode, rank, world)
        am = oracle_absmax(self.O, w).reshape(w.out_features, w.in_features // w.blocksize)
        packed = np.asarray(w.packed).reshape(w.out_features, w.in_features // 2)
        return (packed[r0:r0 + rows, c0 // 2:(c0 + cols) // 2].copy().reshape(-1),
                am[r0:r0 + rows, c0 // w.blocksize:(c0 + cols) // w.blocksize].copy().reshape(-1),
                w.quant_map, rows, cols, w.blocksize)

    def fuse(self, *hs):
        return (np.concatenate([h[0] for h in hs]), np.concatenate([h[1] for h in hs]), hs[0][2],
                sum(h[3] for h in hs), hs[0][4], hs[0][5])

    def empty(self, *shape, dtype=torch.bfloat16):
        return torch.empty(*shape, dtype=dtype)

    def forward(self, h, x, out, seq_len):
        packed, am, qmap, N, K, bs = h
        xb = x.contiguous().view(torch.uint16).numpy()
        y = self.O.forward(packed, qmap, am, xb, seq_len, N, K, bs)
        out.copy_(torch.from_numpy(y.reshape(seq_len, N)).view(torch.bfloat16))

    def gate_up_swiglu(self, h, x, out, seq_len, ff):
        packed, am, qmap, N, K, bs = h
        if N != 2 * ff or ff % 16:
            return False
        xb = x.contiguous().view(torch.uint16).numpy()
        if seq_len == 1:
            y = self.O.gemv_gate_up_swiglu(packed, qmap, am, xb.reshape(-1), ff, K, bs).reshape(1, ff)
        else:
            y = self.O.swiglu_rows(self.O.forward(packed, qmap, am, xb, seq_len, N, K, bs), seq_len, ff)
        out.copy_(torch.from_numpy(y).view(torch.bfloat16))
        return True


    def make_dense(self, weight):
        return weight.contiguous()

    def dense_forward(self, h, x, out, seq_len):
        y = self.O.gemm_bf16w(h.view(torch.uint16).numpy(), x.contiguous().view(torch.uint16).numpy(), seq_len,
                              h.shape[0], h.shape[1])
        out.copy_(torch.from_numpy(y.reshape(seq_len, h.shape[0])).view(torch.bfloat16))

    def argmax(self, logits, n, result, index_offset=0):
        from oracle import backend_numpy
        bits = logits.reshape(-1)[:n].contiguous().view(torch.uint16).numpy()
        result.copy_(torch.tensor([backend_numpy.argmax(bits, index_offset)], dtype=torch.int32))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from oracle import nf4_oracle as O
        O.set_num_threads(2)
        H, FF = 256, 512
        gate, up, down = make_weight(1, FF, H), make_weight(2, FF, H), make_weight(3, H, FF)
        be = OracleBackend()
        x = synth.gaussian_activation(4, M, H)
        mlp = sharded.ShardedNf4Mlp(gate, up, down, be)
        y = mlp.forward(x)
        # column-parallel with gather and row-parallel on their own
        col = sharded.ColumnParallelNf4Linear(gate, be)
        g_full = col.forward(x, gather=True)
        row = sharded.RowParallelNf4Linear(down, be)
        mid = synth.gaussian_activation(5, M, FF)
        cols = FF // world
        y_row = row.forward(mid[:, rank * cols:(rank + 1) * cols].contiguous())
        if rank == 0:
            q.put(("ok", y.view(torch.uint16).numpy(), g_full.view(torch.uint16).numpy(),
                   y_row.view(torch.uint16).numpy()))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover - surfaced in the parent
        if rank == 0:
            q.put(("err", repr(e)))
        raise


@pytest.mark.parametrize("M", [1, 3])
def test_sharded_mlp_two_gloo_ranks(oracle, M):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
    assert res[0] == "ok", res
    _, y, g_full, y_row = res
    # unsharded oracle
    H, FF = 256, 512
    gate, up, down = make_weight(1, FF, H), make_weight(2, FF, H), make_weight(3, H, FF)
    x = synth.gaussian_activation(4, M, H).view(torch.uint16).numpy()
    packed = np.concatenate([gate.packed, up.packed])
    am = np.concatenate([oracle_absmax(oracle, gate), oracle_absmax(oracle, up)])
    if M == 1:
        mid = oracle.gemv_gate_up_swiglu(packed, gate.quant_map, am, x.reshape(-1), FF, H, 64).reshape(1, FF)
    else:
        mid = oracle.swiglu_rows(oracle.forward(packed, gate.quant_map, am, x, M, 2 * FF, H, 64), M, FF)
    want = bits_to_f32(oracle.forward(down.packed, down.quant_map, oracle_absmax(oracle, down), mid,
                                      M, H, FF, 64))
    got = bits_to_f32(y)
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    want_g = oracle.forward(gate.packed, gate.quant_map, oracle_absmax(oracle, gate), x, M, FF, H, 64)
    assert np.array_equal(g_full, want_g)  # row shards are independent: exact
    mid5 = synth.gaussian_activation(5, M, FF).view(torch.uint16).numpy()
    want_r = bits_to_f32(oracle.forward(down.packed, down.quant_map, oracle_absmax(oracle, down),
                                        mid5, M, H, FF, 64))
    assert np.abs(bits_to_f32(y_row) - want_r).max() <= 2e-2 * np.abs(want_r).max()


def test_shard_rules():
    w = make_weight(9, 96, 256)
    assert sharded.shard_bounds(w, sharded.ROWS, 1, 2) == (48, 48, 0, 256)
    assert sharded.shard_bounds(w, sharded.COLS, 3, 4) == (0, 96, 192, 64)
    with pytest.raises(ValueError):
        sharded.shard_bounds(w, sharded.COLS, 0, 8)   # 32 columns < blocksize
    with pytest.raises(ValueError):
        sharded.shard_bounds(w, sharded.ROWS, 0, 5)
    with pytest.raises(ValueError):
        sharded.shard_bounds(w, sharded.ROWS, 2, 2)


def _handle_worker(rank, world, port, absent, q):
    """Rank `absent` (if any) leaves before the exchange, as a rank that died during set-up."""
    import datetime
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
        if rank == absent:
            q.put((rank, "left"))
            return  # never joins the collective (no destroy: the others must not be helped out)
        mine = bytes([rank]) * 64
        try:
            got = sharded.exchange_handles(None, mine)
            q.put((rank, "ok", got))
        except Exception as e:
            q.put((rank, "raised", type(e).__name__))
    except Exception as e:  # pragma: no cover
        q.put((rank, "err", repr(e)))


@pytest.mark.parametrize("absent", [None, 1])
def test_handle_exchange_and_a_rank_that_never_arrives(absent):
    """The host side of make_peer_buffer: every rank gets every rank's 64-byte handle in rank
    order; when one rank never arrives, the others get an exception after the group's timeout
    instead of waiting for ever."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_handle_worker, args=(r, world, port, absent, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        item = q.get(timeout=120)
        res[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():  # pragma: no cover
            p.terminate()
    if absent is None:
        for r in range(world):
            assert res[r][0] == "ok", res
            assert res[r][1] == [bytes([i]) * 64 for i in range(world)]
    else:
        assert res[absent][0] == "left"
        assert res[0][0] == "raised", res


def test_mis_sized_shards_are_refused_on_the_host():
    w = make_weight(10, 100, 192)
    with pytest.raises(ValueError):
        sharded.check_shardable(w, sharded.ROWS, 3)   # 100 rows over 3 ranks
    with pytest.raises(ValueError):
        sharded.check_shardable(w, sharded.COLS, 2)   # 96 columns per rank: not a multiple of 64
    with pytest.raises(ValueError):
        sharded.shard_bounds(w, sharded.ROWS, 2, 2)   # rank outside the group
    be = OracleBackend()
    with pytest.raises(ValueError):
        be.make_shard(w, sharded.COLS, 0, 2)


def _head_worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        g = torch.Generator().manual_seed(77)
        w = (torch.randn(512, 128, generator=g) * 0.05).to(torch.bfloat16)
        w[300] = w[40]                      # two equal rows in different shards: the smaller index must win
        x = synth.gaussian_activation(78, 1, 128)
        head = sharded.VocabParallelHead(w, OracleBackend())
        toks = [int(head.greedy(x)[0])]
        x2 = (w[40].float() * 8).to(torch.bfloat16).reshape(1, -1)   # aligned with rows 40 and 300
        toks.append(int(head.greedy(x2)[0]))
        if rank == 0:
            q.put(("ok", toks))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        if rank == 0:
            q.put(("err", repr(e)))
        raise


def test_vocab_parallel_head_two_gloo_ranks(oracle):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_head_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
    assert res[0] == "ok", res
    g = torch.Generator().manual_seed(77)
    w = (torch.randn(512, 128, generator=g) * 0.05).to(torch.bfloat16)
    w[300] = w[40]
    x = synth.gaussian_activation(78, 1, 128)
    x2 = (w[40].float() * 8).to(torch.bfloat16).reshape(1, -1)
    for xi, tok in zip((x, x2), res[1]):
        from oracle import backend_numpy
        logits = oracle.gemm_bf16w(w.view(torch.uint16).numpy(), xi.view(torch.uint16).numpy(), 1, 512, 128)
        assert tok == backend_numpy.argmax(logits)   # ties as the reference's single reduction resolves them
    assert res[1][1] == 40
    with pytest.raises(ValueError):
        sharded.check_shardable(make_weight(1, 96, 64), sharded.ROWS, 5)
