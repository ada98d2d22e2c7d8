"""Multi-GPU layer on real GPUs: one process per GPU, NCCL. Skipped with fewer than 2 GPUs.

Checks the Megatron-style MLP (gate|up row-sharded with local SwiGLU -> down column-sharded ->
one all-reduce) against the unsharded CPU oracle at decode (M = 1) and prefill (M = 256) sizes.
"""
import os
import socket

import numpy as np
import pytest
import torch

from aila_b200 import synth
from tests.helpers import bits_to_f32, make_weight, oracle_absmax

pytestmark = pytest.mark.gpu

H, FF = 1024, 2048


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from aila_b200 import sharded
        be = sharded.CudaBackend(rank)
        gate, up, down = make_weight(1, FF, H), make_weight(2, FF, H), make_weight(3, H, FF)
        mlp = sharded.ShardedNf4Mlp(gate, up, down, be)
        outs = {}
        for M in (1, 256):
            x = synth.gaussian_activation(10 + M, M, H).cuda()
            y = mlp.forward(x)
            torch.cuda.synchronize()
            outs[M] = y.cpu().view(torch.uint16).numpy()
        # fused exchange: the down projection stores its row sums into every rank's buffer over
        # NVLink and a small kernel adds them up - several eager calls (the exchange alternates
        # between two buffer halves), then the same calls replayed from a CUDA graph
        peers = be.make_peer_buffer(None, H)
        fused = sharded.ShardedNf4Mlp(gate, up, down, be, peers=peers)
        x1 = synth.gaussian_activation(11, 1, H).cuda()
        ys = [fused.forward(x1) for _ in range(5)]
        torch.cuda.synchronize()
        be.scratch.check()
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                yg = fused.forward(x1)
                yg2 = fused.forward(yg[:, :H].contiguous())
            for _ in range(3):
                g.replay()
            st.synchronize()
        be.scratch.check()
        y_chain = fused.forward(fused.forward(x1)[:, :H].contiguous())
        torch.cuda.synchronize()
        be.scratch.check()
        same = all(torch.equal(ys[0], t) for t in ys[1:]) and torch.equal(ys[0], yg) \
            and torch.equal(y_chain, yg2)
        mine = ys[0].clone()
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        same = same and all(torch.equal(mine, t) for t in everyone)
        # the same MLP as ONE launch per rank (gate|up -> down -> exchange inside the chained kernel)
        yc = [fused.forward_chained(x1).clone() for _ in range(4)]
        torch.cuda.synchronize()
        be.scratch.check()
        same = same and all(torch.equal(yc[0], t) for t in yc[1:])
        dist.all_gather(everyone, yc[0])
        same = same and all(torch.equal(yc[0], t) for t in everyone)
        chained_err = float((yc[0].float() - ys[0].float()).abs().max() / ys[0].float().abs().max())
        same = same and chained_err < 1e-2
        outs["chained"] = yc[0].cpu().view(torch.uint16).numpy()
        # a tall, narrow row-parallel linear: its grid exceeds the SM count, so the exchange takes
        # the two-kernel form (publish, then a reducer kernel) instead of the single launch
        tall = make_weight(4, 20000, 128 * world)
        rp = sharded.RowParallelNf4Linear(tall, be, peers=None)
        peers_tall = be.make_peer_buffer(None, 20000)
        rp_fused = sharded.RowParallelNf4Linear(tall, be, peers=peers_tall)
        xt = synth.gaussian_activation(12, 1, 128 * world).cuda()
        xt_local = xt[:, rank * 128:(rank + 1) * 128].contiguous()
        yt_ref = rp.forward(xt_local)
        yt = [rp_fused.forward(xt_local) for _ in range(3)]
        torch.cuda.synchronize()
        be.scratch.check()
        tall_err = float((yt[0].float() - yt_ref.float()).abs().max() / yt_ref.float().abs().max())
        same = same and all(torch.equal(yt[0], t) for t in yt[1:]) and tall_err < 1e-2
        peers_tall.close()
        # the output head with its vocabulary split over the ranks: the exchanged (value, index)
        # pairs must pick the token that the whole head picks on one GPU
        gen = torch.Generator().manual_seed(31)
        wh = (torch.randn(4096, H, generator=gen) * 0.05).to(torch.bfloat16)
        xh = synth.gaussian_activation(32, 1, H).cuda()
        head = sharded.VocabParallelHead(wh, be)
        tok = int(head.greedy(xh)[0])
        whole = be.make_dense(wh)
        full_logits = be.empty(1, 4096)
        be.dense_forward(whole, xh, full_logits, 1)
        whole_tok = be.empty(1, dtype=torch.int32)
        be.argmax(full_logits, 4096, whole_tok)
        same = same and tok == int(whole_tok.cpu()[0])
        outs["fused"] = ys[0].cpu().view(torch.uint16).numpy()
        outs["fused_consistent"] = bool(same)
        peers.close()
        if rank == 0:
            q.put(("ok", outs))
        dist.barrier()
    except Exception as e:  # pragma: no cover
        if rank == 0:
            q.put(("err", repr(e)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_mlp_nccl(oracle, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
    assert res[0] == "ok", res
    gate, up, down = make_weight(1, FF, H), make_weight(2, FF, H), make_weight(3, H, FF)
    packed = np.concatenate([gate.packed, up.packed])
    am = np.concatenate([oracle_absmax(oracle, gate), oracle_absmax(oracle, up)])
    assert res[1].pop("fused_consistent"), "fused exchange: results differ between calls or ranks"
    fused_bits = res[1].pop("fused")
    chained_bits = res[1].pop("chained")
    for M, got in res[1].items():
        x = synth.gaussian_activation(10 + M, M, H).view(torch.uint16).numpy()
        if M == 1:
            mid = oracle.gemv_gate_up_swiglu(packed, gate.quant_map, am, x.reshape(-1), FF, H, 64).reshape(1, FF)
        else:
            mid = oracle.swiglu_rows(oracle.forward(packed, gate.quant_map, am, x, M, 2 * FF, H, 64), M, FF)
        want = bits_to_f32(oracle.forward(down.packed, down.quant_map, oracle_absmax(oracle, down),
                                          mid, M, H, FF, 64))
        err = np.abs(bits_to_f32(got) - want).max()
        assert err <= 2e-2 * np.abs(want).max(), (M, err)
        if M == 1:
            err = np.abs(bits_to_f32(fused_bits) - want).max()
            assert err <= 2e-2 * np.abs(want).max(), ("fused", err)
            err = np.abs(bits_to_f32(chained_bits) - want).max()
            assert err <= 2e-2 * np.abs(want).max(), ("chained", err)
            # (not bit-equal to the library route, which rounds every rank's partial sum to bf16
            # before the all-reduce; the fused route adds the fp32 partial sums and rounds once)


def _skip_worker(rank, world, port, q):
    """Step 1: both ranks call. Step 2: rank 1 leaves the call out (between steps, nothing of it in
    flight); rank 0's wait runs out after a few milliseconds and the launch reports it. Step 3:
    fresh exchange buffers, both ranks call, the numbers are those of step 1."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from aila_b200 import _lib, sharded
        be = sharded.CudaBackend(rank)
        w = make_weight(21, 512, 256 * world)
        x = synth.gaussian_activation(22, 1, 256 * world).cuda()
        xl = x[:, rank * 256:(rank + 1) * 256].contiguous()
        peers = be.make_peer_buffer(None, 512)
        rp = sharded.RowParallelNf4Linear(w, be, peers=peers)
        y1 = rp.forward(xl).clone()
        torch.cuda.synchronize()
        be.scratch.check()
        dist.barrier()
        torch.cuda.synchronize()
        status = None
        if rank == 0:
            be.scratch.set_wait_limit(20_000_000)  # about 10 ms
            rp.forward(xl)
            torch.cuda.synchronize()
            try:
                be.scratch.check()
            except _lib.Nf4Error as e:
                status = e.status
            be.scratch.set_wait_limit(2_000_000_000)
        dist.barrier()  # rank 1 learns on the host that the step is over
        torch.cuda.synchronize()
        peers.close()
        peers = be.make_peer_buffer(None, 512)
        rp = sharded.RowParallelNf4Linear(w, be, peers=peers)
        y3 = rp.forward(xl)
        torch.cuda.synchronize()
        be.scratch.check()
        same = torch.equal(y1, y3)
        peers.close()
        if rank == 0:
            q.put(("ok", status, bool(same)))
        dist.barrier()
    except Exception as e:  # pragma: no cover
        if rank == 0:
            q.put(("err", repr(e)))
        raise
    finally:
        dist.destroy_process_group()


def test_rank_that_skips_a_call_times_the_other_out():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from aila_b200 import _lib
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_skip_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
    assert res[0] == "ok", res
    assert res[1] == _lib.ERR_KERNEL_TIMEOUT, res
    assert res[2], "after new exchange buffers the result must be that of the first step"
