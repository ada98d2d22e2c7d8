#!/usr/bin/env python
"""Benchmark of the NF4 linear hot path on B200.

Headline workload: the fused gate+up+SiLU NF4 decode GEMV, M = 1, K = 2560, gate and up each
2560 -> 9728, blocksize 64 with double-quantised absmax. One STEP = one pass over LAYERS distinct
copies of that fused weight (LAYERS * 25.7 MB, far larger than the 126 MB L2, so every pass
streams from HBM), run as ONE chained launch (aila_nf4_chain_run) replayed from a CUDA graph.

  value        whole-job NF4 weight GB/s with inputs resident in HBM (all ranks' bytes / max time)
  roofline     algorithmic bytes of one operation / average time per operation inside the chained
               launch, against the measured HBM peak
  per_call     the same 36 operations as 36 separate C-ABI calls (one launch each)
  cfg1         36 plain 2560 -> 9728 linears, chained
  stack        the decode-step linear stack of a 36-layer GQA transformer (144 linears in one
               chained launch) plus the bf16 lm_head and argmax
  e2e          the headline metric through the host-buffer C-ABI call (H2D x, chain, D2H y, sync)
  prefill      the second half of the metric: the M = 2048 NF4 prefill GEMM pair in TFLOP/s
  tp           the sharded large-model linears (MLP, q, o) at M = 1 and M = 2048
  cpu_baseline / --impl reference: the CPU restatement of the reference kernels on host cores

Usage: python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
       python bench.py --profile-case chain|per_call|batch|batch32|dense|prefill   (small runs for ncu)
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, FF = 2560, 9728          # Qwen3-4B MLP shapes
LAYERS = 36
PREFILL_M = 2048
METRIC = "nf4_gemv_weight_bandwidth"
UNIT = "GB/s"
WORKLOAD = "cfg2 fused gate+up+SiLU NF4 GEMV, M=1, K=2560, 2x9728 rows, bs64 double-quant"

# ncu dram__bytes_read.sum + dram__bytes_write.sum per operation of the dominant kernel: one
# capture of a chained launch of 8 operations (python bench.py --profile-case chain), 208.04 MB
# read + 3.82 MB written, divided by 8. Traffic grows in proportion to the operations.
NCU_TRAFFIC_BYTES_PER_OP = 26_483_264


def weight_bytes(n: int, k: int) -> int:
    """nibbles + u8 absmax codes + fp32 second-level scales of one NF4 [n, k] weight."""
    blocks = n * k // 64
    return n * k // 2 + blocks + 4 * ((blocks + 255) // 256)


GATE_UP_WEIGHT_BYTES = 2 * weight_bytes(FF, H)                 # 25,694,080
GATE_UP_ALGO_BYTES = GATE_UP_WEIGHT_BYTES + 2 * H + 2 * FF     # + x + y = 25,718,656
CFG1_ALGO_BYTES = weight_bytes(FF, H) + 2 * H + 2 * FF         # 12,871,616


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tf=d["bf16_tflops"], tf_sus=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sus=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([s.strip() for s in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
                for n, v in zip(names, s[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU arm: the C restatement of the reference kernels (the reference's SYCL sources cannot be
# built in this image), all host cores
# ------------------------------------------------------------------------------------------
def _cpu_inputs():
    import numpy as np
    import torch

    from aila_b200 import synth
    from oracle import nf4_oracle as O
    O.build()
    O.set_num_threads(os.cpu_count() or 1)  # launchers such as torchrun pin OMP_NUM_THREADS=1
    g = synth.synth_linear(synth.seed_for(2, 0, "gate"), FF, H)
    u = synth.synth_linear(synth.seed_for(2, 0, "up"), FF, H)
    am = np.concatenate([O.expand_absmax(w.absmax_codes, w.nested_quant_map, w.nested_absmax,
                                         w.nested_blocksize, w.nested_offset) for w in (g, u)])
    packed = np.concatenate([g.packed, u.packed])
    x = synth.gaussian_activation(2009, H).view(torch.uint16).numpy()
    return O, g, packed, am, x


def cpu_baselines(min_seconds: float = 8.0, max_reps: int = 400):
    """cfg2 (the headline), cfg1 and a bounded sample of the prefill route on the host cores."""
    import numpy as np
    import torch
    O, g, packed, am, x = _cpu_inputs()

    def best_mean(fn, seconds):
        for _ in range(2):
            fn()
        reps, t0, best = 0, time.perf_counter(), 1e9
        while reps < max_reps and (time.perf_counter() - t0 < seconds or reps < 3):
            t1 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t1)
            reps += 1
        return (time.perf_counter() - t0) / reps, best, reps

    mean, best, reps = best_mean(lambda: O.gemv_gate_up_swiglu(packed, g.quant_map, am, x, FF, H, 64),
                                 min_seconds)
    out = dict(value=GATE_UP_WEIGHT_BYTES / mean / 1e9, unit=UNIT, cores=O.num_threads(), kind="port",
               best_ms=best * 1e3, mean_ms=mean * 1e3,
               build="gcc -O2 -march=x86-64-v3 -fopenmp -ffp-contract=off (oracle/Makefile)",
               sample=f"{reps} passes of one cfg2 fused gate+up+SiLU GEMV (2x[9728,2560] NF4), "
                      f"scalar C port of the reference SYCL kernel, OpenMP over rows")
    half = packed[: packed.size // 2]
    mean1, _, reps1 = best_mean(lambda: O.gemv(half, g.quant_map, am[: am.size // 2], x, FF, H, 64), 3.0)
    out["cfg1"] = dict(value=weight_bytes(FF, H) / mean1 / 1e9, unit=UNIT, mean_ms=mean1 * 1e3,
                       sample=f"{reps1} passes of one 2560->9728 GEMV")
    # the reference's M > 1 route at blocksize 64: dequantise to bf16 (its kernel, transcribed), then
    # a bf16 matmul with fp32 accumulation (torch CPU = oneDNN, the library family it calls)
    m_cpu = 256
    xs = torch.randn(m_cpu, H, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    t0 = time.perf_counter()
    w_nk = O.dequantize_nk(packed, g.quant_map, am, 2 * FF, H, 64)
    t_deq = time.perf_counter() - t0
    wt = torch.from_numpy(w_nk.view(np.int16).copy()).view(torch.bfloat16)
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    _ = xs @ wt.t()
    t_mm = time.perf_counter() - t0
    out["prefill_route"] = dict(value=2.0 * m_cpu * 2 * FF * H / (t_deq + t_mm) / 1e12, unit="TFLOP/s",
                                dequant_ms=t_deq * 1e3, matmul_ms=t_mm * 1e3,
                                sample=f"gate|up 2560->19456 at M={m_cpu} (1/8 of cfg3's rows): transcribed "
                                       f"dequantize_weight + torch CPU bf16 matmul, one pass")
    return out


def run_reference(args):
    """--impl reference: the reference's own algorithm on the host cores. Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    O, g, packed, am, x = _cpu_inputs()
    for _ in range(max(args.warmup, 1)):
        O.gemv_gate_up_swiglu(packed, g.quant_map, am, x, FF, H, 64)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.gemv_gate_up_swiglu(packed, g.quant_map, am, x, FF, H, 64)
    dt = (time.perf_counter() - t0) / args.steps
    val = GATE_UP_WEIGHT_BYTES / dt / 1e9
    sample = ("each step = ONE cfg2 fused gate+up+SiLU GEMV (1/36 of the GPU arm's step), "
              "scalar C port of the reference kernel, OpenMP over rows")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "50 MB working set on host caches; CPU arm"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
def _rolled(w, shift):
    """A copy of a quantised weight with its rows rotated: distinct memory, same value distribution."""
    import numpy as np
    if shift == 0:
        return w
    n, k = w.out_features, w.in_features
    return dataclasses.replace(
        w, packed=np.roll(np.asarray(w.packed).reshape(n, k // 2), shift, 0).reshape(-1),
        absmax_codes=np.roll(np.asarray(w.absmax_codes).reshape(n, k // 64), shift, 0).reshape(-1))


def _lin(w, local):
    from aila_b200.linear import Bnb4BitLinear
    l = Bnb4BitLinear()
    assert l.init(w, local), l.last_error
    return l


def _fuse(*ls):
    from aila_b200.linear import Bnb4BitLinear
    f = Bnb4BitLinear()
    assert f.init_fused_rows(*ls), f.last_error
    for l in ls:
        l.close()
    return f


def _graph(fn, stream):
    """fn captured in a CUDA graph (after one eager run); returns the replay callable."""
    import torch
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
    return g.replay


def _time_stream(fn, stream, reps, warm=3):
    import torch
    with torch.cuda.stream(stream):
        for _ in range(warm):
            fn()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            fn()
        b.record(stream)
        stream.synchronize()
    return a.elapsed_time(b) * 1e3 / reps  # us


def _max_rel_err(got_bits, want_bits):
    """max |got - want| / max |want| of two bf16 bit arrays."""
    import numpy as np

    def f32(a):
        return (np.ascontiguousarray(a, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    g, w = f32(got_bits), f32(want_bits)
    return float(np.abs(g - w).max() / max(np.abs(w).max(), 1e-30))


def _bits(t):
    import torch
    return t.detach().cpu().contiguous().view(torch.uint16).numpy()


# ------------------------------------------------------------------------------------------
def tp_linears(rank, world, local, stream):
    """The large-model linears (hidden 5120, intermediate 25600; q 5120->8192, o 8192->5120) sharded
    over `world` GPUs, at M = 1 and M = 2048. MLP: gate|up by rows with local SwiGLU, down by
    columns, one sum exchange. q by rows (column-parallel, no exchange), o by columns (row-parallel,
    one sum exchange). Strong scaling: total work fixed, ideal = t(1) / world. Every result is
    compared with the CPU oracle on the UNSHARDED weights (M = 2048: sampled rows)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from aila_b200 import sharded, synth
    from oracle import nf4_oracle as O
    O.build()
    O.set_num_threads(max(1, (os.cpu_count() or world) // world))
    H5, FF5, Q5 = 5120, 25600, 8192
    dev = torch.device("cuda", local)
    gate = synth.synth_linear(synth.seed_for(5, 0, "gate"), FF5, H5)
    up = synth.synth_linear(synth.seed_for(5, 0, "up"), FF5, H5)
    down = synth.synth_linear(synth.seed_for(5, 0, "down"), H5, FF5)
    wq = synth.synth_linear(synth.seed_for(5, 0, "q"), Q5, H5)
    wo = synth.synth_linear(synth.seed_for(5, 0, "o"), H5, Q5)
    be = sharded.CudaBackend(local)
    be.scratch.ensure(2048, FF5, 2 * FF5 // world, True)
    g_r, u_r = be.make_shard(gate, sharded.ROWS, rank, world), be.make_shard(up, sharded.ROWS, rank, world)
    gate_up, local_ff = be.fuse(g_r, u_r), FF5 // world
    dn = be.make_shard(down, sharded.COLS, rank, world)
    q_r = be.make_shard(wq, sharded.ROWS, rank, world)
    o_r = be.make_shard(wo, sharded.COLS, rank, world)
    local_q = Q5 // world

    def am(w):
        return O.expand_absmax(w.absmax_codes, w.nested_quant_map, w.nested_absmax, w.nested_blocksize,
                               w.nested_offset)

    out = {"workload": "cfg5 linears: MLP 5120 -> 2x25600 -> 5120 (gate|up row-sharded + local SwiGLU, down "
                       "column-sharded, one sum exchange), q 5120->8192 row-sharded, o 8192->5120 column-sharded",
           "world": world, "scaling": "strong",
           "fields": "M1_mlp_chained_us: gate|up -> down -> exchange as ONE launch per rank; "
                     "M1_mlp_fused_exchange_us: two launches, exchange folded into the second; "
                     "*_with_exchange_us: library all-reduce; *_with_reduce_scatter_us: library reduce-scatter, "
                     "result sharded by batch rows; *_efficiency = t(unsharded on one GPU) / (world x best sharded time)"}
    parity = 0.0

    def allmax(v):
        if world == 1:
            return float(v)
        t = torch.tensor([float(v)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    peers = be.make_peer_buffer(None, H5) if world > 1 else None
    peers_chain = be.make_peer_buffer(None, H5) if world > 1 else None
    # the unsharded linears on this GPU: t(1) of the strong-scaling efficiencies below
    if world > 1:
        gu_full = be.fuse(be.make_shard(gate, sharded.ROWS, 0, 1), be.make_shard(up, sharded.ROWS, 0, 1))
        dn_full = be.make_shard(down, sharded.COLS, 0, 1)
    for M, reps in ((1, 100), (2048, 10)):
        x = synth.gaussian_activation(5009 + M, M, H5).to(dev)
        xo = synth.gaussian_activation(5019 + M, M, Q5).to(dev)
        xo_local = xo[:, rank * local_q:(rank + 1) * local_q].contiguous()
        mid = be.empty(M, local_ff)
        part = be.empty(M, H5)
        yq = be.empty(M, local_q)
        yo = be.empty(M, H5)
        y_fused = be.empty(1, H5)

        def mlp_compute():
            assert be.gate_up_swiglu(gate_up, x, mid, M, local_ff)
            be.forward(dn, mid, part, M)

        def exchange(t):
            if world == 1:
                return
            if M <= 64:  # fp32 exchange for decode-sized messages
                acc = t.float()
                dist.all_reduce(acc)
                t.copy_(acc)
            else:
                dist.all_reduce(t)

        def mlp_full():
            mlp_compute()
            exchange(part)

        def mlp_fused():
            assert be.gate_up_swiglu(gate_up, x, mid, 1, local_ff)
            be.forward_allreduce(dn, peers, mid, y_fused)

        y_chain = be.empty(1, H5)
        chain = None
        if M == 1:
            try:  # gate|up -> down (-> exchange) as ONE launch per rank
                chain = be.make_chain([dict(linear=gate_up, ff_dim=local_ff, x=x), dict(linear=dn, y=y_chain)],
                                      peers_chain)
            except Exception as e:  # (unsharded, the 25600 input columns of down are beyond the chained kernel)
                out["M1_mlp_chained_note"] = f"not applicable at world {world}: {e}"

        rs_out = be.empty(max(1, M // world), H5)

        def mlp_reduce_scatter():  # the sum arrives sharded by rows of the batch: half the NVLink bytes
            mlp_compute()
            dist.reduce_scatter_tensor(rs_out, part)

        def q_proj():
            be.forward(q_r, x, yq, M)

        def o_compute():
            be.forward(o_r, xo_local, yo, M)

        def o_full():
            o_compute()
            exchange(yo)

        def timed(fn):
            try:
                run = _graph(fn, stream)
            except Exception:
                torch.cuda.synchronize()
                run = fn
            if world > 1:
                dist.barrier()
            return allmax(_time_stream(run, stream, reps))

        t_c, t_f = timed(mlp_compute), timed(mlp_full)
        out[f"M{M}_mlp_compute_us"], out[f"M{M}_mlp_with_exchange_us"] = t_c, t_f
        out[f"M{M}_mlp_collective_us"] = t_f - t_c
        out[f"M{M}_q_us"] = timed(q_proj)
        t_oc, t_of = timed(o_compute), timed(o_full)
        out[f"M{M}_o_compute_us"], out[f"M{M}_o_with_exchange_us"] = t_oc, t_of
        if M == 1 and world > 1:
            out["M1_mlp_fused_exchange_us"] = timed(mlp_fused)
        if chain is not None:
            out["M1_mlp_chained_us"] = timed(chain.run)
        if M > 1 and world > 1 and M % world == 0:
            out[f"M{M}_mlp_with_reduce_scatter_us"] = timed(mlp_reduce_scatter)
        if world > 1:
            mid_f, y_f = be.empty(M, FF5), be.empty(M, H5)

            def mlp_unsharded():
                assert be.gate_up_swiglu(gu_full, x, mid_f, M, FF5)
                be.forward(dn_full, mid_f, y_f, M)

            t1 = timed(mlp_unsharded)
            out[f"M{M}_mlp_unsharded_one_gpu_us"] = t1
            best = min(v for k, v in out.items() if k.startswith(f"M{M}_mlp_") and k.endswith("_us")
                       and "compute" not in k and "collective" not in k and "unsharded" not in k)
            out[f"M{M}_mlp_efficiency"] = t1 / (world * best)
            del mid_f, y_f
        # ---- parity against the oracle on the unsharded weights
        with torch.cuda.stream(stream):
            if M > 1 and world > 1 and M % world == 0:
                mlp_reduce_scatter()  # (before mlp_full: both leave their input in `part`)
            mlp_full()
            o_full()
            q_proj()
            if M == 1 and world > 1:
                mlp_fused()
            if chain is not None:
                chain.run()
            stream.synchronize()
        be.scratch.check()
        rows = [0] if M == 1 else [0, 1029, 2047]
        xs, xos = _bits(x)[rows], _bits(xo)[rows]
        gu_packed = np.concatenate([gate.packed, up.packed])
        gu_am = np.concatenate([am(gate), am(up)])
        if M == 1:
            mid_w = O.gemv_gate_up_swiglu(gu_packed, gate.quant_map, gu_am, xs[0], FF5, H5, 64)
            y_w = O.gemv(down.packed, down.quant_map, am(down), mid_w, H5, FF5, 64).reshape(1, -1)
            q_w = O.gemv(wq.packed, wq.quant_map, am(wq), xs[0], Q5, H5, 64).reshape(1, -1)
            o_w = O.gemv(wo.packed, wo.quant_map, am(wo), xos[0], H5, Q5, 64).reshape(1, -1)
        else:
            # the reference's M > 1 route on the sampled rows: bf16-rounded weights, bf16 GEMM
            n_r = len(rows)
            w_gu = O.dequantize_nk(gu_packed, gate.quant_map, gu_am, 2 * FF5, H5, 64)
            mid_w = O.swiglu_rows(O.gemm_bf16w(w_gu, xs, n_r, 2 * FF5, H5), n_r, FF5)
            del w_gu
            y_w = O.gemm_bf16w(O.dequantize_nk(down.packed, down.quant_map, am(down), H5, FF5, 64), mid_w,
                               n_r, H5, FF5)
            q_w = O.gemm_bf16w(O.dequantize_nk(wq.packed, wq.quant_map, am(wq), Q5, H5, 64), xs, n_r, Q5, H5)
            o_w = O.gemm_bf16w(O.dequantize_nk(wo.packed, wo.quant_map, am(wo), H5, Q5, 64), xos, n_r, H5, Q5)
        for i, r in enumerate(rows):
            parity = max(parity, _max_rel_err(_bits(part)[r], y_w[i]), _max_rel_err(_bits(yo)[r], o_w[i]),
                         _max_rel_err(_bits(yq)[r], q_w[i][rank * local_q:(rank + 1) * local_q]))
            if M == 1 and world > 1:
                parity = max(parity, _max_rel_err(_bits(y_fused)[0], y_w[i]))
            if chain is not None:
                parity = max(parity, _max_rel_err(_bits(y_chain)[0], y_w[i]))
            if M > 1 and world > 1 and M % world == 0:
                per = M // world
                if rank * per <= r < (rank + 1) * per:
                    parity = max(parity, _max_rel_err(_bits(rs_out)[r - rank * per], y_w[i]))
        if chain is not None:
            chain.close()
    out["parity_max_rel_err"] = allmax(parity)
    out["parity_bound"] = 2e-2
    if peers is not None:
        dist.barrier()
        peers.close()
        peers_chain.close()
    return out


def decode_stack(local, stream, batches=(4, 8, 16, 32)):
    """cfg4: the NF4 linears of one decode step of a 36-layer GQA transformer (hidden 2560, q 4096,
    k/v 1024, ff 9728): per layer fused qkv 2560->6144, o 4096->2560, fused gate|up+SiLU
    2560->2x9728, down 9728->2560; each linear gets its own N(0,1) input. 144 operations, 1.87 GB
    of weights per step: as one chained launch, as 144 separate calls, and followed by the bf16
    lm_head 2560->151936 (0.78 GB, dense GEMV) and the greedy argmax over its logits."""
    import torch

    from aila_b200 import synth
    from aila_b200.linear import Bnb4BitLinear, Bnb4BitLinearScratch, DecodeChain, Linear, argmax
    dev = torch.device("cuda", local)
    HID, Q, KV, F, VOCAB = 2560, 4096, 1024, 9728, 151936
    shapes = {"q": (Q, HID), "k": (KV, HID), "v": (KV, HID), "o": (HID, Q), "gate": (F, HID),
              "up": (F, HID), "down": (HID, F)}
    base = {k: synth.synth_linear(synth.seed_for(4, 0, k), *v) for k, v in shapes.items()}
    layers = []
    for i in range(36):
        w = {k: _rolled(v, 16 * i) for k, v in base.items()}
        layers.append((_fuse(_lin(w["q"], local), _lin(w["k"], local), _lin(w["v"], local)), _lin(w["o"], local),
                       _fuse(_lin(w["gate"], local), _lin(w["up"], local)), _lin(w["down"], local)))
    scratch = Bnb4BitLinearScratch(local)
    scratch.ensure(1, F, 2 * F, False)
    x_h = synth.gaussian_activation(4009, 1, HID).to(dev)
    x_q = synth.gaussian_activation(4019, 1, Q).to(dev)
    x_f = synth.gaussian_activation(4029, 1, F).to(dev)
    y_qkv = torch.empty(1, Q + 2 * KV, dtype=torch.bfloat16, device=dev)
    y_h = torch.empty(1, HID, dtype=torch.bfloat16, device=dev)
    y_f = torch.empty(1, F, dtype=torch.bfloat16, device=dev)
    ops = []
    for qkv, o, gu, dn in layers:
        ops += [dict(linear=qkv, x=x_h, y=y_qkv), dict(linear=o, x=x_q, y=y_h),
                dict(linear=gu, ff_dim=F, x=x_h, y=y_f), dict(linear=dn, x=x_f, y=y_h)]
    chain = DecodeChain(scratch, ops)

    def per_call():
        for qkv, o, gu, dn in layers:
            qkv.forward(scratch, x_h, y_qkv, 1)
            o.forward(scratch, x_q, y_h, 1)
            assert Bnb4BitLinear.try_forward_decode_gate_up_swiglu(gu, scratch, x_h, y_f, F)
            dn.forward(scratch, x_f, y_h, 1)

    us = _time_stream(_graph(chain.run, stream), stream, 20)
    us_calls = _time_stream(_graph(per_call, stream), stream, 10)
    scratch.check()
    # small batches (batched decode kernel: up to 32 rows per launch, one pass over the weights)
    batch = {}
    for M in batches:
        xb_h = synth.gaussian_activation(4100 + M, M, HID).to(dev)
        xb_q = synth.gaussian_activation(4200 + M, M, Q).to(dev)
        xb_f = synth.gaussian_activation(4300 + M, M, F).to(dev)
        yb_qkv = torch.empty(M, Q + 2 * KV, dtype=torch.bfloat16, device=dev)
        yb_h = torch.empty(M, HID, dtype=torch.bfloat16, device=dev)
        yb_f = torch.empty(M, F, dtype=torch.bfloat16, device=dev)

        def step_m():
            for qkv, o, gu, dn in layers:
                qkv.forward(scratch, xb_h, yb_qkv, M)
                o.forward(scratch, xb_q, yb_h, M)
                assert Bnb4BitLinear.try_forward_decode_gate_up_swiglu(gu, scratch, xb_h, yb_f, F, seq_len=M)
                dn.forward(scratch, xb_f, yb_h, M)

        batch[f"M{M}_us_per_step"] = _time_stream(_graph(step_m, stream), stream, 5)
    scratch.check()
    # the bf16 lm_head of the same model and the token choice; four distinct heads so that
    # consecutive timed launches do not find the weight in L2 (values drawn on the device)
    g = torch.Generator(device=dev).manual_seed(synth.seed_for(4, 0, "lm_head"))
    heads = []
    for _ in range(4):
        h = Linear()
        h.init((torch.randn(VOCAB, HID, generator=g, device=dev) * 0.02).to(torch.bfloat16), HID, VOCAB, local)
        heads.append(h)
    logits = torch.empty(1, VOCAB, dtype=torch.bfloat16, device=dev)
    token = torch.zeros(1, dtype=torch.int32, device=dev)

    def head_only():
        for h in heads:
            h.forward(scratch, x_h, logits, 1)

    def full_step():
        chain.run()
        heads[0].forward(scratch, y_h, logits, 1)
        argmax(logits, VOCAB, token)

    us_head = _time_stream(_graph(head_only, stream), stream, 10) / len(heads)
    us_full = _time_stream(_graph(full_step, stream), stream, 20)
    head_bytes = VOCAB * HID * 2
    wbytes = 36 * (weight_bytes(Q + 2 * KV, HID) + weight_bytes(HID, Q) + 2 * weight_bytes(F, HID) +
                   weight_bytes(HID, F))
    pk = peaks()
    # the whole decode step of the same model through the backend skeleton (embedding, per-head
    # norm + RoPE + cache append, attention, the linears, lm_head, argmax), host-driven, greedy
    from aila_b200.backend import Qwen3Bnb4Backend, Qwen3Config
    cfgm = Qwen3Config(hidden_size=HID, intermediate_size=F, num_hidden_layers=36, num_attention_heads=32,
                       num_key_value_heads=8, head_dim=128, vocab_size=VOCAB)
    ones = torch.ones(HID, dtype=torch.bfloat16)
    model = Qwen3Bnb4Backend(cfgm, local, max_seq_len=256)
    model.load((torch.randn(VOCAB, HID, generator=g, device=dev) * 0.02).to(torch.bfloat16),
               [dict(qkv=t[0], o=t[1], gate_up=t[2], down=t[3], input_ln=ones, post_attn_ln=ones,
                     q_norm=torch.ones(128, dtype=torch.bfloat16), k_norm=torch.ones(128, dtype=torch.bfloat16))
                for t in layers], ones, heads[0])
    n_prompt, n_gen = 16, 48
    with torch.cuda.stream(stream):
        model.forward(torch.arange(1, n_prompt + 1, dtype=torch.int32))
        tok = model.greedy_token()
        stream.synchronize()
        t0 = time.perf_counter()
        for _ in range(n_gen):
            model.forward(tok)
            tok = model.greedy_token()
        stream.synchronize()
        tok_s = n_gen / (time.perf_counter() - t0)
        model.generate(4)  # captures the step
        stream.synchronize()
        t0 = time.perf_counter()
        model.generate(n_gen)
        stream.synchronize()
        tok_s_graph = n_gen / (time.perf_counter() - t0)
    model.scratch.check()
    model.close()
    for t in layers:
        for l in t:
            l.close()
    return {"workload": "cfg4 NF4 linear stack, M=1: 36 x {qkv 2560->6144, o 4096->2560, "
                        "gate|up+SiLU 2560->2x9728, down 9728->2560}, one chained launch of 144 operations",
            "operations_per_step": 144, "launches_per_step": 1,
            "weight_bytes_per_step": wbytes, "us_per_step": us, "weight_GBps": wbytes / us / 1e3,
            "frac_of_measured_hbm": wbytes / us / 1e3 / pk["hbm"],
            "per_call": {"launches_per_step": 144, "us_per_step": us_calls,
                         "frac_of_measured_hbm": wbytes / us_calls / 1e3 / pk["hbm"]},
            "small_batch": batch,
            "backend_decode": {"what": "whole decode steps of the 36-layer model through "
                                       "aila_b200.backend.Qwen3Bnb4Backend (4 launches per layer, driven from "
                                       "Python, greedy), context 16..64, wall clock", "tokens_per_s": tok_s,
                               "tokens_per_s_graph": tok_s_graph,
                               "graph": "generate(): one captured step (position and token stay on the device) "
                                        "replayed per token, context 68..116"},
            "lm_head": {"workload": "bf16 dense GEMV 2560 -> 151936, 4 distinct weights in turn",
                        "us": us_head, "weight_GBps": head_bytes / us_head / 1e3,
                        "frac_of_measured_hbm": head_bytes / us_head / 1e3 / pk["hbm"]},
            "with_lm_head_and_argmax": {"launches_per_step": 3, "us_per_step": us_full,
                                        "weight_bytes_per_step": wbytes + head_bytes,
                                        "weight_GBps": (wbytes + head_bytes) / us_full / 1e3,
                                        "frac_of_measured_hbm": (wbytes + head_bytes) / us_full / 1e3 / pk["hbm"]}}


# ------------------------------------------------------------------------------------------
def profile_case(case: str):
    """Small, self-terminating runs of one kernel each, for capture under ncu (a few launches, well
    under a GB on the device except `dense`)."""
    import torch

    from aila_b200 import synth
    from aila_b200.linear import Bnb4BitLinear, Bnb4BitLinearScratch, DecodeChain, Linear
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    scratch = Bnb4BitLinearScratch(0)
    gate = synth.synth_linear(synth.seed_for(2, 0, "gate"), FF, H)
    up = synth.synth_linear(synth.seed_for(2, 0, "up"), FF, H)
    x = synth.gaussian_activation(2009, 1, H).to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if case in ("chain", "per_call", "batch", "batch32"):
        n = 8  # 8 x 25.7 MB = 206 MB of weights: larger than L2
        fused = [_fuse(_lin(_rolled(gate, 16 * i), 0), _lin(_rolled(up, 16 * i), 0)) for i in range(n)]
        M = {"batch": 8, "batch32": 32}.get(case, 1)
        xm = synth.gaussian_activation(2109, M, H).to(dev)
        outs = [torch.empty(M, FF, dtype=torch.bfloat16, device=dev) for _ in range(n)]
        chain = DecodeChain(scratch, [dict(linear=f, ff_dim=FF, x=x, y=o) for f, o in zip(fused, outs)]) \
            if case == "chain" else None
        for _ in range(3):
            flush.zero_()
            if chain is not None:
                chain.run()
            else:
                for f, o in zip(fused, outs):
                    assert Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, xm, o, FF, seq_len=M)
    elif case == "prefill":
        down = _lin(synth.synth_linear(synth.seed_for(3, 0, "down"), H, FF), 0)
        gu = _fuse(_lin(gate, 0), _lin(up, 0))
        scratch.ensure(PREFILL_M, FF, 2 * FF, True)
        xm = synth.gaussian_activation(3009, PREFILL_M, H).to(dev)
        mid = torch.empty(PREFILL_M, FF, dtype=torch.bfloat16, device=dev)
        ym = torch.empty(PREFILL_M, H, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            flush.zero_()
            assert Bnb4BitLinear.try_forward_decode_gate_up_swiglu(gu, scratch, xm, mid, FF, seq_len=PREFILL_M)
            down.forward(scratch, mid, ym, PREFILL_M)
    elif case == "dense":
        VOCAB = 151936
        g = torch.Generator(device=dev).manual_seed(7)
        head = Linear()
        head.init((torch.randn(VOCAB, H, generator=g, device=dev) * 0.02).to(torch.bfloat16), H, VOCAB, 0)
        logits = torch.empty(1, VOCAB, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            flush.zero_()
            head.forward(scratch, x, logits, 1)
    else:
        raise SystemExit(f"unknown profile case {case}")
    torch.cuda.synchronize()
    scratch.check()
    print(json.dumps({"profile_case": case, "status": "ok"}))


# ------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-tp", action="store_true", help="skip the sharded cfg5 linears")
    ap.add_argument("--no-stack", action="store_true", help="skip the cfg4 decode linear stack")
    ap.add_argument("--stack", action="store_true", help="time the cfg4 stack also when N > 1 (rank 0)")
    ap.add_argument("--profile-case", default=None)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.profile_case:
        return profile_case(args.profile_case)

    import numpy as np
    import torch
    import torch.distributed as dist

    from aila_b200 import synth
    from aila_b200.linear import Bnb4BitLinear, Bnb4BitLinearScratch, DecodeChain

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        torch.set_num_threads(max(1, (os.cpu_count() or world) // world))  # torchrun pins 1
    pk = peaks()
    layers = args.layers

    # ---- weights: one genuinely quantised gate/up pair; the other copies are row-rolled
    # versions of the same bytes (distinct memory, same value distribution).
    gate = synth.synth_linear(synth.seed_for(2, 0, "gate"), FF, H)
    up = synth.synth_linear(synth.seed_for(2, 0, "up"), FF, H)
    linears = [_fuse(_lin(_rolled(gate, 16 * i), local), _lin(_rolled(up, 16 * i), local)) for i in range(layers)]
    gates = [_lin(_rolled(gate, 16 * i + 8), local) for i in range(layers)]
    scratch = Bnb4BitLinearScratch(local)
    scratch.ensure(1, H, 2 * FF, False)
    x = synth.gaussian_activation(2009, 1, H).to(dev)
    outs = [torch.empty(1, FF, dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    stream = torch.cuda.Stream(dev)
    chain = DecodeChain(scratch, [dict(linear=f, ff_dim=FF, x=x, y=o) for f, o in zip(linears, outs)])
    replay = _graph(chain.run, stream)

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            replay()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        with ClockSampler(local) as clocks:
            ev[0].record(stream)
            for i in range(args.steps):
                replay()
                ev[i + 1].record(stream)
            stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    total_ms = ev[0].elapsed_time(ev[-1])
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    scratch.check()
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * layers * GATE_UP_WEIGHT_BYTES / (ms_per_step * 1e-3) / 1e9
    op_us = ms_per_step * 1e3 / layers
    achieved = GATE_UP_ALGO_BYTES / (op_us * 1e-6) / 1e9

    # ---- what was timed is right: layer 0 (and the last one) against the CPU oracle
    parity = None
    if rank == 0:
        O, g0, packed, am, xb = _cpu_inputs()
        want = O.gemv_gate_up_swiglu(packed, g0.quant_map, am, xb, FF, H, 64)
        parity = _max_rel_err(_bits(outs[0]).reshape(-1), want)
        assert parity <= 2e-2, f"timed output differs from the oracle: {parity}"

    # ---- the same operations as separate calls (one launch each), and cfg1 chained
    def per_call():
        for f, o in zip(linears, outs):
            assert Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x, o, FF)

    call_us = _time_stream(_graph(per_call, stream), stream, max(5, args.steps // 2)) / layers
    outs1 = [torch.empty(1, FF, dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    chain1 = DecodeChain(scratch, [dict(linear=f, x=x, y=o) for f, o in zip(gates, outs1)])
    cfg1_us = _time_stream(_graph(chain1.run, stream), stream, max(5, args.steps // 2)) / layers
    scratch.check()

    # ---- end to end through the host-buffer C-ABI calls
    xh = synth.gaussian_activation(2009, 1, H).pin_memory()
    yh = torch.empty(1, FF, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    with torch.cuda.stream(stream):
        for _ in range(2):
            chain.run_host(xh, yh)
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            chain.run_host(xh, yh)
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        assert torch.equal(yh.view(torch.uint16), outs[-1].cpu().view(torch.uint16))
        for f in linears[:2]:
            f.gate_up_swiglu_host(scratch, xh, yh, 1, FF)
        t0 = time.perf_counter()
        for _ in range(3):
            for f in linears:
                f.gate_up_swiglu_host(scratch, xh, yh, 1, FF)
        torch.cuda.synchronize()
        e2e_call_s = (time.perf_counter() - t0) / 3
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = world * layers * GATE_UP_WEIGHT_BYTES / e2e_s / 1e9
    chain.close()
    chain1.close()
    for f in gates:
        f.close()

    # ---- prefill GEMM pair (cfg3), rank 0 only
    prefill = None
    if not args.no_prefill and rank == 0:
        down_w = synth.synth_linear(synth.seed_for(3, 0, "down"), H, FF)
        down = _lin(down_w, local)
        gu = linears[0]
        scratch.ensure(PREFILL_M, FF, 2 * FF, True)
        xm = synth.gaussian_activation(3009, PREFILL_M, H).to(dev)
        mid = torch.empty(PREFILL_M, FF, dtype=torch.bfloat16, device=dev)
        ym = torch.empty(PREFILL_M, H, dtype=torch.bfloat16, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

        def pair():
            assert Bnb4BitLinear.try_forward_decode_gate_up_swiglu(gu, scratch, xm, mid, FF,
                                                                   seq_len=PREFILL_M)
            down.forward(scratch, mid, ym, PREFILL_M)

        with torch.cuda.stream(stream):
            for _ in range(3):
                pair()
            stream.synchronize()
            reps = 10
            tot = 0.0
            for _ in range(reps):
                flush.zero_()  # L2 flush between timed iterations
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                pair()
                b.record(stream)
                stream.synchronize()
                tot += a.elapsed_time(b)
        ms = tot / reps
        flops = 2.0 * PREFILL_M * (2 * FF) * H + 2.0 * PREFILL_M * H * FF
        tf = flops / (ms * 1e-3) / 1e12
        scratch.check()
        prefill = {"metric": "nf4_prefill_gemm_pair", "value": tf, "unit": "TFLOP/s",
                   "ms": ms, "workload": "cfg3: X[2048,2560] -> gate_up 2x9728 (+SwiGLU) -> down 2560; "
                                         "includes the NF4 -> bf16 dequantisation of both weights",
                   "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["tf"], "unit": "TFLOP/s",
                                "frac": tf / pk["tf"], "frac_of_sustained": tf / pk["tf_sus"] if pk["tf_sus"] else None,
                                "peak_source": pk["source"] + " burst"},
                   "l2": "256 MB flush between iterations"}
        down.close()
        del flush, xm, mid, ym
    for f in linears:
        f.close()
    linears = []
    torch.cuda.empty_cache()

    stack = None
    if rank == 0 and not args.no_stack and (world == 1 or args.stack):
        try:
            stack = decode_stack(local, stream)
        except Exception as e:  # keep the headline line even if an extra fails
            stack = {"error": repr(e)[:300]}
        torch.cuda.empty_cache()
    tp = None
    if not args.no_tp:
        try:
            tp = tp_linears(rank, world, local, stream)
        except Exception as e:
            tp = {"error": repr(e)[:300]}

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    cpu = None
    if not args.no_cpu and world == 1:
        cpu = cpu_baselines()

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x nf4 -> f32 accumulate",
        "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "layers_per_step": layers, "bytes_per_step": layers * GATE_UP_ALGO_BYTES,
                   "l2": f"inputs larger than L2: {layers} distinct weight copies = "
                         f"{layers * GATE_UP_WEIGHT_BYTES / 1e6:.0f} MB per step",
                   "launch": f"one chained launch of {layers} operations per step (aila_nf4_chain_run), "
                             "replayed from a CUDA graph", "parallelism": f"replicas x{world}"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                     "frac": achieved / pk["hbm"], "traffic": NCU_TRAFFIC_BYTES_PER_OP * layers,
                     "peak_source": pk["source"], "operation_us": op_us,
                     "algorithmic_bytes_per_launch": GATE_UP_ALGO_BYTES * layers,
                     "operations_per_launch": layers,
                     "algorithmic_bytes_per_operation": GATE_UP_ALGO_BYTES,
                     "traffic_per_operation": NCU_TRAFFIC_BYTES_PER_OP,
                     "frac_of_nominal_8TBps": achieved / 8000.0},
        "per_call": {"what": "the same operations as separate aila_nf4_forward_gate_up_swiglu calls "
                             "(one launch each, CUDA graph)", "launch_us": call_us,
                     "frac": GATE_UP_ALGO_BYTES / call_us / 1e3 / pk["hbm"]},
        "cfg1": {"workload": "cfg1 NF4 GEMV 2560 -> 9728, M=1: 36 distinct weights, one chained launch",
                 "operation_us": cfg1_us, "algorithmic_bytes_per_operation": CFG1_ALGO_BYTES,
                 "frac": CFG1_ALGO_BYTES / cfg1_us / 1e3 / pk["hbm"]},
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": 2 * H, "d2h_bytes_per_step": 2 * FF,
                "note": "aila_nf4_chain_run_host: pinned H2D copy of x, the chained launch, D2H copy of the "
                        "last operation's output, one stream sync",
                "per_call_value": layers * GATE_UP_WEIGHT_BYTES / e2e_call_s / 1e9,
                "per_call_note": "aila_nf4_forward_gate_up_swiglu_host per layer: H2D x, kernel storing y "
                                 "into the pinned host buffer, sync - 36 times per step"},
        "parity_max_rel_err_layer0": parity,
        "gpu_launches": args.steps,
        "clocks": clocks.summary(),
        "step_ms_min_max": [min(step_ms), max(step_ms)],
    }
    if cpu:
        line["cpu_baseline"] = cpu
    if prefill:
        line["prefill"] = prefill
    if tp:
        line["tp"] = tp
    if stack:
        line["stack"] = stack
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
