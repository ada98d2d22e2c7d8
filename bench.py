#!/usr/bin/env python
"""Benchmark of the NF4 linear hot path on B200.

Headline workload (BASELINE.json configs[1]): the fused gate+up+SiLU NF4 decode GEMV,
M = 1, K = 2560, gate and up each 2560 -> 9728, blocksize 64 with double-quantised absmax.
One STEP = one pass over LAYERS distinct copies of that fused weight (LAYERS * 25.7 MB, far
larger than the 126 MB L2, so every pass streams from HBM), replayed from a CUDA graph.

  value     whole-job NF4 weight GB/s with inputs resident in HBM (all ranks' bytes / max time)
  roofline  algorithmic bytes of one launch / average launch time, against the measured HBM peak
  e2e       the same metric through the host-buffer C-ABI call (H2D x, kernel, D2H y per call)
  prefill   the second half of BASELINE.json's metric: cfg3 NF4 prefill GEMM pair in TFLOP/s
  cpu_baseline / --impl reference: the CPU restatement of the reference kernels on host cores

Usage: python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, FF = 2560, 9728          # cfg2 / cfg3 shapes (Qwen3-4B MLP)
LAYERS = 36
PREFILL_M = 2048
METRIC = "nf4_gemv_weight_bandwidth"
UNIT = "GB/s"

# ncu dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the
# capture summarised under profiles/ (None until a capture exists for the current kernel).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 25750528  # profiles/gemv_stream_cfg2_ncu.md


def weight_bytes(n: int, k: int) -> int:
    """nibbles + u8 absmax codes + fp32 second-level scales of one NF4 [n, k] weight."""
    blocks = n * k // 64
    return n * k // 2 + blocks + 4 * ((blocks + 255) // 256)


GATE_UP_WEIGHT_BYTES = 2 * weight_bytes(FF, H)                 # 25,694,080
GATE_UP_ALGO_BYTES = GATE_UP_WEIGHT_BYTES + 2 * H + 2 * FF     # + x + y = 25,718,656


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
def cpu_gate_up_baseline(min_seconds: float = 10.0, max_reps: int = 400):
    """Times the CPU restatement of the reference's fused gate+up+SiLU GEMV on all host cores."""
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
    for _ in range(3):
        O.gemv_gate_up_swiglu(packed, g.quant_map, am, x, FF, H, 64)
    reps, t0, best = 0, time.perf_counter(), 1e9
    while reps < max_reps and (time.perf_counter() - t0 < min_seconds or reps < 5):
        t1 = time.perf_counter()
        O.gemv_gate_up_swiglu(packed, g.quant_map, am, x, FF, H, 64)
        best = min(best, time.perf_counter() - t1)
        reps += 1
    mean = (time.perf_counter() - t0) / reps
    return dict(value=GATE_UP_WEIGHT_BYTES / mean / 1e9, unit=UNIT, cores=O.num_threads(),
                kind="port", best_ms=best * 1e3, mean_ms=mean * 1e3,
                sample=f"{reps} passes of one cfg2 fused gate+up+SiLU GEMV (2x[9728,2560] NF4), "
                       f"scalar C port of the reference SYCL kernel, OpenMP over rows")


def run_reference(args):
    """--impl reference: the reference's own algorithm on the host cores (CPU port; the SYCL
    sources cannot be built in this image). Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
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
        "config": {"workload": "cfg2 fused gate+up+SiLU NF4 GEMV, M=1, K=2560, 2x9728 rows, bs64 double-quant",
                   "l2": "50 MB working set on host caches; CPU arm"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)



# ------------------------------------------------------------------------------------------
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


def tp_mlp_latency(rank, world, local, stream):
    """cfg5 MLP (hidden 5120, intermediate 25600) sharded over `world` GPUs: gate|up by rows with
    local SwiGLU, down by columns, one all-reduce. Per-layer latency at M = 1 and M = 2048, with
    and without the collective. Strong scaling: total work fixed, ideal = t(1)/world."""
    import torch
    import torch.distributed as dist

    from aila_b200 import sharded, synth
    H5, FF5 = 5120, 25600
    gate = synth.synth_linear(synth.seed_for(5, 0, "gate"), FF5, H5)
    up = synth.synth_linear(synth.seed_for(5, 0, "up"), FF5, H5)
    down = synth.synth_linear(synth.seed_for(5, 0, "down"), H5, FF5)
    be = sharded.CudaBackend(local)
    be.scratch.ensure(2048, FF5, 2 * FF5 // world, True)
    if world > 1:
        mlp = sharded.ShardedNf4Mlp(gate, up, down, be)
        gate_up, dn, local_ff = mlp.gate_up, mlp.down, mlp.local_ff
    else:
        g, u = be.make_shard(gate, 0, 0, 1), be.make_shard(up, 0, 0, 1)
        gate_up, dn, local_ff = be.fuse(g, u), be.make_shard(down, 1, 0, 1), FF5
    out = {"workload": "cfg5 MLP 5120 -> 2x25600 -> 5120, NF4; gate|up row-sharded + local SwiGLU, "
                       "down column-sharded, one all-reduce", "world": world, "scaling": "strong"}
    for M, reps in ((1, 200), (2048, 10)):
        x = synth.gaussian_activation(5009 + M, M, H5).to(torch.device("cuda", local))
        mid = be.empty(M, local_ff)
        part = be.empty(M, H5)

        def compute():
            assert be.gate_up_swiglu(gate_up, x, mid, M, local_ff)
            be.forward(dn, mid, part, M)

        acc32 = torch.empty(M, H5, dtype=torch.float32, device=part.device) if M <= 64 else None

        def full():
            compute()
            if acc32 is not None:  # fp32 exchange for decode-sized messages
                acc32.copy_(part)
                dist.all_reduce(acc32)
                part.copy_(acc32)
            else:
                dist.all_reduce(part)

        def graphed(fn):
            """Replays fn from a CUDA graph when capture works (NCCL included), else eager."""
            try:
                with torch.cuda.stream(stream):
                    fn()
                    stream.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        fn()
                return g.replay, "cuda graph"
            except Exception:
                torch.cuda.synchronize()
                return fn, "eager"

        if world > 1:
            dist.barrier()
        run_c, how_c = graphed(compute)
        t_c = _time_stream(run_c, stream, reps)
        if world > 1:
            dist.barrier()
            run_f, how_f = graphed(full)
            dist.barrier()
            t_f = _time_stream(run_f, stream, reps)
            out[f"M{M}_launch"] = f"compute: {how_c}; with all-reduce: {how_f}"
        else:
            t_f = t_c
            out[f"M{M}_launch"] = how_c
        if world > 1:
            t = torch.tensor([t_c, t_f], device=torch.device("cuda", local))
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_c, t_f = float(t[0]), float(t[1])
        out[f"M{M}_compute_us"] = t_c
        out[f"M{M}_with_allreduce_us"] = t_f
        if world > 1 and M == 1 and os.environ.get("AILA_BENCH_FUSED_TP", "1") != "0":
            # the exchange folded into the down GEMV: fp32 row sums stored into every rank's
            # buffer over NVLink, summed by a small kernel (no library collective). A failure on
            # any rank is reported instead of the number; the collectives below stay matched.
            t_x, how_x, err = 0.0, "", ""
            peers = None
            dev_t = torch.device("cuda", local)
            y1 = be.empty(1, H5)

            def fused():
                assert be.gate_up_swiglu(gate_up, x, mid, 1, local_ff)
                be.forward_allreduce(dn, peers, mid, y1)

            try:  # set-up and one checked call; every rank must get through it before any timing
                peers = be.make_peer_buffer(None, H5)
                with torch.cuda.stream(stream):
                    fused()
                    stream.synchronize()
                be.scratch.check()
            except Exception as e:  # noqa: BLE001
                err = repr(e)[:200]
            ok = torch.tensor([0.0 if err else 1.0], device=dev_t)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok[0]) > 0.5:
                try:
                    run_x, how_x = graphed(fused)
                    t_x = _time_stream(run_x, stream, reps)
                    torch.cuda.synchronize()
                    be.scratch.check()
                except Exception as e:  # noqa: BLE001
                    err = repr(e)[:200]
            elif not err:
                err = "set-up failed on another rank"
            t = torch.tensor([t_x, 0.0 if err else 1.0], device=dev_t)
            dist.all_reduce(t[:1], op=dist.ReduceOp.MAX)
            dist.all_reduce(t[1:], op=dist.ReduceOp.MIN)
            if float(t[1]) > 0.5:
                out["M1_fused_exchange_us"] = float(t[0])
                out["M1_fused_launch"] = how_x
            else:
                out["M1_fused_exchange_error"] = err or "failed on another rank"
            dist.barrier()
            if peers is not None:
                peers.close()
    be.scratch.check()
    return out


def decode_stack(local, stream):
    """cfg4: the NF4 linears of one decode step of a 36-layer GQA transformer (hidden 2560, q 4096,
    k/v 1024, ff 9728): per layer fused qkv 2560->6144, o 4096->2560, fused gate|up+SiLU
    2560->2x9728, down 9728->2560; each linear gets its own N(0,1) input. One CUDA graph of 144
    launches, 1.87 GB of weights per step; then the same plus the bf16 lm_head 2560->151936
    (0.78 GB, dense GEMV) and the greedy argmax over its logits."""
    import dataclasses

    import numpy as np
    import torch

    from aila_b200 import synth
    from aila_b200.linear import Bnb4BitLinear, Bnb4BitLinearScratch, Linear, argmax
    dev = torch.device("cuda", local)
    HID, Q, KV, F, VOCAB = 2560, 4096, 1024, 9728, 151936
    shapes = {"q": (Q, HID), "k": (KV, HID), "v": (KV, HID), "o": (HID, Q), "gate": (F, HID),
              "up": (F, HID), "down": (HID, F)}
    base = {k: synth.synth_linear(synth.seed_for(4, 0, k), *v) for k, v in shapes.items()}

    def rolled(w, shift):
        n, k = w.out_features, w.in_features
        return dataclasses.replace(
            w, packed=np.roll(np.asarray(w.packed).reshape(n, k // 2), shift, 0).reshape(-1),
            absmax_codes=np.roll(np.asarray(w.absmax_codes).reshape(n, k // 64), shift, 0).reshape(-1))

    def lin(w):
        l = Bnb4BitLinear()
        assert l.init(w, local), l.last_error
        return l

    def fuse(*ls):
        f = Bnb4BitLinear()
        assert f.init_fused_rows(*ls), f.last_error
        for l in ls:
            l.close()
        return f

    layers = []
    for i in range(36):
        w = {k: rolled(v, 16 * i) for k, v in base.items()}
        layers.append((fuse(lin(w["q"]), lin(w["k"]), lin(w["v"])), lin(w["o"]),
                       fuse(lin(w["gate"]), lin(w["up"])), lin(w["down"])))
    scratch = Bnb4BitLinearScratch(local)
    scratch.ensure(1, F, 2 * F, False)
    x_h = synth.gaussian_activation(4009, 1, HID).to(dev)
    x_q = synth.gaussian_activation(4019, 1, Q).to(dev)
    x_f = synth.gaussian_activation(4029, 1, F).to(dev)
    y_qkv = torch.empty(1, Q + 2 * KV, dtype=torch.bfloat16, device=dev)
    y_h = torch.empty(1, HID, dtype=torch.bfloat16, device=dev)
    y_f = torch.empty(1, F, dtype=torch.bfloat16, device=dev)

    def step():
        for qkv, o, gu, dn in layers:
            qkv.forward(scratch, x_h, y_qkv, 1)
            o.forward(scratch, x_q, y_h, 1)
            assert Bnb4BitLinear.try_forward_decode_gate_up_swiglu(gu, scratch, x_h, y_f, F)
            dn.forward(scratch, x_f, y_h, 1)

    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
    us = _time_stream(graph.replay, stream, 20)
    scratch.check()
    # small batches through the batched decode kernel (eight rows per launch)
    batch = {}
    for M in (4, 8, 16, 32):
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

        with torch.cuda.stream(stream):
            step_m()
            stream.synchronize()
            gm = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gm, stream=stream):
                step_m()
        batch[f"M{M}_us_per_step"] = _time_stream(gm.replay, stream, 10)
        del gm
    scratch.check()
    # the bf16 lm_head of the same model and the token choice, alone and behind the stack
    g = torch.Generator().manual_seed(synth.seed_for(4, 0, "lm_head"))
    head_w = (torch.randn(VOCAB, HID, generator=g) * 0.02).to(torch.bfloat16)
    head = Linear()
    head.init(head_w, HID, VOCAB, local)
    del head_w
    logits = torch.empty(1, VOCAB, dtype=torch.bfloat16, device=dev)
    token = torch.zeros(1, dtype=torch.int32, device=dev)
    # three more heads so that consecutive timed launches do not find the weight in L2
    heads = [head]
    for _ in range(3):
        h = Linear()
        h.init((torch.randn(VOCAB, HID, generator=g) * 0.02).to(torch.bfloat16), HID, VOCAB, local)
        heads.append(h)

    def head_only():
        for h in heads:
            h.forward(scratch, x_h, logits, 1)

    def full_step():
        step()
        head.forward(scratch, y_h, logits, 1)
        argmax(logits, VOCAB, token)

    with torch.cuda.stream(stream):
        head_only()
        full_step()
        stream.synchronize()
        g_head = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_head, stream=stream):
            head_only()
        g_full = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_full, stream=stream):
            full_step()
    us_head = _time_stream(g_head.replay, stream, 10) / len(heads)
    us_full = _time_stream(g_full.replay, stream, 20)
    head_bytes = VOCAB * HID * 2
    wbytes = 36 * (weight_bytes(Q + 2 * KV, HID) + weight_bytes(HID, Q) + 2 * weight_bytes(F, HID) +
                   weight_bytes(HID, F))
    pk = peaks()
    return {"workload": "cfg4 NF4 linear stack, M=1: 36 x {qkv 2560->6144, o 4096->2560, "
                        "gate|up+SiLU 2560->2x9728, down 9728->2560}", "launches_per_step": 144,
            "weight_bytes_per_step": wbytes, "us_per_step": us, "weight_GBps": wbytes / us / 1e3,
            "frac_of_measured_hbm": wbytes / us / 1e3 / pk["hbm"],
            "small_batch": batch,
            "lm_head": {"workload": "bf16 dense GEMV 2560 -> 151936, 4 distinct weights in turn",
                        "us": us_head, "weight_GBps": head_bytes / us_head / 1e3,
                        "frac_of_measured_hbm": head_bytes / us_head / 1e3 / pk["hbm"]},
            "with_lm_head_and_argmax": {"us_per_step": us_full,
                                        "weight_bytes_per_step": wbytes + head_bytes,
                                        "weight_GBps": (wbytes + head_bytes) / us_full / 1e3,
                                        "frac_of_measured_hbm": (wbytes + head_bytes) / us_full / 1e3 / pk["hbm"]}}

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
    ap.add_argument("--no-tp", action="store_true", help="skip the sharded cfg5 MLP latency (N > 1)")
    ap.add_argument("--tp", action="store_true", help="also time the cfg5 MLP at N = 1")
    ap.add_argument("--stack", action="store_true", help="also time the cfg4 decode linear stack")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import numpy as np
    import torch
    import torch.distributed as dist

    from aila_b200 import synth
    from aila_b200.linear import Bnb4BitLinear, Bnb4BitLinearScratch

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
    linears = []
    for i in range(layers):
        def rolled(w, shift):
            if shift == 0:
                return w
            import dataclasses
            rows = np.asarray(w.packed).reshape(FF, H // 2)
            codes = np.asarray(w.absmax_codes).reshape(FF, H // 64)
            return dataclasses.replace(w, packed=np.roll(rows, shift, 0).reshape(-1),
                                       absmax_codes=np.roll(codes, shift, 0).reshape(-1))
        lg, lu, f = Bnb4BitLinear(), Bnb4BitLinear(), Bnb4BitLinear()
        assert lg.init(rolled(gate, 16 * i), local), lg.last_error
        assert lu.init(rolled(up, 16 * i), local), lu.last_error
        assert f.init_fused_rows(lg, lu), f.last_error
        lg.close()
        lu.close()
        linears.append(f)
    scratch = Bnb4BitLinearScratch(local)
    scratch.ensure(1, H, 2 * FF, False)
    x = synth.gaussian_activation(2009, 1, H).to(dev)
    outs = [torch.empty(1, FF, dtype=torch.bfloat16, device=dev) for _ in range(layers)]

    stream = torch.cuda.Stream(dev)

    def one_pass():
        for f, o in zip(linears, outs):
            ok = Bnb4BitLinear.try_forward_decode_gate_up_swiglu(f, scratch, x, o, FF)
            assert ok

    with torch.cuda.stream(stream):
        one_pass()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        for _ in range(args.warmup):
            graph.replay()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        with ClockSampler(local) as clocks:
            ev[0].record(stream)
            for i in range(args.steps):
                graph.replay()
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
    launch_us = ms_per_step * 1e3 / layers
    achieved = GATE_UP_ALGO_BYTES / (launch_us * 1e-6) / 1e9

    # ---- end to end through the host-buffer C-ABI call
    xh = synth.gaussian_activation(2009, 1, H).pin_memory()
    yh = torch.empty(1, FF, dtype=torch.bfloat16).pin_memory()
    with torch.cuda.stream(stream):
        for _ in range(2):
            for f in linears:
                f.gate_up_swiglu_host(scratch, xh, yh, 1, FF)
        e2e_steps = max(3, min(args.steps, 20))
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            for f in linears:
                f.gate_up_swiglu_host(scratch, xh, yh, 1, FF)
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = world * layers * GATE_UP_WEIGHT_BYTES / e2e_s / 1e9

    # ---- parity spot check of what was timed (one layer against the oracle is done in tests;
    # here only finiteness so the bench never reports numbers for garbage)
    assert torch.isfinite(outs[0].float()).all() and torch.isfinite(yh.float()).all()

    # ---- prefill GEMM pair (cfg3), rank 0 only
    prefill = None
    if not args.no_prefill and rank == 0:
        down_w = synth.synth_linear(synth.seed_for(3, 0, "down"), H, FF)
        down = Bnb4BitLinear()
        assert down.init(down_w, local), down.last_error
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
                                         "includes NF4->bf16 dequant pass of both weights",
                   "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["tf"], "unit": "TFLOP/s",
                                "frac": tf / pk["tf"], "peak_source": pk["source"] + " burst"},
                   "l2": "256 MB flush between iterations"}

    tp = None
    if (world > 1 and not args.no_tp) or args.tp:
        for f in linears:
            f.close()
        linears = []
        try:
            tp = tp_mlp_latency(rank, world, local, stream)
        except Exception as e:  # keep the headline line even if the extra fails
            tp = {"error": repr(e)}
    stack = None
    if args.stack and rank == 0:
        for f in linears:
            f.close()
        linears = []
        try:
            stack = decode_stack(local, stream)
        except Exception as e:
            stack = {"error": repr(e)}

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    cpu = None
    if not args.no_cpu and world == 1:
        cpu = cpu_gate_up_baseline()

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x nf4 -> f32 accumulate",
        "data": "synthetic",
        "config": {"workload": "cfg2 fused gate+up+SiLU NF4 GEMV, M=1, K=2560, 2x9728 rows, bs64 double-quant",
                   "layers_per_step": layers, "bytes_per_step": layers * GATE_UP_ALGO_BYTES,
                   "l2": f"inputs larger than L2: {layers} distinct weight copies = "
                         f"{layers * GATE_UP_WEIGHT_BYTES / 1e6:.0f} MB per step",
                   "launch": "CUDA graph of the C-ABI calls", "parallelism": f"replicas x{world}"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                     "frac": achieved / pk["hbm"], "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "peak_source": pk["source"], "launch_us": launch_us,
                     "algorithmic_bytes_per_launch": GATE_UP_ALGO_BYTES,
                     "frac_of_nominal_8TBps": achieved / 8000.0},
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": layers * 2 * H,
                "d2h_bytes_per_step": layers * 2 * FF,
                "note": "aila_nf4_forward_gate_up_swiglu_host per layer: pinned H2D copy of x, kernel "
                        "whose epilogue stores y straight into the pinned host buffer (the D2H "
                        "bytes cross PCIe as the kernel's stores), stream sync"},
        "gpu_launches": args.steps * layers,
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
