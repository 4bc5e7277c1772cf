#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference ...                    (the CPU arm: numpy statement on host cores)

Workload ("scale-out" configuration): 8 scenes x 120 000 unique voxels sampled uniformly in
a [41,1600,1408] grid (seed 4, one generator stream per scene), 3x3x3 submanifold conv,
C_in = C_out = 128, fp16 with fp32 accumulation.  A step is forward + input gradient +
weight gradient over the batch.  Scenes are sharded over the ranks (weights replicated, no
collective for forward / input gradient); the fp32 weight-gradient partials [128,27,128]
are summed by one NCCL all-reduce and cast to fp16.  Total work is fixed: strong scaling.

The timed loop replays CUDA graphs of the step over rotating buffer sets whose footprint
exceeds the 126 MB L2, so HBM figures are cold-cache.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_SCENES = 8
VOXELS_PER_SCENE = 120000
C_IN = C_OUT = 128
KV = 27
METRIC = "sparse-conv effective TFLOP/s (fwd+dgrad+wgrad, fp16, C=K=128, 3x3x3 subm)"
WORKLOAD = "scale-out: 8 scenes x 120k voxels, grid [41,1600,1408], seed 4, fwd+dgrad+wgrad fp16 C=K=128"
L2_BYTES = 126 * 1024 * 1024


def host_features(n_in, n_out, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n_in, C_IN), dtype=np.float32).astype(np.float16)
    dout = rng.standard_normal((n_out, C_OUT), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((KV, C_IN, C_OUT), dtype=np.float32) / np.sqrt(KV * C_IN)).astype(np.float16)
    return x, dout, np.ascontiguousarray(w.transpose(2, 0, 1))  # weight in the [K, kv, C] layout


def op_bytes(n_rows, num_tiles, C=C_IN, K=C_OUT, es=2):
    """Algorithmic bytes of one launch: features in + out, weights, neighbour table, mask + sort."""
    fwd = n_rows * C * es + n_rows * K * es + KV * C * K * es + 4 * KV * n_rows + 8 * n_rows
    wgrad = n_rows * C * es + n_rows * K * es + KV * C * K * es + 4 * KV * n_rows + 4 * n_rows + 4 * num_tiles
    return fwd, wgrad


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def finish(self):
        self._halt.set()
        self.join(timeout=1.0)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ----------------------------------------------------------------------------------------
# CPU arm: the reference's numpy statement of the op on the host cores
# ----------------------------------------------------------------------------------------
def cpu_sample_step(O, x, dout, w, indices):
    t = time.perf_counter()
    O.np_forward(x, w, indices)
    O.np_dgrad(dout, w, indices, x.shape[0])
    O.np_wgrad(dout, x, indices)
    return time.perf_counter() - t


def cpu_setup(voxels):
    from cumm_b200 import workloads as W
    from oracle import oracle as O
    tb = W.build_tables(W.sample_coords(voxels, [4, 0]))
    x, dout, w = host_features(tb.n_in, tb.n_out, [4, 100])
    return O, tb, x, dout, w


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    voxels = VOXELS_PER_SCENE
    O, tb, x, dout, w = cpu_setup(voxels)
    flops = 3 * 2 * tb.num_pairs * C_IN * C_OUT
    for _ in range(max(args.warmup, 1)):
        cpu_sample_step(O, x, dout, w, tb.indices)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_sample_step(O, x, dout, w, tb.indices)
    dt = (time.perf_counter() - t0) / args.steps
    val = flops / dt / 1e12
    cores = os.cpu_count()
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"one scene of {voxels} voxels per step (1/8 of the batch), numpy gather-"
                                   "matmul-scatter with the BLAS thread pool; the reference's own kernels and CPU "
                                   "simulator need its code generator, which is not installable offline"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "voxels_per_s": 3 * tb.n_out / dt,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scenes", type=int, default=N_SCENES,
                    help="scenes in the batch (default: the 8 of the benchmark configuration; other values are for experiments)")
    ap.add_argument("--no-extras", action="store_true", help="skip the single-scene configurations and CPU baseline")
    ap.add_argument("--single-scene-only", action="store_true",
                    help="run only the 150k-voxel single-scene configurations (few launches: the profiling case)")
    ap.add_argument("--reps", type=int, default=20, help="timed launches per op in the single-scene configurations")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from cumm_b200 import _lib
    from cumm_b200.layer import DeviceTables, SparseConvLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    if args.single_scene_only:
        st = torch.cuda.Stream(device=dev)
        print(json.dumps({"single_scene": single_scene_configs(torch, dev, st, reps=args.reps, warm=1)}), flush=True)
        return

    # ---- shard scenes over ranks
    n_scenes = args.scenes
    per = n_scenes // world if n_scenes % world == 0 else None
    if per is None:
        ids = [b for b in range(n_scenes) if b % world == rank]
    else:
        ids = list(range(rank * per, (rank + 1) * per))
    # neighbour tables of this rank's scenes, built on the GPU (bit-identical to the host generator:
    # tests/test_gpu_pairgen.py); the batch index keeps neighbours inside their scene
    from types import SimpleNamespace
    from cumm_b200 import workloads as W
    from cumm_b200.pairgen import build_tables_gpu
    coords_h = np.concatenate([W.sample_coords(VOXELS_PER_SCENE, [4, b], batch=b) for b in ids])
    tg = build_tables_gpu(torch.from_numpy(coords_h).to(dev), n_scenes, W.GRID)
    torch.cuda.synchronize()
    tb = SimpleNamespace(n_in=tg.n_in, n_out=tg.n_out, num_pairs=int((tg.indices >= 0).sum().item()))
    tg.num_pairs = tb.num_pairs
    x_h, dout_h, w_h = host_features(tb.n_in, tb.n_out, [4, 100, rank])
    _, _, w_h = host_features(8, 8, [4, 100])  # identical weights on every rank
    num_tiles = (tb.n_out + 127) // 128
    fwd_bytes, wgrad_bytes = op_bytes(tb.n_out, num_tiles)
    step_bytes = 2 * fwd_bytes + wgrad_bytes
    nsets = max(2, int(np.ceil(2.2 * L2_BYTES / step_bytes)))
    nsets = min(nsets, 12)

    stream = torch.cuda.Stream(device=dev)
    sets = []
    with torch.cuda.stream(stream):
        w_d = torch.from_numpy(w_h).to(dev)
        for i in range(nsets):
            t = tg.clone()  # every buffer set reads its own copy of the tables
            x = torch.from_numpy(x_h).to(dev)
            dout = torch.from_numpy(dout_h).to(dev)
            out = torch.zeros((tb.n_out, C_OUT), dtype=torch.float16, device=dev)
            din = torch.zeros((tb.n_in, C_IN), dtype=torch.float16, device=dev)
            dw32 = torch.zeros((C_OUT, KV, C_IN), dtype=torch.float32, device=dev)
            dw16 = torch.zeros((C_OUT, KV, C_IN), dtype=torch.float16, device=dev)
            layer = SparseConvLayer(t, w_d, x, out, dout, din, dw32, stream=stream.cuda_stream)
            sets.append(dict(t=t, x=x, dout=dout, out=out, din=din, dw32=dw32, dw16=dw16, layer=layer))
    stream.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)

    def step_kernels(s, events=None):
        L = s["layer"]
        if events:
            events[0].record(stream)
        L.fwd.launch()
        if events:
            events[1].record(stream)
        L.dgrad.launch()
        if events:
            events[2].record(stream)
        L.wgrad.launch()
        if events:
            events[3].record(stream)

    # The one exchange step of the path: sum the fp32 weight-gradient partials over ranks and cast.
    # Default: this library's one-shot sum through NVLink peer memory (cb2_peer_allreduce); with
    # CUMM_B200_ALLREDUCE=nccl, or if the peer buffers cannot be set up, NCCL all-reduce + cast.
    peer_ar, exchange_kind = None, "nccl all-reduce + cast"
    if world > 1:
        ok = 0
        if os.environ.get("CUMM_B200_ALLREDUCE", "peer") == "peer":
            try:
                from cumm_b200.peer_allreduce import PeerAllReduce
                peer_ar = PeerAllReduce.over_process_group(C_OUT * KV * C_IN, dev)
                ok = 1
            except Exception as e:  # noqa: BLE001 - any set-up failure means: use NCCL, and say so
                print(f"[rank {rank}] peer-memory sum unavailable ({e!r}); using NCCL", file=sys.stderr, flush=True)
        agreed = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed[0]) == 1:
            exchange_kind = "one-shot sum through NVLink peer memory (own kernel), fp16 cast fused"
        else:
            peer_ar = None

    def exchange(s, cuda_stream):
        if peer_ar is not None:
            peer_ar(s["dw32"], out_f16=s["dw16"], stream=cuda_stream)
        else:
            if world > 1:
                dist.all_reduce(s["dw32"])
            s["dw16"].copy_(s["dw32"])

    def step_tail(s, events=None):
        exchange(s, stream.cuda_stream)
        if events:
            events[4].record(stream)

    def step_ops(s, events=None):
        step_kernels(s, events)
        step_tail(s, events)

    # warm-up outside graphs (first-call set-up: attributes, status buffer, NCCL channels)
    with torch.cuda.stream(stream):
        for s in sets:
            step_ops(s)
    stream.synchronize()
    assert _lib.device_status() == 0, "kernel status word set during warm-up"

    # Single GPU: the whole step is one graph.  Several GPUs with the peer-memory sum: still one
    # graph -- forward, weight gradient, then the sum on a forked stream beside the input gradient
    # -- so a step costs the host one launch (at 8 GPUs a step is ~0.1 ms of GPU work: an eager
    # sequence of launches and events per step was slower than one GPU).  With NCCL: graph A =
    # forward + weight gradient, the all-reduce + cast eagerly on a side stream (NCCL stays out
    # of capture), graph B = input gradient on the main stream.
    graphs, graphs_b = [], []
    side = torch.cuda.Stream(device=dev)
    one_graph = world == 1 or peer_ar is not None
    with torch.cuda.stream(stream):
        for s in sets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                if world == 1:
                    step_kernels(s)
                    step_tail(s)
                elif one_graph:
                    s["layer"].fwd.launch()
                    s["layer"].wgrad.launch()
                    side.wait_stream(stream)
                    with torch.cuda.stream(side):
                        exchange(s, side.cuda_stream)
                    s["layer"].dgrad.launch()
                    stream.wait_stream(side)
                else:
                    s["layer"].fwd.launch()
                    s["layer"].wgrad.launch()
            graphs.append(g)
            if not one_graph:
                gb = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gb, stream=stream):
                    s["layer"].dgrad.launch()
                graphs_b.append(gb)
    stream.synchronize()
    ev_a = [torch.cuda.Event() for _ in range(nsets)]
    ev_b = [torch.cuda.Event() for _ in range(nsets)]

    def replay(i):
        k = i % nsets
        graphs[k].replay()
        if not one_graph:
            ev_a[k].record(stream)
            with torch.cuda.stream(side):
                side.wait_event(ev_a[k])
                exchange(sets[k], side.cuda_stream)
                ev_b[k].record(side)
            graphs_b[k].replay()
            stream.wait_event(ev_b[k])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            replay(i)
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    launches0 = _lib.launch_count()
    e0, e1 = ev(), ev()
    with torch.cuda.stream(stream):
        if world > 1:
            # The ranks leave the host barrier up to milliseconds apart, and a step ends in a
            # rendezvous of all GPUs: one more untimed step lines the GPUs' timelines up (its
            # exchange completes at the same moment everywhere), so the start events are
            # simultaneous and the K timed steps do not include one rank waiting for another's host.
            replay(args.warmup)
        e0.record(stream)
        for i in range(args.steps):
            replay(i)
        e1.record(stream)
    barrier()
    clocks = sampler.finish()
    ms_total = e0.elapsed_time(e1)
    # graph replays do not pass through the library's launch counter: per step forward, backward
    # input, and the three kernels of the weight gradient (plan, main, reduce)
    gpu_launches = 5 * args.steps
    del launches0

    # per-op durations, live, events between the launches (not graph-captured)
    op_ms = np.zeros(4)
    reps = max(5, min(args.steps, 20))
    with torch.cuda.stream(stream):
        for i in range(reps):
            evs = [ev() for _ in range(5)]
            step_ops(sets[i % nsets], evs)
            stream.synchronize()
            op_ms += [evs[j].elapsed_time(evs[j + 1]) for j in range(4)]
    op_ms /= reps
    if peer_ar is not None:
        # Between events the exchange also holds the wait for the slowest rank's eager launches;
        # the kernel's own clock readings (start to finish of the last call on this rank) are the
        # figure that belongs beside the other kernels.
        op_ms[3] = peer_ar.last_call_ns()["done"] * 1e-6
    status = _lib.device_status()

    ms_step = ms_total / args.steps
    t = torch.tensor([ms_step, float(tb.num_pairs), float(tb.n_out), float(status)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms_step, pairs_total, rows_total, status = float(tmax[0]), float(tsum[1]), float(tsum[2]), int(tmax[3])
    else:
        pairs_total, rows_total = float(tb.num_pairs), float(tb.n_out)
    flops_step = 3 * 2 * pairs_total * C_IN * C_OUT
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers (features in, weight gradient out)
    s0 = sets[0]
    x_pin = torch.from_numpy(x_h).pin_memory()
    dout_pin = torch.from_numpy(dout_h).pin_memory()
    dw_pin = torch.empty((C_OUT, KV, C_IN), dtype=torch.float16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        s0["x"].copy_(x_pin, non_blocking=True)
        s0["dout"].copy_(dout_pin, non_blocking=True)
        step_ops(s0)
        dw_pin.copy_(s0["dw16"], non_blocking=True)

    with torch.cuda.stream(stream):
        e2e_step()
    barrier()
    a0, a1 = ev(), ev()
    with torch.cuda.stream(stream):
        a0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        a1.record(stream)
    barrier()
    e2e_ms = a0.elapsed_time(a1) / e2e_steps
    if world > 1:
        tt = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt[0])
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
    h2d = x_pin.numel() * 2 + dout_pin.numel() * 2
    d2h = dw_pin.numel() * 2

    line = None
    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
        names = ["forward", "backward_input", "backward_weight(+reduce)", "allreduce+cast"]
        dom = int(np.argmax(op_ms[:3]))
        dom_bytes = [fwd_bytes, fwd_bytes, wgrad_bytes][dom]
        # DRAM bytes per output row from the ncu launch list of this command
        # (profiles/bench_step_launch_list.md): 459.9 MB (forward), 460.1 MB (backward input) and
        # 534.7 MB (backward weight: plan + main + reduce) per launch at 960 000 rows
        traffic = [479.1, 479.3, 557.0][dom] * tb.n_out
        achieved = dom_bytes / (op_ms[dom] * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "scenes_per_rank": len(ids), "rows_per_rank": tb.n_out,
                       "pairs_total": pairs_total, "parallelism": f"scene-sharded x{world}, wgrad fp32 all-reduce",
                       "l2": f"rotating {nsets} buffer sets ({nsets * step_bytes / 1e6:.0f} MB touched) > 126 MB L2",
                       "timed_region": "one CUDA graph per step (N>1: the exchange on a forked stream beside dgrad)" if one_graph else "graph(fwd+wgrad), then NCCL all-reduce + cast eagerly on a side stream overlapped with graph(dgrad)",
                       "exchange": exchange_kind if world > 1 else "none (one GPU)",
                       "exchange_last_call_ns_rank0": peer_ar.last_call_ns() if peer_ar is not None else None},
            "voxels_per_s": 3 * rows_total / (ms_step * 1e-3),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms},
            "gpu_launches": gpu_launches,
            "roofline": {"bound": "hbm", "kernel": names[dom], "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "peak_source": peak_src, "traffic": traffic,
                         "traffic_source": "ncu dram__bytes_read+write per row at 960k rows, scaled by rows",
                         "algorithmic_bytes_per_launch": dom_bytes, "us_per_launch": op_ms[dom] * 1e3},
            "per_op_us": {names[i]: op_ms[i] * 1e3 for i in range(4)},
            "per_op_gbs": {names[i]: [fwd_bytes, fwd_bytes, wgrad_bytes][i] / (op_ms[i] * 1e-3) / 1e9 for i in range(3)},
            "status_word": status,
        }

    if rank == 0 and world == 1 and not args.no_extras:
        line["single_scene"] = single_scene_configs(torch, dev, stream)
        line["cpu_baseline"] = cpu_baseline()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def single_scene_configs(torch, dev, stream, reps=20, warm=3):
    """The 150 000-voxel single-scene configurations, each op timed alone: fp16 C=K=128
    fwd/dgrad/wgrad and int8 stride-2 fwd.  Launches rotate over buffer sets whose combined
    footprint exceeds the 126 MB L2, so every launch reads its inputs from HBM."""
    from cumm_b200 import _lib
    from cumm_b200 import workloads as W
    from cumm_b200.layer import DeviceTables, SparseConvLayer
    res = {}
    coords = W.sample_coords(150000, 1)
    hbm_peak = 6531.0
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        hbm_peak = float(json.loads(pk.read_text()).get("hbm_gbs", hbm_peak))
    NSETS = 4

    def time_calls(calls):
        """Average duration of one launch: the launches of one pass over the rotating sets
        are captured in a CUDA graph and replayed back to back, so the figure holds the
        kernel and the gap to the next kernel on the stream, not the host's launch path."""
        ts = []
        with torch.cuda.stream(stream):
            for i in range(warm * len(calls)):
                calls[i % len(calls)].launch()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for c in calls:
                    c.launch()
            g.replay()
            stream.synchronize()
            for i in range(reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                g.replay()
                b.record(stream)
                stream.synchronize()
                ts.append(a.elapsed_time(b) / len(calls))
        return float(np.median(ts)) * 1e3  # us

    layers = []
    with torch.cuda.stream(stream):
        tb = W.build_tables(coords)
        rng = np.random.default_rng(2)
        xh = rng.standard_normal((tb.n_in, 128), dtype=np.float32).astype(np.float16)
        dh = rng.standard_normal((tb.n_out, 128), dtype=np.float32).astype(np.float16)
        w = torch.from_numpy((rng.standard_normal((128, 27, 128), dtype=np.float32) / 58.8).astype(np.float16)).to(dev)
        for _ in range(NSETS):
            x = torch.from_numpy(xh).to(dev)
            dout = torch.from_numpy(dh).to(dev)
            out = torch.zeros((tb.n_out, 128), dtype=torch.float16, device=dev)
            din = torch.zeros_like(x)
            dw = torch.zeros((128, 27, 128), dtype=torch.float16, device=dev)
            t = DeviceTables.from_host(tb, dev)
            layers.append(SparseConvLayer(t, w, x, out, dout, din, dw, stream=stream.cuda_stream))
    stream.synchronize()
    fb, wb = op_bytes(tb.n_out, (tb.n_out + 127) // 128)
    flops = 2 * tb.num_pairs * 128 * 128
    for L in layers:  # the weight gradient reads the forward pass's tile masks
        L.fwd.launch()
    for name, calls, nbytes in (("fp16_forward", [L.fwd for L in layers], fb),
                                ("fp16_backward_input", [L.dgrad for L in layers], fb),
                                ("fp16_backward_weight", [L.wgrad for L in layers], wb)):
        us = time_calls(calls)
        warm_us = time_calls([calls[0]] * NSETS)  # one buffer set over and over: the 95 MB working set stays in L2
        res[name] = {"us": us, "eff_tflops": flops / us / 1e6, "gbs": nbytes / us / 1e3,
                     "frac_hbm_measured": nbytes / us / 1e3 / hbm_peak, "gvoxels_per_s": tb.n_out / us / 1e3,
                     "us_warm_l2": warm_us}
    del layers
    res["gather_gemm_27_calls_c64"] = config1_gather_gemm(torch, dev, stream, coords, time_calls, hbm_peak, NSETS)
    # int8 stride-2 regular conv, k=3, pad=1
    layers3 = []
    with torch.cuda.stream(stream):
        tb3 = W.build_tables(coords, stride=(2, 2, 2), subm=False)
        rng = np.random.default_rng(3)
        x8h = rng.integers(-127, 128, (tb3.n_in, 128)).astype(np.int8)
        w8 = torch.from_numpy(rng.integers(-127, 128, (128, 27, 128)).astype(np.int8)).to(dev)
        sc = torch.from_numpy(rng.uniform(1e-3, 1e-2, 128).astype(np.float32)).to(dev)
        bi = torch.from_numpy(rng.standard_normal(128).astype(np.float32)).to(dev)
        for _ in range(NSETS):
            x8 = torch.from_numpy(x8h).to(dev)
            o8 = torch.zeros((tb3.n_out, 128), dtype=torch.int8, device=dev)
            t3 = DeviceTables.from_host(tb3, dev)
            L3 = SparseConvLayer(t3, w8, x8, o8, stream=stream.cuda_stream)
            L3.prepare_int8(sc, bi)
            layers3.append(L3)
    stream.synchronize()
    b3 = tb3.n_in * 128 + tb3.n_out * 128 + 27 * 128 * 128 + 4 * 27 * tb3.n_out + 8 * tb3.n_out + 2 * 128 * 4
    us = time_calls([L.fwd for L in layers3])
    warm_us = time_calls([layers3[0].fwd] * NSETS)
    ops = 2 * tb3.num_pairs * 128 * 128
    res["int8_forward_stride2"] = {"us": us, "eff_tops": ops / us / 1e6, "gbs": b3 / us / 1e3,
                                   "frac_hbm_measured": b3 / us / 1e3 / hbm_peak, "gvoxels_per_s": tb3.n_out / us / 1e3,
                                   "us_warm_l2": warm_us}
    res["table_generation"] = time_table_generation(torch, dev, stream, coords)
    res["l2"] = f"rotating {NSETS} buffer sets per configuration (> 126 MB L2)"
    res["timing"] = f"CUDA graph of {NSETS} back-to-back launches (one per buffer set), events around a replay, / {NSETS}"
    res["status_word"] = _lib.device_status()
    return res


def time_table_generation(torch, dev, stream, coords):
    """Neighbour tables of the 150 000-voxel scene built on the GPU (hash build, probe, masks,
    stable sort, backward tables): device time by CUDA events around the whole call, which
    includes its allocations and, for the strided case, the one synchronisation that returns
    the number of active outputs."""
    from cumm_b200 import workloads as W
    from cumm_b200.pairgen import build_tables_gpu
    out = {}
    with torch.cuda.stream(stream):
        cd = torch.from_numpy(coords).to(dev)
        for name, kw in (("submanifold", {}), ("stride2", {"stride": (2, 2, 2), "subm": False})):
            ts = []
            for i in range(6):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                t = build_tables_gpu(cd, 1, W.GRID, stream=stream.cuda_stream, **kw)
                b.record(stream)
                stream.synchronize()
                if i:
                    ts.append(a.elapsed_time(b) * 1e3)
            # int32 traffic the tables amount to: coordinates in, both index tables, masks and orders out
            nbytes = 16 * t.n_in + 4 * 27 * (t.n_in + t.n_out) + 8 * (t.n_in + t.n_out)
            us = float(np.median(ts))
            out[name] = {"us": us, "n_out": t.n_out, "table_bytes": nbytes, "gbs": nbytes / us / 1e3}
    return out


def config1_gather_gemm(torch, dev, stream, coords, time_calls, hbm_peak, nsets):
    """The native (non-mask) sparse convolution of the 150 000-voxel scene at C = K = 64: one
    gather-GEMM-scatter GemmParams call per filter offset that has pairs, accumulating with
    beta = 1 into a pre-zeroed output, as cumm/gemm/main_real_spconv.py:309-403 does.  The
    figure is the time of the whole sequence of calls."""
    from cumm_b200 import workloads as W
    from cumm_b200.tensorview import float16, float32
    from cumm_b200.tensorview.gemm import GemmAlgoDesp, GemmParams, ShuffleStrideType, prepare_gemm
    tb = W.build_tables(coords)
    C = K = 64
    rng = np.random.default_rng(1)
    xh = rng.standard_normal((tb.n_in, C), dtype=np.float32).astype(np.float16)
    wh = (rng.standard_normal((K, 27, C), dtype=np.float32) / np.sqrt(27 * C)).astype(np.float16)
    d = GemmAlgoDesp()
    d.dtype_a = d.dtype_b = d.dtype_c = float16
    d.dacc = d.dcomp = float32
    d.trans_a, d.trans_b, d.trans_c = False, True, False
    d.tile_shape = [128, 64, 64]  # C = K = 64: the narrowest tiles
    d.warp_tile_shape = [128, 64, 64]
    d.tensorop = [128, 64, 16]
    d.num_stage = 3
    d.algo = "Blackwell"
    d.shuffle_type = ShuffleStrideType.ShuffleAC
    d.element_per_access_a = d.element_per_access_b = d.element_per_access_c = 8
    pairs = []
    for f in range(27):
        o_idx = np.nonzero(tb.indices[f] >= 0)[0].astype(np.int32)
        if len(o_idx):
            pairs.append((f, tb.indices[f][o_idx].astype(np.int32), o_idx))
    n_pairs = sum(len(o) for _, _, o in pairs)
    sequences = []
    with torch.cuda.stream(stream):
        w = torch.from_numpy(wh).to(dev)
        idx_dev = [(f, torch.from_numpy(i).to(dev), torch.from_numpy(o).to(dev)) for f, i, o in pairs]
        for _ in range(nsets):
            x = torch.from_numpy(xh).to(dev)
            out = torch.zeros((tb.n_out, K), dtype=torch.float16, device=dev)
            calls = []
            for f, i_idx, o_idx in idx_dev:
                p = GemmParams()
                p.algo_desp = d
                p.a, p.b, p.c = x, w[:, f, :], out
                p.a_inds, p.c_inds = i_idx, o_idx
                p.beta = 1.0
                p.stream = stream.cuda_stream
                calls.append(prepare_gemm(p))
            sequences.append(calls)
    stream.synchronize()

    class Sequence:
        def __init__(self, calls):
            self.calls = calls

        def launch(self):
            for c in self.calls:
                c.launch()

    us = time_calls([Sequence(c) for c in sequences])
    nbytes = tb.n_in * C * 2 + tb.n_out * K * 2 + 27 * C * K * 2 + 8 * n_pairs
    return {"us": us, "calls": len(pairs), "pairs": int(n_pairs), "eff_tflops": 2 * n_pairs * C * K / us / 1e6,
            "gbs": nbytes / us / 1e3, "frac_hbm_measured": nbytes / us / 1e3 / hbm_peak}


def cpu_baseline():
    """The numpy statement of one scene's step on the host cores, a bounded sample."""
    O, tb, x, dout, w = cpu_setup(VOXELS_PER_SCENE)
    cpu_sample_step(O, x, dout, w, tb.indices)
    n, t_total = 0, 0.0
    while t_total < 10.0 and n < 20:
        t_total += cpu_sample_step(O, x, dout, w, tb.indices)
        n += 1
    dt = t_total / n
    flops = 3 * 2 * tb.num_pairs * C_IN * C_OUT
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{n} steps over one scene of {VOXELS_PER_SCENE} voxels (1/8 of the batch), numpy "
                      "gather-matmul-scatter, BLAS thread pool", "ms_per_sample_step": dt * 1e3}


if __name__ == "__main__":
    main()
