#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference ...                    (the CPU arm: numpy statement on host cores)

Workload ("scale-out" configuration): 8 scenes x 120 000 unique voxels sampled uniformly in
a [41,1600,1408] grid (seed 4, one generator stream per scene), 3x3x3 submanifold conv,
C_in = C_out = 128, fp16 with fp32 accumulation.  A step is forward + input gradient +
weight gradient over the batch.  Scenes are sharded over the ranks (weights replicated, no
collective for forward / input gradient); the fp32 weight-gradient partials [128,27,128]
are summed over the ranks (one exchange step) and cast to fp16.  Total work is fixed: strong
scaling.

The three operators of a step are independent of each other, so a step is one CUDA graph with
three branches (each kernel bounded to a share of the SMs, `max_ctas`) unless
`--schedule sequential` asks for one after the other.  The timed loop replays the graphs over
rotating buffer sets whose footprint exceeds the 126 MB L2, so HBM figures are cold-cache; it
is repeated `--repeats` times and the median is the headline.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import hashlib
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
# SM shares of the three kernels when they run side by side (forward, backward input, backward
# weight), picked from measured step times: with several GPUs the exchange follows the weight
# gradient, so that branch gets more SMs the smaller a GPU's share of the rows is (2 GPUs:
# measured there; 4 and 8: from one GPU running a rank's rows with a world-of-one exchange).
_WORLD = int(os.environ.get("WORLD_SIZE", "1"))
SHARES = tuple(int(v) for v in os.environ.get(
    "CUMM_B200_BENCH_SHARES",
    "48,48,52" if _WORLD == 1 else "46,46,56" if _WORLD <= 2 else "42,42,64" if _WORLD <= 4 else "40,40,68").split(","))
# Several GPUs: the weight gradient runs first on the whole GPU, then forward and backward input side
# by side on these shares while the exchange runs on the SMs they leave free.
MULTI_GPU_SCHEDULE = os.environ.get("CUMM_B200_BENCH_MULTI", "branches")  # or "wgrad_first"
PAIR_SHARES = tuple(int(v) for v in os.environ.get("CUMM_B200_BENCH_PAIR_SHARES", "68,68").split(","))


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


def base_config(world, scenes, rows_per_rank, pairs_total):
    return {"workload": WORKLOAD, "scenes": scenes, "scenes_per_rank": scenes // max(world, 1),
            "rows_per_rank": rows_per_rank, "pairs_total": pairs_total,
            "parallelism": f"scene-sharded x{world}, wgrad fp32 partial sums exchanged"}


def hbm_peak():
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
        if "hbm_gbs" in peaks:
            return float(peaks["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback 6650 GB/s"


def csrc_digest():
    h = hashlib.sha256()
    for f in sorted((ROOT / "cumm_b200" / "csrc").glob("*.cu*")):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()[:16]


def measured_traffic():
    """DRAM bytes per output row of each kernel, from the ncu capture recorded in
    profiles/traffic.json, and whether the kernel sources have changed since that capture."""
    p = ROOT / "profiles" / "traffic.json"
    if not p.exists():
        return None, None
    t = json.loads(p.read_text())
    return t, t.get("csrc_sha256") != csrc_digest()


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
            time.sleep(0.002)

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
# CPU arm: the reference's numpy statement of the op on the host cores, over the whole batch
# ----------------------------------------------------------------------------------------
def cpu_setup(scenes=N_SCENES, voxels=VOXELS_PER_SCENE):
    from cumm_b200 import workloads as W
    from oracle import oracle as O
    tabs = [W.build_tables(W.sample_coords(voxels, [4, b], batch=b)) for b in range(scenes)]
    _, _, w = host_features(8, 8, [4, 100])
    feats = [host_features(voxels, voxels, [4, 100, b])[:2] for b in range(scenes)]
    return O, tabs, feats, w


def cpu_batch_step(O, tabs, feats, w):
    """forward + input gradient + weight gradient of every scene of the batch; returns seconds."""
    t = time.perf_counter()
    dw = None
    for tb, (x, dout) in zip(tabs, feats):
        O.np_forward(x, w, tb.indices)
        O.np_dgrad(dout, w, tb.indices, x.shape[0])
        d = O.np_wgrad(dout, x, tb.indices)
        dw = d if dw is None else dw + d
    return time.perf_counter() - t


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    O, tabs, feats, w = cpu_setup(args.scenes)
    pairs = float(sum(tb.num_pairs for tb in tabs))
    rows = sum(tb.n_out for tb in tabs)
    flops = 3 * 2 * pairs * C_IN * C_OUT
    for _ in range(max(args.warmup, 1)):
        cpu_batch_step(O, tabs, feats, w)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_batch_step(O, tabs, feats, w)
    dt = (time.perf_counter() - t0) / args.steps
    val = flops / dt / 1e12
    cores = os.cpu_count()
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": base_config(world, args.scenes, rows // world, pairs),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"the whole batch per step ({args.scenes} scenes x {VOXELS_PER_SCENE} voxels), numpy "
                                   "gather-matmul-scatter with the BLAS thread pool; the reference's own kernels and CPU "
                                   "simulator need its code generator, which is not installable offline"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "voxels_per_s": 3 * rows / dt,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline(scenes=N_SCENES):
    """The numpy statement of the batch's step on the host cores, a bounded sample."""
    O, tabs, feats, w = cpu_setup(scenes)
    cpu_batch_step(O, tabs, feats, w)
    n, t_total = 0, 0.0
    while t_total < 12.0 and n < 10:
        t_total += cpu_batch_step(O, tabs, feats, w)
        n += 1
    dt = t_total / n
    flops = 3 * 2 * float(sum(tb.num_pairs for tb in tabs)) * C_IN * C_OUT
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{n} steps over the whole batch ({scenes} scenes x {VOXELS_PER_SCENE} voxels), numpy "
                      "gather-matmul-scatter, BLAS thread pool", "ms_per_sample_step": dt * 1e3}


# ----------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--repeats", type=int, default=10, help="how many times the K-step timed loop is run (median reported)")
    ap.add_argument("--schedule", default=os.environ.get("CUMM_B200_BENCH_SCHEDULE", "concurrent"),
                    choices=["concurrent", "sequential"],
                    help="the three operators of a step side by side on SM shares, or one after the other")
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
    from cumm_b200.layer import SparseConvLayer
    from cumm_b200.tensorview.gemm import ConvOpType

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
    from cumm_b200 import workloads as W
    from cumm_b200.pairgen import build_tables_gpu
    coords_h = np.concatenate([W.sample_coords(VOXELS_PER_SCENE, [4, b], batch=b) for b in ids])
    tg = build_tables_gpu(torch.from_numpy(coords_h).to(dev), n_scenes, W.GRID)
    torch.cuda.synchronize()
    n_in, n_out = tg.n_in, tg.n_out
    num_pairs = int((tg.indices >= 0).sum().item())
    tg.num_pairs = num_pairs
    feats = [host_features(VOXELS_PER_SCENE, VOXELS_PER_SCENE, [4, 100, b])[:2] for b in ids]
    x_h = np.concatenate([f[0] for f in feats])
    dout_h = np.concatenate([f[1] for f in feats])
    _, _, w_h = host_features(8, 8, [4, 100])  # identical weights on every rank
    num_tiles = (n_out + 127) // 128
    fwd_bytes, wgrad_bytes = op_bytes(n_out, num_tiles)
    step_bytes = 2 * fwd_bytes + wgrad_bytes
    nsets = max(2, int(np.ceil(2.2 * L2_BYTES / step_bytes)))
    nsets = min(nsets, 12)
    concurrent = args.schedule == "concurrent"
    shares = {ConvOpType.Forward: SHARES[0], ConvOpType.BackwardInput: SHARES[1], ConvOpType.BackwardWeight: SHARES[2]}

    stream = torch.cuda.Stream(device=dev)
    s_dgrad, s_wgrad = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    sets = []
    with torch.cuda.stream(stream):
        w_d = torch.from_numpy(w_h).to(dev)
        for i in range(nsets):
            t = tg.clone()  # every buffer set reads its own copy of the tables
            x = torch.from_numpy(x_h).to(dev)
            dout = torch.from_numpy(dout_h).to(dev)
            out = torch.zeros((n_out, C_OUT), dtype=torch.float16, device=dev)
            din = torch.zeros((n_in, C_IN), dtype=torch.float16, device=dev)
            dw16 = torch.zeros((C_OUT, KV, C_IN), dtype=torch.float16, device=dev)
            # one GPU: the weight gradient writes fp16 itself; several: fp32 partials for the exchange
            dw32 = torch.zeros((C_OUT, KV, C_IN), dtype=torch.float32, device=dev) if world > 1 else None
            dw = dw32 if world > 1 else dw16
            alone = SparseConvLayer(t, w_d, x, out, dout, din, dw, stream=stream.cuda_stream)
            shared = SparseConvLayer(t, w_d, x, out, dout, din, dw, stream=stream.cuda_stream, cta_shares=shares)
            pair = SparseConvLayer(t, w_d, x, out, dout, din, None, stream=stream.cuda_stream,
                                   cta_shares={ConvOpType.Forward: PAIR_SHARES[0], ConvOpType.BackwardInput: PAIR_SHARES[1]})
            sets.append(dict(t=t, x=x, dout=dout, out=out, din=din, dw32=dw32, dw16=dw16, alone=alone, shared=shared,
                             pair=pair))
    stream.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)

    # The one exchange step of the path: sum the fp32 weight-gradient partials over ranks and cast.
    # Default: this library's sum through NVLink peer memory (cb2_peer_allreduce); with
    # CUMM_B200_ALLREDUCE=nccl, or if the peer buffers cannot be set up, NCCL all-reduce + cast.
    peer_ar, exchange_kind = None, "nccl all-reduce + cast"
    if world > 1:
        ok = 0
        if os.environ.get("CUMM_B200_ALLREDUCE", "peer") == "peer":
            try:
                from cumm_b200.peer_allreduce import PeerAllReduce
                peer_ar = PeerAllReduce.over_process_group(C_OUT * KV * C_IN, dev)
                # its CTAs go to the SMs the convolution kernels leave free, not beside them
                peer_ar.own_sm_smem_bytes = 12 * 1024
                ok = 1
            except Exception as e:  # noqa: BLE001 - any set-up failure means: use NCCL, and say so
                print(f"[rank {rank}] peer-memory sum unavailable ({e!r}); using NCCL", file=sys.stderr, flush=True)
        agreed = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed[0]) == 1:
            exchange_kind = "sum through NVLink peer memory (own kernel: reduce-scatter + all-gather by plain peer stores), fp16 cast fused"
        else:
            peer_ar = None

    def exchange(s, cuda_stream):
        if world == 1:
            return
        if peer_ar is not None:
            peer_ar(s["dw32"], out_f16=s["dw16"], stream=cuda_stream)
        else:
            red = s["dw32"].clone()
            dist.all_reduce(red)
            s["dw16"].copy_(red)

    def step_sequential(s, events=None):
        """Eager, one operator after the other on the main stream, full grids (per-op timings)."""
        L = s["alone"]
        for i, call in enumerate((L.fwd, L.dgrad, L.wgrad)):
            if events:
                events[i].record(stream)
            call.launch()
        if events:
            events[3].record(stream)
        exchange(s, stream.cuda_stream)
        if events:
            events[4].record(stream)

    def step_branches(s):
        """One GPU: the step as three branches: forward on the main stream, input gradient and
        weight gradient on two others, joined at the end.  Several GPUs: the weight gradient first,
        on the whole GPU, then three branches: the exchange of its partial sums, forward and
        input gradient (the two convolutions leave the exchange a few SMs of its own)."""
        s_dgrad.wait_stream(stream)
        s_wgrad.wait_stream(stream)
        if world == 1 or MULTI_GPU_SCHEDULE == "branches":
            L = s["shared"]
            L.fwd.launch()
            with torch.cuda.stream(s_wgrad):
                L.wgrad.launch(s_wgrad.cuda_stream)
                exchange(s, s_wgrad.cuda_stream)
            with torch.cuda.stream(s_dgrad):
                L.dgrad.launch(s_dgrad.cuda_stream)
        else:
            s["alone"].wgrad.launch()
            s_dgrad.wait_stream(stream)
            s_wgrad.wait_stream(stream)
            with torch.cuda.stream(s_wgrad):
                exchange(s, s_wgrad.cuda_stream)
            s["pair"].fwd.launch()
            with torch.cuda.stream(s_dgrad):
                s["pair"].dgrad.launch(s_dgrad.cuda_stream)
        stream.wait_stream(s_dgrad)
        stream.wait_stream(s_wgrad)

    # warm-up outside graphs (first-call set-up: attributes, status buffer, plans, NCCL channels)
    with torch.cuda.stream(stream):
        for s in sets:
            step_sequential(s)
            step_branches(s)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "kernel status word set during warm-up"
    l0 = _lib.launch_count()
    with torch.cuda.stream(stream):
        step_branches(sets[0]) if concurrent else step_sequential(sets[0])
    torch.cuda.synchronize()
    launches_per_step = _lib.launch_count() - l0

    # Graph capture.  One GPU, or several with the peer-memory sum: the whole step is one graph.
    # With NCCL the all-reduce stays outside capture (a captured NCCL all-reduce hung a 2-GPU run
    # here): graph A = forward + weight gradient, the all-reduce + cast eagerly on a side stream,
    # graph B = input gradient.
    graphs, graphs_b = [], []
    side = torch.cuda.Stream(device=dev)
    one_graph = world == 1 or peer_ar is not None
    with torch.cuda.stream(stream):
        for s in sets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                if one_graph:
                    if concurrent:
                        step_branches(s)
                    else:
                        L = s["alone"]
                        L.fwd.launch()
                        L.wgrad.launch()
                        if world > 1:
                            side.wait_stream(stream)
                            with torch.cuda.stream(side):
                                exchange(s, side.cuda_stream)
                        L.dgrad.launch()
                        if world > 1:
                            stream.wait_stream(side)
                else:
                    s["alone"].fwd.launch()
                    s["alone"].wgrad.launch()
            graphs.append(g)
            if not one_graph:
                gb = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gb, stream=stream):
                    s["alone"].dgrad.launch()
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

    # ---- the exchange's result, checked against the rank-ordered sum (untimed)
    exchange_verified = None
    if world > 1:
        exchange_verified = verify_exchange(torch, dist, dev, stream, sets, exchange, replay, peer_ar is not None, world)

    # ---- timed region: K steps, repeated; device time by CUDA events, max over ranks per repeat
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    rep_ms = []
    for r in range(max(1, args.repeats)):
        barrier()
        e0, e1 = ev(), ev()
        with torch.cuda.stream(stream):
            if world > 1:
                # The ranks leave the host barrier up to milliseconds apart, and a step ends in a
                # rendezvous of all GPUs: one more untimed step lines the GPUs' timelines up, so the
                # start events are simultaneous and the K timed steps do not include one rank
                # waiting for another's host.
                replay(args.warmup)
            e0.record(stream)
            for i in range(args.steps):
                replay(i)
            e1.record(stream)
        barrier()
        rep_ms.append(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.finish()
    # the exchange kernel's own clock readings in the last timed step (graph replay, ranks in step)
    exchange_in_step_ns = peer_ar.last_call_ns() if peer_ar is not None else None
    rep_t = torch.tensor(rep_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(rep_t, op=dist.ReduceOp.MAX)
    rep_ms = rep_t.cpu().numpy()
    ms_step = float(np.median(rep_ms))
    gpu_launches = int(launches_per_step) * args.steps * len(rep_ms)

    # per-op durations, live, events between eager launches with full grids (each operator alone)
    op_ms = np.zeros(4)
    reps = max(5, min(args.steps, 20))
    with torch.cuda.stream(stream):
        for i in range(reps):
            evs = [ev() for _ in range(5)]
            step_sequential(sets[i % nsets], evs)
            stream.synchronize()
            op_ms += [evs[j].elapsed_time(evs[j + 1]) for j in range(4)]
    op_ms /= reps
    if peer_ar is not None:
        # Between events of eager launches the exchange also holds the wait for the slowest rank's
        # host; the kernel's own clock readings in the last timed step (start to finish on this
        # rank) are the figure that belongs beside the other kernels.
        op_ms[3] = exchange_in_step_ns["done"] * 1e-6
    status = _lib.device_status()

    t = torch.tensor([float(num_pairs), float(n_out), float(status)], dtype=torch.float64, device=dev)
    if world > 1:
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        pairs_total, rows_total, status = float(tsum[0]), float(tsum[1]), int(tmax[2])
    else:
        pairs_total, rows_total = float(num_pairs), float(n_out)
    flops_step = 3 * 2 * pairs_total * C_IN * C_OUT
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers: both feature tensors in, all three
    # results (output rows, input gradient, weight gradient) back, every step
    s0 = sets[0]
    x_pin = torch.from_numpy(x_h).pin_memory()
    dout_pin = torch.from_numpy(dout_h).pin_memory()
    out_pin = torch.empty((n_out, C_OUT), dtype=torch.float16).pin_memory()
    din_pin = torch.empty((n_in, C_IN), dtype=torch.float16).pin_memory()
    dw_pin = torch.empty((C_OUT, KV, C_IN), dtype=torch.float16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    # Double-buffered: the copies in of step i+1 and the copies out of step i run on streams of their
    # own beside the kernels, so the two directions of the host link are busy at the same time.  Every
    # step still copies its own inputs in and its own results out; events order the three streams.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    done_in = [ev() for _ in range(2)]
    done_run = [ev() for _ in range(2)]
    done_out = [ev() for _ in range(2)]

    def e2e_step(i):
        k = i % 2
        sk = sets[k]
        # the set's inputs are free once the step that last used the set has run
        s_in.wait_event(done_run[k])
        with torch.cuda.stream(s_in):
            sk["x"].copy_(x_pin, non_blocking=True)
            sk["dout"].copy_(dout_pin, non_blocking=True)
            done_in[k].record(s_in)
        # the set's results are free once they have been copied out
        stream.wait_event(done_in[k])
        stream.wait_event(done_out[k])
        replay(k)
        done_run[k].record(stream)
        s_out.wait_event(done_run[k])
        with torch.cuda.stream(s_out):
            out_pin.copy_(sk["out"], non_blocking=True)
            din_pin.copy_(sk["din"], non_blocking=True)
            dw_pin.copy_(sk["dw16"], non_blocking=True)
            done_out[k].record(s_out)

    with torch.cuda.stream(stream):
        for k in range(2):
            done_run[k].record(stream)
            done_out[k].record(stream)
        e2e_step(0)
        e2e_step(1)
        stream.wait_event(done_out[0])
        stream.wait_event(done_out[1])
    barrier()
    a0, a1 = ev(), ev()
    with torch.cuda.stream(stream):
        a0.record(stream)
        s_in.wait_event(a0)
        for i in range(e2e_steps):
            e2e_step(i)
        stream.wait_event(done_out[0])
        stream.wait_event(done_out[1])
        a1.record(stream)
    barrier()
    e2e_ms = a0.elapsed_time(a1) / e2e_steps
    if world > 1:
        tt = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt[0])
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
    h2d = x_pin.numel() * 2 + dout_pin.numel() * 2
    d2h = (out_pin.numel() + din_pin.numel() + dw_pin.numel()) * 2

    line = None
    if rank == 0:
        peak, peak_src = hbm_peak()
        names = ["forward", "backward_input", "backward_weight", "exchange+cast"]
        dom = int(np.argmax(op_ms[:3]))
        dom_bytes = [fwd_bytes, fwd_bytes, wgrad_bytes][dom]
        achieved = dom_bytes / (op_ms[dom] * 1e-3) / 1e9
        tr, stale = measured_traffic()
        traffic = None
        if tr is not None:
            traffic = float(tr["dram_bytes_per_row"][names[dom]]) * n_out
        cfg = base_config(world, n_scenes, n_out, pairs_total)
        run = {}
        run.update({
            "l2": f"rotating {nsets} buffer sets ({nsets * step_bytes / 1e6:.0f} MB touched) > 126 MB L2",
            "schedule": (f"one CUDA graph per step, three branches side by side (max_ctas {SHARES[0]}/{SHARES[1]}/{SHARES[2]}: "
                         "forward / backward input / backward weight" + (", the exchange after it on the SMs it frees)" if world > 1 else ")")
                         if concurrent and one_graph and (world == 1 or MULTI_GPU_SCHEDULE == "branches") else
                         f"one CUDA graph per step: backward weight on the whole GPU, then forward / backward input side by "
                         f"side (max_ctas {PAIR_SHARES[0]}/{PAIR_SHARES[1]}) with the exchange on the SMs they leave free"
                         if concurrent and one_graph else
                         "one CUDA graph per step, operators one after the other" if one_graph else
                         "graph(fwd+wgrad), then NCCL all-reduce + cast eagerly on a side stream overlapped with graph(dgrad)"),
            "exchange": exchange_kind if world > 1 else "none (one GPU)",
            "exchange_verified": exchange_verified,
            "exchange_last_call_ns_rank0": exchange_in_step_ns,
            "timed_region": f"{len(rep_ms)} repeats of {args.steps} steps; ms_per_step is the median repeat",
        })
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": cfg, "run": run,
            "repeats": {"n": len(rep_ms), "ms_per_step_min": float(rep_ms.min()), "ms_per_step_max": float(rep_ms.max()),
                        "spread": float((rep_ms.max() - rep_ms.min()) / ms_step)},
            "voxels_per_s": 3 * rows_total / (ms_step * 1e-3),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms,
                    "how": "every step: inputs from pinned host memory, the step, all three results back to pinned host "
                           "memory; two buffer sets, copies in / kernels / copies out on three streams"},
            "gpu_launches": gpu_launches,
            "roofline": {"bound": "hbm", "kernel": names[dom] + " (alone, full grid)", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src, "traffic": traffic,
                         "traffic_source": None if tr is None else tr.get("source"), "traffic_stale": stale,
                         "algorithmic_bytes_per_launch": dom_bytes, "us_per_launch": op_ms[dom] * 1e3},
            "roofline_step": {"bound": "hbm", "what": "all three operators of the timed step (this rank's rows)",
                              "algorithmic_bytes_per_step": step_bytes,
                              "achieved": step_bytes / (ms_step * 1e-3) / 1e9, "unit": "GB/s",
                              "frac": step_bytes / (ms_step * 1e-3) / 1e9 / peak},
            "per_op_us": {names[i]: op_ms[i] * 1e3 for i in range(4)},
            "per_op_gbs": {names[i]: [fwd_bytes, fwd_bytes, wgrad_bytes][i] / (op_ms[i] * 1e-3) / 1e9 for i in range(3)},
            "status_word": status,
        }

    if rank == 0 and world == 1 and not args.no_extras:
        line["single_scene"] = single_scene_configs(torch, dev, stream)
        line["config0"] = config0_dense_gemm(torch, dev, stream)
        line["cpu_baseline"] = cpu_baseline(n_scenes)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if exchange_verified is False:
        sys.exit(3)


def verify_exchange(torch, dist, dev, stream, sets, exchange, replay, bit_exact, world):
    """Compares what the exchange delivers with the fp32 partials of all ranks summed in rank
    order (gathered with NCCL, added on the device), outside the timed region: three eager
    calls on fresh rank-dependent data (both slot parities of the peer-memory kernel), then the
    buffers a graph replay left behind.  The peer-memory kernel must match bit for bit and every
    rank must hold identical fp16 results; the NCCL variant is held to fp32 round-off."""
    rank = dist.get_rank()
    ok = True

    def check(s, what):
        nonlocal ok
        parts = [torch.empty_like(s["dw32"]) for _ in range(world)]
        dist.all_gather(parts, s["dw32"])
        acc = parts[0].clone()
        for r in range(1, world):
            acc += parts[r]
        want16 = acc.to(torch.float16)
        got16 = s["dw16"]
        if bit_exact:
            good = bool(torch.equal(got16.view(torch.int16), want16.view(torch.int16)))
        else:
            good = bool(torch.allclose(got16.float(), want16.float(), rtol=2e-3, atol=1e-3))
        all16 = [torch.empty_like(got16) for _ in range(world)]
        dist.all_gather(all16, got16)
        same = all(bool(torch.equal(all16[0].view(torch.int16), a.view(torch.int16))) for a in all16)
        if not (good and same):
            ok = False
            bad = int((got16.float() != want16.float()).sum())
            print(f"[rank {rank}] exchange check failed ({what}): {bad} entries differ from the rank-ordered sum; "
                  f"identical on all ranks: {same}", file=sys.stderr, flush=True)

    s = sets[0]
    keep = s["dw32"].clone()
    with torch.cuda.stream(stream):
        for call in range(3):
            g = torch.Generator(device=dev)
            g.manual_seed(1000 * call + rank)
            s["dw32"].copy_(torch.randn(s["dw32"].shape, generator=g, device=dev) * (1.0 + rank))
            s["dw16"].zero_()
            exchange(s, stream.cuda_stream)
            stream.synchronize()
            check(s, f"eager call {call}")
        s["dw32"].copy_(keep)
        for i in range(2):
            replay(i)
        stream.synchronize()
        for i in range(2):
            check(sets[i % len(sets)], f"after graph replay of set {i % len(sets)}")
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(int(flag[0]) == 1)


def config0_dense_gemm(torch, dev, stream):
    """The simulator-sized dense GEMM (A [128,64] x B [64,128] fp16, fp32 accumulation, alpha 1,
    beta 0): its time on the GPU through GemmParams with no index lists, beside a single-core
    numpy tile-loop restatement of the data flow of the reference's CPU simulator (64x64x32
    tiles), which stands in for the simulator itself (it needs the reference's code generator)."""
    from cumm_b200.tensorview import float16, float32
    from cumm_b200.tensorview.gemm import GemmAlgoDesp, GemmParams, ShuffleStrideType, prepare_gemm
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (128, 64)).astype(np.float32).astype(np.float16)
    b = rng.uniform(-1, 1, (64, 128)).astype(np.float32).astype(np.float16)
    d = GemmAlgoDesp()
    d.dtype_a = d.dtype_b = d.dtype_c = float16
    d.dacc = d.dcomp = float32
    d.trans_a, d.trans_b, d.trans_c = False, False, False
    d.tile_shape = [128, 128, 64]
    d.warp_tile_shape = [128, 128, 64]
    d.tensorop = [128, 128, 16]
    d.num_stage = 3
    d.algo = "Blackwell"
    d.shuffle_type = ShuffleStrideType.NoShuffle
    d.element_per_access_a = d.element_per_access_b = d.element_per_access_c = 8
    with torch.cuda.stream(stream):
        p = GemmParams()
        p.algo_desp = d
        p.a, p.b = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
        p.c = torch.zeros((128, 128), dtype=torch.float16, device=dev)
        p.stream = stream.cuda_stream
        call = prepare_gemm(p)
        for _ in range(5):
            call.launch()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for _ in range(20):
                call.launch()
        ts = []
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            g.replay()
            e1.record(stream)
            stream.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / 20)
        got = p.c.cpu().numpy()
    t0 = time.perf_counter()
    n = 0
    while time.perf_counter() - t0 < 2.0:
        want = O.np_dense_gemm_tiled(a, b)
        n += 1
    cpu_us = (time.perf_counter() - t0) / n * 1e6
    err = float(np.abs(got.astype(np.float32) - want.astype(np.float32)).max())
    flop = 2 * 128 * 128 * 64
    return {"workload": "dense GEMM 128x128x64 fp16, fp32 accumulation, alpha 1 beta 0, seed 0",
            "gpu_us_per_call": float(np.median(ts)), "gpu_gflops": flop / float(np.median(ts)) / 1e3,
            "gpu_timing": "CUDA graph of 20 back-to-back calls, events around a replay, / 20 (launch-bound by construction)",
            "cpu_us_per_call": cpu_us, "cpu_gflops": flop / cpu_us / 1e3, "cpu_cores": 1,
            "cpu_kind": "single-core numpy tile loop restating the reference simulator's data flow (64x64x32 tiles); "
                        "the simulator itself is not importable without the reference's code generator",
            "max_abs_diff_gpu_vs_cpu": err}


def single_scene_configs(torch, dev, stream, reps=20, warm=3):
    """The 150 000-voxel single-scene configurations: fp16 C=K=128 forward / input gradient /
    weight gradient, each alone and the three side by side as one step; the 27-call
    gather-GEMM-scatter sequence at C=K=64; int8 stride-2 forward.  Launches rotate over
    buffer sets whose combined footprint exceeds the 126 MB L2, so every launch reads its
    inputs from HBM."""
    from cumm_b200 import _lib
    from cumm_b200 import workloads as W
    from cumm_b200.layer import DeviceTables, SparseConvLayer
    from cumm_b200.tensorview.gemm import ConvOpType
    res = {}
    coords = W.sample_coords(150000, 1)
    peak, _ = hbm_peak()
    NSETS = 4

    def time_graph(capture, per):
        """Median duration of one replay of the captured work, divided by `per`."""
        ts = []
        with torch.cuda.stream(stream):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                capture()
            g.replay()
            stream.synchronize()
            for i in range(reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                g.replay()
                b.record(stream)
                stream.synchronize()
                ts.append(a.elapsed_time(b) / per)
        return float(np.median(ts)) * 1e3  # us

    def time_calls(calls):
        """Average duration of one launch: the launches of one pass over the rotating sets
        are captured in a CUDA graph and replayed back to back, so the figure holds the
        kernel and the gap to the next kernel on the stream, not the host's launch path."""
        with torch.cuda.stream(stream):
            for i in range(warm * len(calls)):
                calls[i % len(calls)].launch()
            stream.synchronize()

        def capture():
            for c in calls:
                c.launch()
        return time_graph(capture, len(calls))

    layers, shared = [], []
    shares = {ConvOpType.Forward: SHARES[0], ConvOpType.BackwardInput: SHARES[1], ConvOpType.BackwardWeight: SHARES[2]}
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
            shared.append(SparseConvLayer(t, w, x, out, dout, din, dw, stream=stream.cuda_stream, cta_shares=shares))
    stream.synchronize()
    fb, wb = op_bytes(tb.n_out, (tb.n_out + 127) // 128)
    flops = 2 * tb.num_pairs * 128 * 128
    for name, calls, nbytes in (("fp16_forward", [L.fwd for L in layers], fb),
                                ("fp16_backward_input", [L.dgrad for L in layers], fb),
                                ("fp16_backward_weight", [L.wgrad for L in layers], wb)):
        us = time_calls(calls)
        warm_us = time_calls([calls[0]] * NSETS)  # one buffer set over and over: the 95 MB working set stays in L2
        res[name] = {"us": us, "eff_tflops": flops / us / 1e6, "gbs": nbytes / us / 1e3,
                     "frac_hbm_measured": nbytes / us / 1e3 / peak, "gvoxels_per_s": tb.n_out / us / 1e3,
                     "us_warm_l2": warm_us}
    # the whole layer step (forward + input gradient + weight gradient) as three branches
    s2, s3 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def step_branches(L):
        s2.wait_stream(stream)
        s3.wait_stream(stream)
        L.fwd.launch()
        with torch.cuda.stream(s3):
            L.wgrad.launch(s3.cuda_stream)
        with torch.cuda.stream(s2):
            L.dgrad.launch(s2.cuda_stream)
        stream.wait_stream(s2)
        stream.wait_stream(s3)

    with torch.cuda.stream(stream):
        for L in shared:
            step_branches(L)
        stream.synchronize()
    us = time_graph(lambda: [step_branches(L) for L in shared], NSETS)
    sb = 2 * fb + wb
    res["fp16_step_three_branches"] = {"us": us, "eff_tflops": 3 * flops / us / 1e6, "gbs": sb / us / 1e3,
                                       "frac_hbm_measured": sb / us / 1e3 / peak,
                                       "gvoxels_per_s": 3 * tb.n_out / us / 1e3,
                                       "what": f"forward, backward input and backward weight side by side (max_ctas "
                                               f"{SHARES[0]}/{SHARES[1]}/{SHARES[2]}), one graph of {NSETS} steps over "
                                               "rotating buffer sets, per step",
                                       "sequential_sum_us": sum(res[k]["us"] for k in ("fp16_forward", "fp16_backward_input",
                                                                                       "fp16_backward_weight"))}
    del layers, shared
    res["gather_gemm_27_calls_c64"] = config1_gather_gemm(torch, dev, stream, coords, time_calls, peak, NSETS)
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
                                   "frac_hbm_measured": b3 / us / 1e3 / peak, "gvoxels_per_s": tb3.n_out / us / 1e3,
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
        # the submanifold builder needs no synchronisation, so a pipeline can capture it: the same
        # launches replayed from a CUDA graph (the eager figure above is mostly launch latency)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            t = build_tables_gpu(cd, 1, W.GRID, stream=stream.cuda_stream)
        ts = []
        for i in range(6):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            g.replay()
            b.record(stream)
            stream.synchronize()
            if i:
                ts.append(a.elapsed_time(b) * 1e3)
        out["submanifold"]["us_as_cuda_graph"] = float(np.median(ts))
        out["submanifold"]["gbs_as_cuda_graph"] = out["submanifold"]["table_bytes"] / out["submanifold"]["us_as_cuda_graph"] / 1e3
    return out


def config1_gather_gemm(torch, dev, stream, coords, time_calls, peak, nsets):
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
    sequences, param_sets = [], []
    with torch.cuda.stream(stream):
        w = torch.from_numpy(wh).to(dev)
        idx_dev = [(f, torch.from_numpy(i).to(dev), torch.from_numpy(o).to(dev)) for f, i, o in pairs]
        for _ in range(nsets):
            x = torch.from_numpy(xh).to(dev)
            out = torch.zeros((tb.n_out, K), dtype=torch.float16, device=dev)
            calls, plist = [], []
            for f, i_idx, o_idx in idx_dev:
                p = GemmParams()
                p.algo_desp = d
                p.a, p.b, p.c = x, w[:, f, :], out
                p.a_inds, p.c_inds = i_idx, o_idx
                p.beta = 1.0
                p.stream = stream.cuda_stream
                calls.append(prepare_gemm(p))
                plist.append(p)
            sequences.append(calls)
            param_sets.append(plist)
    stream.synchronize()

    class Sequence:
        def __init__(self, calls):
            self.calls = calls

        def launch(self):
            for c in self.calls:
                c.launch()

    us = time_calls([Sequence(c) for c in sequences])
    nbytes = tb.n_in * C * 2 + tb.n_out * K * 2 + 27 * C * K * 2 + 8 * n_pairs
    res = {"us": us, "calls": len(pairs), "pairs": int(n_pairs), "eff_tflops": 2 * n_pairs * C * K / us / 1e6,
           "gbs": nbytes / us / 1e3, "frac_hbm_measured": nbytes / us / 1e3 / peak}
    # the same calls handed over as one layer (cb2_gemm_sequence_run): one launch over a neighbour
    # table scattered from the pair lists (built on the first launch, outside the timed replays)
    from cumm_b200.sequence import prepare_gemm_sequence
    with torch.cuda.stream(stream):
        one = [prepare_gemm_sequence(params, stream=stream.cuda_stream) for params in param_sets]
    stream.synchronize()
    us1 = time_calls(one)
    res["one_launch"] = {"us": us1, "eff_tflops": 2 * n_pairs * C * K / us1 / 1e6, "gbs": nbytes / us1 / 1e3,
                         "frac_hbm_measured": nbytes / us1 / 1e3 / peak,
                         "what": "the 27 GemmParams of the layer through cb2_gemm_sequence_run (tables reused)"}
    return res


if __name__ == "__main__":
    main()
