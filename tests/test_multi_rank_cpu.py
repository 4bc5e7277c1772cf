"""The N > 1 path on CPU: two gloo ranks shard the scenes, compute their share of the layer
with the oracle, and combine the weight-gradient partial sums with one all-reduce.  The
result must equal the single-process result over the whole batch (forward / input-gradient
rows concatenate, the weight gradient is the rank-ordered fp32 sum)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from cumm_b200 import workloads as W
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    grid = (6, 16, 16)
    n_scenes, per = 4, 4 // world
    ids = list(range(rank * per, (rank + 1) * per))
    tabs = [W.build_tables(W.sample_coords(400, [9, b], grid, batch=b), grid=grid) for b in ids]
    tb = W.concat_scenes(tabs) if len(tabs) > 1 else tabs[0]
    C, K = 16, 24
    rng = np.random.default_rng([9, 100])
    w = (rng.standard_normal((K, 27, C)) / 8).astype(np.float16)
    feats = [np.random.default_rng([9, 200, b]).standard_normal((400, C)).astype(np.float16) for b in ids]
    douts = [np.random.default_rng([9, 300, b]).standard_normal((400, K)).astype(np.float16) for b in ids]
    x, dout = np.concatenate(feats), np.concatenate(douts)
    mo = np.zeros((tb.n_out + 127) // 128, np.uint32)
    out = O.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort, mask_out=mo)
    din = O.mask_igemm(dout, w, np.zeros((tb.n_in, C), np.float16), tb.indices_bwd, tb.mask_bwd,
                       tb.mask_argsort_bwd, is_dgrad=True)
    dw32 = O.mask_igemm_wgrad(dout, x, None, tb.indices, mo, tb.mask_argsort,
                              out_f32=np.zeros((K, 27, C), np.float32))
    t = torch.from_numpy(dw32)
    dist.all_reduce(t)  # the one exchange step of the path
    np.savez(Path(tmp) / f"rank{rank}.npz", out=out, din=din, dw=t.numpy().astype(np.float16), pairs=tb.num_pairs)
    dist.destroy_process_group()


def test_two_ranks_match_single_process(tmp_path, oracle):
    import torch.multiprocessing as mp
    from cumm_b200 import workloads as W
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    # single process over all four scenes
    grid = (6, 16, 16)
    tabs = [W.build_tables(W.sample_coords(400, [9, b], grid, batch=b), grid=grid) for b in range(4)]
    tb = W.concat_scenes(tabs)
    C, K = 16, 24
    w = (np.random.default_rng([9, 100]).standard_normal((K, 27, C)) / 8).astype(np.float16)
    x = np.concatenate([np.random.default_rng([9, 200, b]).standard_normal((400, C)).astype(np.float16) for b in range(4)])
    dout = np.concatenate([np.random.default_rng([9, 300, b]).standard_normal((400, K)).astype(np.float16) for b in range(4)])
    mo = np.zeros((tb.n_out + 127) // 128, np.uint32)
    out = oracle.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort, mask_out=mo)
    din = oracle.mask_igemm(dout, w, np.zeros((tb.n_in, C), np.float16), tb.indices_bwd, tb.mask_bwd,
                            tb.mask_argsort_bwd, is_dgrad=True)
    dw = oracle.np_wgrad(dout, x, tb.indices)
    assert sum(int(p["pairs"]) for p in parts) == tb.num_pairs
    # rows are owned by exactly one rank: concatenation is exact up to fp32 summation order
    np.testing.assert_allclose(np.concatenate([p["out"] for p in parts]).astype(np.float32), out.astype(np.float32),
                               rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(np.concatenate([p["din"] for p in parts]).astype(np.float32), din.astype(np.float32),
                               rtol=2e-3, atol=2e-3)
    for p in parts:  # every rank holds the same reduced gradient
        np.testing.assert_allclose(p["dw"].astype(np.float32), dw, rtol=1e-2, atol=1e-2)
    assert (parts[0]["dw"] == parts[1]["dw"]).all()
