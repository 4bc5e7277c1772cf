"""The peer-memory sum on one GPU: a world of one (scatter to itself, reduce, gather), and a wait
that runs out (data that nothing sends) reported through the status word; and, where the box
has two GPUs, a world of two processes checked against the rank-ordered sum (``bench.py --gpus N``
makes the same check at every N before it times anything)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_world_of_one_sums_and_casts(cuda_lib):
    import torch
    from cumm_b200 import _lib
    from cumm_b200.peer_allreduce import PeerAllReduce
    numel = 128 * 27 * 128
    buf = torch.zeros(PeerAllReduce.buffer_bytes(numel, 1), dtype=torch.uint8, device="cuda")
    ar = PeerAllReduce(numel, 0, 1, [buf.data_ptr()], keep=buf)
    for call in range(3):  # both parities, the call number only grows
        src = torch.randn(numel, device="cuda") * (call + 1)
        o16 = torch.zeros(numel, dtype=torch.float16, device="cuda")
        o32 = torch.zeros(numel, dtype=torch.float32, device="cuda")
        ar(src, o16, o32)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        assert torch.equal(o32, src)
        assert torch.equal(o16, src.to(torch.float16))


def test_data_that_nothing_sends_times_out(cuda_lib):
    import torch
    from cumm_b200 import _lib
    from cumm_b200.peer_allreduce import PeerAllReduce
    numel = 4096
    n = PeerAllReduce.buffer_bytes(numel, 2)
    own = torch.zeros(n, dtype=torch.uint8, device="cuda")
    other = torch.zeros(n, dtype=torch.uint8, device="cuda")  # stands for a GPU that never answers
    ar = PeerAllReduce(numel, 0, 2, [own.data_ptr(), other.data_ptr()], keep=(own, other), timeout_ns=20_000_000)
    src = torch.ones(numel, device="cuda")
    o32 = torch.full((numel,), 7.0, device="cuda")
    ar(src, None, o32)
    torch.cuda.synchronize()
    assert _lib.device_status() == 1, "the wait must give up and say so"
    assert _lib.device_status() == 0
    assert (o32 == 7.0).all(), "outputs stay untouched when the sum did not happen"
    # the context is still usable
    assert float((src + 1).sum()) == 2.0 * numel


def test_bad_arguments(cuda_lib):
    import torch
    from cumm_b200.peer_allreduce import PeerAllReduce
    with pytest.raises(ValueError):
        PeerAllReduce.buffer_bytes(0, 2)
    with pytest.raises(ValueError):
        PeerAllReduce(10, 0, 1, [256])
    buf = torch.zeros(PeerAllReduce.buffer_bytes(16, 1), dtype=torch.uint8, device="cuda")
    ar = PeerAllReduce(16, 0, 1, [buf.data_ptr()], keep=buf)
    with pytest.raises(RuntimeError, match="must not empty"):
        ar(torch.zeros(16, device="cuda"))


def _two_gpu_worker(rank, world, port, numel, result_path):
    import os
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from cumm_b200 import _lib
    from cumm_b200.peer_allreduce import PeerAllReduce
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = True
    try:
        ar = PeerAllReduce.over_process_group(numel, dev)
        for call in range(4):  # both parities of the buffers, twice
            g = torch.Generator(device=dev)
            g.manual_seed(100 * call + rank)
            src = torch.randn(numel, generator=g, device=dev) * (1.0 + 3.0 * rank)
            o16 = torch.zeros(numel, dtype=torch.float16, device=dev)
            o32 = torch.zeros(numel, dtype=torch.float32, device=dev)
            ar(src, o16, o32)
            torch.cuda.synchronize()
            parts = [torch.empty_like(src) for _ in range(world)]
            dist.all_gather(parts, src)
            want = parts[0].clone()
            for r in range(1, world):
                want += parts[r]  # the kernel's order: GPU 0 first
            ok = ok and _lib.device_status() == 0
            ok = ok and bool(torch.equal(o32.view(torch.int32), want.view(torch.int32)))
            ok = ok and bool(torch.equal(o16.view(torch.int16), want.to(torch.float16).view(torch.int16)))
    finally:
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            Path(result_path).write_text("ok" if int(flag[0]) == 1 else "mismatch")
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("numel", [128 * 27 * 128, 4 * 1031])
def test_two_gpus_sum_matches_rank_ordered_sum(cuda_lib, tmp_path, numel):
    """Two processes, one GPU each: every call's result equals the fp32 sum taken in GPU order,
    bit for bit, as fp32 and as fp16, on both GPUs (an odd shard size included)."""
    import socket
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "result.txt"
    mp.spawn(_two_gpu_worker, args=(2, port, numel, str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"
