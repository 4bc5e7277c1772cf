"""The peer-memory sum on one GPU: a world of one (push to itself, flag, reduce), and a wait
that runs out (a flag that nothing sets) reported through the status word.  Worlds of several
GPUs are exercised by ``bench.py --gpus N``."""
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
    for call in range(3):  # both parities, flags only grow
        src = torch.randn(numel, device="cuda") * (call + 1)
        o16 = torch.zeros(numel, dtype=torch.float16, device="cuda")
        o32 = torch.zeros(numel, dtype=torch.float32, device="cuda")
        ar(src, o16, o32)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        assert torch.equal(o32, src)
        assert torch.equal(o16, src.to(torch.float16))


def test_a_flag_that_nothing_sets_times_out(cuda_lib):
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
