"""Sum of one fp32 tensor per GPU through NVLink peer memory (``cb2_peer_allreduce``): the one
exchange step of the row-sharded convolution, the weight-gradient partial sums (reduce-scatter
then all-gather by plain peer stores, every element summed once in GPU order).

One process per GPU.  The buffers come from ``torch.distributed._symmetric_memory`` (plumbing:
it allocates memory every GPU of the node can map and exchanges the handles); the data
movement and the reduction are this package's own kernel."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

from . import _lib


class PeerAllReduce:
    """``__call__(src_f32, out_f16=None, out_f32=None, stream=0)`` enqueues one sum; every rank
    must make the same sequence of calls with tensors of the ``numel`` given here.  A call can be
    captured in a CUDA graph: the call number that pairs the ranks' calls lives in the buffers."""

    def __init__(self, numel: int, rank: int, world: int, peer_ptrs: Sequence[int], keep=None,
                 timeout_ns: int = 0, own_sm_smem_bytes: int = 0):
        if numel % 4:
            raise ValueError("numel must be a multiple of 4")
        self.numel, self.rank, self.world = int(numel), int(rank), int(world)
        self._ptrs = (ctypes.c_void_p * world)(*[int(p) for p in peer_ptrs])
        self._keep = keep
        self._timeout_ns = int(timeout_ns)
        # see cb2_peer_allreduce_args.own_sm_smem_bytes: keeps the kernel's CTAs off SMs that
        # persistent convolution kernels occupy
        self.own_sm_smem_bytes = int(own_sm_smem_bytes)
        self._L = _lib.load()

    @staticmethod
    def buffer_bytes(numel: int, world: int) -> int:
        n = _lib.load().cb2_peer_allreduce_buffer_size(int(numel), int(world))
        if n == 0:
            raise ValueError(f"bad numel / world ({numel}, {world})")
        return int(n)

    @classmethod
    def over_process_group(cls, numel: int, device, group=None, timeout_ns: int = 0) -> "PeerAllReduce":
        """Allocates and maps the buffers of all ranks of ``group`` (default: the world)."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        nbytes = cls.buffer_bytes(numel, world)
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # nobody pushes before every buffer is zero
        return cls(numel, rank, world, [int(p) for p in hdl.buffer_ptrs], keep=(buf, hdl), timeout_ns=timeout_ns)

    def __call__(self, src_f32, out_f16=None, out_f32=None, stream: int = 0) -> None:
        if src_f32.numel() != self.numel:
            raise ValueError("source size differs from the size this object was made for")
        a = _lib.PeerAllreduceArgs()
        a.peer_buffers = ctypes.cast(self._ptrs, ctypes.POINTER(ctypes.c_void_p))
        a.rank, a.world = self.rank, self.world
        a.src = src_f32.data_ptr()
        a.out_f32 = out_f32.data_ptr() if out_f32 is not None else None
        a.out_f16 = out_f16.data_ptr() if out_f16 is not None else None
        a.numel, a.timeout_ns = self.numel, self._timeout_ns
        a.own_sm_smem_bytes = self.own_sm_smem_bytes
        _lib.raise_for(self._L.cb2_peer_allreduce(ctypes.byref(a), ctypes.c_void_p(int(stream))))

    def last_call_ns(self):
        """Global-timer readings of the last call on this rank, relative to its start: when its
        shards had been sent, when every rank's shard had arrived, when its own shard was summed
        and sent out, when every rank's sums had arrived, when it finished (synchronises)."""
        import torch
        buf = self._keep[0] if isinstance(self._keep, tuple) else self._keep
        torch.cuda.synchronize(buf.device)
        st = buf[2560:2560 + 48].view(torch.int64).cpu().tolist()
        return {"scattered": st[1] - st[0], "shards_seen": st[2] - st[0], "reduced": st[3] - st[0],
                "results_seen": st[4] - st[0], "done": st[5] - st[0]}
