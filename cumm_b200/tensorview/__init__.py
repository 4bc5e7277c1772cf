"""Minimal tensor plumbing behind the operator surface.

The reference's operators take ``tv::Tensor`` (include/tensorview/tensor.h:181); here the
callers' tensors are ``torch.Tensor`` on a CUDA device, or a non-owning :class:`Tensor`
made by :func:`from_blob` (the reference's ``tv.from_blob``, cumm/tensorview_bind.py:752-763).
Only what the GEMM / sparse-conv parameter records need is provided: data pointer, shape,
strides (in elements), dtype code and device.

dtype codes are the reference's ``tv::DType`` values (include/tensorview/dtypes.h:39-55).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

float32 = 0
int32 = 1
int16 = 2
int8 = 3
float64 = 4
bool_ = 5
uint8 = 6
float16 = 7
int64 = 8
uint16 = 9
uint32 = 10
uint64 = 11
bfloat16 = 12
tf32 = 13
unknown = -1

_ITEMSIZE = {float32: 4, int32: 4, int16: 2, int8: 1, float64: 8, bool_: 1, uint8: 1, float16: 2,
             int64: 8, uint16: 2, uint32: 4, uint64: 8, bfloat16: 2, tf32: 4}

# short names used in algorithm-name strings (tv::dtype_short_str, include/tensorview/dtypes.h)
_SHORT = {float32: "f32", int32: "s32", int16: "s16", int8: "s8", float64: "f64", bool_: "b1",
          uint8: "u8", float16: "f16", int64: "s64", uint16: "u16", uint32: "u32", uint64: "u64",
          bfloat16: "bf16", tf32: "tf32"}


def dtype_short_str(code: int) -> str:
    return _SHORT.get(int(code), "unk")


def itemsize(code: int) -> int:
    return _ITEMSIZE[int(code)]


def _torch_dtype_code(dt) -> int:
    import torch
    table = {torch.float32: float32, torch.int32: int32, torch.int16: int16, torch.int8: int8,
             torch.float64: float64, torch.bool: bool_, torch.uint8: uint8, torch.float16: float16,
             torch.int64: int64, torch.bfloat16: bfloat16}
    for name, code in (("uint16", uint16), ("uint32", uint32), ("uint64", uint64)):
        if hasattr(torch, name):
            table[getattr(torch, name)] = code
    return table[dt]


class Tensor:
    """Non-owning view of device memory (the callee never frees caller memory)."""

    def __init__(self, ptr: int, shape: Sequence[int], dtype: int, device: int = 0,
                 stride: Optional[Sequence[int]] = None, keepalive=None):
        self._ptr = int(ptr)
        self.shape: List[int] = [int(s) for s in shape]
        self.dtype = int(dtype)
        self.device = int(device)
        if stride is None:
            stride = []
            acc = 1
            for s in reversed(self.shape):
                stride.append(acc)
                acc *= s
            stride = list(reversed(stride))
        self.stride_ = [int(s) for s in stride]
        self._keepalive = keepalive

    # -- the subset of tv::Tensor's interface the parameter records use
    def data_ptr(self) -> int:
        return self._ptr

    def byte_pointer(self) -> int:
        return self._ptr

    def empty(self) -> bool:
        return self._ptr == 0 or any(s == 0 for s in self.shape) and len(self.shape) > 0 and self._ptr == 0

    def dim(self, i: int) -> int:
        return self.shape[i]

    def stride(self, i: int) -> int:
        return self.stride_[i]

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def nbytes(self) -> int:
        return self.size() * itemsize(self.dtype)

    def view(self, shape: Sequence[int]) -> "Tensor":
        shape = list(shape)
        if -1 in shape:
            known = 1
            for s in shape:
                if s != -1:
                    known *= s
            shape[shape.index(-1)] = self.size() // max(known, 1)
        return Tensor(self._ptr, shape, self.dtype, self.device, keepalive=self._keepalive)

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={dtype_short_str(self.dtype)}, device={self.device})"


def from_blob(ptr: int, shape: Sequence[int], dtype: int, device: int = 0,
              stride: Optional[Sequence[int]] = None) -> Tensor:
    return Tensor(ptr, shape, dtype, device, stride)


def as_view(t) -> Optional[Tensor]:
    """Normalise a torch tensor / Tensor / None to a :class:`Tensor` (None when empty)."""
    if t is None:
        return None
    if isinstance(t, Tensor):
        return None if t._ptr == 0 else t
    # torch tensor
    if t.numel() == 0 and t.dim() <= 1:
        return None
    if not t.is_cuda:
        raise RuntimeError("tensors must live on a CUDA device (there is no CPU path)")
    return Tensor(t.data_ptr(), list(t.shape), _torch_dtype_code(t.dtype), t.device.index or 0,
                  list(t.stride()), keepalive=t)


class CUDAKernelTimer:
    """Named CUDA-event pairs with a namespace stack: the per-call ``timer`` of ``GemmParams`` /
    ``ConvParams`` (tv::CUDAKernelTimer, include/tensorview/profile/cuda_profiler.h:225-405).  When
    a call's params carry an enabled timer, the launch is bracketed by one event pair on the
    call's stream, filed under the kernel's algorithm name, as the reference's
    ``CUDAKernelTimerGuard`` does (cuda_profiler.h:408-440; cumm/conv/main.py:708).  Durations
    are in milliseconds.  A name can be recorded once: use a fresh timer (or ``push`` another
    namespace) for a second call of the same kernel."""

    def __init__(self, enable: bool = True):
        self.enable = bool(enable)
        self._ns: List[str] = []
        self._events = {}
        self._pairs = {}

    def push(self, name: str) -> None:
        if self.enable:
            self._ns.append(name)

    def pop(self) -> None:
        if self.enable:
            if not self._ns:
                raise RuntimeError("you pop value from empty namespaces")
            self._ns.pop()

    def _unique(self, name: str) -> str:
        cur = ".".join(self._ns)
        if not name:
            return cur
        return f"{cur}.{name}" if cur else name

    def record(self, name: str, stream: int = 0) -> None:
        if not self.enable:
            return
        import torch
        unique = self._unique(name)
        if unique in self._events:
            raise RuntimeError(f"your name {unique} already exists")
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.ExternalStream(int(stream)) if stream else torch.cuda.current_stream())
        self._events[unique] = ev

    def insert_pair(self, name: str, start: str, stop: str) -> str:
        if not self.enable:
            return ""
        name, start, stop = self._unique(name), self._unique(start), self._unique(stop)
        if name in self._pairs:
            raise RuntimeError(f"your name {name} already exists")
        self._pairs[name] = (start, stop)
        return name

    def has_pair(self, name: str) -> bool:
        return self._unique(name) in self._pairs

    def sync_all_event(self) -> None:
        for ev in self._events.values():
            ev.synchronize()

    def get_pair_duration(self, name: str) -> float:
        if name not in self._pairs:
            raise RuntimeError(f"can't find your pair {name}")
        a, b = (self._events[k] for k in self._pairs[name])
        a.synchronize()
        b.synchronize()
        return float(a.elapsed_time(b))

    def get_all_pair_time(self):
        self.sync_all_event()
        return {k: float(self._events[a].elapsed_time(self._events[b])) for k, (a, b) in self._pairs.items()}

    get_all_pair_duration = get_all_pair_time


class _TimerGuard:
    """``with _TimerGuard(name, timer, stream):`` -- tv::CUDAKernelTimerGuard."""

    def __init__(self, name: str, timer: Optional[CUDAKernelTimer], stream: int = 0):
        self.name, self.timer, self.stream = name, timer, stream
        self.active = timer is not None and getattr(timer, "enable", False)

    def __enter__(self):
        if self.active:
            if self.name:
                self.timer.push(self.name)
            self.pair = self.timer.insert_pair("", "start", "stop")
            self.timer.record("start", self.stream)
        return self

    def __exit__(self, *exc):
        if self.active:
            self.timer.record("stop", self.stream)
            if self.name:
                self.timer.pop()
        return False
