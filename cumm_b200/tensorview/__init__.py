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
