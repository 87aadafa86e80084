"""Tensor handle wrapper (reference: python/llaisys/tensor.py:14-97)."""
from __future__ import annotations

from ctypes import c_size_t, c_ssize_t
from typing import Sequence, Tuple

from .libllaisys import LIB_LLAISYS, DataType, DeviceType


class Tensor:
    def __init__(self, shape: Sequence[int] | None = None, dtype: DataType = DataType.F32,
                 device: DeviceType = DeviceType.CPU, device_id: int = 0, tensor=None):
        if tensor:
            self._tensor = tensor
            return
        dims = tuple(shape) if shape is not None else ()
        arr = (c_size_t * len(dims))(*dims) if dims else None
        self._tensor = LIB_LLAISYS.tensorCreate(arr, len(dims), int(dtype), int(device), int(device_id))

    def __del__(self):
        handle = getattr(self, "_tensor", None)
        if handle is not None:
            LIB_LLAISYS.tensorDestroy(handle)
            self._tensor = None

    def ndim(self) -> int:
        return int(LIB_LLAISYS.tensorGetNdim(self._tensor))

    def shape(self) -> Tuple[int, ...]:
        buf = (c_size_t * self.ndim())()
        LIB_LLAISYS.tensorGetShape(self._tensor, buf)
        return tuple(buf)

    def strides(self) -> Tuple[int, ...]:
        buf = (c_ssize_t * self.ndim())()
        LIB_LLAISYS.tensorGetStrides(self._tensor, buf)
        return tuple(buf)

    def dtype(self) -> DataType:
        return DataType(LIB_LLAISYS.tensorGetDataType(self._tensor))

    def device_type(self) -> DeviceType:
        return DeviceType(LIB_LLAISYS.tensorGetDeviceType(self._tensor))

    def device_id(self) -> int:
        return int(LIB_LLAISYS.tensorGetDeviceId(self._tensor))

    def data_ptr(self) -> int:
        return LIB_LLAISYS.tensorGetData(self._tensor)

    def lib_tensor(self):
        return self._tensor

    def debug(self) -> None:
        LIB_LLAISYS.tensorDebug(self._tensor)

    def __repr__(self) -> str:
        return (f"<Tensor shape={self.shape()}, dtype={self.dtype().name}, "
                f"device={self.device_type().name}:{self.device_id()}>")

    def load(self, data) -> None:
        """Copies from host memory at `data` (an address or an object with data_ptr())."""
        if hasattr(data, "data_ptr"):
            data = data.data_ptr()
        LIB_LLAISYS.tensorLoad(self._tensor, data)

    def is_contiguous(self) -> bool:
        return bool(LIB_LLAISYS.tensorIsContiguous(self._tensor))

    def view(self, *shape: int) -> "Tensor":
        arr = (c_size_t * len(shape))(*shape)
        return Tensor(tensor=LIB_LLAISYS.tensorView(self._tensor, arr, len(shape)))

    def permute(self, *perm: int) -> "Tensor":
        assert len(perm) == self.ndim()
        arr = (c_size_t * len(perm))(*perm)
        return Tensor(tensor=LIB_LLAISYS.tensorPermute(self._tensor, arr))

    def slice(self, dim: int, start: int, end: int) -> "Tensor":
        return Tensor(tensor=LIB_LLAISYS.tensorSlice(self._tensor, dim, start, end))
