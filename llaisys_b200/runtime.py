"""Device runtime table as a Python object (reference: python/llaisys/runtime.py:6-68)."""
from __future__ import annotations

from . import libllaisys as _l
from .libllaisys import LIB_LLAISYS


def _addr(p) -> int | None:
    """Accepts an int address, a ctypes pointer, or anything with data_ptr() (Tensor, torch.Tensor)."""
    if p is None:
        return None
    if hasattr(p, "data_ptr"):
        p = p.data_ptr()
    if hasattr(p, "value"):
        p = p.value
    return int(p) if p is not None else None


class RuntimeAPI:
    def __init__(self, device_type: _l.DeviceType):
        self._api = LIB_LLAISYS.llaisysGetRuntimeAPI(_l.llaisysDeviceType_t(device_type))

    def get_device_count(self) -> int:
        return self._api.contents.get_device_count()

    def set_device(self, device_id: int) -> None:
        self._api.contents.set_device(device_id)

    def device_synchronize(self) -> None:
        self._api.contents.device_synchronize()

    def create_stream(self):
        return self._api.contents.create_stream()

    def destroy_stream(self, stream) -> None:
        self._api.contents.destroy_stream(stream)

    def stream_synchronize(self, stream) -> None:
        self._api.contents.stream_synchronize(stream)

    def malloc_device(self, size: int):
        return self._api.contents.malloc_device(size)

    def free_device(self, ptr) -> None:
        self._api.contents.free_device(ptr)

    def malloc_host(self, size: int):
        return self._api.contents.malloc_host(size)

    def free_host(self, ptr) -> None:
        self._api.contents.free_host(ptr)

    def memcpy_sync(self, dst, src, size: int, kind: _l.MemcpyKind) -> None:
        self._api.contents.memcpy_sync(_addr(dst), _addr(src), size, _l.llaisysMemcpyKind_t(kind))

    def memcpy_async(self, dst, src, size: int, kind: _l.MemcpyKind, stream) -> None:
        self._api.contents.memcpy_async(_addr(dst), _addr(src), size, _l.llaisysMemcpyKind_t(kind), stream)


def set_context_runtime(device_type: _l.DeviceType, device_id: int = 0) -> None:
    """Makes (device_type, device_id) current for the calling thread."""
    LIB_LLAISYS.llaisysSetContextRuntime(_l.llaisysDeviceType_t(device_type), device_id)


def context_stream() -> int | None:
    """Address of the stream the calling thread's current runtime queues operators on (None on CPU)."""
    return LIB_LLAISYS.llaisysGetContextStream()
