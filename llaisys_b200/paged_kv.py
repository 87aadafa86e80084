"""Paged KV cache: block manager plus append / gather / attention over pages.

Thin wrapper over the status-returning entry points of include/llaisys/paged_kv.h; a non-zero status
becomes a LlaisysError carrying the code and the library's message. Bulk arguments (q, out, k_rows, ...)
may be llaisys Tensors, torch tensors, or raw addresses -- anything with data_ptr() -- in the cache's device
memory; index arguments are Python sequences or numpy int32 arrays on the host.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int32
from enum import IntEnum
from typing import Sequence

import numpy as np

from .libllaisys import LIB_LLAISYS, DataType, DeviceType, Status, llaisysPagedKV_t
from .runtime import _addr

_I32P = ctypes.POINTER(c_int32)


class Kernel(IntEnum):
    """LLAISYS_KERNEL_* of include/llaisys/paged_kv.h: the kernel that served an attention call."""
    NONE = 0
    CPU = 1
    GENERIC = 2
    DECODE_TMA = 3
    DECODE_TMA_FUSED = 4
    DECODE_CP_ASYNC = 5
    PREFILL_TC = 6


def last_attention_kernel() -> Kernel:
    """Kernel of the calling thread's most recent attention call (any cache, or Ops.self_attention)."""
    return Kernel(LIB_LLAISYS.llaisysLastAttentionKernel())


class LlaisysError(RuntimeError):
    def __init__(self, status: int, message: str):
        self.status = Status(status)
        super().__init__(f"{self.status.name}: {message}")


def _check(status: int) -> None:
    if status != 0:
        raise LlaisysError(status, LIB_LLAISYS.llaisysGetLastError().decode())


def _i32(values) -> tuple[np.ndarray, ctypes.Array]:
    arr = np.ascontiguousarray(values, dtype=np.int32)
    return arr, arr.ctypes.data_as(_I32P)


def _i32_address(values) -> tuple[np.ndarray, int]:
    """The same for the per-step call, where the few microseconds of building a ctypes pointer object count: the
    array (kept alive by the caller's frame) and its address as a plain integer."""
    arr = values if (type(values) is np.ndarray and values.dtype == np.int32 and values.flags.c_contiguous) else \
        np.ascontiguousarray(values, dtype=np.int32)
    return arr, arr.__array_interface__["data"][0]


class PagedKVCache:
    """Fixed pool of pages with a free list and per-sequence block tables.

    Pool layout: pool[layer][page][K|V][nkvh][page_size][head_dim]. Token `pos` of a sequence lives in page
    table[seq][pos // page_size], slot pos % page_size.
    """

    def __init__(self, num_pages: int, nkvh: int, head_dim: int, *, page_size: int = 16, nlayer: int = 1,
                 dtype: DataType = DataType.BF16, device: DeviceType = DeviceType.CPU, device_id: int = 0,
                 max_seqs: int = 256, max_pages_per_seq: int | None = None):
        self.num_pages, self.nkvh, self.head_dim = num_pages, nkvh, head_dim
        self.page_size, self.nlayer, self.dtype = page_size, nlayer, DataType(dtype)
        self.device, self.device_id = DeviceType(device), device_id
        self.max_seqs = max_seqs
        self.max_pages_per_seq = max_pages_per_seq if max_pages_per_seq is not None else num_pages
        handle = llaisysPagedKV_t()
        self._kv = None
        _check(LIB_LLAISYS.llaisysPagedKVCreate(byref(handle), int(device), device_id, int(dtype), nlayer, num_pages,
                                                page_size, nkvh, head_dim, max_seqs, self.max_pages_per_seq))
        self._kv = handle

    def close(self) -> None:
        if self._kv is not None:
            LIB_LLAISYS.llaisysPagedKVDestroy(self._kv)
            self._kv = None

    def __del__(self):
        self.close()

    # ---- block manager ----
    def add_seq(self) -> int:
        seq = c_int32(-1)
        _check(LIB_LLAISYS.llaisysPagedKVSeqAdd(self._kv, byref(seq)))
        return seq.value

    def reserve(self, seq: int, n_tokens: int) -> None:
        _check(LIB_LLAISYS.llaisysPagedKVSeqReserve(self._kv, seq, n_tokens))

    def assign_pages(self, seq: int, pages: Sequence[int]) -> None:
        arr, ptr = _i32(pages)
        _check(LIB_LLAISYS.llaisysPagedKVSeqAssignPages(self._kv, seq, ptr, arr.size))

    def free_seq(self, seq: int) -> None:
        _check(LIB_LLAISYS.llaisysPagedKVSeqFree(self._kv, seq))

    # ---- prefix sharing ----

    def publish(self, seq: int, tokens: Sequence[int]) -> None:
        """Makes the sequence's full pages findable under the ids of the tokens they hold."""
        arr = np.ascontiguousarray(tokens, dtype=np.int64)
        _check(LIB_LLAISYS.llaisysPagedKVSeqPublish(self._kv, seq, arr.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                                                    arr.size))

    def match_prefix(self, seq: int, tokens: Sequence[int]) -> int:
        """Attaches published pages matching the longest whole-page prefix of `tokens` to the empty sequence `seq`;
        -> tokens covered."""
        arr = np.ascontiguousarray(tokens, dtype=np.int64)
        matched = ctypes.c_size_t(0)
        _check(LIB_LLAISYS.llaisysPagedKVSeqMatchPrefix(self._kv, seq, arr.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                                                        arr.size, ctypes.byref(matched)))
        return int(matched.value)

    def fork(self, parent: int, n_tokens: int) -> int:
        """New sequence sharing the parent's first n_tokens (whole pages by reference, a partial last page copied)."""
        child = ctypes.c_int32(-1)
        _check(LIB_LLAISYS.llaisysPagedKVSeqFork(self._kv, parent, n_tokens, ctypes.byref(child)))
        return child.value

    def page_ref_count(self, page: int) -> int:
        return int(LIB_LLAISYS.llaisysPagedKVPageRefCount(self._kv, page))

    def num_cached_pages(self) -> int:
        return int(LIB_LLAISYS.llaisysPagedKVNumCachedPages(self._kv))

    def num_free_pages(self) -> int:
        return int(LIB_LLAISYS.llaisysPagedKVNumFreePages(self._kv))

    def num_seqs(self) -> int:
        return int(LIB_LLAISYS.llaisysPagedKVNumSeqs(self._kv))

    def seq_num_pages(self, seq: int) -> int:
        return int(LIB_LLAISYS.llaisysPagedKVSeqNumPages(self._kv, seq))

    def seq_pages(self, seq: int) -> list[int]:
        n = self.seq_num_pages(seq)
        if n < 0:
            raise LlaisysError(Status.NO_SEQ, f"sequence {seq} does not exist")
        buf = (c_int32 * max(n, 1))()
        _check(LIB_LLAISYS.llaisysPagedKVSeqPages(self._kv, seq, buf, n))
        return list(buf[:n])

    # ---- device views ----
    def pool_ptr(self, layer: int = 0) -> int:
        return LIB_LLAISYS.llaisysPagedKVPoolData(self._kv, layer)

    def layer_bytes(self) -> int:
        return int(LIB_LLAISYS.llaisysPagedKVLayerBytes(self._kv))

    def block_table_ptr(self) -> int:
        return LIB_LLAISYS.llaisysPagedKVBlockTableData(self._kv)

    def set_launch_overlap(self, enable: bool) -> None:
        """Opt in to programmatic dependent launch of append / decode (see llaisysPagedKVSetLaunchOverlap)."""
        _check(LIB_LLAISYS.llaisysPagedKVSetLaunchOverlap(self._kv, 1 if enable else 0))

    def last_kernel(self) -> "Kernel":
        """Which kernel served this cache's most recent attention call."""
        return Kernel(LIB_LLAISYS.llaisysPagedKVLastKernel(self._kv))

    def flush(self) -> None:
        _check(LIB_LLAISYS.llaisysPagedKVFlush(self._kv))

    def check(self) -> None:
        """Synchronises and raises LlaisysError(KERNEL) if a kernel skipped out-of-range metadata."""
        _check(LIB_LLAISYS.llaisysPagedKVCheck(self._kv))

    # ---- data path: host index arrays ----
    def append(self, layer: int, k_rows, v_rows, seq_ids, positions) -> None:
        s, sp = _i32(seq_ids)
        p, pp = _i32(positions)
        if s.size != p.size:
            raise ValueError("seq_ids and positions must have the same length")
        _check(LIB_LLAISYS.llaisysPagedKVAppend(self._kv, layer, _addr(k_rows), _addr(v_rows), sp, pp, s.size))

    def gather(self, layer: int, seq: int, n_tokens: int, k_out, v_out) -> None:
        _check(LIB_LLAISYS.llaisysPagedKVGather(self._kv, layer, seq, n_tokens, _addr(k_out), _addr(v_out)))

    def decode(self, layer: int, out, q, seq_ids, kv_lens, nh: int, scale: float) -> None:
        s, sp = _i32(seq_ids)
        l, lp = _i32(kv_lens)
        if s.size != l.size:
            raise ValueError("seq_ids and kv_lens must have the same length")
        _check(LIB_LLAISYS.llaisysPagedAttentionDecode(self._kv, layer, _addr(out), _addr(q), sp, lp, s.size, nh,
                                                       scale))

    def decode_step_host(self, layer: int, out, q, k_new, v_new, seq_ids, kv_lens, nh: int, scale: float) -> None:
        """One decode step from host buffers, synchronous: k_new[i] / v_new[i] become token kv_lens[i] - 1 of sequence
        seq_ids[i], then out[i] = attention of q[i] over kv_lens[i] tokens. out, q, k_new, v_new are HOST tensors
        (pinned ones copy asynchronously); seq_ids / kv_lens may be int32 numpy arrays (used as they are) or lists."""
        s, sp = _i32_address(seq_ids)
        l, lp = _i32_address(kv_lens)
        if s.size != l.size:
            raise ValueError("seq_ids and kv_lens must have the same length")
        _check(LIB_LLAISYS.llaisysPagedDecodeStepHost(self._kv, layer, _addr(out), _addr(q), _addr(k_new), _addr(v_new),
                                                      sp, lp, s.size, nh, scale))

    def decode_partial(self, layer: int, part, q, seq_ids, kv_lens, nh: int, scale: float) -> None:
        s, sp = _i32(seq_ids)
        l, lp = _i32(kv_lens)
        if s.size != l.size:
            raise ValueError("seq_ids and kv_lens must have the same length")
        _check(LIB_LLAISYS.llaisysPagedAttentionDecodePartial(self._kv, layer, _addr(part), _addr(q), sp, lp, s.size,
                                                              nh, scale))

    def prefill(self, layer: int, out, q, seq_ids, q_lens, kv_lens, nh: int, scale: float) -> None:
        s, sp = _i32(seq_ids)
        ql, qlp = _i32(q_lens)
        l, lp = _i32(kv_lens)
        if not (s.size == ql.size == l.size):
            raise ValueError("seq_ids, q_lens and kv_lens must have the same length")
        _check(LIB_LLAISYS.llaisysPagedAttentionPrefill(self._kv, layer, _addr(out), _addr(q), sp, qlp, lp, s.size,
                                                        nh, scale))

    # ---- data path: device index arrays, explicit stream ----
    def append_dev(self, layer: int, k_rows, v_rows, seq_ids_dev, positions_dev, n_rows: int, stream) -> None:
        _check(LIB_LLAISYS.llaisysPagedKVAppendDev(self._kv, layer, _addr(k_rows), _addr(v_rows), _addr(seq_ids_dev),
                                                   _addr(positions_dev), n_rows, stream))

    def rope_append_dev(self, layer: int, q_out, qkv, bias, seq_ids_dev, positions_dev, n_rows: int, nh: int,
                        theta: float, stream) -> None:
        """Bias + rotary embedding + append over a packed q|k|v projection (device index arrays, explicit stream)."""
        _check(LIB_LLAISYS.llaisysPagedKVRopeAppendDev(self._kv, layer, _addr(q_out), _addr(qkv),
                                                       _addr(bias) if bias is not None else None, _addr(seq_ids_dev),
                                                       _addr(positions_dev), n_rows, nh, theta, stream))

    def decode_dev(self, layer: int, out, q, seq_ids_dev, kv_lens_dev, n_seqs: int, max_kv_len: int, nh: int,
                   scale: float, stream) -> None:
        _check(LIB_LLAISYS.llaisysPagedAttentionDecodeDev(self._kv, layer, _addr(out), _addr(q), _addr(seq_ids_dev),
                                                          _addr(kv_lens_dev), n_seqs, max_kv_len, nh, scale, stream))

    def decode_step_dev(self, layer: int, out, q, k_new, v_new, seq_ids_dev, kv_lens_dev, n_seqs: int, max_kv_len: int,
                        nh: int, scale: float, stream) -> None:
        """One decode step in one launch: k_new[i] / v_new[i] become token kv_lens[i] - 1 of sequence i, then attention of
        q[i] over its kv_lens[i] tokens (device index arrays, explicit stream)."""
        _check(LIB_LLAISYS.llaisysPagedDecodeStepDev(self._kv, layer, _addr(out), _addr(q), _addr(k_new), _addr(v_new),
                                                     _addr(seq_ids_dev), _addr(kv_lens_dev), n_seqs, max_kv_len, nh, scale,
                                                     stream))

    def decode_partial_dev(self, layer: int, part, q, seq_ids_dev, kv_lens_dev, n_seqs: int, max_kv_len: int,
                           nh: int, scale: float, stream) -> None:
        _check(LIB_LLAISYS.llaisysPagedAttentionDecodePartialDev(self._kv, layer, _addr(part), _addr(q),
                                                                 _addr(seq_ids_dev), _addr(kv_lens_dev), n_seqs,
                                                                 max_kv_len, nh, scale, stream))

    def prefill_dev(self, layer: int, out, q, seq_ids_dev, q_starts_dev, kv_lens_dev, n_seqs: int, total_q: int,
                    max_q_len: int, max_kv_len: int, nh: int, scale: float, stream) -> None:
        _check(LIB_LLAISYS.llaisysPagedAttentionPrefillDev(self._kv, layer, _addr(out), _addr(q), _addr(seq_ids_dev),
                                                           _addr(q_starts_dev), _addr(kv_lens_dev), n_seqs, total_q,
                                                           max_q_len, max_kv_len, nh, scale, stream))


def lse_merge(out, parts, n_parts: int, n_rows: int, head_dim: int, *, dtype: DataType,
              device: DeviceType = DeviceType.CPU, device_id: int = 0) -> None:
    """Merges n_parts partial results float [n_parts, n_rows, head_dim + 2] into out [n_rows, head_dim]."""
    _check(LIB_LLAISYS.llaisysLseMerge(int(device), device_id, _addr(out), int(dtype), _addr(parts), n_parts, n_rows,
                                       head_dim))


def decode_no_alloc(out, q, pool_layer, block_table_dev, table_stride: int, num_pages: int, seq_ids_dev, kv_lens_dev,
                    n_seqs: int, max_kv_len: int, nh: int, nkvh: int, scale: float, *, dtype: DataType = DataType.BF16,
                    device_id: int = 0, error_flag_dev=None, stream=None) -> None:
    """Split-KV decode over a caller-owned page pool with no device allocation inside the library.

    For servers that have committed all free HBM to their own pool, or decode loops that cannot take the
    device-wide stall of an allocation: the kernel's scratch is a fixed array in the library image. Limits:
    n_seqs * nkvh <= 512, head_dim 128, 16-token pages, BF16/F16. All calls on a device share that array, so
    calls must be ordered on the GPU; the first call on a device should come before any stream capture.
    """
    _check(LIB_LLAISYS.llaisysPagedAttentionDecodeNoAlloc(
        device_id, _addr(out), _addr(q), _addr(pool_layer), _addr(block_table_dev), table_stride, num_pages,
        _addr(seq_ids_dev), _addr(kv_lens_dev), n_seqs, max_kv_len, nh, nkvh, int(dtype), scale,
        _addr(error_flag_dev), stream))


def decode_no_alloc_status(device_id: int = 0, stream=None) -> int:
    """Synchronises the stream and returns (and clears) the error bits that decode_no_alloc calls WITHOUT an error word
    of their own have collected on the device: 0 = none, 1 = an out-of-range page index was skipped."""
    flags = c_int32(0)
    _check(LIB_LLAISYS.llaisysPagedAttentionDecodeNoAllocStatus(device_id, stream, byref(flags)))
    return int(flags.value)
