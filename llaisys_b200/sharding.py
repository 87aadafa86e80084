"""Multi-GPU partitioning of the KV-cache path, one process per GPU over torch.distributed.

Two modes, matching how the path shards:
  * a batch of sequences: whole sequences go to ranks (longest-first bin packing); every rank owns its page
    pool and block tables and there is NO data-path collective;
  * one very long sequence: the KV range is cut into page-aligned slices, one per rank; each rank runs the
    partial decode over its slice and the (o, m, l) partials are merged after ONE all-gather
    (NCCL over NVLink on GPUs, gloo on CPU ranks) -- or, on the GPUs of one node, after every rank has written
    its partial straight into the other ranks' exchange buffers over NVLink (`PeerExchange`, peer stores into
    IPC-mapped memory; no kernel ever READS another GPU's memory).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from .libllaisys import DataType, DeviceType
from .paged_kv import PagedKVCache, lse_merge

_TORCH_DTYPE = {DataType.F32: torch.float32, DataType.F16: torch.float16, DataType.BF16: torch.bfloat16}


def shard_sequences(ctx_lens: Sequence[int], world: int) -> list[list[int]]:
    """Assigns sequence indices to ranks, longest first onto the least loaded rank (ties: lowest rank)."""
    loads = [0] * world
    shards: list[list[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(ctx_lens)), key=lambda i: (-ctx_lens[i], i)):
        r = min(range(world), key=lambda r: (loads[r], r))
        shards[r].append(i)
        loads[r] += ctx_lens[i]
    return [sorted(s) for s in shards]


def kv_range(total_tokens: int, world: int, rank: int, page_size: int = 16) -> tuple[int, int]:
    """Token range [lo, hi) of `rank`: page-aligned cuts, pages spread as evenly as possible."""
    pages = -(-total_tokens // page_size)
    base, extra = divmod(pages, world)
    lo_page = rank * base + min(rank, extra)
    hi_page = lo_page + base + (1 if rank < extra else 0)
    return min(lo_page * page_size, total_tokens), min(hi_page * page_size, total_tokens)


def split_decode(cache: PagedKVCache, layer: int, out: torch.Tensor, q: torch.Tensor, seq_ids: Sequence[int],
                 local_kv_lens: Sequence[int], nh: int, scale: float, group=None) -> None:
    """Decode over a KV range split across the ranks of `group`.

    Every rank passes the same q [n_seqs, nh, d] and its LOCAL sequences / lengths (the slice of each sequence
    its cache holds; 0 is allowed). Each rank computes partials, all ranks gather them, and every rank merges
    into `out` [n_seqs, nh, d].
    """
    n_seqs, d = q.shape[0], q.shape[-1]
    world = dist.get_world_size(group)
    part = torch.empty((n_seqs, nh, d + 2), dtype=torch.float32, device=q.device)
    cache.decode_partial(layer, part, q, seq_ids, local_kv_lens, nh, scale)
    if cache.device == DeviceType.NVIDIA:
        # the partial was queued on the library's stream; the collective runs on torch's
        torch.cuda.current_stream().wait_stream(torch.cuda.ExternalStream(_context_stream()))
    # [world * n_seqs, nh, d + 2]: rank r's partial occupies rows [r * n_seqs, (r + 1) * n_seqs)
    gathered = torch.empty((world * n_seqs, nh, d + 2), dtype=torch.float32, device=q.device)
    dist.all_gather_into_tensor(gathered, part, group=group)
    if cache.device == DeviceType.NVIDIA:
        torch.cuda.ExternalStream(_context_stream()).wait_stream(torch.cuda.current_stream())
    lse_merge(out, gathered, world, n_seqs * nh, d, dtype=cache.dtype, device=cache.device,
              device_id=cache.device_id)


class PeerExchange:
    """Per-rank exchange buffer for split-KV decode through peer memory (include/llaisys/paged_kv.h,
    llaisysPeerExchange*): every rank creates one, the IPC handles travel through the process group, and each
    `split_decode` step is then partial decode + peer stores + flags + merge, all on the library's stream
    (capturable in a CUDA graph). One process per GPU, all on one node."""

    def __init__(self, max_rows: int, head_dim: int, *, device_id: int, group=None):
        import ctypes

        from .libllaisys import LIB_LLAISYS
        from .paged_kv import _check

        self.group = group
        # without a process group: a single rank exchanging with itself (the same kernels, one GPU)
        self._solo = not (dist.is_available() and dist.is_initialized())
        self.rank, self.world = (0, 1) if self._solo else (dist.get_rank(group), dist.get_world_size(group))
        slot = -(-max_rows * (head_dim + 2) // 4) * 4
        self._ex = ctypes.c_void_p()
        _check(LIB_LLAISYS.llaisysPeerExchangeCreate(ctypes.byref(self._ex), device_id, self.rank, self.world, slot))
        mine = ctypes.create_string_buffer(64)
        _check(LIB_LLAISYS.llaisysPeerExchangeHandle(self._ex, mine))
        if self._solo:
            return
        handles: list = [None] * self.world
        dist.all_gather_object(handles, mine.raw, group=group)
        _check(LIB_LLAISYS.llaisysPeerExchangeConnect(self._ex, ctypes.create_string_buffer(b"".join(handles), 64 * self.world)))
        dist.barrier(group=group)  # nobody pushes before everybody has mapped everybody

    def split_decode(self, cache: PagedKVCache, layer: int, out, q, seq_ids_dev, kv_lens_dev, n_seqs: int,
                     max_kv_len: int, nh: int, scale: float, stream) -> None:
        """Decode over a KV range split across the ranks: every rank passes the same q and its LOCAL sequences and
        lengths as device int32 arrays (0 is a valid length); out [n_seqs, nh, d] is the merged result on every rank."""
        from .libllaisys import LIB_LLAISYS
        from .paged_kv import _addr, _check

        _check(LIB_LLAISYS.llaisysPagedAttentionDecodeSplitDev(cache._kv, layer, _addr(out), _addr(q), _addr(seq_ids_dev),
                                                               _addr(kv_lens_dev), n_seqs, max_kv_len, nh, scale,
                                                               self._ex, stream))

    def set_wait_limit(self, polls: int) -> None:
        """Polls (about half a microsecond each) after which a merge stops waiting for a peer's values; the default is about a second."""
        from .libllaisys import LIB_LLAISYS
        from .paged_kv import _check

        _check(LIB_LLAISYS.llaisysPeerExchangeSetWaitLimit(self._ex, polls))

    def status(self, stream) -> int:
        """Synchronises the stream; 0, or 1 when a wait for a peer ran out since the last call (which clears it)."""
        from .libllaisys import LIB_LLAISYS

        return int(LIB_LLAISYS.llaisysPeerExchangeStatus(self._ex, stream))

    def check(self, stream) -> None:
        """Synchronises the stream and raises if a wait for a peer ran out."""
        from .libllaisys import LIB_LLAISYS

        status = LIB_LLAISYS.llaisysPeerExchangeStatus(self._ex, stream)
        if status != 0:
            raise RuntimeError(f"peer exchange: a wait for another rank ran out (status {status})")

    def close(self) -> None:
        from .libllaisys import LIB_LLAISYS

        if getattr(self, "_ex", None):
            if not self._solo:
                dist.barrier(group=self.group)  # nobody unmaps while a peer may still write
                LIB_LLAISYS.llaisysPeerExchangeDisconnect(self._ex)
                dist.barrier(group=self.group)  # nobody releases its buffer while a peer still maps it
            LIB_LLAISYS.llaisysPeerExchangeDestroy(self._ex)
            self._ex = None


def _context_stream() -> int:
    from .runtime import context_stream

    return int(context_stream() or 0)
