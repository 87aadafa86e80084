"""Iteration-level batching engine over a Qwen2 model (include/llaisys/serving.h). The reference has no counterpart:
it describes a request queue with continuous batching and a prefix-matching KV-cache pool as future work
(README.md:415-424)."""
from __future__ import annotations

import ctypes
from ctypes import c_int64, c_size_t, c_void_p
from typing import Iterable, Sequence

import numpy as np

from .libllaisys import LIB_LLAISYS, LlaisysEngineEvent
from .paged_kv import _check


class Engine:
    """submit() requests at any time; every step() runs one batched model step over all running requests (decode tokens
    and prompt chunks mixed) and returns the tokens it produced as (request id, token, finished) triples."""

    def __init__(self, model, *, max_batch: int = 64, max_tokens_per_step: int = 4096, prefill_chunk: int = 512):
        self._model = model  # the engine borrows the model (if the model is destroyed first, the engine's calls fail cleanly)
        self._engine = c_void_p()
        _check(LIB_LLAISYS.llaisysEngineCreate(ctypes.byref(self._engine), model._model, max_batch, max_tokens_per_step,
                                               prefill_chunk))
        self._events = (LlaisysEngineEvent * max_batch)()
        self._cap = max_batch

    def close(self) -> None:
        if getattr(self, "_engine", None):
            LIB_LLAISYS.llaisysEngineDestroy(self._engine)
            self._engine = None

    def __del__(self):
        self.close()

    def submit(self, prompt: Sequence[int], max_new_tokens: int, end_token: int = -1) -> int:
        arr = np.ascontiguousarray(prompt, dtype=np.int64)
        rid = c_int64(0)
        _check(LIB_LLAISYS.llaisysEngineSubmit(self._engine, arr.ctypes.data_as(ctypes.POINTER(c_int64)), arr.size,
                                               max_new_tokens, end_token, ctypes.byref(rid)))
        return rid.value

    def step(self) -> list[tuple[int, int, bool]]:
        n = c_size_t(0)
        _check(LIB_LLAISYS.llaisysEngineStep(self._engine, self._events, self._cap, ctypes.byref(n)))
        return [(e.request, e.token, bool(e.finished)) for e in self._events[: n.value]]

    def cancel(self, request: int) -> None:
        _check(LIB_LLAISYS.llaisysEngineCancel(self._engine, request))

    @property
    def num_waiting(self) -> int:
        return int(LIB_LLAISYS.llaisysEngineNumWaiting(self._engine))

    @property
    def num_running(self) -> int:
        return int(LIB_LLAISYS.llaisysEngineNumRunning(self._engine))

    @property
    def counters(self) -> dict:
        names = ("steps", "prompt_tokens_from_cache", "tokens_computed")
        return {name: int(LIB_LLAISYS.llaisysEngineCounter(self._engine, i)) for i, name in enumerate(names)}

    def run(self, arrivals: Iterable[tuple[int, Sequence[int], int]] = ()) -> dict[int, list[int]]:
        """Drives the engine to completion. arrivals: (step index at which the request arrives, prompt, max_new_tokens),
        sorted by step. -> generated tokens per request, keyed by arrival order (0, 1, ...)."""
        pending = list(arrivals)
        ids: dict[int, int] = {}
        out: dict[int, list[int]] = {}
        it = 0
        while pending or self.num_waiting or self.num_running:
            while pending and pending[0][0] <= it:
                _, prompt, max_new = pending.pop(0)
                rid = self.submit(prompt, max_new)
                ids[rid] = len(ids)
                out[ids[rid]] = []
            for rid, token, _ in self.step():
                out[ids[rid]].append(token)
            it += 1
        return out
