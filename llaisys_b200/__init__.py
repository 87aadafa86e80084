"""llaisys_b200 -- B200-native implementation of the LLAISYS KV-cache / self-attention path.

The public names are the reference frontend's (python/llaisys/__init__.py:1-20): RuntimeAPI, DeviceType,
DataType, MemcpyKind, Stream, Tensor, Ops. `PagedKVCache`, `lse_merge` and `LlaisysError` are new: the
reference has no KV cache. A program written against the reference package can switch with
`import llaisys_b200 as llaisys`.
"""
from .libllaisys import DataType, DeviceType, MemcpyKind, Status
from .libllaisys import llaisysStream_t as Stream
from .runtime import RuntimeAPI, context_stream, set_context_runtime
from .tensor import Tensor
from .ops import Ops
from .paged_kv import (Kernel, LlaisysError, PagedKVCache, decode_no_alloc, decode_no_alloc_status, last_attention_kernel,
                       lse_merge)
from . import models
from .serving import Engine

__all__ = [
    "RuntimeAPI", "DeviceType", "DataType", "MemcpyKind", "Stream", "Tensor", "Ops", "models", "Engine",
    "PagedKVCache", "lse_merge", "decode_no_alloc", "decode_no_alloc_status", "LlaisysError", "Status", "Kernel",
    "last_attention_kernel", "context_stream", "set_context_runtime",
]
