"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark configurations.

No public dataset is involved anywhere on this path: values are N(0, 1) drawn in f32 from one seeded CPU
generator per configuration and cast once to the run dtype, so the GPU and the oracle see identical bits;
context lengths are uniform integers; physical pages are a prefix of a random permutation of the pool.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

NH, NKVH, D, PAGE = 12, 2, 128, 16
POOL_PAGES = 16384


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def randn(shape, dtype: torch.dtype, g: torch.Generator) -> torch.Tensor:
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)


@dataclass
class DecodeBatch:
    """One decode step: per sequence a context length (INCLUDING the row being appended), the cached rows
    [ctx - 1, nkvh, d], the new row, and one query."""
    ctx: list[int]
    pages: list[list[int]]          # physical pages per sequence
    k: list[torch.Tensor]           # per sequence [ctx, nkvh, d] (last row = the appended one)
    v: list[torch.Tensor]
    q: torch.Tensor                 # [B, nh, d]
    scale: float


def config1(seed: int = 1):
    """f32 single decode step: q [1, 12, 128], k/v [513, 2, 128] (512 cached + 1 appended), scale 1/sqrt(128)."""
    g = _gen(seed)
    q = randn((1, NH, D), torch.float32, g)
    k = randn((513, NKVH, D), torch.float32, g)
    v = randn((513, NKVH, D), torch.float32, g)
    return q, k, v, 1.0 / D ** 0.5


def decode_batch(batch: int, lo: int, hi: int, seed: int, dtype=torch.bfloat16, pool_pages: int = POOL_PAGES,
                 nh: int = NH, nkvh: int = NKVH, d: int = D, page: int = PAGE) -> DecodeBatch:
    """Config-2 style batch: ctx ~ U{lo..hi} after the append, pages = prefix of a random permutation."""
    g = _gen(seed)
    ctx = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    perm = torch.randperm(pool_pages, generator=g).tolist()
    pages, at = [], 0
    for c in ctx:
        n = -(-c // page)
        pages.append(perm[at:at + n])
        at += n
    assert at <= pool_pages, "pool too small for this batch"
    k = [randn((c, nkvh, d), dtype, g) for c in ctx]
    v = [randn((c, nkvh, d), dtype, g) for c in ctx]
    q = randn((batch, nh, d), dtype, g)
    return DecodeBatch(ctx, pages, k, v, q, 1.0 / d ** 0.5)


def config2(seed: int = 2, **kw) -> DecodeBatch:
    """Batch 32, ctx ~ U{128..4096}, page 16, pool 16384 pages, 12/2 heads, d 128, bf16."""
    return decode_batch(32, 128, 4096, seed, **kw)


@dataclass
class PrefillBatch:
    """Chunked prefill: per sequence an existing context C and a new chunk of `chunk` tokens."""
    context: list[int]
    chunk: int
    pages: list[list[int]]
    k: list[torch.Tensor]           # per sequence [C + chunk, nkvh, d]
    v: list[torch.Tensor]
    q: list[torch.Tensor]           # per sequence [chunk, nh, d]
    scale: float


def prefill_batch(batch: int, max_context: int, chunk: int, seed: int, dtype=torch.bfloat16,
                  pool_pages: int = POOL_PAGES, nh: int = NH, nkvh: int = NKVH, d: int = D,
                  page: int = PAGE) -> PrefillBatch:
    g = _gen(seed)
    context = torch.randint(0, max_context + 1, (batch,), generator=g).tolist()
    perm = torch.randperm(pool_pages, generator=g).tolist()
    pages, at = [], 0
    for c in context:
        n = -(-(c + chunk) // page)
        pages.append(perm[at:at + n])
        at += n
    assert at <= pool_pages, "pool too small for this batch"
    k = [randn((c + chunk, nkvh, d), dtype, g) for c in context]
    v = [randn((c + chunk, nkvh, d), dtype, g) for c in context]
    q = [randn((chunk, nh, d), dtype, g) for _ in context]
    return PrefillBatch(context, chunk, pages, k, v, q, 1.0 / d ** 0.5)


def config3(seed: int = 3, **kw) -> PrefillBatch:
    """Batch 8, existing context ~ U{0..8192}, 512-token chunk appended then attended causally, bf16."""
    return prefill_batch(8, 8192, 512, seed, **kw)
