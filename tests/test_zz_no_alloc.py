"""llaisysPagedAttentionDecodeNoAlloc against the cache's own decode entry point.

The no-allocation variant exists for callers whose process has no HBM left to give (all of it is in their own
page pool) or that cannot take an allocator's device-wide stall inside a decode loop; its scratch is a static
array shared by every call. This file is collected last on purpose: a run that stops at the first failure has
then already run every other test. It passes on its own in a fresh process and after the rest of the suite.
"""
import pytest
import torch

import llaisys_b200 as llaisys
from llaisys_b200 import LlaisysError, Status
from oracle import attention, workloads
from tests import helpers

NVIDIA = llaisys.DeviceType.NVIDIA


@pytest.mark.gpu
def test_no_alloc_decode_matches_cache_decode_on_two_calls_in_a_row(cuda_device):
    batch = workloads.decode_batch(9, 1, 2500, seed=41, pool_pages=2048)
    cache, seqs = helpers.build_cache(NVIDIA, "bf16", batch.pages, num_pages=2048, nkvh=2, d=128)
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, NVIDIA)
    cache.flush()
    stream = llaisys.context_stream()
    ids = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    max_pages = max(len(p) for p in batch.pages)

    # call 1: full contexts; call 2: every context cut to a different length and a different query, so stale
    # partials or counters from call 1 would show
    g = torch.Generator().manual_seed(99)
    cases = [(batch.ctx, batch.q), ([max(1, c // 3) for c in batch.ctx], workloads.randn(batch.q.shape, torch.bfloat16, g))]
    for ctx, q_host in cases:
        lens = torch.tensor(ctx, dtype=torch.int32, device="cuda")
        q = q_host.cuda()
        expect = torch.empty_like(q)
        cache.decode_dev(0, expect, q, ids, lens, len(seqs), max(ctx), 12, batch.scale, stream)
        cache.check()
        got = torch.full_like(q, float("nan"))
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        llaisys.decode_no_alloc(got, q, cache.pool_ptr(0), cache.block_table_ptr(), max_pages, 2048, ids, lens,
                                len(seqs), max(ctx), 12, 2, batch.scale, error_flag_dev=flag, stream=stream)
        llaisys.RuntimeAPI(NVIDIA).stream_synchronize(stream)
        assert int(flag.item()) == 0
        got, expect = got.cpu(), expect.cpu()
        assert not got.float().isnan().any()
        # the two entry points run different kernels (cp.async ring vs TMA ring) with the same f32 mathematics:
        # they agree to one bf16 ulp of the output, the tolerance the decode tests use against the f64 oracle
        assert helpers.max_abs(got, expect) <= 8e-3 * max(1.0, expect.float().abs().max().item())
        for i in range(len(seqs)):
            ref = attention.self_attention(q_host[i:i + 1], batch.k[i][:ctx[i]], batch.v[i][:ctx[i]], batch.scale)
            assert helpers.max_abs(got[i:i + 1], ref) <= helpers.MAX_ABS["bf16"]


@pytest.mark.gpu
def test_no_alloc_decode_rejects_sizes_beyond_the_static_scratch(cuda_device):
    q = torch.zeros((300, 12, 128), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros(300, dtype=torch.int32, device="cuda")
    pool = torch.zeros(8 * 2 * 2 * 16 * 128, dtype=torch.bfloat16, device="cuda")
    table = torch.zeros((300, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(LlaisysError) as e:  # 300 sequences x 2 kv heads > 512 pairs
        llaisys.decode_no_alloc(q, q, pool, table, 4, 8, ids, ids, 300, 64, 12, 2, 0.1, stream=llaisys.context_stream())
    assert e.value.status == Status.INVALID and "512" in str(e.value)
    with pytest.raises(LlaisysError) as e:  # f32 pools are not covered
        llaisys.decode_no_alloc(q, q, pool, table, 4, 8, ids, ids, 4, 64, 12, 2, 0.1, dtype=llaisys.DataType.F32,
                                stream=llaisys.context_stream())
    assert e.value.status == Status.UNSUPPORTED
