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


@pytest.mark.gpu
def test_no_alloc_decode_without_sequence_ids_and_without_an_error_word(cuda_device):
    """seq_ids_dev = NULL (row i of the block table is sequence i) and error_flag_dev = NULL: the kernel's error bits
    are then collected inside the library and llaisysPagedAttentionDecodeNoAllocStatus is how a caller sees them -- a
    page index out of range must show up there (once), not vanish, and a clean call must leave it at zero."""
    nseq, pages_per, pool_pages = 3, 4, 32
    g = torch.Generator().manual_seed(7)
    ctx = [64, 37, 1]
    table = torch.zeros((nseq, pages_per), dtype=torch.int32)
    perm = torch.randperm(pool_pages, generator=g).tolist()
    pool = torch.zeros((pool_pages, 2, 2, 16, 128), dtype=torch.bfloat16)  # [page][K|V][kvh][slot][d]
    ks = [workloads.randn((c, 2, 128), torch.bfloat16, g) for c in ctx]
    vs = [workloads.randn((c, 2, 128), torch.bfloat16, g) for c in ctx]
    for s in range(nseq):
        for j in range(pages_per):
            table[s, j] = perm[s * pages_per + j]
        for t in range(ctx[s]):
            page = int(table[s, t // 16])
            pool[page, 0, :, t % 16] = ks[s][t]
            pool[page, 1, :, t % 16] = vs[s][t]
    q_host = workloads.randn((nseq, 12, 128), torch.bfloat16, g)
    pool_d, table_d, q = pool.cuda(), table.cuda(), q_host.cuda()
    lens = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    stream = llaisys.context_stream()
    assert llaisys.decode_no_alloc_status(0, stream) == 0
    got = torch.full_like(q, float("nan"))
    llaisys.decode_no_alloc(got, q, pool_d, table_d, pages_per, pool_pages, None, lens, nseq, max(ctx), 12, 2, 128 ** -0.5,
                            error_flag_dev=None, stream=stream)
    assert llaisys.decode_no_alloc_status(0, stream) == 0
    got = got.cpu()
    for i in range(nseq):
        ref = attention.self_attention(q_host[i:i + 1], ks[i], vs[i], 128 ** -0.5)
        assert helpers.max_abs(got[i:i + 1], ref) <= helpers.MAX_ABS["bf16"], i
    # a block-table entry outside the pool: skipped, flagged, reported once
    bad = table.clone()
    bad[0, 1] = pool_pages + 5
    llaisys.decode_no_alloc(torch.empty_like(q), q, pool_d, bad.cuda(), pages_per, pool_pages, None, lens, nseq, max(ctx), 12, 2,
                            128 ** -0.5, error_flag_dev=None, stream=stream)
    assert llaisys.decode_no_alloc_status(0, stream) == 1
    assert llaisys.decode_no_alloc_status(0, stream) == 0


@pytest.mark.gpu
def test_no_alloc_decode_on_a_device_that_is_not_current(cuda_device):
    """The call makes its device current while it runs and puts the caller's device back."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with torch.cuda.device(1):
        q = torch.randn((2, 12, 128), device="cuda:1").bfloat16()
        pool = torch.randn((8, 2, 2, 16, 128), device="cuda:1").bfloat16()
        table = torch.tensor([[0, 1], [2, 3]], dtype=torch.int32, device="cuda:1")
        lens = torch.tensor([20, 32], dtype=torch.int32, device="cuda:1")
        got = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
    torch.cuda.set_device(0)
    llaisys.decode_no_alloc(got, q, pool, table, 2, 8, None, lens, 2, 32, 12, 2, 128 ** -0.5, device_id=1, stream=None)
    assert torch.cuda.current_device() == 0
    with torch.cuda.device(1):
        torch.cuda.synchronize()
    qh, ph = q.cpu(), pool.cpu()
    for i, n in enumerate((20, 32)):
        k = torch.cat([ph[int(table[i, j]), 0].transpose(0, 1) for j in range(2)])[:n].contiguous()
        v = torch.cat([ph[int(table[i, j]), 1].transpose(0, 1) for j in range(2)])[:n].contiguous()
        ref = attention.self_attention(qh[i:i + 1], k, v, 128 ** -0.5)
        assert helpers.max_abs(got[i:i + 1].cpu(), ref) <= helpers.MAX_ABS["bf16"]
