"""Paged append / gather / attention through the C ABI against the oracle, on a CPU cache here and -- marked
gpu -- on a B200. Append and gather must be bit-exact; attention within the bound of the dtype."""
import numpy as np
import pytest
import torch

import llaisys_b200 as llaisys
from llaisys_b200 import LlaisysError, Status
from oracle import attention, workloads
from oracle.paged import PagedCacheModel
from tests import helpers

CPU, NVIDIA = llaisys.DeviceType.CPU, llaisys.DeviceType.NVIDIA


def words(t: torch.Tensor) -> np.ndarray:
    w = helpers.tensor_words(t).numpy()
    return w.view(np.uint32 if w.itemsize == 4 else np.uint16)


def check_append_gather_bit_exact(device, dname, batch: workloads.DecodeBatch, pool_pages, nlayer=2):
    dev = helpers.torch_device(device)
    nkvh, d = batch.k[0].shape[1], batch.k[0].shape[2]
    cache, seqs = helpers.build_cache(device, dname, batch.pages, num_pages=pool_pages, nkvh=nkvh, d=d, nlayer=nlayer)
    model = PagedCacheModel(pool_pages, 16, nkvh, d, word_dtype=np.uint32 if dname == "f32" else np.uint16,
                            max_seqs=len(seqs))
    for pages in batch.pages:
        model.assign_pages(model.add_seq(), pages)
    layer = nlayer - 1
    # two appends: all but the last row of every sequence (a "prefill"), then the last rows (a "decode step")
    last = [c - 1 for c in batch.ctx]
    helpers.append_all(cache, layer, seqs, batch.k, batch.v, device, hi=last)
    helpers.append_all(cache, layer, seqs, batch.k, batch.v, device, lo=last)
    for i, s in enumerate(seqs):
        model.append(words(batch.k[i]), words(batch.v[i]), [i] * batch.ctx[i], range(batch.ctx[i]))
    for i, s in enumerate(seqs):
        k_out = torch.empty_like(batch.k[i], device=dev)
        v_out = torch.empty_like(batch.v[i], device=dev)
        cache.gather(layer, s, batch.ctx[i], k_out, v_out)
        cache.check()
        mk, mv = model.gather(i, batch.ctx[i])
        assert np.array_equal(words(k_out.cpu()), mk) and np.array_equal(words(v_out.cpu()), mv)
        assert torch.equal(helpers.tensor_words(k_out.cpu()), helpers.tensor_words(batch.k[i]))
        assert torch.equal(helpers.tensor_words(v_out.cpu()), helpers.tensor_words(batch.v[i]))
    # the whole pool, byte for byte, equals the model's (untouched slots stay zero), and layer 0 is untouched
    pool = torch.empty(cache.layer_bytes(), dtype=torch.uint8)
    api = llaisys.RuntimeAPI(device)
    kind = llaisys.MemcpyKind.H2H if device == CPU else llaisys.MemcpyKind.D2H
    api.memcpy_sync(pool.data_ptr(), cache.pool_ptr(layer), pool.numel(), kind)
    assert np.array_equal(pool.numpy(), model.pool.reshape(-1).view(np.uint8))
    api.memcpy_sync(pool.data_ptr(), cache.pool_ptr(0), pool.numel(), kind)
    assert not pool.any()
    return cache, seqs


def check_decode(device, dname, batch: workloads.DecodeBatch, pool_pages, tol=None):
    dev = helpers.torch_device(device)
    nh, d = batch.q.shape[1], batch.q.shape[2]
    cache, seqs = helpers.build_cache(device, dname, batch.pages, num_pages=pool_pages, nkvh=batch.k[0].shape[1], d=d)
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, device)
    out = torch.empty_like(batch.q, device=dev)
    cache.decode(0, out, batch.q.to(dev), seqs, batch.ctx, nh, batch.scale)
    cache.check()
    out = out.cpu()
    bound = tol or helpers.MAX_ABS[dname]
    ulp = {"f32": 1e-6, "f16": 1e-3, "bf16": 8e-3}[dname]
    for i in range(len(seqs)):
        q = batch.q[i:i + 1]
        expect = attention.self_attention(q, batch.k[i], batch.v[i], batch.scale)
        assert helpers.max_abs(out[i:i + 1], expect) <= bound, (i, batch.ctx[i])
        f64 = attention.self_attention_f64(q, batch.k[i], batch.v[i], batch.scale)
        assert helpers.max_abs(out[i:i + 1], f64) <= ulp * max(1.0, f64.abs().max().item()), (i, batch.ctx[i])
    # partial variant + merge over one part reproduces the same result
    part = torch.empty((len(seqs), nh, d + 2), dtype=torch.float32, device=dev)
    cache.decode_partial(0, part, batch.q.to(dev), seqs, batch.ctx, nh, batch.scale)
    merged = torch.empty_like(batch.q, device=dev)
    llaisys.lse_merge(merged, part, 1, len(seqs) * nh, d, dtype=helpers.LL_DTYPE[dname], device=device)
    cache.check()
    assert helpers.max_abs(merged.cpu(), out) <= ulp
    return cache, seqs


def check_prefill(device, dname, batch: workloads.PrefillBatch, pool_pages, repeats=0):
    dev = helpers.torch_device(device)
    nh, d = batch.q[0].shape[1], batch.q[0].shape[2]
    cache, seqs = helpers.build_cache(device, dname, batch.pages, num_pages=pool_pages, nkvh=batch.k[0].shape[1], d=d)
    # existing context first, then the chunk (appended, then attended causally)
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, device, hi=batch.context)
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, device, lo=batch.context)
    q = torch.cat(batch.q).contiguous()
    out = torch.empty_like(q, device=dev)
    q_lens = [batch.chunk] * len(seqs)
    kv_lens = [c + batch.chunk for c in batch.context]
    cache.prefill(0, out, q.to(dev), seqs, q_lens, kv_lens, nh, batch.scale)
    cache.check()
    # the kernel is deterministic: repeated launches must give the same bits (a synchronisation race inside it shows
    # up as rows that differ from run to run, most easily in the tiles that run last, alone on their SM)
    for _ in range(repeats):
        again = torch.empty_like(q, device=dev)
        cache.prefill(0, again, q.to(dev), seqs, q_lens, kv_lens, nh, batch.scale)
        cache.check()
        assert torch.equal(helpers.tensor_words(again.cpu()), helpers.tensor_words(out.cpu()))
    out = out.cpu()
    ulp = {"f32": 1e-6, "f16": 1e-3, "bf16": 8e-3}[dname]
    for i in range(len(seqs)):
        got = out[i * batch.chunk:(i + 1) * batch.chunk]
        expect = attention.self_attention(batch.q[i], batch.k[i], batch.v[i], batch.scale)
        assert helpers.max_abs(got, expect) <= helpers.MAX_ABS[dname], (i, batch.context[i])
        f64 = attention.self_attention_f64(batch.q[i], batch.k[i], batch.v[i], batch.scale)
        assert helpers.max_abs(got, f64) <= ulp * max(1.0, f64.abs().max().item()), (i, batch.context[i])


# ---- CPU cache --------------------------------------------------------------------------------------

@pytest.mark.parametrize("dname", ["bf16", "f16", "f32"])
def test_append_gather_bit_exact_cpu(dname):
    batch = workloads.decode_batch(6, 1, 70, seed=11, dtype=helpers.TORCH_DTYPE[dname], pool_pages=64)
    check_append_gather_bit_exact(CPU, dname, batch, 64)


@pytest.mark.parametrize("dname", ["bf16", "f16", "f32"])
def test_decode_cpu(dname):
    batch = workloads.decode_batch(5, 1, 90, seed=12, dtype=helpers.TORCH_DTYPE[dname], pool_pages=64)
    check_decode(CPU, dname, batch, 64)


def test_decode_gqa_and_head_dim_variants_cpu():
    for nh, nkvh, d in ((8, 8, 64), (4, 1, 32), (6, 2, 8)):
        batch = workloads.decode_batch(3, 1, 40, seed=13, dtype=torch.float32, pool_pages=32, nh=nh, nkvh=nkvh, d=d)
        check_decode(CPU, "f32", batch, 32)


@pytest.mark.parametrize("dname", ["bf16", "f32"])
def test_prefill_cpu(dname):
    batch = workloads.prefill_batch(3, 40, 9, seed=14, dtype=helpers.TORCH_DTYPE[dname], pool_pages=32)
    check_prefill(CPU, dname, batch, 32)


def test_prefill_with_empty_context_and_ragged_chunks_cpu():
    g = torch.Generator().manual_seed(3)
    cache = llaisys.PagedKVCache(16, 2, 128, dtype=llaisys.DataType.F32, max_seqs=3)
    seqs, ks, vs, qs, q_lens, kv_lens = [], [], [], [], [1, 5, 0], [33, 5, 0]
    for ql, kl in zip(q_lens, kv_lens):
        s = cache.add_seq()
        cache.reserve(s, kl)
        seqs.append(s)
        ks.append(workloads.randn((kl, 2, 128), torch.float32, g))
        vs.append(workloads.randn((kl, 2, 128), torch.float32, g))
        qs.append(workloads.randn((ql, 12, 128), torch.float32, g))
    helpers.append_all(cache, 0, seqs, ks, vs, CPU)
    q = torch.cat(qs)
    out = torch.full_like(q, 7.0)
    cache.prefill(0, out, q, seqs, q_lens, kv_lens, 12, 0.1)
    at = 0
    for i, ql in enumerate(q_lens):
        if ql:
            assert helpers.max_abs(out[at:at + ql], attention.self_attention(qs[i], ks[i], vs[i], 0.1)) <= 1e-5
        at += ql


def test_data_path_argument_errors_cpu():
    cache = llaisys.PagedKVCache(8, 2, 128, dtype=llaisys.DataType.BF16, max_seqs=2)
    s = cache.add_seq()
    cache.reserve(s, 16)
    rows = torch.zeros((1, 2, 128), dtype=torch.bfloat16)
    q = torch.zeros((1, 12, 128), dtype=torch.bfloat16)
    cases = [
        (lambda: cache.append(0, rows, rows, [s], [16]), Status.INVALID),        # position beyond reserved pages
        (lambda: cache.append(0, rows, rows, [s], [-1]), Status.INVALID),
        (lambda: cache.append(0, rows, rows, [s + 1], [0]), Status.NO_SEQ),      # unknown sequence
        (lambda: cache.append(1, rows, rows, [s], [0]), Status.INVALID),         # layer out of range
        (lambda: cache.decode(0, q, q, [s], [17], 12, 1.0), Status.INVALID),     # kv_len beyond capacity
        (lambda: cache.decode(0, q, q, [s], [1], 11, 1.0), Status.INVALID),      # nh not a multiple of nkvh
        (lambda: cache.prefill(0, q, q, [s], [2], [1], 12, 1.0), Status.INVALID),  # q_len > kv_len
        (lambda: cache.gather(0, s, 17, rows, rows), Status.INVALID),
    ]
    for call, status in cases:
        with pytest.raises(LlaisysError) as e:
            call()
        assert e.value.status == status
    cache.append(0, rows, rows, [s], [15])  # still usable after the errors
    cache.decode(0, q, q, [s], [0], 12, 1.0)  # zero-length context: output is zero, not NaN
    assert not q.float().abs().any()
    cache.check()


def check_decode_step_host(device, pinned=False):
    """The one-call host-buffer step must leave the cache and the output exactly as append + decode do, with pageable
    and with page-locked host buffers."""
    dev = helpers.torch_device(device)
    batch = workloads.decode_batch(5, 1, 300, seed=8, pool_pages=128)
    nkvh, d, nh = workloads.NKVH, workloads.D, workloads.NH
    outs = []
    for fused in (False, True):
        cache, seqs = helpers.build_cache(device, "bf16", batch.pages, num_pages=128, nkvh=nkvh, d=d)
        last = [c - 1 for c in batch.ctx]
        helpers.append_all(cache, 0, seqs, batch.k, batch.v, device, hi=last)
        k_new = torch.stack([k[-1] for k in batch.k]).contiguous()
        v_new = torch.stack([v[-1] for v in batch.v]).contiguous()
        out = torch.empty_like(batch.q)
        if fused:
            q_host = batch.q
            if pinned:
                out, q_host, k_new, v_new = (t.pin_memory() for t in (out, batch.q, k_new, v_new))
            cache.decode_step_host(0, out, q_host, k_new, v_new, np.asarray(seqs, np.int32),
                                   np.asarray(batch.ctx, np.int32), nh, batch.scale)
        else:
            cache.append(0, k_new.to(dev), v_new.to(dev), seqs, last)
            out_d = torch.empty_like(batch.q, device=dev)
            cache.decode(0, out_d, batch.q.to(dev), seqs, batch.ctx, nh, batch.scale)
            out = out_d.cpu()
        cache.check()
        k_all = torch.empty_like(batch.k[0], device=dev)
        v_all = torch.empty_like(batch.v[0], device=dev)
        cache.gather(0, seqs[0], batch.ctx[0], k_all, v_all)
        outs.append((out.clone(), k_all.cpu(), v_all.cpu()))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(helpers.tensor_words(a), helpers.tensor_words(b))
    expect = attention.self_attention(batch.q[:1], batch.k[0], batch.v[0], batch.scale)
    assert (outs[1][0][:1].float() - expect.float()).abs().max().item() <= 2e-2
    with pytest.raises(LlaisysError):  # position 0 of a sequence needs kv_len >= 1
        cache.decode_step_host(0, out, batch.q, k_new, v_new, np.asarray(seqs, np.int32),
                               np.zeros(len(seqs), np.int32), nh, batch.scale)


@pytest.mark.gpu
def test_decode_step_host_many_sequences_nvidia(cuda_device):
    """300 sequences: beyond the 256 whose index arrays travel with the launch, so the step uploads them; page-locked
    buffers. Output against the oracle, appended rows bit-exact."""
    n = 300
    g = torch.Generator().manual_seed(33)
    ctx = torch.randint(1, 40, (n,), generator=g).tolist()
    cache = llaisys.PagedKVCache(3 * n, 2, 128, dtype=llaisys.DataType.BF16, device=NVIDIA, max_seqs=n, max_pages_per_seq=3)
    seqs, ks, vs = [], [], []
    for c in ctx:
        s = cache.add_seq()
        cache.reserve(s, c)
        seqs.append(s)
        ks.append(workloads.randn((c, 2, 128), torch.bfloat16, g))
        vs.append(workloads.randn((c, 2, 128), torch.bfloat16, g))
    helpers.append_all(cache, 0, seqs, ks, vs, NVIDIA, hi=[c - 1 for c in ctx])
    q = workloads.randn((n, 12, 128), torch.bfloat16, g).pin_memory()
    k_new = torch.stack([k[-1] for k in ks]).contiguous().pin_memory()
    v_new = torch.stack([v[-1] for v in vs]).contiguous().pin_memory()
    out = torch.empty_like(q).pin_memory()
    cache.decode_step_host(0, out, q, k_new, v_new, np.asarray(seqs, np.int32), np.asarray(ctx, np.int32), 12, 128 ** -0.5)
    cache.check()
    assert cache.last_kernel() == llaisys.Kernel.DECODE_TMA_FUSED
    for i in (0, 7, 255, 256, 299):
        expect = attention.self_attention(q[i:i + 1], ks[i], vs[i], 128 ** -0.5)
        assert helpers.max_abs(out[i:i + 1], expect) <= helpers.MAX_ABS["bf16"], i
        k_out = torch.empty_like(ks[i], device="cuda")
        v_out = torch.empty_like(vs[i], device="cuda")
        cache.gather(0, seqs[i], ctx[i], k_out, v_out)
        assert torch.equal(helpers.tensor_words(k_out.cpu()), helpers.tensor_words(ks[i]))
        assert torch.equal(helpers.tensor_words(v_out.cpu()), helpers.tensor_words(vs[i]))


def test_decode_step_host_cpu():
    check_decode_step_host(CPU)


@pytest.mark.gpu
@pytest.mark.parametrize("pinned", [False, True])
def test_decode_step_host_nvidia(cuda_device, pinned):
    check_decode_step_host(NVIDIA, pinned)


def check_one_launch_step(device, lens, pool_pages=256, dname="bf16", nh=12, nkvh=2):
    """llaisysPagedDecodeStepDev (append the step's row and attend, one launch on NVIDIA) must leave the pool and the
    output exactly as llaisysPagedKVAppendDev + llaisysPagedAttentionDecodeDev do, and match the oracle."""
    dev = helpers.torch_device(device)
    dt = helpers.TORCH_DTYPE[dname]
    g = torch.Generator().manual_seed(sum(lens) + len(lens))
    perm = torch.randperm(pool_pages, generator=g).tolist()
    pages, at = [], 0
    for c in lens:
        n = -(-c // 16)
        pages.append(perm[at:at + n])
        at += n
    ks = [workloads.randn((c, nkvh, 128), dt, g) for c in lens]
    vs = [workloads.randn((c, nkvh, 128), dt, g) for c in lens]
    q = workloads.randn((len(lens), nh, 128), dt, g)
    k_new = torch.stack([k[-1] for k in ks]).contiguous().to(dev)
    v_new = torch.stack([v[-1] for v in vs]).contiguous().to(dev)
    scale = 128 ** -0.5
    results = []
    for one_launch in (False, True):
        cache, seqs = helpers.build_cache(device, dname, pages, num_pages=pool_pages, nkvh=nkvh, d=128)
        helpers.append_all(cache, 0, seqs, ks, vs, device, hi=[c - 1 for c in lens])
        cache.flush()
        ids = torch.tensor(seqs, dtype=torch.int32, device=dev)
        kv = torch.tensor(lens, dtype=torch.int32, device=dev)
        out = torch.full(q.shape, float("nan"), dtype=dt, device=dev)
        stream = llaisys.context_stream() if device == NVIDIA else None
        if one_launch:
            cache.decode_step_dev(0, out, q.to(dev), k_new, v_new, ids, kv, len(lens), max(lens), nh, scale, stream)
            if device == NVIDIA:
                assert cache.last_kernel() == llaisys.Kernel.DECODE_TMA_FUSED
        else:
            cache.append_dev(0, k_new, v_new, ids, kv - 1, len(lens), stream)
            cache.decode_dev(0, out, q.to(dev), ids, kv, len(lens), max(lens), nh, scale, stream)
        cache.check()
        pool = torch.empty(cache.layer_bytes(), dtype=torch.uint8)
        kind = llaisys.MemcpyKind.H2H if device == CPU else llaisys.MemcpyKind.D2H
        llaisys.RuntimeAPI(device).memcpy_sync(pool.data_ptr(), cache.pool_ptr(0), pool.numel(), kind)
        results.append((out.cpu(), pool))
    assert torch.equal(results[0][1], results[1][1]), "the pool differs from append + decode"
    assert torch.equal(helpers.tensor_words(results[0][0]), helpers.tensor_words(results[1][0]))
    out = results[1][0]
    for i, c in enumerate(lens):
        expect = attention.self_attention(q[i:i + 1], ks[i], vs[i], scale)
        assert helpers.max_abs(out[i:i + 1], expect) <= helpers.MAX_ABS[dname], (i, c)


def test_one_launch_step_cpu():
    check_one_launch_step(CPU, [1, 2, 16, 17, 40], pool_pages=32)


@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_one_launch_step_nvidia(cuda_device, dname):
    """New rows in every slot position: the only token of a sequence, the last slot of a page, the first slot of a fresh
    page; short and long sequences in one batch, so that several pairs end inside one CTA's span and long ones are cut."""
    check_one_launch_step(NVIDIA, [1, 2, 15, 16, 17, 31, 32, 33, 300, 1000, 48, 1, 64, 65], dname=dname)
    check_one_launch_step(NVIDIA, [2000, 5, 777], pool_pages=256, dname=dname, nh=16)
    check_one_launch_step(NVIDIA, [33] * 40, pool_pages=256, dname=dname, nh=4, nkvh=4)


@pytest.mark.gpu
def test_one_launch_step_north_star_shape_nvidia(cuda_device):
    """The shape the headline number is quoted on -- 64 sequences x 4096 tokens, 12/2 heads, bf16, all 16384 pages of the
    pool in a random permutation -- through the one-launch step, against the oracle: every output row within 2e-2 and
    one output ulp of the float64 result, the appended rows bit-exact, and the kernel the TMA decode kernel."""
    g = torch.Generator().manual_seed(64)
    n, ctx = 64, 4096
    perm = torch.randperm(workloads.POOL_PAGES, generator=g).tolist()
    pages = [perm[i * 256:(i + 1) * 256] for i in range(n)]
    ks = [workloads.randn((ctx, 2, 128), torch.bfloat16, g) for _ in range(n)]
    vs = [workloads.randn((ctx, 2, 128), torch.bfloat16, g) for _ in range(n)]
    q = workloads.randn((n, 12, 128), torch.bfloat16, g)
    cache, seqs = helpers.build_cache(NVIDIA, "bf16", pages, num_pages=workloads.POOL_PAGES, nkvh=2, d=128)
    helpers.append_all(cache, 0, seqs, ks, vs, NVIDIA, hi=[ctx - 1] * n)
    cache.flush()
    ids = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    kv = torch.full((n,), ctx, dtype=torch.int32, device="cuda")
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    k_new = torch.stack([k[-1] for k in ks]).cuda()
    v_new = torch.stack([v[-1] for v in vs]).cuda()
    scale = 128 ** -0.5
    cache.decode_step_dev(0, out, q.cuda(), k_new, v_new, ids, kv, n, ctx, 12, scale, llaisys.context_stream())
    cache.check()
    assert cache.last_kernel() == llaisys.Kernel.DECODE_TMA_FUSED
    out = out.cpu()
    for i in range(n):
        expect = attention.self_attention(q[i:i + 1], ks[i], vs[i], scale)
        assert helpers.max_abs(out[i:i + 1], expect) <= helpers.MAX_ABS["bf16"], i
        f64 = attention.self_attention_f64(q[i:i + 1], ks[i], vs[i], scale)
        assert helpers.max_abs(out[i:i + 1], f64) <= 8e-3 * max(1.0, f64.abs().max().item()), i
    for i in (0, 31, 63):
        k_out = torch.empty_like(ks[i], device="cuda")
        v_out = torch.empty_like(vs[i], device="cuda")
        cache.gather(0, seqs[i], ctx, k_out, v_out)
        cache.check()
        assert torch.equal(helpers.tensor_words(k_out.cpu()), helpers.tensor_words(ks[i]))
        assert torch.equal(helpers.tensor_words(v_out.cpu()), helpers.tensor_words(vs[i]))
    # the plain decode call on the same cache: same kernel without the append, same bits
    again = torch.empty_like(q, device="cuda")
    cache.decode_dev(0, again, q.cuda(), ids, kv, n, ctx, 12, scale, llaisys.context_stream())
    cache.check()
    assert cache.last_kernel() == llaisys.Kernel.DECODE_TMA
    assert torch.equal(helpers.tensor_words(again.cpu()), helpers.tensor_words(out))


@pytest.mark.gpu
def test_one_long_sequence_131072_tokens_nvidia(cuda_device):
    """One layer of the long-context configuration on one GPU: a single 131072-token sequence (8192 pages), decode and
    partial decode against the float64 oracle (walked in key ranges to bound its memory)."""
    g = torch.Generator().manual_seed(131072)
    total = 131072
    k = workloads.randn((total, 2, 128), torch.bfloat16, g)
    v = workloads.randn((total, 2, 128), torch.bfloat16, g)
    q = workloads.randn((1, 12, 128), torch.bfloat16, g)
    cache = llaisys.PagedKVCache(total // 16, 2, 128, dtype=llaisys.DataType.BF16, device=NVIDIA, max_seqs=1,
                                 max_pages_per_seq=total // 16)
    s = cache.add_seq()
    cache.assign_pages(s, torch.randperm(total // 16, generator=g).tolist())
    helpers.append_all(cache, 0, [s], [k], [v], NVIDIA)
    out = torch.empty_like(q, device="cuda")
    scale = 128 ** -0.5
    cache.decode(0, out, q.cuda(), [s], [total], 12, scale)
    cache.check()
    assert cache.last_kernel() == llaisys.Kernel.DECODE_TMA
    f64 = attention.decode_attention_f64_chunked(q, k, v, scale)
    assert helpers.max_abs(out.cpu(), f64) <= 8e-3 * max(1.0, f64.abs().max().item())


@pytest.mark.gpu
def test_back_to_back_one_launch_steps_with_launch_overlap_nvidia(cuda_device):
    """Twenty one-launch steps queued without any host synchronisation, programmatic dependent launch on, on ONE layer:
    step t + 1 reads the row step t wrote, sometimes in the same page and sometimes (lengths cross several page
    boundaries) in the page before its own last one. Every step must match the oracle."""
    steps, nseq = 20, 6
    batch = workloads.decode_batch(nseq, 60, 900, seed=71, pool_pages=512)
    cache, seqs = helpers.build_cache(NVIDIA, "bf16", [p for p in batch.pages], num_pages=512, nkvh=2, d=128)
    cache.set_launch_overlap(True)
    start = [c - steps for c in batch.ctx]
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, NVIDIA, hi=start)
    cache.flush()
    stream = llaisys.context_stream()
    ids = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(72)
    qs = [workloads.randn((nseq, 12, 128), torch.bfloat16, g) for _ in range(steps)]
    len_dev = [torch.tensor([st + t + 1 for st in start], dtype=torch.int32, device="cuda") for t in range(steps)]
    k_new = [torch.stack([batch.k[i][start[i] + t] for i in range(nseq)]).cuda() for t in range(steps)]
    v_new = [torch.stack([batch.v[i][start[i] + t] for i in range(nseq)]).cuda() for t in range(steps)]
    q_dev = [q.cuda() for q in qs]
    outs = [torch.full((nseq, 12, 128), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(steps)]
    torch.cuda.synchronize()
    for t in range(steps):
        cache.decode_step_dev(0, outs[t], q_dev[t], k_new[t], v_new[t], ids, len_dev[t], nseq, max(batch.ctx), 12,
                              batch.scale, stream)
    cache.check()
    for t in range(steps):
        got = outs[t].cpu()
        for i in range(nseq):
            n = start[i] + t + 1
            expect = attention.self_attention(qs[t][i:i + 1], batch.k[i][:n], batch.v[i][:n], batch.scale)
            assert helpers.max_abs(got[i:i + 1], expect) <= helpers.MAX_ABS["bf16"], (t, i)
    for i in range(nseq):
        k_out = torch.empty_like(batch.k[i], device="cuda")
        v_out = torch.empty_like(batch.v[i], device="cuda")
        cache.gather(0, seqs[i], batch.ctx[i], k_out, v_out)
        assert torch.equal(helpers.tensor_words(k_out.cpu()), helpers.tensor_words(batch.k[i]))
        assert torch.equal(helpers.tensor_words(v_out.cpu()), helpers.tensor_words(batch.v[i]))


def test_host_step_rejects_a_sequence_named_twice_cpu():
    cache = llaisys.PagedKVCache(8, 2, 128, dtype=llaisys.DataType.BF16, max_seqs=2)
    s = cache.add_seq()
    cache.reserve(s, 16)
    rows = torch.zeros((2, 2, 128), dtype=torch.bfloat16)
    q = torch.zeros((2, 12, 128), dtype=torch.bfloat16)
    with pytest.raises(LlaisysError) as e:
        cache.decode_step_host(0, q.clone(), q, rows, rows, np.asarray([s, s], np.int32), np.asarray([3, 3], np.int32), 12, 1.0)
    assert e.value.status == Status.INVALID and "twice" in str(e.value)
    cache.decode_step_host(0, q[:1].clone(), q[:1], rows[:1], rows[:1], np.asarray([s], np.int32), np.asarray([3], np.int32), 12, 1.0)


def test_lse_merge_cpu():
    g = torch.Generator().manual_seed(9)
    q = workloads.randn((1, 12, 128), torch.float32, g)
    k = workloads.randn((200, 2, 128), torch.float32, g)
    v = workloads.randn((200, 2, 128), torch.float32, g)
    cuts = [0, 0, 50, 127, 200]
    parts = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        o, m, l = attention.partial_attention_f64(q, k[a:b], v[a:b], 0.09)
        parts.append(torch.cat([o, m[:, None], l[:, None]], dim=1).float())
    parts = torch.stack(parts).contiguous()  # [P, 12, 130]
    out = torch.empty((12, 128), dtype=torch.float32)
    llaisys.lse_merge(out, parts, len(cuts) - 1, 12, 128, dtype=llaisys.DataType.F32)
    assert helpers.max_abs(out, attention.self_attention_f64(q, k, v, 0.09)[0]) <= 1e-6


# ---- NVIDIA cache -----------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["bf16", "f16", "f32"])
def test_append_gather_bit_exact_nvidia(cuda_device, dname):
    batch = workloads.decode_batch(8, 1, 300, seed=21, dtype=helpers.TORCH_DTYPE[dname], pool_pages=256)
    check_append_gather_bit_exact(NVIDIA, dname, batch, 256)


@pytest.mark.gpu
def test_append_gather_config2_full_size_nvidia(cuda_device):
    """Configuration 2 at full size: 32 sequences, ctx ~ U{128..4096}, 16384-page pool, random page permutation."""
    batch = workloads.config2()
    check_append_gather_bit_exact(NVIDIA, "bf16", batch, workloads.POOL_PAGES, nlayer=2)


@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["bf16", "f16", "f32"])
def test_decode_small_nvidia(cuda_device, dname):
    batch = workloads.decode_batch(7, 1, 700, seed=22, dtype=helpers.TORCH_DTYPE[dname], pool_pages=512)
    check_decode(NVIDIA, dname, batch, 512)


@pytest.mark.gpu
def test_decode_config2_full_size_nvidia(cuda_device):
    check_decode(NVIDIA, "bf16", workloads.config2(), workloads.POOL_PAGES)


@pytest.mark.gpu
def test_decode_gqa_and_head_dim_variants_nvidia(cuda_device):
    for nh, nkvh, d, dt, dname in ((8, 8, 64, torch.float32, "f32"), (4, 1, 32, torch.float16, "f16"),
                                   (16, 2, 128, torch.bfloat16, "bf16"), (2, 2, 128, torch.bfloat16, "bf16"),
                                   (14, 2, 128, torch.float16, "f16")):
        batch = workloads.decode_batch(4, 1, 600, seed=23, dtype=dt, pool_pages=256, nh=nh, nkvh=nkvh, d=d)
        check_decode(NVIDIA, dname, batch, 256)


@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["bf16", "f32"])
def test_prefill_small_nvidia(cuda_device, dname):
    batch = workloads.prefill_batch(4, 300, 37, seed=24, dtype=helpers.TORCH_DTYPE[dname], pool_pages=256)
    check_prefill(NVIDIA, dname, batch, 256)


@pytest.mark.gpu
def test_prefill_config3_reduced_nvidia(cuda_device):
    """Configuration 3's shape with a shorter context bound so the CPU oracle finishes in seconds:
    8 sequences, context ~ U{0..1024}, 512-token chunk."""
    check_prefill(NVIDIA, "bf16", workloads.prefill_batch(8, 1024, 512, seed=3, pool_pages=2048), 2048)


@pytest.mark.gpu
def test_prefill_config3_full_size_nvidia(cuda_device):
    """Configuration 3 at full size: 8 sequences, context ~ U{0..8192}, 512-token chunk, 16384-page pool
    (the CPU oracle needs a few seconds per long sequence)."""
    check_prefill(NVIDIA, "bf16", workloads.config3(), workloads.POOL_PAGES, repeats=10)


@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_prefill_ragged_chunks_and_block_boundaries_nvidia(cuda_device, dname):
    """Chunks and contexts on both sides of the kernel's tile sizes (128 query rows, 64-key blocks, 16-token pages),
    a chunk with no context, a one-token chunk, and a sequence without a chunk, in one ragged batch."""
    g = torch.Generator().manual_seed(17)
    dt = helpers.TORCH_DTYPE[dname]
    q_lens = [1, 127, 128, 129, 300, 64, 0, 5]
    ctxs = [200, 0, 63, 64, 65, 1000, 30, 15]
    kv_lens = [c + q for c, q in zip(ctxs, q_lens)]
    cache = llaisys.PagedKVCache(512, 2, 128, dtype=helpers.LL_DTYPE[dname], device=NVIDIA, max_seqs=len(q_lens),
                                 max_pages_per_seq=80)
    seqs, ks, vs, qs = [], [], [], []
    for ql, kl in zip(q_lens, kv_lens):
        s = cache.add_seq()
        cache.reserve(s, kl)
        seqs.append(s)
        ks.append(workloads.randn((kl, 2, 128), dt, g))
        vs.append(workloads.randn((kl, 2, 128), dt, g))
        qs.append(workloads.randn((ql, 12, 128), dt, g))
    helpers.append_all(cache, 0, seqs, ks, vs, NVIDIA)
    q = torch.cat(qs).cuda()
    out = torch.full_like(q, float("nan"))
    cache.prefill(0, out, q, seqs, q_lens, kv_lens, 12, 128 ** -0.5)
    cache.check()
    out = out.cpu()
    assert not out.float().isnan().any()
    at = 0
    for i, ql in enumerate(q_lens):
        if ql:
            expect = attention.self_attention(qs[i], ks[i], vs[i], 128 ** -0.5)
            assert helpers.max_abs(out[at:at + ql], expect) <= helpers.MAX_ABS[dname], (i, ql, kv_lens[i])
            f64 = attention.self_attention_f64(qs[i], ks[i], vs[i], 128 ** -0.5)
            ulp = {"f16": 1e-3, "bf16": 8e-3}[dname]
            assert helpers.max_abs(out[at:at + ql], f64) <= ulp * max(1.0, f64.abs().max().item()), (i, ql)
        at += ql


@pytest.mark.gpu
@pytest.mark.parametrize("nh,nkvh,ctx,chunk", [(12, 2, 6000, 256), (7, 1, 3000, 130), (4, 4, 9000, 64)])
def test_prefill_one_long_sequence_split_over_ctas_nvidia(cuda_device, nh, nkvh, ctx, chunk):
    """One sequence with a long context: a handful of tiles for a whole GPU, so the kernel cuts every tile's key range
    into pieces run by different CTAs and merges their partial results. The merged rows must match the oracle, and
    -- the merge order being fixed, not the order in which the pieces finish -- be the same bits on every launch."""
    g = torch.Generator().manual_seed(nh * 1000 + ctx)
    kv_len = ctx + chunk
    cache = llaisys.PagedKVCache((kv_len + 15) // 16 + 4, nkvh, 128, dtype=llaisys.DataType.BF16, device=NVIDIA, max_seqs=1,
                                 max_pages_per_seq=(kv_len + 15) // 16)
    s = cache.add_seq()
    cache.reserve(s, kv_len)
    k = workloads.randn((kv_len, nkvh, 128), torch.bfloat16, g)
    v = workloads.randn((kv_len, nkvh, 128), torch.bfloat16, g)
    qh = workloads.randn((chunk, nh, 128), torch.bfloat16, g)
    helpers.append_all(cache, 0, [s], [k], [v], NVIDIA)
    q = qh.cuda()
    out = torch.full_like(q, float("nan"))
    cache.prefill(0, out, q, [s], [chunk], [kv_len], nh, 128 ** -0.5)
    cache.check()
    for _ in range(5):
        again = torch.full_like(q, float("nan"))
        cache.prefill(0, again, q, [s], [chunk], [kv_len], nh, 128 ** -0.5)
        cache.check()
        assert torch.equal(helpers.tensor_words(again.cpu()), helpers.tensor_words(out.cpu()))
    out = out.cpu()
    assert not out.float().isnan().any()
    expect = attention.self_attention(qh, k, v, 128 ** -0.5)
    assert helpers.max_abs(out, expect) <= helpers.MAX_ABS["bf16"]


@pytest.mark.gpu
def test_prefill_tiles_of_very_different_lengths_in_one_batch_nvidia(cuda_device):
    """Contexts from 100 to 10500 tokens in one batch of 256-row chunks: the kernel cuts the line of all tiles' blocks
    into equal pieces, so the long tiles run over two to five CTAs each (their partial results are merged from shared
    memory, one, two or four trips for the other fragments) while one CTA takes half a dozen short tiles. Every row
    must match the oracle and, the merge order being fixed, be the same bits on every launch."""
    g = torch.Generator().manual_seed(77)
    ctxs = [10500, 700, 3000, 100, 5200, 1500, 8000, 6100]
    chunk = 256
    kv_lens = [c + chunk for c in ctxs]
    pages = sum((l + 15) // 16 for l in kv_lens) + 8
    cache = llaisys.PagedKVCache(pages, 2, 128, dtype=llaisys.DataType.BF16, device=NVIDIA, max_seqs=len(ctxs),
                                 max_pages_per_seq=max((l + 15) // 16 for l in kv_lens))
    seqs, ks, vs, qs = [], [], [], []
    for kl in kv_lens:
        s = cache.add_seq()
        cache.reserve(s, kl)
        seqs.append(s)
        ks.append(workloads.randn((kl, 2, 128), torch.bfloat16, g))
        vs.append(workloads.randn((kl, 2, 128), torch.bfloat16, g))
        qs.append(workloads.randn((chunk, 12, 128), torch.bfloat16, g))
    helpers.append_all(cache, 0, seqs, ks, vs, NVIDIA)
    q = torch.cat(qs).cuda()
    q_lens = [chunk] * len(ctxs)
    out = torch.full_like(q, float("nan"))
    cache.prefill(0, out, q, seqs, q_lens, kv_lens, 12, 128 ** -0.5)
    cache.check()
    assert cache.last_kernel() == llaisys.Kernel.PREFILL_TC
    for _ in range(5):
        again = torch.full_like(q, float("nan"))
        cache.prefill(0, again, q, seqs, q_lens, kv_lens, 12, 128 ** -0.5)
        cache.check()
        assert torch.equal(helpers.tensor_words(again.cpu()), helpers.tensor_words(out.cpu()))
    out = out.cpu()
    assert not out.float().isnan().any()
    for i in range(len(ctxs)):
        expect = attention.self_attention(qs[i], ks[i], vs[i], 128 ** -0.5)
        assert helpers.max_abs(out[i * chunk:(i + 1) * chunk], expect) <= helpers.MAX_ABS["bf16"], (i, ctxs[i])


@pytest.mark.gpu
def test_prefill_many_short_sequences_and_one_long_chunk_nvidia(cuda_device):
    """More sequences than the kernel has threads per CTA (its prologue sums and scans the sequences' block counts in
    rounds of one sequence per thread), most with a chunk of one to three rows, some with none, and one whole prompt
    of 1500 rows without context (12 row blocks of one sequence)."""
    g = torch.Generator().manual_seed(29)
    n = 300
    q_lens = [int(x) for x in torch.randint(0, 4, (n,), generator=g)]
    ctxs = [int(x) for x in torch.randint(0, 90, (n,), generator=g)]
    q_lens[137], ctxs[137] = 1500, 0
    kv_lens = [c + q for c, q in zip(ctxs, q_lens)]
    pages = sum((l + 15) // 16 for l in kv_lens) + 8
    cache = llaisys.PagedKVCache(pages, 2, 128, dtype=llaisys.DataType.BF16, device=NVIDIA, max_seqs=n, max_pages_per_seq=96)
    seqs, ks, vs, qs = [], [], [], []
    for ql, kl in zip(q_lens, kv_lens):
        s = cache.add_seq()
        cache.reserve(s, kl)
        seqs.append(s)
        ks.append(workloads.randn((kl, 2, 128), torch.bfloat16, g))
        vs.append(workloads.randn((kl, 2, 128), torch.bfloat16, g))
        qs.append(workloads.randn((ql, 12, 128), torch.bfloat16, g))
    helpers.append_all(cache, 0, seqs, ks, vs, NVIDIA)
    q = torch.cat(qs).cuda()
    out = torch.full_like(q, float("nan"))
    cache.prefill(0, out, q, seqs, q_lens, kv_lens, 12, 128 ** -0.5)
    cache.check()
    out = out.cpu()
    assert not out.float().isnan().any()
    at = 0
    for i, ql in enumerate(q_lens):
        if ql:
            expect = attention.self_attention(qs[i], ks[i], vs[i], 128 ** -0.5)
            assert helpers.max_abs(out[at:at + ql], expect) <= helpers.MAX_ABS["bf16"], (i, ql, kv_lens[i])
        at += ql


@pytest.mark.gpu
def test_back_to_back_steps_with_launch_overlap_nvidia(cuda_device):
    """Sixteen decode steps queued without any host synchronisation, with programmatic dependent launch enabled: each
    step appends one new row per sequence and attends over the grown context. Every step's output must match the
    oracle -- the kernels may only overlap in the parts that do not depend on their predecessor."""
    steps, nseq = 16, 5
    batch = workloads.decode_batch(nseq, 40, 900, seed=61, pool_pages=512)
    cache, seqs = helpers.build_cache(NVIDIA, "bf16", [p for p in batch.pages], num_pages=512, nkvh=2, d=128)
    cache.set_launch_overlap(True)
    start = [c - steps for c in batch.ctx]  # context before the first step
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, NVIDIA, hi=start)
    cache.flush()
    stream = llaisys.context_stream()
    ids = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(62)
    qs = [workloads.randn((nseq, 12, 128), torch.bfloat16, g) for _ in range(steps)]
    # everything the kernels index with is prepared before the first launch
    pos_dev = [torch.tensor([st + t for st in start], dtype=torch.int32, device="cuda") for t in range(steps)]
    len_dev = [torch.tensor([st + t + 1 for st in start], dtype=torch.int32, device="cuda") for t in range(steps)]
    k_new = [torch.stack([batch.k[i][start[i] + t] for i in range(nseq)]).cuda() for t in range(steps)]
    v_new = [torch.stack([batch.v[i][start[i] + t] for i in range(nseq)]).cuda() for t in range(steps)]
    q_dev = [q.cuda() for q in qs]
    outs = [torch.full((nseq, 12, 128), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(steps)]
    torch.cuda.synchronize()
    for t in range(steps):
        cache.append_dev(0, k_new[t], v_new[t], ids, pos_dev[t], nseq, stream)
        cache.decode_dev(0, outs[t], q_dev[t], ids, len_dev[t], nseq, max(batch.ctx), 12, batch.scale, stream)
    cache.check()
    for t in range(steps):
        got = outs[t].cpu()
        for i in range(nseq):
            n = start[i] + t + 1
            expect = attention.self_attention(qs[t][i:i + 1], batch.k[i][:n], batch.v[i][:n], batch.scale)
            assert helpers.max_abs(got[i:i + 1], expect) <= helpers.MAX_ABS["bf16"], (t, i)


@pytest.mark.gpu
def test_back_to_back_prefill_chunks_with_launch_overlap_nvidia(cuda_device):
    """Six rounds of "append a chunk per sequence, attend over the grown context" on ONE layer, queued without any host
    synchronisation and with programmatic dependent launch on: the chunk kernel may do its set-up under the append
    before it, the next append may be scheduled under the chunk kernel, and yet every round must match the oracle."""
    rounds, chunk, nseq = 6, 150, 3
    g = torch.Generator().manual_seed(71)
    start = [700, 0, 2300]
    total = [s + rounds * chunk for s in start]
    ks = [workloads.randn((n, 2, 128), torch.bfloat16, g) for n in total]
    vs = [workloads.randn((n, 2, 128), torch.bfloat16, g) for n in total]
    cache = llaisys.PagedKVCache(sum((n + 15) // 16 for n in total) + 4, 2, 128, dtype=llaisys.DataType.BF16, device=NVIDIA,
                                 max_seqs=nseq, max_pages_per_seq=max((n + 15) // 16 for n in total))
    seqs = []
    for n in total:
        s = cache.add_seq()
        cache.reserve(s, n)
        seqs.append(s)
    helpers.append_all(cache, 0, seqs, ks, vs, NVIDIA, hi=start)
    cache.flush()
    stream = llaisys.context_stream()
    ids = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    starts = torch.tensor([i * chunk for i in range(nseq + 1)], dtype=torch.int32, device="cuda")
    qs = [workloads.randn((nseq * chunk, 12, 128), torch.bfloat16, g) for _ in range(rounds)]
    # everything the kernels index with is prepared before the first launch
    row_seq = torch.repeat_interleave(ids, chunk)
    row_pos, lens, k_new, v_new = [], [], [], []
    for r in range(rounds):
        row_pos.append(torch.cat([torch.arange(st + r * chunk, st + (r + 1) * chunk, dtype=torch.int32) for st in start]).cuda())
        lens.append(torch.tensor([st + (r + 1) * chunk for st in start], dtype=torch.int32, device="cuda"))
        k_new.append(torch.cat([ks[i][start[i] + r * chunk:start[i] + (r + 1) * chunk] for i in range(nseq)]).cuda())
        v_new.append(torch.cat([vs[i][start[i] + r * chunk:start[i] + (r + 1) * chunk] for i in range(nseq)]).cuda())
    q_dev = [q.cuda() for q in qs]
    outs = [torch.full((nseq * chunk, 12, 128), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(rounds)]
    torch.cuda.synchronize()
    cache.set_launch_overlap(True)
    for r in range(rounds):
        cache.append_dev(0, k_new[r], v_new[r], row_seq, row_pos[r], nseq * chunk, stream)
        cache.prefill_dev(0, outs[r], q_dev[r], ids, starts, lens[r], nseq, nseq * chunk, chunk, max(total), 12, 128 ** -0.5,
                          stream)
    cache.check()
    assert cache.last_kernel() == llaisys.Kernel.PREFILL_TC
    for r in range(rounds):
        got = outs[r].cpu()
        for i in range(nseq):
            n = start[i] + (r + 1) * chunk
            expect = attention.self_attention(qs[r][i * chunk:(i + 1) * chunk], ks[i][:n], vs[i][:n], 128 ** -0.5)
            assert helpers.max_abs(got[i * chunk:(i + 1) * chunk], expect) <= helpers.MAX_ABS["bf16"], (r, i)


@pytest.mark.gpu
def test_kernel_flags_bad_metadata_instead_of_faulting_nvidia(cuda_device):
    """Device-array entry points do no host validation; a position past the block table is skipped and reported
    by check(), and the cache stays usable."""
    cache = llaisys.PagedKVCache(8, 2, 128, dtype=llaisys.DataType.BF16, device=NVIDIA, max_seqs=2,
                                 max_pages_per_seq=2)
    s = cache.add_seq()
    cache.reserve(s, 32)
    cache.flush()
    rows = torch.ones((2, 2, 128), dtype=torch.bfloat16, device="cuda")
    ids = torch.tensor([s, s], dtype=torch.int32, device="cuda")
    pos = torch.tensor([3, 9999], dtype=torch.int32, device="cuda")
    cache.append_dev(0, rows, rows, ids, pos, 2, llaisys.context_stream())
    with pytest.raises(LlaisysError) as e:
        cache.check()
    assert e.value.status == Status.KERNEL
    cache.check()  # flag was cleared
    k_out = torch.empty((4, 2, 128), dtype=torch.bfloat16, device="cuda")
    v_out = torch.empty_like(k_out)
    cache.gather(0, s, 4, k_out, v_out)
    cache.check()
    assert k_out[3].float().eq(1).all() and not k_out[:3].float().abs().any()
