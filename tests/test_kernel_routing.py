"""Which kernel serves which call. The library reports the kernel it queued (llaisysPagedKVLastKernel,
llaisysLastAttentionKernel); these tests pin that report at every benchmark configuration, so a parity test can never
pass on a kernel other than the one the numbers are quoted for. Inside the specialised kernels' domain (16-bit data,
head_dim 128, 16-token pages, at most 8 query heads per kv head) a call they cannot take fails with UNSUPPORTED and a
reason; it is not re-routed to the generic kernel."""
import pytest
import torch

import llaisys_b200 as llaisys
from llaisys_b200 import Kernel, LlaisysError, Status
from oracle import attention, workloads
from tests import helpers

CPU, NVIDIA = llaisys.DeviceType.CPU, llaisys.DeviceType.NVIDIA


def test_cpu_calls_report_the_host_loops():
    batch = workloads.decode_batch(3, 1, 60, seed=41, dtype=torch.float32, pool_pages=32)
    cache, seqs = helpers.build_cache(CPU, "f32", batch.pages, num_pages=32, nkvh=2, d=128)
    assert cache.last_kernel() == Kernel.NONE
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, CPU)
    out = torch.empty_like(batch.q)
    cache.decode(0, out, batch.q, seqs, batch.ctx, 12, batch.scale)
    assert cache.last_kernel() == Kernel.CPU and llaisys.last_attention_kernel() == Kernel.CPU
    q, k, v, scale = workloads.config1()
    helpers.run_self_attention(q, k, v, scale, CPU, "f32")
    assert llaisys.last_attention_kernel() == Kernel.CPU


@pytest.mark.gpu
def test_legacy_operator_routing_nvidia(cuda_device):
    """llaisysSelfAttention on plain tensors: one query -> cp.async split-KV kernel; 16 or more bf16 queries with
    head_dim 128 -> tcgen05 kernel; f32, other head dims and short multi-token queries -> generic kernel."""
    g = torch.Generator().manual_seed(5)

    def run(qlen, total, nh, nkvh, d, dname):
        dt = helpers.TORCH_DTYPE[dname]
        q = workloads.randn((qlen, nh, d), dt, g)
        k = workloads.randn((total, nkvh, d), dt, g)
        v = workloads.randn((total, nkvh, d), dt, g)
        got = helpers.run_self_attention(q, k, v, d ** -0.5, NVIDIA, dname)
        expect = attention.self_attention(q, k, v, d ** -0.5)
        assert helpers.max_abs(got, expect) <= helpers.MAX_ABS[dname]
        return llaisys.last_attention_kernel()

    assert run(1, 513, 12, 2, 128, "bf16") == Kernel.DECODE_CP_ASYNC
    assert run(1, 700, 12, 2, 128, "f16") == Kernel.DECODE_CP_ASYNC
    assert run(16, 16, 12, 2, 128, "bf16") == Kernel.PREFILL_TC
    assert run(200, 650, 12, 2, 128, "f16") == Kernel.PREFILL_TC
    assert run(5, 11, 12, 2, 128, "bf16") == Kernel.GENERIC      # 2..15 queries: a 128-row tile would be padding
    assert run(1, 513, 12, 2, 128, "f32") == Kernel.GENERIC       # configuration 1
    assert run(5, 11, 4, 2, 8, "bf16") == Kernel.GENERIC          # the reference's own test shape
    assert run(1, 40, 18, 2, 128, "bf16") == Kernel.GENERIC       # 9 query heads per kv head


@pytest.mark.gpu
def test_paged_calls_report_their_kernel_nvidia(cuda_device):
    batch = workloads.decode_batch(4, 1, 500, seed=42, pool_pages=256)
    cache, seqs = helpers.build_cache(NVIDIA, "bf16", batch.pages, num_pages=256, nkvh=2, d=128)
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, NVIDIA)
    out = torch.empty_like(batch.q, device="cuda")
    cache.decode(0, out, batch.q.cuda(), seqs, batch.ctx, 12, batch.scale)
    assert cache.last_kernel() == Kernel.DECODE_TMA
    part = torch.empty((4, 12, 130), dtype=torch.float32, device="cuda")
    cache.decode_partial(0, part, batch.q.cuda(), seqs, batch.ctx, 12, batch.scale)
    assert cache.last_kernel() == Kernel.DECODE_TMA
    chunk = min(batch.ctx)
    q = workloads.randn((chunk, 12, 128), torch.bfloat16, torch.Generator().manual_seed(1)).cuda()
    out_c = torch.empty_like(q)
    cache.prefill(0, out_c, q, seqs[:1], [chunk], [batch.ctx[0]], 12, batch.scale)
    assert cache.last_kernel() == Kernel.PREFILL_TC
    cache.check()
    # pools outside the specialised kernels' shapes are the generic kernel's
    for dname, d in (("f32", 128), ("bf16", 64)):
        b2 = workloads.decode_batch(2, 1, 90, seed=43, dtype=helpers.TORCH_DTYPE[dname], pool_pages=32, d=d)
        c2, s2 = helpers.build_cache(NVIDIA, dname, b2.pages, num_pages=32, nkvh=2, d=d)
        helpers.append_all(c2, 0, s2, b2.k, b2.v, NVIDIA)
        o2 = torch.empty_like(b2.q, device="cuda")
        c2.decode(0, o2, b2.q.cuda(), s2, b2.ctx, 12, b2.scale)
        c2.check()
        assert c2.last_kernel() == Kernel.GENERIC


@pytest.mark.gpu
def test_call_the_fast_kernels_cannot_take_is_refused_not_rerouted_nvidia(cuda_device):
    batch = workloads.decode_batch(2, 20, 200, seed=44, pool_pages=64)
    cache, seqs = helpers.build_cache(NVIDIA, "bf16", batch.pages, num_pages=64, nkvh=2, d=128)
    helpers.append_all(cache, 0, seqs, batch.k, batch.v, NVIDIA)
    # a query buffer that starts on an odd 2-byte boundary: the decode kernel loads q in 4-byte words
    flat = torch.zeros(batch.q.numel() + 8, dtype=torch.bfloat16, device="cuda")
    q_odd = flat[1:1 + batch.q.numel()].view(batch.q.shape)
    q_odd.copy_(batch.q)
    out = torch.empty_like(batch.q, device="cuda")
    with pytest.raises(LlaisysError) as e:
        cache.decode(0, out, q_odd, seqs, batch.ctx, 12, batch.scale)
    assert e.value.status == Status.UNSUPPORTED and "aligned" in str(e.value)
    # a chunk whose output is not 16-byte aligned
    chunk = 20
    qc = torch.zeros((chunk, 12, 128), dtype=torch.bfloat16, device="cuda")
    oc = flat.new_zeros(qc.numel() + 8)[1:1 + qc.numel()].view(qc.shape)
    with pytest.raises(LlaisysError) as e:
        cache.prefill(0, oc, qc, seqs[:1], [chunk], [batch.ctx[0]], 12, batch.scale)
    assert e.value.status == Status.UNSUPPORTED
    # the cache is still usable and still on its kernel
    cache.decode(0, out, batch.q.cuda(), seqs, batch.ctx, 12, batch.scale)
    cache.check()
    assert cache.last_kernel() == Kernel.DECODE_TMA


@pytest.mark.gpu
def test_more_sequences_than_one_launch_takes_nvidia(cuda_device):
    """1100 one-page sequences: the decode call is cut into launches of at most 1024 sequences, all on the TMA kernel."""
    n = 1100
    g = torch.Generator().manual_seed(45)
    cache = llaisys.PagedKVCache(n, 2, 128, dtype=llaisys.DataType.BF16, device=NVIDIA, max_seqs=n, max_pages_per_seq=1)
    ctx = torch.randint(1, 17, (n,), generator=g).tolist()
    seqs, ks, vs = [], [], []
    for c in ctx:
        s = cache.add_seq()
        cache.reserve(s, c)
        seqs.append(s)
        ks.append(workloads.randn((c, 2, 128), torch.bfloat16, g))
        vs.append(workloads.randn((c, 2, 128), torch.bfloat16, g))
    helpers.append_all(cache, 0, seqs, ks, vs, NVIDIA)
    q = workloads.randn((n, 12, 128), torch.bfloat16, g)
    out = torch.empty_like(q, device="cuda")
    cache.decode(0, out, q.cuda(), seqs, ctx, 12, 128 ** -0.5)
    cache.check()
    assert cache.last_kernel() == Kernel.DECODE_TMA
    out = out.cpu()
    for i in (0, 1, 511, 1023, 1024, 1099):
        expect = attention.self_attention(q[i:i + 1], ks[i], vs[i], 128 ** -0.5)
        assert helpers.max_abs(out[i:i + 1], expect) <= helpers.MAX_ABS["bf16"], i
