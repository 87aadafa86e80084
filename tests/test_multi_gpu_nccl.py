"""The two multi-GPU modes on real GPUs over NCCL (one process per GPU): whole sequences per rank with no collective,
and one long sequence split by KV range with a single all-gather and the log-sum-exp merge. Needs two or more GPUs in
the box; the same logic runs on CPU ranks over gloo in test_multi_rank_gloo.py."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention, workloads


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import llaisys_b200 as llaisys
    from llaisys_b200 import sharding
    from tests import helpers

    nvidia = llaisys.DeviceType.NVIDIA
    llaisys.set_context_runtime(nvidia, rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        # ---- mode 1: whole sequences per rank ----
        batch = workloads.decode_batch(7, 1, 1200, seed=51, pool_pages=1024)
        mine = sharding.shard_sequences(batch.ctx, world)[rank]
        cache = llaisys.PagedKVCache(1024, 2, 128, dtype=llaisys.DataType.BF16, device=nvidia, device_id=rank,
                                     max_seqs=max(len(mine), 1), max_pages_per_seq=80)
        seqs = []
        for i in mine:
            s = cache.add_seq()
            cache.assign_pages(s, batch.pages[i])
            seqs.append(s)
        dev = torch.device("cuda", rank)
        ids, pos = [], []
        for s, i in zip(seqs, mine):
            ids += [s] * batch.ctx[i]
            pos += list(range(batch.ctx[i]))
        cache.append(0, torch.cat([batch.k[i] for i in mine]).to(dev), torch.cat([batch.v[i] for i in mine]).to(dev), ids, pos)
        q = batch.q[mine].contiguous().to(dev)
        out = torch.empty_like(q)
        cache.decode(0, out, q, seqs, [batch.ctx[i] for i in mine], 12, batch.scale)
        cache.check()
        worst = 0.0
        for n, i in enumerate(mine):
            expect = attention.self_attention(batch.q[i:i + 1], batch.k[i], batch.v[i], batch.scale)
            worst = max(worst, helpers.max_abs(out[n:n + 1].cpu(), expect))

        # ---- mode 2: one long sequence, KV range split across the ranks ----
        g = torch.Generator().manual_seed(78)
        total = 16 * 301 + 9
        qq = workloads.randn((1, 12, 128), torch.bfloat16, g)
        kk = workloads.randn((total, 2, 128), torch.bfloat16, g)
        vv = workloads.randn((total, 2, 128), torch.bfloat16, g)
        lo, hi = sharding.kv_range(total, world, rank)
        cache2 = llaisys.PagedKVCache(512, 2, 128, dtype=llaisys.DataType.BF16, device=nvidia, device_id=rank, max_seqs=1)
        s2 = cache2.add_seq()
        cache2.reserve(s2, hi - lo)
        cache2.append(0, kk[lo:hi].contiguous().to(dev), vv[lo:hi].contiguous().to(dev), [s2] * (hi - lo), list(range(hi - lo)))
        merged = torch.empty((1, 12, 128), dtype=torch.bfloat16, device=dev)
        sharding.split_decode(cache2, 0, merged, qq.to(dev), [s2], [hi - lo], 12, 0.09)
        cache2.check()
        torch.cuda.synchronize()
        full = attention.self_attention_f64(qq, kk, vv, 0.09)
        results[rank] = (mine, worst, helpers.max_abs(merged.cpu(), full), (lo, hi))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.timeout(600)
def test_sequence_sharding_and_kv_range_split_over_nccl():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs in the box")
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, free_port(), results), nprocs=world, join=True)
        assert set(results.keys()) == set(range(world))
        covered = sorted(i for r in range(world) for i in results[r][0])
        assert covered == list(range(7))
        for r in range(world):
            _, worst, merged_err, _ = results[r]
            assert worst <= 2e-2
            assert merged_err <= 8e-3  # one bf16 ulp of the merged output
        assert results[0][3][0] == 0 and results[world - 1][3][1] == 16 * 301 + 9
