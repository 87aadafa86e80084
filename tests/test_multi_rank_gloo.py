"""World-size-2 runs of the two multi-GPU modes on CPU ranks (gloo): sequence sharding with no collective, and
the KV-range split with one all-gather and a log-sum-exp merge."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import llaisys_b200 as llaisys
from llaisys_b200 import sharding
from oracle import attention, workloads
from tests import helpers

CPU = llaisys.DeviceType.CPU


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_sequences_balances_and_covers():
    ctx = [4096, 128, 3000, 2999, 17, 800, 4095, 1]
    for world in (1, 2, 3, 8):
        shards = sharding.shard_sequences(ctx, world)
        assert sorted(i for s in shards for i in s) == list(range(len(ctx)))
        loads = [sum(ctx[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(ctx)


def test_kv_range_is_a_page_aligned_partition():
    for total in (0, 1, 15, 16, 17, 1000, 131072):
        for world in (1, 2, 3, 8):
            cuts = [sharding.kv_range(total, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == total
            for (a, b), (c, _) in zip(cuts[:-1], cuts[1:]):
                assert b == c and a <= b and (b % 16 == 0 or b == total)


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        # ---- mode 1: whole sequences per rank, no collective on the data path ----
        batch = workloads.decode_batch(5, 1, 200, seed=31, pool_pages=128)
        mine = sharding.shard_sequences(batch.ctx, world)[rank]
        cache, seqs = helpers.build_cache(CPU, "bf16", [batch.pages[i] for i in mine], num_pages=128, nkvh=2, d=128)
        helpers.append_all(cache, 0, seqs, [batch.k[i] for i in mine], [batch.v[i] for i in mine], CPU)
        q = batch.q[mine].contiguous()
        out = torch.empty_like(q)
        cache.decode(0, out, q, seqs, [batch.ctx[i] for i in mine], 12, batch.scale)
        worst = 0.0
        for n, i in enumerate(mine):
            expect = attention.self_attention(batch.q[i:i + 1], batch.k[i], batch.v[i], batch.scale)
            worst = max(worst, helpers.max_abs(out[n:n + 1], expect))
        # host-side gather of results only
        gathered = [None] * world
        dist.all_gather_object(gathered, (mine, worst))

        # ---- mode 2: one long sequence, KV range split across ranks ----
        g = torch.Generator().manual_seed(77)
        total = 16 * 37 + 5
        qq = workloads.randn((1, 12, 128), torch.bfloat16, g)
        kk = workloads.randn((total, 2, 128), torch.bfloat16, g)
        vv = workloads.randn((total, 2, 128), torch.bfloat16, g)
        lo, hi = sharding.kv_range(total, world, rank)
        cache2 = llaisys.PagedKVCache(64, 2, 128, dtype=llaisys.DataType.BF16, max_seqs=1)
        s = cache2.add_seq()
        cache2.reserve(s, hi - lo)
        helpers.append_all(cache2, 0, [s], [kk[lo:hi]], [vv[lo:hi]], CPU)
        merged = torch.empty_like(qq)
        sharding.split_decode(cache2, 0, merged, qq, [s], [hi - lo], 12, 0.09)
        full = attention.self_attention_f64(qq, kk, vv, 0.09)
        results[rank] = (gathered, helpers.max_abs(merged, full), (lo, hi))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_ranks_sequence_sharding_and_kv_range_split():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, free_port(), results), nprocs=world, join=True)
        assert set(results.keys()) == {0, 1}
        gathered, err0, r0 = results[0]
        _, err1, r1 = results[1]
        covered = sorted(i for mine, _ in gathered for i in mine)
        assert covered == [0, 1, 2, 3, 4]
        assert all(worst <= 2e-2 for _, worst in gathered)
        assert r0[1] == r1[0] and r0[0] == 0
        assert err0 <= 8e-3 and err1 <= 8e-3  # one bf16 ulp of the merged output


def _worker_missing_rank(rank: int, world: int, ports, results, rank0_gave_up):
    """Step 1 normal; in step 2 rank 1 leaves its collective out (a host-side failure: nothing faults, nobody exits);
    rank 0's all-gather ends with an error after the group's short timeout; both ranks then tear the group down, build a
    new one and step 3 is normal again."""
    import datetime

    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(78)
    total = 16 * 21 + 3
    qq = workloads.randn((1, 12, 128), torch.bfloat16, g)
    kk = workloads.randn((total, 2, 128), torch.bfloat16, g)
    vv = workloads.randn((total, 2, 128), torch.bfloat16, g)
    lo, hi = sharding.kv_range(total, world, rank)
    cache = llaisys.PagedKVCache(64, 2, 128, dtype=llaisys.DataType.BF16, max_seqs=1)
    s = cache.add_seq()
    cache.reserve(s, hi - lo)
    helpers.append_all(cache, 0, [s], [kk[lo:hi]], [vv[lo:hi]], CPU)
    full = attention.self_attention_f64(qq, kk, vv, 0.09)

    def step():
        merged = torch.empty_like(qq)
        sharding.split_decode(cache, 0, merged, qq, [s], [hi - lo], 12, 0.09)
        return helpers.max_abs(merged, full)

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(ports[0]))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    first = step()
    failed = None
    if rank == 0:
        try:
            step()  # rank 1 never joins this one
        except Exception as e:  # the process group's timeout (the kind of exception is the backend's)
            failed = type(e).__name__
        rank0_gave_up.set()
    else:
        rank0_gave_up.wait(timeout=60)  # learns on the host that the step is lost, between steps
    try:
        dist.destroy_process_group()
    except Exception:
        pass  # a group whose collective timed out may refuse an orderly shutdown
    os.environ["MASTER_PORT"] = str(ports[1])
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        third = step()
    finally:
        dist.destroy_process_group()
    results[rank] = (first, failed, third)


@pytest.mark.timeout(300)
def test_a_rank_that_leaves_a_step_out_ends_the_others_collective_with_an_error():
    """Failure detection on the collective path, without a GPU: the process group's timeout is the bounded wait."""
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        gave_up = manager.Event()
        mp.spawn(_worker_missing_rank, args=(world, (free_port(), free_port()), results, gave_up), nprocs=world, join=True)
        assert set(results.keys()) == {0, 1}
        for rank in (0, 1):
            first, _, third = results[rank]
            assert first <= 8e-3 and third <= 8e-3, (rank, first, third)
        assert results[0][1] is not None, "rank 0's collective should have ended with an error"
        assert results[1][1] is None
