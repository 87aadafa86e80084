"""Split-KV decode through peer memory (llaisysPeerExchange*, one process per GPU on one node): every rank must end up
with the attention over the WHOLE sequence, step after step (the slots alternate by step parity, the flags carry the
step number) and when the step is replayed as a CUDA graph. Needs two GPUs; the merge arithmetic itself is covered on
CPU by the LSE-merge tests. With a single rank (no process group) the same two kernels run on one GPU: the decode kernel
stores its partial rows into its own slot and stamps its own flag, the merge waits for that flag. A wait that runs out
is exercised on two GPUs by a rank that leaves one step out: nothing faults, nothing waits without a limit."""
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


def _worker(rank: int, world: int, port: int, results, total: int = 16 * 150 + 5, n_layers: int = 3):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import llaisys_b200 as llaisys
    from llaisys_b200 import sharding
    from tests import helpers

    nvidia = llaisys.DeviceType.NVIDIA
    llaisys.set_context_runtime(nvidia, rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ex = None
    try:
        dev = torch.device("cuda", rank)
        stream = llaisys.context_stream()
        ext = torch.cuda.ExternalStream(stream)
        g = torch.Generator().manual_seed(91)
        nh, nkvh, d = 12, 2, 128  # (default total: the last rank's slice ends inside a page)
        lo, hi = sharding.kv_range(total, world, rank)
        local = hi - lo
        ks = [workloads.randn((total, nkvh, d), torch.bfloat16, g) for _ in range(n_layers)]
        vs = [workloads.randn((total, nkvh, d), torch.bfloat16, g) for _ in range(n_layers)]
        # each "layer" is a sequence of one cache layer, as the long-context benchmark lays them out
        cache = llaisys.PagedKVCache(max(1024, n_layers * (-(-local // 16) + 1)), nkvh, d, dtype=llaisys.DataType.BF16,
                                     device=nvidia, device_id=rank, max_seqs=n_layers, max_pages_per_seq=-(-local // 16) + 1)
        seqs = []
        for layer in range(n_layers):
            s = cache.add_seq()
            cache.reserve(s, local)
            cache.append(0, ks[layer][lo:hi].contiguous().to(dev), vs[layer][lo:hi].contiguous().to(dev), [s] * local,
                         list(range(local)))
            seqs.append(s)
        cache.flush()
        seq_dev = torch.tensor(seqs, dtype=torch.int32, device=dev)
        len_dev = torch.full((n_layers,), local, dtype=torch.int32, device=dev)
        ex = sharding.PeerExchange(n_layers * nh, d, device_id=rank)
        worst = 0.0
        outs = []
        for step in range(5):  # different queries every step: a stale slot or flag would show
            q = workloads.randn((n_layers, nh, d), torch.bfloat16, torch.Generator().manual_seed(1000 + step))
            out = torch.zeros((n_layers, nh, d), dtype=torch.bfloat16, device=dev)
            ex.split_decode(cache, 0, out, q.to(dev), seq_dev, len_dev, n_layers, local, nh, 0.09, stream)
            ex.check(stream)
            cache.check()
            for layer in range(n_layers):
                if total > 20000:  # a full-length layer: the chunked float64 oracle, on the first and the last step only
                    if step not in (0, 4):
                        continue
                    full = attention.decode_attention_f64_chunked(q[layer:layer + 1], ks[layer], vs[layer], 0.09)
                else:
                    full = attention.self_attention_f64(q[layer:layer + 1], ks[layer], vs[layer], 0.09)
                worst = max(worst, helpers.max_abs(out[layer:layer + 1].cpu(), full))
            outs.append(out.cpu())
        # the same step as a CUDA graph, replayed: the step number lives on the device, so replays keep alternating
        # slots; every replay must reproduce the eager result of the same query bit for bit
        q_dev = workloads.randn((n_layers, nh, d), torch.bfloat16, torch.Generator().manual_seed(1004)).to(dev)
        out_g = torch.zeros((n_layers, nh, d), dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=ext):
            ex.split_decode(cache, 0, out_g, q_dev, seq_dev, len_dev, n_layers, local, nh, 0.09, stream)
        same = True
        for _ in range(7):
            out_g.zero_()
            torch.cuda.synchronize()
            with torch.cuda.stream(ext):
                graph.replay()
            ex.check(stream)
            same = same and torch.equal(helpers.tensor_words(out_g.cpu()), helpers.tensor_words(outs[4]))
        dist.barrier()
        results[rank] = (worst, same, (lo, hi))
    finally:
        if ex is not None:
            ex.close()
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.timeout(600)
def test_split_decode_through_peer_memory():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, free_port(), results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            worst, same, _ = results[rank]
            assert worst <= 8e-3, (rank, worst)
            assert same, f"rank {rank}: a graph replay differs from the eager step"


@pytest.mark.gpu
@pytest.mark.timeout(900)
def test_split_decode_of_one_full_131072_token_layer_through_peer_memory():
    """One layer of the long-context configuration at its full length, split over the GPUs of the box (up to 4): the
    merged rows against the float64 oracle over all 131072 tokens, and graph replays bit for bit."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, free_port(), results, 131072, 1), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            worst, same, _ = results[rank]
            assert worst <= 8e-3, (rank, worst)
            assert same, f"rank {rank}: a graph replay differs from the eager step"


@pytest.mark.gpu
def test_single_rank_exchange_on_one_gpu(cuda_device):
    """World size 1: the decode kernel's exchange mode (rows stored into slot 0 of the rank's own buffer, pair counting,
    flag) and the merge kernel, eager for changing queries and lengths and then as a replayed CUDA graph. Lengths cover
    an empty sequence, pairs that fit one CTA and pairs that are cut over many."""
    import llaisys_b200 as llaisys
    from llaisys_b200 import sharding
    from tests import helpers

    nvidia = llaisys.DeviceType.NVIDIA
    stream = llaisys.context_stream()
    ext = torch.cuda.ExternalStream(stream)
    g = torch.Generator().manual_seed(17)
    lens = [3000, 0, 17, 500, 1]
    n = len(lens)
    ks = [workloads.randn((c, 2, 128), torch.bfloat16, g) for c in lens]
    vs = [workloads.randn((c, 2, 128), torch.bfloat16, g) for c in lens]
    cache = llaisys.PagedKVCache(512, 2, 128, dtype=llaisys.DataType.BF16, device=nvidia, max_seqs=n, max_pages_per_seq=200)
    seqs = []
    for c in lens:
        s = cache.add_seq()
        cache.reserve(s, max(c, 1))
        seqs.append(s)
    helpers.append_all(cache, 0, seqs, ks, vs, nvidia)
    cache.flush()
    seq_dev = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    ex = sharding.PeerExchange(n * 12, 128, device_id=0)
    try:
        for step in range(4):
            cut = [c if step % 2 == 0 else c // 2 for c in lens]
            len_dev = torch.tensor(cut, dtype=torch.int32, device="cuda")
            q = workloads.randn((n, 12, 128), torch.bfloat16, torch.Generator().manual_seed(200 + step))
            out = torch.full((n, 12, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
            ex.split_decode(cache, 0, out, q.cuda(), seq_dev, len_dev, n, max(lens), 12, 0.09, stream)
            ex.check(stream)
            cache.check()
            assert cache.last_kernel() == llaisys.Kernel.DECODE_TMA
            out = out.cpu()
            for i, c in enumerate(cut):
                if c == 0:
                    assert not out[i].float().abs().any()
                    continue
                full = attention.self_attention_f64(q[i:i + 1], ks[i][:c], vs[i][:c], 0.09)
                assert helpers.max_abs(out[i:i + 1], full) <= 8e-3, (step, i)
        # graph replays: the step counter lives on the device
        q_dev = workloads.randn((n, 12, 128), torch.bfloat16, torch.Generator().manual_seed(300)).cuda()
        len_dev = torch.tensor(lens, dtype=torch.int32, device="cuda")
        out_g = torch.zeros((n, 12, 128), dtype=torch.bfloat16, device="cuda")
        ex.split_decode(cache, 0, out_g, q_dev, seq_dev, len_dev, n, max(lens), 12, 0.09, stream)
        ex.check(stream)
        eager = out_g.cpu().clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=ext):
            ex.split_decode(cache, 0, out_g, q_dev, seq_dev, len_dev, n, max(lens), 12, 0.09, stream)
        for _ in range(5):
            out_g.zero_()
            torch.cuda.synchronize()
            with torch.cuda.stream(ext):
                graph.replay()
            ex.check(stream)
            assert torch.equal(helpers.tensor_words(out_g.cpu()), helpers.tensor_words(eager))
    finally:
        ex.close()


def _timeout_worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import llaisys_b200 as llaisys
    from llaisys_b200 import sharding
    from tests import helpers

    nvidia = llaisys.DeviceType.NVIDIA
    llaisys.set_context_runtime(nvidia, rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ex = None
    try:
        dev = torch.device("cuda", rank)
        stream = llaisys.context_stream()
        g = torch.Generator().manual_seed(5)
        total = 16 * 64
        k = workloads.randn((total, 2, 128), torch.bfloat16, g)
        v = workloads.randn((total, 2, 128), torch.bfloat16, g)
        q = workloads.randn((1, 12, 128), torch.bfloat16, g)
        lo, hi = sharding.kv_range(total, world, rank)
        cache = llaisys.PagedKVCache(128, 2, 128, dtype=llaisys.DataType.BF16, device=nvidia, device_id=rank, max_seqs=1)
        s = cache.add_seq()
        cache.reserve(s, hi - lo)
        cache.append(0, k[lo:hi].contiguous().to(dev), v[lo:hi].contiguous().to(dev), [s] * (hi - lo), list(range(hi - lo)))
        cache.flush()
        seq_dev = torch.tensor([s], dtype=torch.int32, device=dev)
        len_dev = torch.tensor([hi - lo], dtype=torch.int32, device=dev)
        full = attention.self_attention_f64(q, k, v, 0.09)

        def step(exchange):
            out = torch.zeros((1, 12, 128), dtype=torch.bfloat16, device=dev)
            exchange.split_decode(cache, 0, out, q.to(dev), seq_dev, len_dev, 1, hi - lo, 12, 0.09, stream)
            return out

        ex = sharding.PeerExchange(12, 128, device_id=rank)
        ex.set_wait_limit(1 << 19)  # about a quarter of a second instead of a second
        first = step(ex)
        assert ex.status(stream) == 0
        ok_first = helpers.max_abs(first.cpu(), full) <= 8e-3
        dist.barrier()
        # rank 1 leaves this step out (between steps, nothing of it in flight): rank 0's merge gives up after the limit
        statuses = None
        if rank == 0:
            step(ex)
            statuses = (ex.status(stream), ex.status(stream))  # reported once, then clear
        dist.barrier()
        # the step counters have diverged: every rank closes its exchange and makes a new one
        ex.close()
        ex = sharding.PeerExchange(12, 128, device_id=rank)
        again = step(ex)
        assert ex.status(stream) == 0
        ok_again = helpers.max_abs(again.cpu(), full) <= 8e-3
        cache.check()
        results[rank] = (ok_first, statuses, ok_again)
    finally:
        if ex is not None:
            ex.close()
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.timeout(600)
def test_a_wait_for_a_missing_peer_runs_out_and_the_exchange_recovers():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_timeout_worker, args=(2, free_port(), results), nprocs=2, join=True)
        assert len(results) == 2
        assert results[0][0] and results[1][0], "the normal step before the missing one is wrong"
        assert results[0][1] == (1, 0), f"rank 0 should report one timed-out wait, then nothing: {results[0][1]}"
        assert results[0][2] and results[1][2], "the step after re-creating the exchange is wrong"

