"""Prefix-sharing KV pool (reference-counted pages, publish / match by token prefix, fork with a copied last page):
the block manager against the Python restatement of its contract on random operation sequences, and the data path
(gather, decode attention) over shared pages against the attention oracle."""
import random

import numpy as np
import pytest
import torch

import llaisys_b200 as llaisys
from llaisys_b200 import LlaisysError, Status
from oracle import attention, workloads
from oracle.prefix import PrefixPoolModel
from tests import helpers

CPU, NVIDIA = llaisys.DeviceType.CPU, llaisys.DeviceType.NVIDIA
PAGE = 16


def make_cache(device, num_pages, max_seqs, max_pages_per_seq, dname="bf16", nkvh=2, d=128, nlayer=1):
    return llaisys.PagedKVCache(num_pages, nkvh, d, nlayer=nlayer, dtype=helpers.LL_DTYPE[dname], device=device,
                                max_seqs=max_seqs, max_pages_per_seq=max_pages_per_seq)


def same_state(cache, model: PrefixPoolModel):
    assert cache.num_free_pages() == model.num_free()
    assert cache.num_cached_pages() == len(model.cached)
    assert cache.num_seqs() == len(model.tables)
    for seq, table in model.tables.items():
        assert cache.seq_pages(seq) == table, f"sequence {seq}"
    for page in range(model.num_pages):
        assert cache.page_ref_count(page) == model.ref[page], f"page {page}"


def test_block_manager_matches_the_model_on_random_operations():
    rng = random.Random(7)
    num_pages, max_seqs, mpps = 24, 6, 8
    cache = make_cache(CPU, num_pages, max_seqs, mpps)
    model = PrefixPoolModel(num_pages, PAGE, max_seqs, mpps)
    # a small family of token streams with shared prefixes, so that matches actually happen
    stems = [[rng.randrange(50) for _ in range(160)] for _ in range(3)]
    streams = []
    for stem in stems:
        for cut in (32, 64, 100):
            streams.append(stem[:cut] + [rng.randrange(50, 99) for _ in range(160 - cut)])
    held: dict[int, list[int]] = {}  # live sequence -> the tokens it holds
    for step in range(600):
        op = rng.choice(["new", "new", "grow", "free", "free", "fork", "publish"])
        try:
            if op == "new":
                tokens = rng.choice(streams)[: rng.randrange(1, 128)]
                seq_m = model.add_seq()
                seq = cache.add_seq()
                assert seq == seq_m
                matched = cache.match_prefix(seq, tokens)
                assert matched == model.match(seq, tokens)
                model.reserve(seq, len(tokens))  # the model first: if it refuses, the handler below replays the call
                cache.reserve(seq, len(tokens))
                held[seq] = tokens
            elif op == "grow" and held:
                seq = rng.choice(list(held))
                stream = next(s for s in streams if s[: len(held[seq])] == held[seq]) if any(
                    s[: len(held[seq])] == held[seq] for s in streams) else None
                if stream is None or len(held[seq]) >= 128:
                    continue
                n = min(128, len(held[seq]) + rng.randrange(1, 40))
                model.reserve(seq, n)
                cache.reserve(seq, n)
                held[seq] = stream[:n]
            elif op == "free" and held:
                seq = rng.choice(list(held))
                cache.free_seq(seq)
                model.free_seq(seq)
                del held[seq]
            elif op == "publish" and held:
                seq = rng.choice(list(held))
                cache.publish(seq, held[seq])
                model.publish(seq, held[seq])
            elif op == "fork" and held:
                parent = rng.choice(list(held))
                n = rng.randrange(0, len(held[parent]) + 1)
                child_m, _ = model.fork(parent, n)
                child = cache.fork(parent, n)
                assert child == child_m
                held[child] = held[parent][:n]
        except (MemoryError, KeyError) as exc:  # the model refused: the library must refuse the same call the same way
            want = Status.NO_PAGES if isinstance(exc, MemoryError) else Status.NO_SEQ
            with pytest.raises(LlaisysError) as err:
                if op == "new":
                    if isinstance(exc, KeyError):
                        cache.add_seq()
                    else:
                        cache.reserve(seq, len(tokens))
                elif op == "grow":
                    cache.reserve(seq, n)
                elif op == "fork":
                    cache.fork(parent, n)
            assert err.value.status == want
            if op == "new" and isinstance(exc, MemoryError):  # the sequence exists but could not grow: drop it
                cache.free_seq(seq)
                model.free_seq(seq)
        same_state(cache, model)
    assert len(model.cached) + sum(1 for r in model.ref if r > 1) > 0  # the run did exercise caching or sharing


def fill(cache, seq, k, v, lo, hi, device):
    dev = helpers.torch_device(device)
    ids, pos = [seq] * (hi - lo), list(range(lo, hi))
    cache.append(0, k[lo:hi].contiguous().to(dev), v[lo:hi].contiguous().to(dev), ids, pos)


def check_shared_data(device):
    dev = helpers.torch_device(device)
    g = torch.Generator().manual_seed(11)
    nh, nkvh, d = 12, 2, 128
    cache = make_cache(device, 32, 4, 8)
    tokens = list(range(100, 170))  # 70 tokens: 4 full pages and 6 tokens of a fifth
    k = workloads.randn((70, nkvh, d), torch.bfloat16, g)
    v = workloads.randn((70, nkvh, d), torch.bfloat16, g)
    a = cache.add_seq()
    cache.reserve(a, 70)
    fill(cache, a, k, v, 0, 70, device)
    cache.publish(a, tokens)

    # a second request with the same first 50 tokens finds 3 whole pages (48 tokens) and appends its own rest
    other = tokens[:50] + [7] * 10
    k2 = torch.cat([k[:50], workloads.randn((10, nkvh, d), torch.bfloat16, g)])
    v2 = torch.cat([v[:50], workloads.randn((10, nkvh, d), torch.bfloat16, g)])
    b = cache.add_seq()
    assert cache.match_prefix(b, other) == 48
    assert cache.seq_pages(b) == cache.seq_pages(a)[:3]
    assert [cache.page_ref_count(p) for p in cache.seq_pages(a)] == [2, 2, 2, 1, 1]
    cache.reserve(b, 60)
    fill(cache, b, k2, v2, 48, 60, device)

    # a fork in the middle of the parent's last page copies that page; both sides then grow independently
    c = cache.fork(a, 70)
    assert cache.seq_pages(c)[:4] == cache.seq_pages(a)[:4] and cache.seq_pages(c)[4] != cache.seq_pages(a)[4]
    ka, va = workloads.randn((5, nkvh, d), torch.bfloat16, g), workloads.randn((5, nkvh, d), torch.bfloat16, g)
    kc, vc = workloads.randn((5, nkvh, d), torch.bfloat16, g), workloads.randn((5, nkvh, d), torch.bfloat16, g)
    cache.reserve(a, 75)
    cache.reserve(c, 75)
    full_a, full_va = torch.cat([k, ka]), torch.cat([v, va])
    full_c, full_vc = torch.cat([k, kc]), torch.cat([v, vc])
    fill(cache, a, full_a, full_va, 70, 75, device)
    fill(cache, c, full_c, full_vc, 70, 75, device)

    expect = {a: (full_a, full_va), b: (k2, v2), c: (full_c, full_vc)}
    q = workloads.randn((3, nh, d), torch.bfloat16, g)
    out = torch.empty_like(q, device=dev)
    seqs = [a, b, c]
    lens = [75, 60, 75]
    cache.decode(0, out, q.to(dev), seqs, lens, nh, 1.0 / d ** 0.5)
    cache.check()
    out = out.cpu()
    for i, s in enumerate(seqs):
        ke, ve = expect[s]
        k_out = torch.empty((lens[i], nkvh, d), dtype=torch.bfloat16, device=dev)
        v_out = torch.empty_like(k_out)
        cache.gather(0, s, lens[i], k_out, v_out)
        assert torch.equal(helpers.tensor_words(k_out.cpu()), helpers.tensor_words(ke[: lens[i]]))
        assert torch.equal(helpers.tensor_words(v_out.cpu()), helpers.tensor_words(ve[: lens[i]]))
        want = attention.self_attention(q[i:i + 1], ke[: lens[i]], ve[: lens[i]], 1.0 / d ** 0.5)
        assert (out[i:i + 1].float() - want.float()).abs().max().item() <= 2e-2

    # releasing every holder keeps the published pages findable; a new request still matches them
    for s in seqs:
        cache.free_seq(s)
    assert cache.num_cached_pages() == 4 and cache.num_free_pages() == 32
    e = cache.add_seq()
    assert cache.match_prefix(e, tokens) == 64
    k_out = torch.empty((64, nkvh, d), dtype=torch.bfloat16, device=dev)
    v_out = torch.empty_like(k_out)
    cache.gather(0, e, 64, k_out, v_out)
    cache.check()
    assert torch.equal(helpers.tensor_words(k_out.cpu()), helpers.tensor_words(k[:64]))
    assert torch.equal(helpers.tensor_words(v_out.cpu()), helpers.tensor_words(v[:64]))


def test_shared_pages_hold_the_right_data_cpu():
    check_shared_data(CPU)


def test_cached_pages_are_evicted_oldest_first_and_only_when_needed():
    cache = make_cache(CPU, 6, 4, 6)
    t1, t2 = list(range(32)), list(range(100, 132))
    for toks in (t1, t2):
        s = cache.add_seq()
        cache.reserve(s, 32)
        cache.publish(s, toks)
        cache.free_seq(s)
    assert cache.num_cached_pages() == 4 and cache.num_free_pages() == 6
    s = cache.add_seq()
    # 2 plain free pages first, then the page released longest ago: a freed sequence lets go of its LAST page first, so
    # a chain loses its tail before its root
    cache.reserve(s, 48)
    assert cache.num_cached_pages() == 3
    probe = cache.add_seq()
    assert cache.match_prefix(probe, t1) == 16  # t1's second page is gone, its first still matches
    with pytest.raises(LlaisysError) as err:
        cache.match_prefix(probe, t2)  # not empty any more
    assert err.value.status == Status.INVALID
    probe2 = cache.add_seq()
    assert cache.match_prefix(probe2, t2) == 32
    with pytest.raises(LlaisysError) as err:
        cache.publish(probe2, list(range(64)))  # more tokens than pages
    assert err.value.status == Status.INVALID
    assert cache.num_cached_pages() == 0 and cache.num_free_pages() == 0


@pytest.mark.gpu
def test_shared_pages_hold_the_right_data_nvidia(cuda_device):
    check_shared_data(NVIDIA)
