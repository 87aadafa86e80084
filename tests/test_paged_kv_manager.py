"""Block manager: free list, block tables, error codes -- host logic only, against the numpy model."""
import random

import pytest
from hypothesis import given, settings, strategies as st

import llaisys_b200 as llaisys
from llaisys_b200 import LlaisysError, Status
from oracle.paged import PagedCacheModel


def make(num_pages=64, page=16, max_seqs=8, max_pages_per_seq=None):
    cache = llaisys.PagedKVCache(num_pages, 2, 8, page_size=page, dtype=llaisys.DataType.BF16, max_seqs=max_seqs,
                                 max_pages_per_seq=max_pages_per_seq)
    model = PagedCacheModel(num_pages, page, 2, 8, max_seqs=max_seqs, max_pages_per_seq=max_pages_per_seq)
    return cache, model


def test_reserve_hands_out_pages_in_order_and_is_idempotent():
    cache, _ = make()
    s = cache.add_seq()
    assert cache.seq_num_pages(s) == 0 and cache.num_free_pages() == 64
    cache.reserve(s, 1)
    assert cache.seq_pages(s) == [0]
    cache.reserve(s, 16)  # still one page
    assert cache.seq_pages(s) == [0]
    cache.reserve(s, 17)
    cache.reserve(s, 5)  # never shrinks
    assert cache.seq_pages(s) == [0, 1] and cache.num_free_pages() == 62


def test_pool_exhaustion_is_a_status_and_changes_nothing():
    cache, _ = make(num_pages=4)
    a, b = cache.add_seq(), cache.add_seq()
    cache.reserve(a, 48)
    with pytest.raises(LlaisysError) as e:
        cache.reserve(b, 33)  # needs 3, only 1 free
    assert e.value.status == Status.NO_PAGES
    assert cache.seq_num_pages(b) == 0 and cache.num_free_pages() == 1
    cache.reserve(b, 16)
    assert cache.num_free_pages() == 0


def test_free_returns_pages_and_retires_the_id():
    cache, _ = make(num_pages=8)
    a = cache.add_seq()
    cache.reserve(a, 16 * 3)
    pages = cache.seq_pages(a)
    cache.free_seq(a)
    assert cache.num_free_pages() == 8 and cache.num_seqs() == 0 and cache.seq_num_pages(a) == -1
    for call in (lambda: cache.free_seq(a), lambda: cache.reserve(a, 1), lambda: cache.seq_pages(a)):
        with pytest.raises(LlaisysError) as e:  # double free / use after free
            call()
        assert e.value.status == Status.NO_SEQ
    b = cache.add_seq()
    cache.reserve(b, 16 * 3)
    assert cache.seq_pages(b) == pages  # freed pages come back in their original order


def test_assign_specific_pages():
    cache, _ = make(num_pages=16)
    a, b = cache.add_seq(), cache.add_seq()
    cache.assign_pages(a, [7, 3, 11])
    assert cache.seq_pages(a) == [7, 3, 11] and cache.num_free_pages() == 13
    for bad, status in (([3], Status.NO_PAGES), ([5, 5], Status.NO_PAGES), ([16], Status.INVALID),
                        ([-1], Status.INVALID), ([4, 7], Status.NO_PAGES)):
        with pytest.raises(LlaisysError) as e:
            cache.assign_pages(b, bad)
        assert e.value.status == status
        assert cache.seq_num_pages(b) == 0 and cache.num_free_pages() == 13  # all-or-nothing
    cache.assign_pages(b, [4, 5])
    cache.reserve(b, 16 * 4)  # the free list skips the pages taken by name
    assert cache.seq_pages(b) == [4, 5, 0, 1]


def test_limits():
    cache, _ = make(num_pages=64, max_seqs=2, max_pages_per_seq=3)
    a, b = cache.add_seq(), cache.add_seq()
    with pytest.raises(LlaisysError) as e:
        cache.add_seq()
    assert e.value.status == Status.NO_SEQ
    with pytest.raises(LlaisysError) as e:
        cache.reserve(a, 16 * 3 + 1)
    assert e.value.status == Status.INVALID and cache.seq_num_pages(a) == 0
    with pytest.raises(LlaisysError) as e:
        cache.assign_pages(b, [1, 2, 3, 4])
    assert e.value.status == Status.INVALID


def test_bad_create_arguments():
    for kw in (dict(num_pages=0), dict(nkvh=0), dict(head_dim=0), dict(page_size=0), dict(dtype=llaisys.DataType.I32),
               dict(head_dim=3), dict(device=llaisys.DeviceType.NVIDIA, device_id=99)):
        args = dict(num_pages=4, nkvh=2, head_dim=8, page_size=16, dtype=llaisys.DataType.BF16)
        args.update(kw)
        with pytest.raises(LlaisysError):
            llaisys.PagedKVCache(args.pop("num_pages"), args.pop("nkvh"), args.pop("head_dim"), **args)


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["add", "reserve", "assign", "free"]), st.integers(0, 10 ** 6)),
                min_size=1, max_size=60))
def test_random_operation_sequences_match_the_model(ops):
    cache, model = make(num_pages=24, page=4, max_seqs=5, max_pages_per_seq=10)
    live: list[int] = []
    for op, r in ops:
        rng = random.Random(r)
        if op == "add":
            try:
                expect = model.add_seq()
            except KeyError:
                with pytest.raises(LlaisysError):
                    cache.add_seq()
                continue
            assert cache.add_seq() == expect
            live.append(expect)
        elif not live:
            continue
        elif op == "reserve":
            s, n = rng.choice(live), rng.randint(0, 50)
            try:
                model.reserve(s, n)
            except (ValueError, MemoryError):
                with pytest.raises(LlaisysError):
                    cache.reserve(s, n)
            else:
                cache.reserve(s, n)
        elif op == "assign":
            s = rng.choice(live)
            pages = [rng.randint(0, 23) for _ in range(rng.randint(1, 3))]
            try:
                model.assign_pages(s, pages)
            except (ValueError, MemoryError):
                with pytest.raises(LlaisysError):
                    cache.assign_pages(s, pages)
            else:
                cache.assign_pages(s, pages)
        else:
            s = live.pop(rng.randrange(len(live)))
            model.free_seq(s)
            cache.free_seq(s)
        # invariants: tables equal the model's, no page owned twice, free count consistent
        owned = []
        for s in live:
            assert cache.seq_pages(s) == model.tables[s]
            owned += model.tables[s]
        assert len(owned) == len(set(owned))
        assert cache.num_free_pages() == 24 - len(owned) == len(model.free)
        assert cache.num_seqs() == len(live)
