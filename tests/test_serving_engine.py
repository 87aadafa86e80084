"""Continuous batching engine and prefix reuse at model level: every request must receive exactly the tokens it gets
when generated alone, whatever it was batched with, however its prompt was chunked, and whether or not its first pages
came from the prefix cache (the comparison the reference makes for one sequence against Hugging Face,
test/test_infer.py:83-148, extended to the multi-user service README.md:415-424 describes)."""
import numpy as np
import pytest
import torch

import llaisys_b200 as llaisys
from llaisys_b200 import LlaisysError, Status
from tests.test_qwen2_model import hf_greedy, hf_model, make


def expected(hf, prompts, max_new):
    return [hf_greedy(hf, p, n)[len(p):] for p, n in zip(prompts, max_new)]


def test_engine_matches_single_sequence_generation_cpu():
    cfg, hf = hf_model(seed=21)
    model = make(cfg, hf)
    rng = np.random.default_rng(0)
    lens, max_new = [5, 40, 17, 64, 1, 33], [6, 3, 9, 4, 8, 5]
    prompts = [rng.integers(0, 318, n).tolist() for n in lens]
    want = expected(hf, prompts, max_new)
    model.configure_cache(4, 96)  # 4 live requests at most: the last two wait for a slot
    engine = llaisys.Engine(model, max_batch=4, max_tokens_per_step=48, prefill_chunk=16)
    arrivals = [(0, prompts[0], max_new[0]), (0, prompts[1], max_new[1]), (1, prompts[2], max_new[2]),
                (1, prompts[3], max_new[3]), (2, prompts[4], max_new[4]), (5, prompts[5], max_new[5])]
    got = engine.run(arrivals)
    for i in range(len(prompts)):
        assert got[i] == want[i], f"request {i}"
    c = engine.counters
    assert c["tokens_computed"] == sum(lens) + sum(n - 1 for n in max_new)  # nothing computed twice, nothing skipped
    assert engine.num_running == 0 and engine.num_waiting == 0
    engine.close()
    assert model.add_seq() >= 0  # every sequence slot came back


def test_budget_below_running_requests_starves_nobody_cpu():
    """A step budget smaller than the number of decoding requests: the requests that go without a token rotate, so all of
    them advance together instead of the last ones waiting for the first to finish, and every token is still the one
    the request gets alone."""
    cfg, hf = hf_model(seed=23)
    model = make(cfg, hf)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 318, 3).tolist() for _ in range(4)]
    max_new = [8, 8, 8, 8]
    want = expected(hf, prompts, max_new)
    model.configure_cache(4, 32)
    engine = llaisys.Engine(model, max_batch=4, max_tokens_per_step=2, prefill_chunk=2)
    ids = [engine.submit(p, n) for p, n in zip(prompts, max_new)]
    got = {rid: [] for rid in ids}
    progress_when_first_finished = None
    while engine.num_waiting or engine.num_running:
        for rid, token, finished in engine.step():
            got[rid].append(token)
            if finished and progress_when_first_finished is None:
                progress_when_first_finished = [len(got[r]) for r in ids]
    for rid, w in zip(ids, want):
        assert got[rid] == w
    # when the first request finished, the slowest one was at most a couple of tokens behind (without the rotation the
    # last two requests had not produced anything yet)
    assert min(progress_when_first_finished) >= max(progress_when_first_finished) - 3, progress_when_first_finished
    engine.close()


def test_prefix_reuse_gives_the_same_tokens_and_skips_work_cpu():
    cfg, hf = hf_model(seed=22)
    model = make(cfg, hf)
    rng = np.random.default_rng(1)
    system = rng.integers(0, 318, 50).tolist()  # a shared beginning: 3 whole pages
    prompts = [system + rng.integers(0, 318, n).tolist() for n in (7, 12, 3)]
    want = expected(hf, prompts, [5, 5, 5])
    model.configure_cache(4, 96)
    engine = llaisys.Engine(model, max_batch=4, max_tokens_per_step=256, prefill_chunk=64)
    first = engine.run([(0, prompts[0], 5)])
    assert first[0] == want[0] and engine.counters["prompt_tokens_from_cache"] == 0
    rest = engine.run([(0, prompts[1], 5), (0, prompts[2], 5)])
    assert rest[0] == want[1] and rest[1] == want[2]
    assert engine.counters["prompt_tokens_from_cache"] == 2 * 48
    # the same through the model API
    seq, covered = model.add_seq_with_prefix(prompts[1])
    assert covered == 48  # request 1's pages were published while it ran and stay findable after it finished
    nxt = model.step([seq], [prompts[1][covered:]])
    assert nxt[0] == want[1][0]
    # a prompt that is a whole number of pages, seen before: one token is always left to run
    model.free_seq(seq)
    seq2, covered2 = model.add_seq_with_prefix(prompts[1][:48])
    assert covered2 == 32


def test_engine_argument_errors_and_admission_cpu():
    cfg, hf = hf_model(seed=23)
    model = make(cfg, hf)
    with pytest.raises(LlaisysError):
        llaisys.Engine(model)  # cache not configured
    model.configure_cache(2, 48)  # 2 sequences x 3 pages = 6 pages in the pool
    engine = llaisys.Engine(model, max_batch=2, max_tokens_per_step=128, prefill_chunk=64)
    with pytest.raises(LlaisysError) as err:
        engine.submit([], 4)
    assert err.value.status == Status.INVALID
    with pytest.raises(LlaisysError):
        engine.submit([1, 2, 3], 0)
    with pytest.raises(LlaisysError):
        engine.submit([999], 4)  # token out of range
    with pytest.raises(LlaisysError):
        engine.submit(list(range(40)), 20)  # longer than a sequence can get
    a = engine.submit(list(range(40)), 9)  # 48 tokens: 3 pages
    b = engine.submit(list(range(100, 140)), 9)
    c = engine.submit(list(range(200, 210)), 2)
    events = engine.step()
    assert engine.num_running == 2 and engine.num_waiting == 1  # c waits for a slot, in order
    assert sorted(e[0] for e in events) == [a, b]
    engine.cancel(a)
    with pytest.raises(LlaisysError):
        engine.cancel(a)
    events = engine.step()  # c is admitted into a's slot and prefilled in the same step b decodes
    assert sorted(e[0] for e in events) == [b, c] and engine.num_waiting == 0
    while engine.num_running:
        engine.step()
    assert model.add_seq() >= 0


def test_engine_survives_its_model_being_destroyed_first():
    """Garbage collection may finalise a model before the engine built on it: the engine must then fail cleanly."""
    cfg, hf = hf_model(seed=23)
    model = make(cfg, hf)
    model.configure_cache(2, 48)
    engine = llaisys.Engine(model, max_batch=2, max_tokens_per_step=64, prefill_chunk=64)
    engine.submit(list(range(40)), 9)
    engine.submit(list(range(100, 140)), 9)
    engine.step()  # one request mid-prompt, one decoding
    model.close()
    assert engine.num_running == 0 and engine.num_waiting == 0
    with pytest.raises(LlaisysError) as err:
        engine.submit([1, 2], 2)
    assert err.value.status == Status.INVALID
    engine.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_engine_on_gpu(cuda_device, dtype_name):
    """f32: the engine's tokens equal single-sequence generation on the same device. bf16 (tensor-core prefill, TMA
    decode, batch-dependent GEMM kernels): every generated token must be within the rounding margin of the best token
    under Hugging Face's f32 logits for the same history."""
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
    ldt = {"f32": llaisys.DataType.F32, "bf16": llaisys.DataType.BF16}[dtype_name]
    cfg, hf32 = hf_model(seed=24, std=0.02, num_attention_heads=12, num_key_value_heads=2, hidden_size=1536,
                         intermediate_size=1024)
    hf = hf32.to(tdt).float()
    model = llaisys.models.Qwen2(config=cfg, state_dict=hf.state_dict(), device=llaisys.DeviceType.NVIDIA, dtype=ldt)
    rng = np.random.default_rng(2)
    system = rng.integers(0, 318, 70).tolist()
    prompts = [system + rng.integers(0, 318, n).tolist() for n in (150, 9, 40)] + [rng.integers(0, 318, 200).tolist()]
    max_new = [6, 10, 8, 5]
    model.configure_cache(3, 320)
    engine = llaisys.Engine(model, max_batch=3, max_tokens_per_step=256, prefill_chunk=128)
    got = engine.run([(0, prompts[0], max_new[0]), (2, prompts[1], max_new[1]), (3, prompts[2], max_new[2]),
                      (3, prompts[3], max_new[3])])
    assert engine.counters["prompt_tokens_from_cache"] == 2 * 64
    tol = 2e-3 if dtype_name == "f32" else 0.05
    for i, p in enumerate(prompts):
        assert len(got[i]) == max_new[i]
        with torch.no_grad():
            logits = hf(torch.tensor([p + got[i][:-1]])).logits[0].float()
        for s, token in enumerate(got[i]):
            row = logits[len(p) - 1 + s]
            assert (row.max() - row[token]).item() <= 2 * tol * max(1.0, row.abs().max().item()), (i, s)
    if dtype_name == "f32":
        single = llaisys.models.Qwen2(config=cfg, state_dict=hf.state_dict(), device=llaisys.DeviceType.NVIDIA, dtype=ldt)
        for i, p in enumerate(prompts):
            assert single.generate(p, max_new_tokens=max_new[i], top_k=1)[len(p):] == got[i]
