"""Tensor-parallel Qwen2 (heads and MLP rows sharded over the ranks, two all-reduces per layer): every rank must
produce the tokens and logits of the unsharded model. CPU: two gloo ranks with the host all-reduce callback. GPU: two
NCCL ranks, one per B200 (skipped with fewer than two devices)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]

TP_CFG = dict(num_attention_heads=4, num_key_value_heads=2, hidden_size=512, intermediate_size=768)


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank: int, world: int, port: int, backend: str, dtype_name: str, out_path: str):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    import llaisys_b200 as llaisys
    from tests.test_qwen2_model import hf_model

    gpu = backend == "nccl"
    if gpu:
        torch.cuda.set_device(rank)
        llaisys.set_context_runtime(llaisys.DeviceType.NVIDIA, rank)
    dist.init_process_group(backend, rank=rank, world_size=world,
                            **({"device_id": torch.device("cuda", rank)} if gpu else {}))
    try:
        ldt = {"f32": llaisys.DataType.F32, "bf16": llaisys.DataType.BF16}[dtype_name]
        cfg, hf = hf_model(seed=31, std=0.02 if gpu else 0.08, **(dict(TP_CFG, num_attention_heads=12, hidden_size=1536,
                                                                         intermediate_size=1024) if gpu else TP_CFG))
        model = llaisys.models.Qwen2(config=cfg, state_dict=hf.state_dict(), dtype=ldt,
                                     device=llaisys.DeviceType.NVIDIA if gpu else llaisys.DeviceType.CPU,
                                     device_id=rank if gpu else 0, tp_group=dist.group.WORLD)
        assert model.tp_world == world and model.tp_rank == rank
        rng = np.random.default_rng(5)
        prompts = [rng.integers(0, 318, n).tolist() for n in (37, 5, 64)]
        model.configure_cache(3, 128)
        seqs = [model.add_seq() for _ in prompts]
        nxt = model.step(seqs, prompts)                      # prefill of three ragged prompts
        logits = model.last_logits(3)
        loop = model.decode_loop(seqs, nxt, 6)               # device-side loop (graph replays on NVIDIA)
        torch.save({"next": nxt, "logits": logits, "loop": loop, "prompts": prompts}, f"{out_path}.{rank}")
    finally:
        dist.destroy_process_group()


def run_ranks(world, backend, dtype_name, tmp_path):
    out = str(tmp_path / "tp")
    mp.spawn(worker, args=(world, free_port(), backend, dtype_name, out), nprocs=world, join=True)
    return [torch.load(f"{out}.{r}", weights_only=False) for r in range(world)]


def check_against_unsharded(results, dtype_name, gpu):
    import llaisys_b200 as llaisys
    from tests.test_qwen2_model import hf_logits, hf_model

    cfg, hf = hf_model(seed=31, std=0.02 if gpu else 0.08, **(dict(TP_CFG, num_attention_heads=12, hidden_size=1536,
                                                                     intermediate_size=1024) if gpu else TP_CFG))
    if dtype_name == "bf16":
        hf = hf.to(torch.bfloat16).float()
    tol = {"f32": 2e-3 if gpu else 2e-4, "bf16": 0.05}[dtype_name]
    r0 = results[0]
    for r in results[1:]:  # replicated computation: every rank holds the same answers, bit for bit
        assert r["next"] == r0["next"] and np.array_equal(r["loop"], r0["loop"])
        assert np.array_equal(r["logits"], r0["logits"])
    for i, p in enumerate(r0["prompts"]):
        want = hf_logits(hf, p)[-1]
        got = torch.from_numpy(r0["logits"][i])
        assert (got - want).abs().max().item() < tol * max(1.0, want.abs().max().item())
        fed = p + [r0["next"][i]] + r0["loop"][:-1, i].tolist()
        rows = hf_logits(hf, fed)
        for s, token in enumerate([r0["next"][i]] + r0["loop"][:, i].tolist()):
            row = rows[len(p) - 1 + s]
            margin = (row.max() - row[token]).item()
            assert margin <= 2 * tol * max(1.0, row.abs().max().item()), (i, s, margin)
            if dtype_name == "f32" and not gpu:
                assert token == int(row.argmax())


def test_two_rank_tensor_parallel_model_cpu(tmp_path):
    check_against_unsharded(run_ranks(2, "gloo", "f32", tmp_path), "f32", gpu=False)


def test_sharding_argument_errors():
    import llaisys_b200 as llaisys
    from llaisys_b200.libllaisys import LIB_LLAISYS, LlaisysQwen2Meta
    import ctypes

    meta = LlaisysQwen2Meta(dtype=int(llaisys.DataType.F32), nlayer=1, hs=256, nh=2, nkvh=1, dh=128, di=512, maxseq=64,
                            voc=100, epsilon=1e-6, theta=10000.0, end_token=-1)
    # one KV head cannot be split in two
    assert not LIB_LLAISYS.llaisysQwen2ModelCreateTP(ctypes.byref(meta), 0, 0, 0, 2)
    assert not LIB_LLAISYS.llaisysQwen2ModelCreateTP(ctypes.byref(meta), 0, 0, 3, 2)
    meta.nh, meta.nkvh = 4, 2
    model = LIB_LLAISYS.llaisysQwen2ModelCreateTP(ctypes.byref(meta), 0, 0, 1, 2)
    assert model
    try:
        weights = LIB_LLAISYS.llaisysQwen2ModelWeights(model).contents
        shape = (ctypes.c_size_t * 2)()
        LIB_LLAISYS.tensorGetShape(weights.attn_q_w[0], shape)
        assert tuple(shape) == (2 * 128, 256)
        LIB_LLAISYS.tensorGetShape(weights.mlp_down_w[0], shape)
        assert tuple(shape) == (256, 256)
        # a sharded model refuses to run without its all-reduce
        assert LIB_LLAISYS.llaisysQwen2ModelConfigureCache(model, 1, 32) == 0
        seq = ctypes.c_int32(-1)
        assert LIB_LLAISYS.llaisysQwen2ModelSeqAdd(model, ctypes.byref(seq)) == 0
        ids, n = (ctypes.c_int32 * 1)(seq.value), (ctypes.c_int32 * 1)(1)
        tok, nxt = (ctypes.c_int64 * 1)(3), (ctypes.c_int64 * 1)(0)
        assert LIB_LLAISYS.llaisysQwen2ModelStep(model, ids, n, 1, tok, nxt) == int(llaisys.Status.INVALID)
    finally:
        LIB_LLAISYS.llaisysQwen2ModelDestroy(model)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_two_rank_tensor_parallel_model_nccl(tmp_path, dtype_name):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    check_against_unsharded(run_ranks(2, "nccl", dtype_name, tmp_path), dtype_name, gpu=True)
