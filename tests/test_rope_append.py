"""The fused step before attention (bias + rotary embedding + paged append over a packed q|k|v projection) against
the oracles of its parts: the reference's rope definition (test/ops/rope.py:11-32) for the rotation and the
bit-exact page model for where the rows land."""
import numpy as np
import pytest
import torch

import llaisys_b200 as llaisys
from oracle import ops as oracle_ops
from oracle import workloads
from tests import helpers

CPU, NVIDIA = llaisys.DeviceType.CPU, llaisys.DeviceType.NVIDIA


def run_case(device, dname, *, nh, nkvh, d, ctx, with_bias, theta=10000.0, seed=0, pool_pages=64):
    tdt = helpers.TORCH_DTYPE[dname]
    dev = helpers.torch_device(device)
    g = torch.Generator().manual_seed(seed)
    pages_needed = sum(-(-c // 16) for c in ctx)
    perm = torch.randperm(pool_pages, generator=g).tolist()[:pages_needed]
    pages, at = [], 0
    for c in ctx:
        n = -(-c // 16)
        pages.append(perm[at:at + n])
        at += n
    cache, seqs = helpers.build_cache(device, dname, pages, num_pages=pool_pages, nkvh=nkvh, d=d)
    # rows in a shuffled order: the kernel must honour (sequence, position), not row order
    ids, pos = [], []
    for s, c in zip(seqs, ctx):
        ids += [s] * c
        pos += list(range(c))
    order = torch.randperm(len(ids), generator=g).tolist()
    ids = [ids[i] for i in order]
    pos = [pos[i] for i in order]
    n_rows, width = len(ids), (nh + 2 * nkvh) * d
    qkv = workloads.randn((n_rows, width), tdt, g)
    bias = workloads.randn((width,), tdt, g) if with_bias else None

    ids_d = torch.tensor(ids, dtype=torch.int32, device=dev)
    pos_d = torch.tensor(pos, dtype=torch.int32, device=dev)
    q_out = torch.zeros((n_rows, nh, d), dtype=tdt, device=dev)
    cache.flush()
    stream = llaisys.context_stream() if device == NVIDIA else None
    cache.rope_append_dev(0, q_out, qkv.to(dev), bias.to(dev) if with_bias else None, ids_d, pos_d, n_rows, nh, theta,
                          stream)
    cache.check()

    # expected: f32 arithmetic on the stored values, one rounding (the kernel's contract)
    x = qkv.float() + (bias.float() if with_bias else 0.0)
    x = x.view(n_rows, nh + 2 * nkvh, d)
    p64 = torch.tensor(pos, dtype=torch.int64)
    q_ref = oracle_ops.rope(x[:, :nh], p64, theta).to(tdt)
    k_ref = oracle_ops.rope(x[:, nh:nh + nkvh], p64, theta).to(tdt)
    v_ref = x[:, nh + nkvh:].to(tdt)
    tol = {"f32": 2e-5, "f16": 2e-3, "bf16": 1.6e-2}[dname]  # one unit in the last place of values up to ~4 and sincos error
    assert torch.allclose(q_out.cpu().float(), q_ref.float(), atol=tol, rtol=tol)
    for s, c in zip(seqs, ctx):
        k_out = torch.empty((c, nkvh, d), dtype=tdt, device=dev)
        v_out = torch.empty((c, nkvh, d), dtype=tdt, device=dev)
        cache.gather(0, s, c, k_out, v_out)
        rows = [i for i in range(n_rows) if ids[i] == s]
        rows.sort(key=lambda i: pos[i])
        assert torch.allclose(k_out.cpu().float(), k_ref[rows].float(), atol=tol, rtol=tol)
        if with_bias:
            assert torch.allclose(v_out.cpu().float(), v_ref[rows].float(), atol=tol, rtol=tol)
        else:  # no arithmetic touches v: bit-exact
            assert torch.equal(helpers.tensor_words(v_out.cpu()), helpers.tensor_words(v_ref[rows]))
    return cache


@pytest.mark.parametrize("dname", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("with_bias", [True, False])
def test_rope_append_cpu(dname, with_bias):
    run_case(CPU, dname, nh=12, nkvh=2, d=128, ctx=[37, 1, 16], with_bias=with_bias)


def test_rope_append_other_shapes_cpu():
    run_case(CPU, "f32", nh=4, nkvh=4, d=64, ctx=[5, 33], with_bias=True, theta=1e6)
    run_case(CPU, "bf16", nh=2, nkvh=1, d=8, ctx=[20], with_bias=True)  # half a head row is shorter than a 16-byte vector


def test_rope_append_flags_bad_rows_cpu():
    cache, seqs = helpers.build_cache(CPU, "f32", [[3]], num_pages=8, nkvh=1, d=8)
    qkv = torch.zeros((2, 3 * 8))
    q_out = torch.zeros((2, 1, 8))
    ids = torch.tensor([seqs[0], seqs[0]], dtype=torch.int32)
    pos = torch.tensor([0, 16], dtype=torch.int32)  # position 16 needs a second page the sequence does not own
    cache.flush()
    cache.rope_append_dev(0, q_out, qkv, None, ids, pos, 2, 1, 10000.0, None)
    with pytest.raises(llaisys.LlaisysError):
        cache.check()


@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("with_bias", [True, False])
def test_rope_append_nvidia(cuda_device, dname, with_bias):
    run_case(NVIDIA, dname, nh=12, nkvh=2, d=128, ctx=[333, 1, 16, 77], with_bias=with_bias)


@pytest.mark.gpu
def test_rope_append_other_shapes_nvidia(cuda_device):
    run_case(NVIDIA, "f32", nh=4, nkvh=4, d=64, ctx=[5, 33], with_bias=True, theta=1e6)
    run_case(NVIDIA, "bf16", nh=2, nkvh=1, d=8, ctx=[20], with_bias=True)


@pytest.mark.gpu
def test_rope_append_matches_cpu_backend_nvidia(cuda_device):
    """Same inputs through both backends: q and the pool contents must agree to the last bit in f32 up to the sincos
    implementation (compared at 1e-6), and exactly for v."""
    g = torch.Generator().manual_seed(9)
    n_rows, nh, nkvh, d = 40, 12, 2, 128
    qkv = workloads.randn((n_rows, (nh + 2 * nkvh) * d), torch.float32, g)
    bias = workloads.randn(((nh + 2 * nkvh) * d,), torch.float32, g)
    outs = []
    for device in (CPU, NVIDIA):
        dev = helpers.torch_device(device)
        cache, seqs = helpers.build_cache(device, "f32", [[5, 2, 7]], num_pages=8, nkvh=nkvh, d=d)
        ids = torch.full((n_rows,), seqs[0], dtype=torch.int32, device=dev)
        pos = torch.arange(n_rows, dtype=torch.int32, device=dev)
        q_out = torch.zeros((n_rows, nh, d), device=dev)
        cache.flush()
        cache.rope_append_dev(0, q_out, qkv.to(dev), bias.to(dev), ids, pos, n_rows, nh, 10000.0,
                              llaisys.context_stream() if device == NVIDIA else None)
        cache.check()
        k = torch.empty((n_rows, nkvh, d), device=dev)
        v = torch.empty((n_rows, nkvh, d), device=dev)
        cache.gather(0, seqs[0], n_rows, k, v)
        outs.append((q_out.cpu(), k.cpu(), v.cpu()))
    assert torch.allclose(outs[0][0], outs[1][0], atol=2e-5, rtol=0)
    assert torch.allclose(outs[0][1], outs[1][1], atol=2e-5, rtol=0)
    assert torch.equal(outs[0][2], outs[1][2])
