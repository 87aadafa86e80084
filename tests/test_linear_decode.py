"""Decode-sized projections (at most 128 activation rows): `linear` and `linear_accumulate` against the reference's
definition of linear (test/ops/linear.py:11-12, x . W^T + b) evaluated in float64 on the same rounded inputs. On NVIDIA
these shapes run the hand-written tcgen05 weight-streaming kernel, including its K split over a thread-block cluster."""
import pytest
import torch

import llaisys_b200 as llaisys
from tests import helpers

CPU, NVIDIA = llaisys.DeviceType.CPU, llaisys.DeviceType.NVIDIA

# (rows, K, N, accumulate): the four projections of the 1.5B model at batch 64, then edge shapes: one row, a full 128,
# a ragged row count, a single 64-element K chunk, a K that does not divide evenly among the cluster's CTAs
MODEL_SHAPES = [(64, 1536, 2048, False), (64, 1536, 1536, True), (64, 1536, 17920, False), (64, 8960, 1536, True)]
EDGE_SHAPES = [(1, 1536, 1536, True), (128, 1536, 2048, False), (7, 1024, 1536, True), (33, 64, 64, False),
               (5, 448, 192, True), (100, 128, 128, False), (8, 8960, 1536, True), (16, 4096, 256, False)]


def run_case(device, dname, m, k, n, accumulate, seed=0):
    dt = helpers.TORCH_DTYPE[dname]
    g = torch.Generator().manual_seed(seed + m + k + n)
    x = torch.randn((m, k), generator=g).to(dt)
    w = (torch.randn((n, k), generator=g) * 0.05).to(dt)
    before = torch.randn((m + 4, n), generator=g).to(dt)  # 4 guard rows behind the output must stay untouched
    buf = helpers.to_llaisys(before, device, dname)
    out = buf.slice(0, 0, m)
    x_, w_ = helpers.to_llaisys(x, device, dname), helpers.to_llaisys(w, device, dname)
    if accumulate:
        llaisys.Ops.linear_accumulate(out, x_, w_)
    else:
        llaisys.Ops.linear(out, x_, w_, None)
    got = helpers.from_llaisys(buf, dname)
    exact = x.double() @ w.double().T + (before[:m].double() if accumulate else 0.0)
    assert torch.equal(helpers.tensor_words(got[m:]), helpers.tensor_words(before[m:])), "rows behind the output changed"
    # one rounding to the output type plus f32 accumulation noise
    rtol = {"f32": 2e-6, "f16": 2 ** -10, "bf16": 2 ** -7}[dname]
    atol = {"f32": 2e-5, "f16": 2e-3, "bf16": 1e-2}[dname] * max(1.0, (k / 1024) ** 0.5)
    err = (got[:m].double() - exact).abs()
    bound = atol + rtol * exact.abs()
    assert bool((err <= bound).all()), f"{(m, k, n, accumulate, dname)}: worst excess {(err - bound).max().item():.3e}"


@pytest.mark.parametrize("dname", ["f32", "bf16"])
def test_decode_projections_cpu(dname):
    for m, k, n, acc in [(5, 448, 192, True), (33, 64, 64, False), (7, 1024, 96, True)]:
        run_case(CPU, dname, m, k, n, acc)


@pytest.mark.gpu
@pytest.mark.parametrize("path", ["tc", "default"])
@pytest.mark.parametrize("dname", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("shape", MODEL_SHAPES + EDGE_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_decode_projections_nvidia(cuda_device, dname, shape, path):
    """path "tc" takes the hand-written kernel wherever its shape rules allow (the library otherwise picks it only
    where it measured faster than cuBLAS); "default" is the routing a user gets."""
    llaisys.Ops.set_linear_policy(1 if path == "tc" else 0)
    try:
        run_case(NVIDIA, dname, *shape)
    finally:
        llaisys.Ops.set_linear_policy(0)


@pytest.mark.gpu
def test_decode_projection_is_deterministic_nvidia(cuda_device):
    """The cluster reduction adds the K splits in rank order: the same call twice gives the same bits."""
    llaisys.Ops.set_linear_policy(1)
    g = torch.Generator().manual_seed(3)
    x = torch.randn((64, 8960), generator=g).to(torch.bfloat16)
    w = (torch.randn((1536, 8960), generator=g) * 0.05).to(torch.bfloat16)
    x_, w_ = helpers.to_llaisys(x, NVIDIA, "bf16"), helpers.to_llaisys(w, NVIDIA, "bf16")
    outs = []
    for _ in range(3):
        out = llaisys.Tensor((64, 1536), dtype=llaisys.DataType.BF16, device=NVIDIA)
        llaisys.Ops.linear(out, x_, w_, None)
        outs.append(helpers.tensor_words(helpers.from_llaisys(out, "bf16")))
    llaisys.Ops.set_linear_policy(0)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
