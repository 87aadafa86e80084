"""llaisysSelfAttention against the oracle: the reference's own cases and tolerances
(reference: test/ops/self_attention.py:71-81), the golden vectors, and benchmark configuration 1."""
import pytest
import torch

import llaisys_b200 as llaisys
from oracle import attention, workloads
from tests import helpers

REF_SHAPES = [(2, 2, 1, 1, 4), (5, 11, 4, 2, 8)]
MORE_SHAPES = [(1, 1, 12, 2, 128), (1, 513, 12, 2, 128), (16, 16, 12, 2, 128), (40, 100, 12, 2, 128),
               (3, 35, 8, 8, 64), (7, 7, 6, 1, 32)]


def check_reference_case(device, shape, dname):
    qlen, kvlen, nh, nkvh, hd = shape
    dt = helpers.TORCH_DTYPE[dname]
    g = torch.Generator().manual_seed(hash(shape) % 1000)
    # U[0, 1) like the reference's random_tensor (test/test_utils.py:8-12)
    q = torch.rand((qlen, nh, hd), generator=g).to(dt)
    k = torch.rand((kvlen, nkvh, hd), generator=g).to(dt)
    v = torch.rand((kvlen, nkvh, hd), generator=g).to(dt)
    scale = 1.0 / hd ** 0.5
    expect = attention.self_attention(q, k, v, scale)
    got = helpers.run_self_attention(q, k, v, scale, device, dname)
    tol = helpers.REF_TOL[dname]
    assert got.shape == expect.shape and got.dtype == expect.dtype
    assert torch.allclose(got.float(), expect.float(), atol=tol, rtol=tol), helpers.max_abs(got, expect)


def check_golden(device, name):
    dname, q, k, v, scale, expect, _ = helpers.load_golden(name)
    if q is None:
        q, k, v, scale = workloads.config1()
    got = helpers.run_self_attention(q, k, v, scale, device, dname)
    assert helpers.max_abs(got, expect) <= helpers.MAX_ABS[dname]
    # tighter: an f32-accumulating kernel sits within about one output ulp of the float64 result
    f64 = attention.self_attention_f64(q, k, v, scale)
    ulp = {"f32": 1e-6, "f16": 1e-3, "bf16": 8e-3}[dname]
    assert helpers.max_abs(got, f64) <= ulp * max(1.0, f64.abs().max().item())


@pytest.mark.parametrize("dname", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", REF_SHAPES + MORE_SHAPES)
def test_reference_cases_cpu(shape, dname):
    check_reference_case(llaisys.DeviceType.CPU, shape, dname)


@pytest.mark.parametrize("name", helpers.golden_cases())
def test_golden_cpu(name):
    check_golden(llaisys.DeviceType.CPU, name)


@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", REF_SHAPES + MORE_SHAPES)
def test_reference_cases_nvidia(cuda_device, shape, dname):
    check_reference_case(llaisys.DeviceType.NVIDIA, shape, dname)


@pytest.mark.gpu
@pytest.mark.parametrize("name", helpers.golden_cases())
def test_golden_nvidia(cuda_device, name):
    check_golden(llaisys.DeviceType.NVIDIA, name)


@pytest.mark.gpu
@pytest.mark.parametrize("kvlen", [1, 15, 16, 17, 255, 256, 257, 4096, 5000])
def test_decode_lengths_around_page_and_split_boundaries_nvidia(cuda_device, kvlen):
    """qlen 1 over contiguous bf16 K/V takes the split-KV kernel: lengths on both sides of the page size (16)
    and of the split size."""
    g = torch.Generator().manual_seed(kvlen)
    q = workloads.randn((1, 12, 128), torch.bfloat16, g)
    k = workloads.randn((kvlen, 2, 128), torch.bfloat16, g)
    v = workloads.randn((kvlen, 2, 128), torch.bfloat16, g)
    scale = 1.0 / 128 ** 0.5
    got = helpers.run_self_attention(q, k, v, scale, llaisys.DeviceType.NVIDIA, "bf16")
    assert helpers.max_abs(got, attention.self_attention(q, k, v, scale)) <= helpers.MAX_ABS["bf16"]
    f64 = attention.self_attention_f64(q, k, v, scale)
    assert helpers.max_abs(got, f64) <= 8e-3 * max(1.0, f64.abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["bf16", "f16"])
@pytest.mark.parametrize("qlen,kvlen", [(16, 16), (100, 100), (130, 131), (512, 1024), (300, 2049), (2048, 2048)])
def test_multi_token_queries_over_plain_tensors_nvidia(cuda_device, qlen, kvlen, dname):
    """From 16 query rows on, 16-bit contiguous K/V with head_dim 128 take the tensor-core (tcgen05) kernel through
    tensor maps made over the caller's tensors: lengths that end inside a 16-token tile, inside a 64-key block and
    inside a 128-row query tile, and a square causal case with several query tiles."""
    dt = helpers.TORCH_DTYPE[dname]
    g = torch.Generator().manual_seed(qlen * 7 + kvlen)
    q = workloads.randn((qlen, 12, 128), dt, g)
    k = workloads.randn((kvlen, 2, 128), dt, g)
    v = workloads.randn((kvlen, 2, 128), dt, g)
    scale = 1.0 / 128 ** 0.5
    got = helpers.run_self_attention(q, k, v, scale, llaisys.DeviceType.NVIDIA, dname)
    assert helpers.max_abs(got, attention.self_attention(q, k, v, scale)) <= helpers.MAX_ABS[dname]
    f64 = attention.self_attention_f64(q, k, v, scale)
    ulp = {"f16": 1e-3, "bf16": 8e-3}[dname]
    assert helpers.max_abs(got, f64) <= ulp * max(1.0, f64.abs().max().item())
