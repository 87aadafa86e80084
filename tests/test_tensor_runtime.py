"""Tensor and runtime behaviour, mirroring the reference's test_tensor.py and test_runtime.py
(reference: test/test_tensor.py:8-49, test/test_runtime.py:7-53), on CPU and -- marked gpu -- on NVIDIA."""
import pytest
import torch

import llaisys_b200 as llaisys
from tests import helpers


def read_strided(t: llaisys.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Copies a (possibly strided) llaisys tensor out the way the reference's check_equal does:
    span copy, then as_strided (reference: test/test_utils.py:116-160)."""
    shape, strides = t.shape(), t.strides()
    span = 1 + sum(st * (sh - 1) for sh, st in zip(shape, strides))
    flat = torch.zeros(span, dtype=dtype)
    api = llaisys.RuntimeAPI(t.device_type())
    kind = llaisys.MemcpyKind.H2H if t.device_type() == llaisys.DeviceType.CPU else llaisys.MemcpyKind.D2H
    api.memcpy_sync(flat.data_ptr(), t.data_ptr(), span * flat.element_size(), kind)
    return torch.as_strided(flat, shape, strides)


def check_tensor_ops(device):
    ref = torch.arange(60, dtype=torch.int64).reshape(3, 4, 5)
    t = llaisys.Tensor((3, 4, 5), dtype=llaisys.DataType.I64, device=device)
    t.load(ref.data_ptr())
    assert t.is_contiguous() and t.shape() == (3, 4, 5) and t.strides() == ref.stride()
    assert torch.equal(read_strided(t, torch.int64), ref)

    v, rv = t.view(6, 10), ref.view(6, 10)
    assert v.shape() == rv.shape and v.strides() == rv.stride() and torch.equal(read_strided(v, torch.int64), rv)

    p, rp = t.permute(2, 0, 1), ref.permute(2, 0, 1)
    assert p.shape() == rp.shape and p.strides() == rp.stride() and not p.is_contiguous()
    assert torch.equal(read_strided(p, torch.int64), rp)

    s, rs = t.slice(2, 1, 4), ref[:, :, 1:4]
    assert s.shape() == rs.shape and s.strides() == rs.stride() and not s.is_contiguous()
    assert torch.equal(read_strided(s, torch.int64), rs)

    # a view of a sliced tensor that stays expressible: merge the two leading (still dense) dims
    sv, rsv = s.view(12, 3), rs.reshape(12, 3)
    assert sv.strides() == (5, 1) and torch.equal(read_strided(sv, torch.int64), rsv)
    # views keep the storage alive after the parent handle is gone
    del t, v, p, s
    assert torch.equal(read_strided(sv, torch.int64), rsv)


def check_memcpy_round_trip(device):
    api = llaisys.RuntimeAPI(device)
    n = 1 << 20
    a = torch.randint(0, 255, (n,), dtype=torch.uint8)
    b = torch.zeros_like(a)
    da, db = api.malloc_device(n), api.malloc_device(n)
    host = device == llaisys.DeviceType.CPU
    api.memcpy_sync(da, a.data_ptr(), n, llaisys.MemcpyKind.H2H if host else llaisys.MemcpyKind.H2D)
    api.memcpy_sync(db, da, n, llaisys.MemcpyKind.H2H if host else llaisys.MemcpyKind.D2D)
    api.memcpy_sync(b.data_ptr(), db, n, llaisys.MemcpyKind.H2H if host else llaisys.MemcpyKind.D2H)
    assert torch.equal(a, b)
    api.free_device(da)
    api.free_device(db)


def check_add_and_rearrange(device):
    for dname, tol in (("f32", 1e-5), ("f16", 1e-3), ("bf16", 1e-3)):  # reference: test/ops/add.py:47-51
        for shape in ((2, 3), (512, 4096)):
            a = torch.rand(shape).to(helpers.TORCH_DTYPE[dname])
            b = torch.rand(shape).to(helpers.TORCH_DTYPE[dname])
            a_, b_ = helpers.to_llaisys(a, device, dname), helpers.to_llaisys(b, device, dname)
            c_ = llaisys.Tensor(shape, dtype=helpers.LL_DTYPE[dname], device=device)
            llaisys.Ops.add(c_, a_, b_)
            assert torch.allclose(helpers.from_llaisys(c_, dname), a + b, atol=tol, rtol=tol)
    src = torch.arange(2 * 3 * 4, dtype=torch.float32).reshape(2, 3, 4)
    s_ = helpers.to_llaisys(src, device, "f32").permute(2, 0, 1)
    d_ = llaisys.Tensor((4, 2, 3), dtype=llaisys.DataType.F32, device=device)
    llaisys.Ops.rearrange(d_, s_)
    assert torch.equal(helpers.from_llaisys(d_, "f32"), src.permute(2, 0, 1).contiguous())


def test_tensor_ops_cpu():
    check_tensor_ops(llaisys.DeviceType.CPU)


def test_memcpy_round_trip_cpu():
    check_memcpy_round_trip(llaisys.DeviceType.CPU)


def test_add_and_rearrange_cpu():
    check_add_and_rearrange(llaisys.DeviceType.CPU)


@pytest.mark.gpu
def test_tensor_ops_nvidia(cuda_device):
    check_tensor_ops(llaisys.DeviceType.NVIDIA)


@pytest.mark.gpu
def test_memcpy_round_trip_nvidia(cuda_device):
    check_memcpy_round_trip(llaisys.DeviceType.NVIDIA)


@pytest.mark.gpu
def test_add_and_rearrange_nvidia(cuda_device):
    check_add_and_rearrange(llaisys.DeviceType.NVIDIA)


@pytest.mark.gpu
def test_operator_output_is_visible_to_memcpy_sync_without_synchronize(cuda_device):
    """The reference's tests read results with memcpy_sync straight after an op and hand torch CUDA pointers to
    memcpy_sync(D2D) (reference: test/test_utils.py:27-32, :143-149): both must be ordered correctly."""
    dev = llaisys.DeviceType.NVIDIA
    api = llaisys.RuntimeAPI(dev)
    a = torch.rand((1024, 1024), device="cuda")
    b = torch.rand((1024, 1024), device="cuda")
    a_, b_, c_ = (llaisys.Tensor((1024, 1024), dtype=llaisys.DataType.F32, device=dev) for _ in range(3))
    api.memcpy_sync(a_.data_ptr(), a.data_ptr(), a.numel() * 4, llaisys.MemcpyKind.D2D)
    api.memcpy_sync(b_.data_ptr(), b.data_ptr(), b.numel() * 4, llaisys.MemcpyKind.D2D)
    for _ in range(20):
        llaisys.Ops.add(c_, a_, b_)
    out = torch.zeros_like(a)
    api.memcpy_sync(out.data_ptr(), c_.data_ptr(), out.numel() * 4, llaisys.MemcpyKind.D2D)
    assert torch.equal(out, a + b)
