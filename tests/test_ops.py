"""The six operators around the attention path against the restated oracles, with the reference's shapes and
tolerances (reference: test/ops/{argmax,embedding,linear,rms_norm,rope,swiglu}.py), on CPU and -- marked gpu -- NVIDIA."""
import pytest
import torch

import llaisys_b200 as llaisys
from oracle import ops as oracle_ops
from tests import helpers

CPU, NVIDIA = llaisys.DeviceType.CPU, llaisys.DeviceType.NVIDIA
PREC = {"f32": 1e-5, "f16": 1e-3, "bf16": 1e-2}


def new(shape, dname, device):
    return llaisys.Tensor(tuple(shape), dtype=helpers.LL_DTYPE[dname], device=device)


def put_i64(t: torch.Tensor, device) -> llaisys.Tensor:
    out = llaisys.Tensor(tuple(t.shape), dtype=llaisys.DataType.I64, device=device)
    out.load(t.contiguous().data_ptr())
    return out


def close(got, expect, tol):
    return torch.allclose(got.float(), expect.float(), atol=tol, rtol=tol)


def check_argmax(device):
    for n in (4, 4096, 151936):
        for dname in ("f32", "f16", "bf16"):
            vals = torch.rand(n).to(helpers.TORCH_DTYPE[dname])
            idx, val = oracle_ops.argmax(vals)
            idx_, val_ = llaisys.Tensor((1,), dtype=llaisys.DataType.I64, device=device), new((1,), dname, device)
            llaisys.Ops.argmax(idx_, val_, helpers.to_llaisys(vals, device, dname))
            got_val = helpers.from_llaisys(val_, dname)
            got_idx = helpers.from_llaisys(idx_, "i64")
            assert torch.equal(got_val, val)
            # ties (16-bit values repeat): any index of the maximum is the reference's behaviour; we return the first
            assert vals[got_idx.item()] == val.item() and got_idx.item() == int((vals == val).nonzero()[0])


def check_embedding(device):
    for n, (vocab, d) in ((1, (2, 3)), (50, (512, 4096))):
        for dname in ("f32", "f16", "bf16"):
            w = torch.rand((vocab, d)).to(helpers.TORCH_DTYPE[dname])
            idx = torch.randint(0, vocab, (n,), dtype=torch.int64)
            out_ = new((n, d), dname, device)
            llaisys.Ops.embedding(out_, put_i64(idx, device), helpers.to_llaisys(w, device, dname))
            assert torch.equal(helpers.tensor_words(helpers.from_llaisys(out_, dname)),
                               helpers.tensor_words(oracle_ops.embedding(idx, w)))


def check_linear(device):
    for (m, k, n, use_bias) in ((2, 4, 3, True), (2, 4, 3, False), (512, 4096, 4096, True), (64, 1536, 256, False)):
        for dname in ("f32", "f16", "bf16"):
            dt = helpers.TORCH_DTYPE[dname]
            x, w = torch.rand((m, k)).to(dt), torch.rand((n, k)).to(dt)
            b = torch.rand((n,)).to(dt) if use_bias else None
            out_ = new((m, n), dname, device)
            llaisys.Ops.linear(out_, helpers.to_llaisys(x, device, dname), helpers.to_llaisys(w, device, dname),
                               helpers.to_llaisys(b, device, dname) if use_bias else None)
            assert close(helpers.from_llaisys(out_, dname), oracle_ops.linear(x, w, b), PREC[dname]), (m, k, n, dname)


def check_rms_norm(device):
    for shape in ((1, 4), (512, 4096), (64, 1536)):
        for dname in ("f32", "f16", "bf16"):
            dt = helpers.TORCH_DTYPE[dname]
            x, w = torch.rand(shape).to(dt), torch.rand((shape[1],)).to(dt)
            out_ = new(shape, dname, device)
            llaisys.Ops.rms_norm(out_, helpers.to_llaisys(x, device, dname), helpers.to_llaisys(w, device, dname), 1e-5)
            assert close(helpers.from_llaisys(out_, dname), oracle_ops.rms_norm(x, w, 1e-5), PREC[dname])


def check_rope(device):
    for shape, (lo, hi) in (((2, 1, 4), (0, 2)), ((512, 4, 4096 // 4), (512, 1024)), ((64, 12, 128), (2000, 2064))):
        for dname, tol in (("f32", 1e-4), ("f16", 1e-3), ("bf16", 1e-2)):
            x = torch.rand(shape).to(helpers.TORCH_DTYPE[dname])
            pos = torch.arange(lo, hi, dtype=torch.int64)
            out_ = new(shape, dname, device)
            llaisys.Ops.rope(out_, helpers.to_llaisys(x, device, dname), put_i64(pos, device), 10000.0)
            assert close(helpers.from_llaisys(out_, dname), oracle_ops.rope(x, pos, 10000.0), tol), (shape, dname)


def check_swiglu(device):
    for shape in ((2, 3), (512, 4096)):
        for dname in ("f32", "f16", "bf16"):
            dt = helpers.TORCH_DTYPE[dname]
            gate, up = (torch.rand(shape) * 4 - 2).to(dt), torch.rand(shape).to(dt)
            out_ = new(shape, dname, device)
            llaisys.Ops.swiglu(out_, helpers.to_llaisys(gate, device, dname), helpers.to_llaisys(up, device, dname))
            assert close(helpers.from_llaisys(out_, dname), oracle_ops.swiglu(gate, up), PREC[dname])


CHECKS = [check_argmax, check_embedding, check_linear, check_rms_norm, check_rope, check_swiglu]


@pytest.mark.parametrize("check", CHECKS, ids=lambda f: f.__name__[6:])
def test_op_cpu(check):
    torch.manual_seed(1)
    check(CPU)


@pytest.mark.gpu
@pytest.mark.parametrize("check", CHECKS, ids=lambda f: f.__name__[6:])
def test_op_nvidia(cuda_device, check):
    torch.manual_seed(1)
    check(NVIDIA)
