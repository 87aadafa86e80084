"""The oracle against the committed golden vectors (outputs of the reference's own torch_self_attention), and,
where the reference tree is present, against that function itself."""
from pathlib import Path

import pytest
import torch

from oracle import attention, workloads
from tests import helpers
from tests.golden import make_golden

REFERENCE = helpers.reference_root()


@pytest.mark.parametrize("name", helpers.golden_cases())
def test_oracle_matches_golden(name):
    dname, q, k, v, scale, expect, sha = helpers.load_golden(name)
    if q is None:  # inputs are regenerated from the seed and checked by hash
        assert name == "config1_f32"
        q, k, v, scale = workloads.config1()
    assert make_golden.sha(q, k, v) == sha, "seeded inputs differ from the ones the golden output was made from"
    got = attention.self_attention(q, k, v, scale)
    assert got.dtype == expect.dtype and got.shape == expect.shape
    # Same machine and torch build: bit-equal. A different CPU may sum in another order, so the bound written
    # here is the reference's own tolerance for the dtype.
    tol = helpers.REF_TOL[dname]
    assert torch.allclose(got.float(), expect.float(), atol=tol, rtol=tol)
    # the float64 statement of the same mathematics agrees to rounding of the dtype
    f64 = attention.self_attention_f64(q, k, v, scale)
    assert helpers.max_abs(f64, expect) <= {"f32": 2e-6, "f16": 2e-3, "bf16": 1.6e-2}[dname]


@pytest.mark.skipif(REFERENCE is None, reason="reference tree not available (set LLAISYS_REFERENCE_ROOT)")
@pytest.mark.parametrize("dname", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", [(2, 2, 1, 1, 4), (5, 11, 4, 2, 8), (1, 130, 12, 2, 128), (33, 70, 12, 2, 128)])
def test_oracle_bit_equal_to_reference_function(shape, dname):
    reference = make_golden.load_reference_function(REFERENCE)
    qlen, kvlen, nh, nkvh, hd = shape
    g = torch.Generator().manual_seed(1234)
    dt = helpers.TORCH_DTYPE[dname]
    q = workloads.randn((qlen, nh, hd), dt, g)
    k = workloads.randn((kvlen, nkvh, hd), dt, g)
    v = workloads.randn((kvlen, nkvh, hd), dt, g)
    expect = torch.empty_like(q)
    reference(expect, q, k, v, 1.0 / hd ** 0.5)
    got = attention.self_attention(q, k, v, 1.0 / hd ** 0.5)
    assert torch.equal(helpers.tensor_words(got), helpers.tensor_words(expect))


def test_partial_and_merge_reproduce_full_attention():
    g = torch.Generator().manual_seed(5)
    q = workloads.randn((1, 12, 128), torch.float32, g)
    k = workloads.randn((300, 2, 128), torch.float32, g)
    v = workloads.randn((300, 2, 128), torch.float32, g)
    scale = 1.0 / 128 ** 0.5
    cuts = [0, 0, 17, 160, 300, 300]  # includes empty ranges
    parts = [attention.partial_attention_f64(q, k[a:b], v[a:b], scale) for a, b in zip(cuts[:-1], cuts[1:])]
    o = torch.stack([p[0] for p in parts])
    m = torch.stack([p[1] for p in parts])
    l = torch.stack([p[2] for p in parts])
    merged = attention.lse_merge_f64(o, m, l)
    full = attention.self_attention_f64(q, k, v, scale)[0]
    assert helpers.max_abs(merged, full) < 1e-12
