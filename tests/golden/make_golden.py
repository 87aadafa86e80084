"""Generates tests/golden/self_attention_golden.npz from the REFERENCE's own oracle function.

Run in a checkout that has the reference tree mounted:
    python tests/golden/make_golden.py <root of the reference tree>

The reference defines the operator only as a PyTorch function inside its test file
(test/ops/self_attention.py:11-28, `torch_self_attention`); that file imports the compiled llaisys package at
module level, so the function is lifted out of the source by AST and executed on its own. For every case the
script (1) runs the reference function on seeded inputs, (2) demands that oracle.attention.self_attention
reproduces it BIT FOR BIT on this machine, and (3) stores inputs (small cases) or an input hash (config 1) and the
reference's output. The .npz then pins the oracle wherever the reference tree is absent.
"""
from __future__ import annotations

import ast
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import attention, workloads  # noqa: E402

DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def load_reference_function(ref_root: Path):
    src = (ref_root / "test" / "ops" / "self_attention.py").read_text()
    tree = ast.parse(src)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "torch_self_attention")
    mod = ast.Module(body=[fn], type_ignores=[])
    scope = {"torch": torch}
    exec(compile(mod, "reference:test/ops/self_attention.py", "exec"), scope)
    return scope["torch_self_attention"]


def to_words(t: torch.Tensor) -> np.ndarray:
    """Bit pattern of a tensor as an unsigned integer array (bf16 has no numpy dtype)."""
    t = t.contiguous()
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.view(torch.int16).numpy().view(np.uint16)


def sha(*tensors: torch.Tensor) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(to_words(t).tobytes())
    return h.hexdigest()


def cases():
    """(name, dtype name, q, k, v, scale, store_inputs)"""
    # the reference's own test shapes and input distribution: U[0, 1), three dtypes
    # (test/ops/self_attention.py:71-81, test/test_utils.py:8-12), here with a seed
    for si, (qlen, kvlen, nh, nkvh, hd) in enumerate([(2, 2, 1, 1, 4), (5, 11, 4, 2, 8)]):
        for dname, dt in DTYPES.items():
            g = torch.Generator().manual_seed(100 + si)
            q = torch.rand((qlen, nh, hd), generator=g, dtype=torch.float32).to(dt)
            k = torch.rand((kvlen, nkvh, hd), generator=g, dtype=torch.float32).to(dt)
            v = torch.rand((kvlen, nkvh, hd), generator=g, dtype=torch.float32).to(dt)
            yield f"ref_shape{si}_{dname}", dname, q, k, v, 1.0 / hd ** 0.5, True
    # benchmark configuration 1: f32 decode step, 512 cached + 1 appended rows
    q, k, v, scale = workloads.config1()
    yield "config1_f32", "f32", q, k, v, scale, False
    # small N(0, 1) cases at the production head shape (12 / 2 heads, d 128): decode and a causal chunk whose
    # context is not a multiple of the page size
    for dname in ("bf16", "f16", "f32"):
        dt = DTYPES[dname]
        g = torch.Generator().manual_seed(7)
        q = workloads.randn((1, 12, 128), dt, g)
        k = workloads.randn((41, 2, 128), dt, g)
        v = workloads.randn((41, 2, 128), dt, g)
        yield f"decode41_{dname}", dname, q, k, v, 1.0 / 128 ** 0.5, True
        g = torch.Generator().manual_seed(8)
        q = workloads.randn((7, 12, 128), dt, g)
        k = workloads.randn((23, 2, 128), dt, g)
        v = workloads.randn((23, 2, 128), dt, g)
        yield f"chunk7of23_{dname}", dname, q, k, v, 1.0 / 128 ** 0.5, True


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <root of the reference project's tree>")
    ref_root = Path(sys.argv[1])
    reference = load_reference_function(ref_root)
    out: dict[str, np.ndarray] = {}
    names = []
    for name, dname, q, k, v, scale, store_inputs in cases():
        ref_out = torch.empty_like(q)
        reference(ref_out, q, k, v, scale)
        mine = attention.self_attention(q, k, v, scale)
        assert torch.equal(to_words_t(mine), to_words_t(ref_out)), f"{name}: restatement differs from the reference"
        names.append(name)
        out[f"{name}/out"] = to_words(ref_out)
        out[f"{name}/scale"] = np.float64(scale)
        out[f"{name}/dtype"] = np.array(dname)
        out[f"{name}/sha"] = np.array(sha(q, k, v))
        out[f"{name}/shapes"] = np.array([*q.shape, *k.shape], dtype=np.int64)
        if store_inputs:
            out[f"{name}/q"], out[f"{name}/k"], out[f"{name}/v"] = to_words(q), to_words(k), to_words(v)
        print(f"{name:24s} ok  max|out|={ref_out.float().abs().max().item():.4f}")
    out["names"] = np.array(names)
    out["torch_version"] = np.array(torch.__version__)
    dst = Path(__file__).with_name("self_attention_golden.npz")
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size} bytes), torch {torch.__version__}")


def to_words_t(t: torch.Tensor) -> torch.Tensor:
    return torch.from_numpy(to_words(t).astype(np.int64))


if __name__ == "__main__":
    main()
