"""Shared test plumbing: dtype tables, golden-vector loading, cache filling, comparisons."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

import llaisys_b200 as llaisys

GOLDEN = Path(__file__).with_name("golden") / "self_attention_golden.npz"


def reference_root() -> Path | None:
    """Where the reference project's tree is, if it is available: the directory named by LLAISYS_REFERENCE_ROOT, else a
    checkout called `reference` beside this repository. None (the tests that need it are skipped) otherwise."""
    import os

    cands = [os.environ.get("LLAISYS_REFERENCE_ROOT"), Path(__file__).resolve().parents[2] / "reference"]
    for c in cands:
        if c and (Path(c) / "test" / "ops" / "self_attention.py").is_file():
            return Path(c)
    return None

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
LL_DTYPE = {"f32": llaisys.DataType.F32, "f16": llaisys.DataType.F16, "bf16": llaisys.DataType.BF16,
            "i64": llaisys.DataType.I64, "i32": llaisys.DataType.I32}
# tolerances of the reference's own self-attention test (test/ops/self_attention.py:76-81), atol == rtol
REF_TOL = {"f32": 1e-5, "f16": 1e-3, "bf16": 1e-2}
# end-to-end bound on the benchmark shapes: max-abs error against the reference's definition
MAX_ABS = {"f32": 1e-4, "f16": 5e-3, "bf16": 2e-2}


def words_to_tensor(words: np.ndarray, dname: str) -> torch.Tensor:
    """Inverse of the generator's bit-pattern dump."""
    if dname == "f32":
        return torch.from_numpy(words.view(np.int32).copy()).view(torch.float32)
    return torch.from_numpy(words.view(np.int16).copy()).view(TORCH_DTYPE[dname])


def tensor_words(t: torch.Tensor) -> torch.Tensor:
    """Bit pattern as an integer tensor, for exact comparisons of 16-bit floats."""
    t = t.contiguous()
    return t.view(torch.int32) if t.element_size() == 4 else t.view(torch.int16)


def golden_cases():
    data = np.load(GOLDEN)
    return [str(n) for n in data["names"]]


def load_golden(name: str):
    """-> dtype name, q, k, v (or None when only a hash is stored), scale, expected output, sha, shapes"""
    data = np.load(GOLDEN)
    dname = str(data[f"{name}/dtype"])
    shapes = data[f"{name}/shapes"].tolist()
    qs, ks = tuple(shapes[:3]), tuple(shapes[3:])
    out = words_to_tensor(data[f"{name}/out"], dname).reshape(qs)
    if f"{name}/q" in data:
        q = words_to_tensor(data[f"{name}/q"], dname).reshape(qs)
        k = words_to_tensor(data[f"{name}/k"], dname).reshape(ks)
        v = words_to_tensor(data[f"{name}/v"], dname).reshape(ks)
    else:
        q = k = v = None
    return dname, q, k, v, float(data[f"{name}/scale"]), out, str(data[f"{name}/sha"])


def torch_device(device: llaisys.DeviceType, device_id: int = 0) -> torch.device:
    return torch.device("cpu") if device == llaisys.DeviceType.CPU else torch.device(f"cuda:{device_id}")


def to_llaisys(t: torch.Tensor, device: llaisys.DeviceType, dname: str) -> llaisys.Tensor:
    """Copies a host torch tensor into a fresh llaisys tensor on `device`."""
    t = t.contiguous()
    out = llaisys.Tensor(tuple(t.shape), dtype=LL_DTYPE[dname], device=device)
    out.load(t.data_ptr())
    return out


def from_llaisys(t: llaisys.Tensor, dname: str) -> torch.Tensor:
    """Copies a contiguous llaisys tensor back to a host torch tensor."""
    out = torch.empty(t.shape(), dtype=TORCH_DTYPE.get(dname, torch.int64))
    api = llaisys.RuntimeAPI(t.device_type())
    kind = llaisys.MemcpyKind.D2H if t.device_type() != llaisys.DeviceType.CPU else llaisys.MemcpyKind.H2H
    api.memcpy_sync(out.data_ptr(), t.data_ptr(), out.numel() * out.element_size(), kind)
    return out


def run_self_attention(q, k, v, scale, device: llaisys.DeviceType, dname: str) -> torch.Tensor:
    q_, k_, v_ = (to_llaisys(x, device, dname) for x in (q, k, v))
    o_ = llaisys.Tensor(tuple(q.shape), dtype=LL_DTYPE[dname], device=device)
    llaisys.Ops.self_attention(o_, q_, k_, v_, scale)
    return from_llaisys(o_, dname)


def build_cache(device: llaisys.DeviceType, dname: str, pages_per_seq, *, num_pages: int, nkvh: int, d: int,
                page: int = 16, nlayer: int = 1, max_seqs: int | None = None):
    """Cache whose sequences own exactly the given physical pages. Returns (cache, seq ids)."""
    cache = llaisys.PagedKVCache(num_pages, nkvh, d, page_size=page, nlayer=nlayer, dtype=LL_DTYPE[dname],
                                 device=device, max_seqs=max_seqs or max(len(pages_per_seq), 1),
                                 max_pages_per_seq=max([len(p) for p in pages_per_seq] + [1]))
    seqs = []
    for pages in pages_per_seq:
        s = cache.add_seq()
        cache.assign_pages(s, pages)
        seqs.append(s)
    return cache, seqs


def append_all(cache, layer: int, seqs, ks, vs, device: llaisys.DeviceType, lo=None, hi=None):
    """Appends rows [lo_i, hi_i) of every sequence's K/V (default: all rows) in ONE append call."""
    dev = torch_device(device)
    rows_k, rows_v, ids, pos = [], [], [], []
    for i, (s, k, v) in enumerate(zip(seqs, ks, vs)):
        a = 0 if lo is None else lo[i]
        b = k.shape[0] if hi is None else hi[i]
        rows_k.append(k[a:b])
        rows_v.append(v[a:b])
        ids += [s] * (b - a)
        pos += list(range(a, b))
    if not ids:
        return
    k_rows = torch.cat(rows_k).contiguous().to(dev)
    v_rows = torch.cat(rows_v).contiguous().to(dev)
    cache.append(layer, k_rows, v_rows, ids, pos)
    cache.check()


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.double() - b.double()).abs().max().item() if a.numel() else 0.0
