"""Oracles for the operators around the attention path, restated from the reference's own test oracles.

Each function follows the PyTorch function of the same purpose in the reference's test directory (cited per function);
like those, it computes in the dtype of its inputs unless noted. TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).
The reference holds no golden vectors for these operators; the restatements are pinned by running the reference's
own scripts against this library where the reference tree is mounted (tests/test_reference_scripts.py).
"""
from __future__ import annotations

import torch


def argmax(vals: torch.Tensor):
    """-> (max_idx int64 [1], max_val [1]). Reference: test/ops/argmax.py:11-12 (torch.max over the last dim)."""
    val, idx = torch.max(vals, dim=-1, keepdim=True)
    return idx, val


def embedding(idx: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Row gather. Reference: test/ops/embedding.py:11-12."""
    return weight[idx]


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """x . w^T + bias. Reference: test/ops/linear.py:11-12 (torch.nn.functional.linear)."""
    return torch.nn.functional.linear(x, w, bias)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """w * x * rsqrt(mean(x^2) + eps), every step in x.dtype. Reference: test/ops/rms_norm.py:11-17."""
    mean = torch.mean(torch.pow(x, 2), dim=-1, keepdim=True)
    mean = torch.rsqrt(mean + eps)
    return torch.mul(x, mean) * w


def rope(x: torch.Tensor, pos_ids: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-split rotary embedding, angles in f32. Reference: test/ops/rope.py:11-32."""
    d = x.shape[-1]
    a, b = x[..., : d // 2], x[..., d // 2:]
    positions = pos_ids.to(torch.float32).unsqueeze(1)
    i = torch.arange(0, d // 2, dtype=torch.float32)
    freqs = positions / (theta ** (2 * i / d))
    sin, cos = freqs.sin().unsqueeze(1), freqs.cos().unsqueeze(1)
    y = torch.empty_like(x)
    y[..., : d // 2] = a * cos - b * sin
    y[..., d // 2:] = b * cos + a * sin
    return y


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """up * gate / (1 + exp(-gate)), the exponential in f32. Reference: test/ops/swiglu.py:11-12."""
    return torch.mul(up, gate / (1 + torch.exp(-gate.float()).to(gate.dtype)))
