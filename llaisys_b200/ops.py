"""Operators on Tensor handles (reference: python/llaisys/ops.py:6-55)."""
from __future__ import annotations

from ctypes import c_float

from .libllaisys import LIB_LLAISYS
from .tensor import Tensor


def _h(t: Tensor | None):
    return t.lib_tensor() if t is not None else None


class Ops:
    @staticmethod
    def add(c: Tensor, a: Tensor, b: Tensor) -> None:
        LIB_LLAISYS.llaisysAdd(_h(c), _h(a), _h(b))

    @staticmethod
    def argmax(max_idx: Tensor, max_val: Tensor, vals: Tensor) -> None:
        LIB_LLAISYS.llaisysArgmax(_h(max_idx), _h(max_val), _h(vals))

    @staticmethod
    def embedding(out: Tensor, index: Tensor, weight: Tensor) -> None:
        LIB_LLAISYS.llaisysEmbedding(_h(out), _h(index), _h(weight))

    @staticmethod
    def linear(out: Tensor, inp: Tensor, weight: Tensor, bias: Tensor | None) -> None:
        LIB_LLAISYS.llaisysLinear(_h(out), _h(inp), _h(weight), _h(bias))

    @staticmethod
    def linear_accumulate(out: Tensor, inp: Tensor, weight: Tensor) -> None:
        """out += inp . weight^T (new: the residual add of a decoder block folded into its projection)."""
        LIB_LLAISYS.llaisysLinearAccumulate(_h(out), _h(inp), _h(weight))

    @staticmethod
    def set_linear_policy(policy: int) -> None:
        """Which kernel serves decode-sized projections on NVIDIA, process-wide: 0 = hand-written tcgen05 kernel where it
        measured faster than cuBLAS (default), 1 = wherever its shape rules allow, 2 = always cuBLAS."""
        if LIB_LLAISYS.llaisysSetLinearPolicy(policy) != 0:
            raise ValueError(f"unknown linear policy {policy}")

    @staticmethod
    def rearrange(out: Tensor, inp: Tensor) -> None:
        LIB_LLAISYS.llaisysRearrange(_h(out), _h(inp))

    @staticmethod
    def rms_norm(out: Tensor, inp: Tensor, weight: Tensor, eps: float) -> None:
        LIB_LLAISYS.llaisysRmsNorm(_h(out), _h(inp), _h(weight), c_float(eps))

    @staticmethod
    def rope(out: Tensor, inp: Tensor, pos_ids: Tensor, theta: float) -> None:
        LIB_LLAISYS.llaisysROPE(_h(out), _h(inp), _h(pos_ids), c_float(theta))

    @staticmethod
    def self_attention(attn_val: Tensor, q: Tensor, k: Tensor, v: Tensor, scale: float) -> None:
        """attn_val[qlen, nh, d] = causal_softmax(q . k^T * scale) . v with k, v [total_len, nkvh, d]."""
        LIB_LLAISYS.llaisysSelfAttention(_h(attn_val), _h(q), _h(k), _h(v), c_float(scale))

    @staticmethod
    def swiglu(out: Tensor, gate: Tensor, up: Tensor) -> None:
        LIB_LLAISYS.llaisysSwiGLU(_h(out), _h(gate), _h(up))
