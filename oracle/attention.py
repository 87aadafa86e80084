"""Self-attention oracle: the reference's definition, restated.

Reference: test/ops/self_attention.py:11-28 (`torch_self_attention`), shapes from README.md:244-266.
The reference computes every step in the dtype of its inputs (for bf16 the scores, the scaled scores, the
probabilities and the output are each rounded to bf16; torch accumulates each matmul in f32 internally).
`self_attention` below keeps that step order and dtype so that it reproduces the reference bit for bit on one
machine; `self_attention_f64` is the same mathematics in float64 for tight checks of f32-accumulating kernels.
"""
from __future__ import annotations

import torch


def causal_visible(qlen: int, kvlen: int) -> torch.Tensor:
    """bool [qlen, kvlen]: key j is visible to query i iff j <= i + (kvlen - qlen).

    Reference: test/ops/self_attention.py:18 -- ones(L, S).tril(diagonal=S - L).
    """
    i = torch.arange(qlen).unsqueeze(1)
    j = torch.arange(kvlen).unsqueeze(0)
    return j <= i + (kvlen - qlen)


def self_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q [qlen, nh, d], k [kvlen, nkvh, d], v [kvlen, nkvh, dv] -> [qlen, nh, dv], all in q.dtype.

    Step by step as the reference (line numbers of test/ops/self_attention.py):
      :12-14  move heads to the front: [heads, len, d]
      :16-19  additive bias in the query dtype: 0 where visible, -inf elsewhere
      :22-23  GQA: repeat each kv head nh // nkvh times, so query head h reads kv head h // (nh // nkvh)
      :25     scores = q @ k^T * scale      (matmul, then a separate multiply, both rounded to q.dtype)
      :26     scores += bias
      :27     softmax over keys
      :28     probabilities @ v, heads back to the middle
    """
    qh, kh, vh = q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1)
    qlen, kvlen = qh.size(1), kh.size(1)
    bias = torch.zeros(qlen, kvlen, dtype=q.dtype)
    bias.masked_fill_(~causal_visible(qlen, kvlen), float("-inf"))
    group = qh.size(0) // kh.size(0)
    kh = kh.repeat_interleave(group, dim=0)
    vh = vh.repeat_interleave(group, dim=0)
    scores = torch.matmul(qh, kh.transpose(1, 2)) * scale
    scores += bias
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, vh).transpose(0, 1).contiguous()


def self_attention_f64(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """Same mathematics on the given (already rounded) inputs, carried in float64; returns float64."""
    out = self_attention(q.double(), k.double(), v.double(), scale)
    return out


def partial_attention_f64(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float):
    """Decode query q [1, nh, d] over a KV range: (o [nh, d], m [nh], l [nh]) in float64.

    o is normalised over the range, m = max scaled score, l = sum exp(score - m): the triple a KV-range shard
    hands to the log-sum-exp merge. An empty range gives o = 0, m = -inf, l = 0.
    """
    nh, d = q.size(1), q.size(2)
    if k.size(0) == 0:
        return (torch.zeros(nh, d, dtype=torch.float64), torch.full((nh,), float("-inf"), dtype=torch.float64),
                torch.zeros(nh, dtype=torch.float64))
    group = nh // k.size(1)
    kh = k.double().transpose(0, 1).repeat_interleave(group, dim=0)  # [nh, len, d]
    vh = v.double().transpose(0, 1).repeat_interleave(group, dim=0)
    s = torch.einsum("hd,hld->hl", q[0].double(), kh) * scale
    m = s.max(dim=1).values
    p = torch.exp(s - m.unsqueeze(1))
    l = p.sum(dim=1)
    o = torch.einsum("hl,hld->hd", p, vh) / l.unsqueeze(1)
    return o, m, l


def lse_merge_f64(o: torch.Tensor, m: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
    """Merges partials o [P, R, d], m [P, R], l [P, R] -> [R, d] (float64): weights l * exp(m - max m)."""
    o, m, l = o.double(), m.double(), l.double()
    m_safe = torch.where(l > 0, m, torch.full_like(m, float("-inf")))
    m_all = m_safe.max(dim=0).values
    m_all = torch.where(torch.isinf(m_all), torch.zeros_like(m_all), m_all)
    w = torch.where(l > 0, l * torch.exp(m_safe - m_all.unsqueeze(0)), torch.zeros_like(l))
    tot = w.sum(dim=0)
    num = (w.unsqueeze(-1) * o).sum(dim=0)
    return torch.where(tot.unsqueeze(-1) > 0, num / tot.clamp_min(1e-300).unsqueeze(-1), torch.zeros_like(num))


def decode_attention_f64_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                                 chunk: int = 16384) -> torch.Tensor:
    """self_attention_f64 for ONE query over a very long context, in bounded memory: the keys are walked in ranges of
    `chunk` tokens (partial_attention_f64) and the ranges merged (lse_merge_f64). q [1, nh, d] -> float64 [1, nh, d].
    Equal to self_attention_f64 up to float64 rounding; the whole-context version would repeat K and V per query head
    in float64 (3 GB at 131072 tokens)."""
    assert q.size(0) == 1
    os_, ms, ls = [], [], []
    for lo in range(0, k.size(0), chunk):
        o, m, l = partial_attention_f64(q, k[lo:lo + chunk], v[lo:lo + chunk], scale)
        os_.append(o)
        ms.append(m)
        ls.append(l)
    return lse_merge_f64(torch.stack(os_), torch.stack(ms), torch.stack(ls)).unsqueeze(0)
