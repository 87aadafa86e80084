"""CPU oracle for the KV-cache / self-attention path. TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this package, and only as the
checker or as the timed CPU baseline. Nothing under llaisys_b200/ imports it.

Pinning status
  * attention.self_attention  restates the reference's own definition of the operator, the PyTorch function
    `torch_self_attention` (reference: test/ops/self_attention.py:11-28). The reference holds no golden vectors
    for it (its tests compare live against that function on unseeded inputs), so the restatement is pinned by
    running the reference function itself: tests/golden/make_golden.py imports it from the reference tree,
    demands bit-equality with this restatement on seeded inputs, and commits the reference's outputs as
    fixtures (tests/golden/self_attention_golden.npz).
  * paged.*  (block manager, append, gather) has no counterpart in the reference -- PARITY UNPINNED by the
    reference. It is pinned by its own invariant instead: append followed by gather returns the appended rows
    bit for bit, and attention over gathered rows equals attention over the original rows.
"""
