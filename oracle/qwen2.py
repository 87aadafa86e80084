"""Oracle for the Qwen2 decoder: the model composed from the operator oracles, with a contiguous per-sequence K/V cache.

The reference declares the model (include/llaisys/models/qwen2.h:7-40) and leaves it unimplemented; what it must
compute is fixed by the reference's end-to-end test, which compares generated tokens with Hugging Face's
Qwen2ForCausalLM under greedy settings (test/test_infer.py:83-148). This file restates that architecture -- RMSNorm,
q/k/v projections with bias, half-split RoPE, causal GQA attention, output projection, SwiGLU MLP, final norm, untied
vocabulary projection -- on oracle/ops.py and oracle/attention.py, i.e. on the reference's own per-operator
definitions. TEST INFRASTRUCTURE ONLY (see oracle/__init__.py). Pinned in tests/test_qwen2_model.py against
transformers' Qwen2ForCausalLM on seeded random weights (f32: same greedy tokens, logits within 2e-4).
"""
from __future__ import annotations

import torch

from . import attention, ops


class Qwen2Oracle:
    def __init__(self, config: dict, state_dict: dict, dtype: torch.dtype = torch.float32):
        self.cfg = config
        self.dtype = dtype
        self.w = {k: v.detach().to("cpu", dtype) for k, v in state_dict.items()}
        if "lm_head.weight" not in self.w:
            self.w["lm_head.weight"] = self.w["model.embed_tokens.weight"]
        self.nlayer = int(config["num_hidden_layers"])
        self.nh = int(config["num_attention_heads"])
        self.nkvh = int(config.get("num_key_value_heads", self.nh))
        self.dh = int(config.get("head_dim") or config["hidden_size"] // self.nh)
        self.eps = float(config.get("rms_norm_eps", 1e-6))
        self.theta = float(config.get("rope_theta", 10000.0))
        self.reset()

    def reset(self) -> None:
        self.k = [None] * self.nlayer
        self.v = [None] * self.nlayer
        self.length = 0

    def forward(self, tokens: list[int]) -> torch.Tensor:
        """Appends tokens to the cached sequence; -> logits [voc] of the last token."""
        w, n = self.w, len(tokens)
        pos = torch.arange(self.length, self.length + n, dtype=torch.int64)
        x = ops.embedding(torch.tensor(tokens, dtype=torch.int64), w["model.embed_tokens.weight"])
        for i in range(self.nlayer):
            p = f"model.layers.{i}."
            h = ops.rms_norm(x, w[p + "input_layernorm.weight"], self.eps)
            q = ops.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(n, self.nh, self.dh)
            k = ops.linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(n, self.nkvh, self.dh)
            v = ops.linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(n, self.nkvh, self.dh)
            q, k = ops.rope(q, pos, self.theta), ops.rope(k, pos, self.theta)
            self.k[i] = k if self.k[i] is None else torch.cat([self.k[i], k])
            self.v[i] = v if self.v[i] is None else torch.cat([self.v[i], v])
            a = attention.self_attention(q, self.k[i], self.v[i], 1.0 / self.dh ** 0.5).reshape(n, self.nh * self.dh)
            x = x + ops.linear(a, w[p + "self_attn.o_proj.weight"], None)
            h = ops.rms_norm(x, w[p + "post_attention_layernorm.weight"], self.eps)
            gate = ops.linear(h, w[p + "mlp.gate_proj.weight"], None)
            up = ops.linear(h, w[p + "mlp.up_proj.weight"], None)
            x = x + ops.linear(ops.swiglu(gate, up), w[p + "mlp.down_proj.weight"], None)
        self.length += n
        last = ops.rms_norm(x[-1:], w["model.norm.weight"], self.eps)
        return ops.linear(last, w["lm_head.weight"], None)[0]

    def generate(self, prompt: list[int], n_new: int) -> list[int]:
        self.reset()
        out, feed = list(prompt), list(prompt)
        for _ in range(n_new):
            token = int(self.forward(feed).argmax())
            out.append(token)
            feed = [token]
        return out
