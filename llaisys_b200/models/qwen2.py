"""Qwen2 on the C model API (reference: python/llaisys/models/qwen2.py:9-33 declares this class with an empty
constructor and a generate() that returns []; test/test_infer.py:57-80 is how it is called).

The constructor reads a Hugging Face checkpoint directory (config.json + *.safetensors) exactly as the reference's
skeleton starts to, or takes a config dict and a state dict directly (random-init weights for tests and benchmarks).
generate() follows the Hugging Face convention the reference's test compares against: it returns prompt + new tokens.
"""
from __future__ import annotations

import ctypes
import itertools
import json
from ctypes import c_float, c_int, c_int32, c_int64
from pathlib import Path
from typing import Mapping, Sequence

import numpy as np

from ..libllaisys import LIB_LLAISYS, DataType, DeviceType, LlaisysQwen2Meta
from ..paged_kv import _check

_TORCH_DTYPE_NAMES = {"bfloat16": DataType.BF16, "float16": DataType.F16, "float32": DataType.F32}


def _torch_dtype(dtype: DataType):
    import torch
    return {DataType.BF16: torch.bfloat16, DataType.F16: torch.float16, DataType.F32: torch.float32}[dtype]


class Qwen2:
    def __init__(self, model_path=None, device: DeviceType = DeviceType.CPU, *, device_id: int = 0,
                 config: Mapping | None = None, state_dict: Mapping | None = None, dtype: DataType | None = None,
                 max_seq_len: int | None = None, tp_group=None):
        """tp_group: a torch.distributed process group (gloo for CPU models, nccl for NVIDIA) whose ranks share this
        model by tensor parallelism: every rank constructs it with the same checkpoint and then makes the same calls;
        each loads only its slices of the attention and MLP matrices."""
        if model_path is not None:
            model_path = Path(model_path)
            config = json.loads((model_path / "config.json").read_text())
        if config is None:
            raise ValueError("Qwen2 needs a checkpoint directory or a config")
        if dtype is None:
            dtype = _TORCH_DTYPE_NAMES.get(str(config.get("torch_dtype", config.get("dtype", "bfloat16"))), DataType.BF16)
        nh = int(config["num_attention_heads"])
        hs = int(config["hidden_size"])
        eos = config.get("eos_token_id", -1)
        if isinstance(eos, (list, tuple)):
            eos = eos[0]
        self.meta = LlaisysQwen2Meta(
            dtype=int(dtype), nlayer=int(config["num_hidden_layers"]), hs=hs, nh=nh,
            nkvh=int(config.get("num_key_value_heads", nh)), dh=int(config.get("head_dim") or hs // nh),
            di=int(config["intermediate_size"]),
            maxseq=int(max_seq_len or config.get("max_position_embeddings", 4096)),
            voc=int(config["vocab_size"]), epsilon=float(config.get("rms_norm_eps", 1e-6)),
            theta=float(config.get("rope_theta", 10000.0)), end_token=int(-1 if eos is None else eos))
        self.dtype = dtype
        self.device = device
        self.device_id = device_id
        self.tp_rank, self.tp_world = 0, 1
        if tp_group is not None:
            import torch.distributed as dist
            self.tp_rank, self.tp_world = dist.get_rank(tp_group), dist.get_world_size(tp_group)
        if self.tp_world > 1:
            self._model = LIB_LLAISYS.llaisysQwen2ModelCreateTP(ctypes.byref(self.meta), int(device), device_id,
                                                                self.tp_rank, self.tp_world)
        else:
            ids = (c_int * 1)(device_id)
            self._model = LIB_LLAISYS.llaisysQwen2ModelCreate(ctypes.byref(self.meta), int(device), ids, 1)
        if not self._model:
            raise RuntimeError("llaisysQwen2ModelCreate failed: " + (LIB_LLAISYS.llaisysGetLastError() or b"").decode())
        if self.tp_world > 1:
            self._connect(tp_group)
        self._weights = LIB_LLAISYS.llaisysQwen2ModelWeights(self._model).contents
        self._loaded: set[str] = set()
        self._tied_embedding = None
        if model_path is not None:
            import safetensors
            for file in sorted(model_path.glob("*.safetensors")):
                with safetensors.safe_open(file, framework="pt", device="cpu") as data:
                    for name in data.keys():
                        self._load(name, data.get_tensor(name))
        if state_dict is not None:
            for name, value in state_dict.items():
                self._load(name, value)
        if model_path is not None or state_dict is not None:
            if "lm_head.weight" not in self._loaded and "model.embed_tokens.weight" in self._loaded:
                self._load("lm_head.weight", self._tied_embedding)  # tie_word_embeddings checkpoints
            missing = self._expected_names() - self._loaded
            if missing:
                raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {sorted(missing)[:3]}")
        self._tied_embedding = None

    # ---- weights -----------------------------------------------------------------------------------------------------

    _LAYER_SLOTS = {
        "input_layernorm.weight": "attn_norm_w", "self_attn.q_proj.weight": "attn_q_w",
        "self_attn.q_proj.bias": "attn_q_b", "self_attn.k_proj.weight": "attn_k_w",
        "self_attn.k_proj.bias": "attn_k_b", "self_attn.v_proj.weight": "attn_v_w",
        "self_attn.v_proj.bias": "attn_v_b", "self_attn.o_proj.weight": "attn_o_w",
        "post_attention_layernorm.weight": "mlp_norm_w", "mlp.gate_proj.weight": "mlp_gate_w",
        "mlp.up_proj.weight": "mlp_up_w", "mlp.down_proj.weight": "mlp_down_w",
    }
    _TOP_SLOTS = {"model.embed_tokens.weight": "in_embed", "lm_head.weight": "out_embed",
                  "model.norm.weight": "out_norm_w"}

    def _expected_names(self) -> set[str]:
        names = set(self._TOP_SLOTS)
        for i in range(self.meta.nlayer):
            names |= {f"model.layers.{i}.{suffix}" for suffix in self._LAYER_SLOTS}
        return names

    def _handle(self, name: str):
        if name in self._TOP_SLOTS:
            return getattr(self._weights, self._TOP_SLOTS[name])
        parts = name.split(".")
        if len(parts) > 3 and parts[0] == "model" and parts[1] == "layers" and parts[2].isdigit():
            slot = self._LAYER_SLOTS.get(".".join(parts[3:]))
            layer = int(parts[2])
            if slot is not None and layer < self.meta.nlayer:
                return getattr(self._weights, slot)[layer]
        return None

    def _connect(self, group) -> None:
        """Gives the sharded model its all-reduce: NCCL on the model's stream for NVIDIA (the unique id travels through
        the process group), a callback into the (gloo) process group for CPU."""
        import torch
        import torch.distributed as dist

        if self.device == DeviceType.NVIDIA:
            box = [None]
            if self.tp_rank == 0:
                uid = ctypes.create_string_buffer(128)
                _check(LIB_LLAISYS.llaisysNcclUniqueId(uid))
                box[0] = uid.raw
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0), group=group)
            uid = ctypes.create_string_buffer(box[0], 128)
            _check(LIB_LLAISYS.llaisysQwen2ModelSetAllReduceNccl(self._model, uid))
            return
        torch_types = {int(DataType.F32): torch.float32, int(DataType.F16): torch.float16,
                       int(DataType.BF16): torch.bfloat16}

        def all_reduce(buf, count, dtype, _user):
            try:
                tdt = torch_types[dtype]
                raw = (ctypes.c_char * (count * torch.empty((), dtype=tdt).element_size())).from_address(buf)
                tensor = torch.frombuffer(raw, dtype=tdt)
                if tdt == torch.float32:
                    dist.all_reduce(tensor, group=group)
                else:  # sum 16-bit activations in f32, as NCCL does internally
                    wide = tensor.float()
                    dist.all_reduce(wide, group=group)
                    tensor.copy_(wide)
                return 0
            except Exception:  # never unwind through the C frames
                import traceback
                traceback.print_exc()
                return 1

        from ..libllaisys import ALL_REDUCE_FN
        self._all_reduce_cb = ALL_REDUCE_FN(all_reduce)  # keep the trampoline alive as long as the model
        _check(LIB_LLAISYS.llaisysQwen2ModelSetAllReduceCallback(self._model, self._all_reduce_cb, None))

    def _load(self, name: str, value) -> None:
        """Copies one checkpoint tensor (torch, any float dtype, host or device) into the model's weight of that name;
        names the model has no slot for (rotary caches and the like) are skipped."""
        handle = self._handle(name)
        if handle is None:
            return
        shape = self._shape_of(handle)
        host = value.detach()
        if self.tp_world > 1 and tuple(host.shape) != shape and host.ndim == len(shape):
            # this rank's slice: the one dimension that is tp_world times the model's (rows of q/k/v/gate/up and their
            # biases, columns of the output and down projections)
            for dim, (have, want) in enumerate(zip(host.shape, shape)):
                if have == want * self.tp_world:
                    host = host.narrow(dim, self.tp_rank * want, want)
        host = host.to(device="cpu", dtype=_torch_dtype(self.dtype)).contiguous()
        if tuple(host.shape) != shape:
            raise ValueError(f"{name}: checkpoint shape {tuple(host.shape)} != model shape {shape}")
        LIB_LLAISYS.tensorLoad(handle, host.data_ptr())
        if name == "model.embed_tokens.weight":
            self._tied_embedding = host
        self._loaded.add(name)

    def load_tensor(self, name: str, value) -> None:
        """Public form of the loader for callers that stream weights in one at a time (Hugging Face names)."""
        self._load(name, value)

    @staticmethod
    def _shape_of(handle) -> tuple[int, ...]:
        ndim = int(LIB_LLAISYS.tensorGetNdim(handle))
        buf = (ctypes.c_size_t * ndim)()
        LIB_LLAISYS.tensorGetShape(handle, buf)
        return tuple(buf)

    def close(self) -> None:
        if getattr(self, "_model", None):
            LIB_LLAISYS.llaisysQwen2ModelDestroy(self._model)
            self._model = None

    def __del__(self):
        self.close()

    # ---- the reference's call: one prompt in, prompt + completion out ----------------------------------------------------

    def generate(self, inputs: Sequence[int], max_new_tokens: int | None = None, top_k: int = 1, top_p: float = 0.8,
                 temperature: float = 0.8, seed: int | None = None) -> list[int]:
        """Greedy when top_k == 1 (the argmax is taken on the device); otherwise temperature / top-k / top-p sampling
        on the host from the step's logits. Stops after max_new_tokens or at the model's end token (kept in the
        output, as Hugging Face's generate does)."""
        inputs = [int(t) for t in inputs]
        if not inputs:
            return []
        if max_new_tokens is None:
            max_new_tokens = max(0, int(self.meta.maxseq) - len(inputs))
        _check(LIB_LLAISYS.llaisysQwen2ModelReset(self._model))
        rng = np.random.default_rng(seed)
        out = list(inputs)
        feed = inputs
        for _ in range(max_new_tokens):
            arr = (c_int64 * len(feed))(*feed)
            token = int(LIB_LLAISYS.llaisysQwen2ModelInfer(self._model, arr, len(feed)))
            if top_k != 1:
                token = self._sample(self.last_logits()[0], top_k, top_p, temperature, rng)
            out.append(token)
            if token == self.meta.end_token:
                break
            feed = [token]
        return out

    @staticmethod
    def _sample(logits: np.ndarray, top_k: int, top_p: float, temperature: float, rng) -> int:
        scores = logits.astype(np.float64) / max(float(temperature), 1e-6)
        order = np.argsort(-scores, kind="stable")
        if top_k and top_k > 0:
            order = order[:top_k]
        probs = np.exp(scores[order] - scores[order[0]])
        probs /= probs.sum()
        if 0.0 < top_p < 1.0:
            keep = int(np.searchsorted(np.cumsum(probs), top_p, side="left")) + 1
            order, probs = order[:keep], probs[:keep] / probs[:keep].sum()
        return int(order[rng.choice(len(order), p=probs)])

    # ---- batched sequences ----------------------------------------------------------------------------------------------

    def configure_cache(self, max_seqs: int, max_tokens: int) -> None:
        _check(LIB_LLAISYS.llaisysQwen2ModelConfigureCache(self._model, max_seqs, max_tokens))

    def add_seq(self) -> int:
        seq = c_int32(-1)
        _check(LIB_LLAISYS.llaisysQwen2ModelSeqAdd(self._model, ctypes.byref(seq)))
        return seq.value

    def add_seq_with_prefix(self, tokens: Sequence[int]) -> tuple[int, int]:
        """New sequence that reuses cached K/V of earlier sequences starting with the same tokens (whole pages, leaving
        at least one token to run). -> (sequence id, tokens already covered); feed tokens[covered:] to step()."""
        arr = np.ascontiguousarray(tokens, dtype=np.int64)
        seq, matched = c_int32(-1), ctypes.c_size_t(0)
        _check(LIB_LLAISYS.llaisysQwen2ModelSeqAddWithPrefix(self._model, arr.ctypes.data_as(ctypes.POINTER(c_int64)),
                                                             arr.size, ctypes.byref(seq), ctypes.byref(matched)))
        return seq.value, int(matched.value)

    def free_seq(self, seq: int) -> None:
        _check(LIB_LLAISYS.llaisysQwen2ModelSeqFree(self._model, seq))

    def step(self, seq_ids: Sequence[int], tokens: Sequence[Sequence[int]]) -> list[int]:
        """Appends tokens[i] to sequence seq_ids[i] (any mix of prefill chunks and single decode tokens) and returns
        the greedy next token of every sequence."""
        n = len(seq_ids)
        if len(tokens) != n:
            raise ValueError("one token list per sequence")
        ids = np.ascontiguousarray(seq_ids, dtype=np.int32)
        # (one pass over the token lists: building an array per sequence and concatenating them cost more than the
        # library call's own host work in a 64-sequence decode step)
        counts = np.fromiter(map(len, tokens), dtype=np.int32, count=n)
        flat = np.fromiter(itertools.chain.from_iterable(tokens), dtype=np.int64, count=int(counts.sum()))
        nxt = np.zeros(n, dtype=np.int64)
        _check(LIB_LLAISYS.llaisysQwen2ModelStep(
            self._model, ids.ctypes.data_as(ctypes.POINTER(c_int32)), counts.ctypes.data_as(ctypes.POINTER(c_int32)), n,
            flat.ctypes.data_as(ctypes.POINTER(c_int64)), nxt.ctypes.data_as(ctypes.POINTER(c_int64))))
        return nxt.tolist()

    def decode_loop(self, seq_ids: Sequence[int], first_tokens: Sequence[int], n_steps: int) -> np.ndarray:
        """n_steps greedy steps with the loop state kept on the device; returns int64 [n_steps, n_seqs]."""
        n = len(seq_ids)
        ids = np.ascontiguousarray(seq_ids, dtype=np.int32)
        first = np.ascontiguousarray(first_tokens, dtype=np.int64)
        if first.shape != (n,):
            raise ValueError("one first token per sequence")
        out = np.zeros((n_steps, n), dtype=np.int64)
        _check(LIB_LLAISYS.llaisysQwen2ModelDecodeLoop(
            self._model, ids.ctypes.data_as(ctypes.POINTER(c_int32)), n, first.ctypes.data_as(ctypes.POINTER(c_int64)),
            n_steps, out.ctypes.data_as(ctypes.POINTER(c_int64))))
        return out

    def last_logits(self, n_seqs: int = 1) -> np.ndarray:
        """float32 [n_seqs, voc] logits of the most recent step (n_seqs = that step's sequence count)."""
        out = np.zeros((n_seqs, int(self.meta.voc)), dtype=np.float32)
        _check(LIB_LLAISYS.llaisysQwen2ModelLastLogits(self._model, out.ctypes.data_as(ctypes.POINTER(c_float)), out.size))
        return out

    @property
    def last_loop_ms(self) -> float:
        """Device milliseconds per decode step of the last decode_loop()."""
        return float(LIB_LLAISYS.llaisysQwen2ModelLastLoopMs(self._model))
