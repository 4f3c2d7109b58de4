"""Flat parameter storage and HF name mapping.

All parameters of a model live in ONE contiguous buffer per role (bf16/fp32 working weights, fp32 main
gradients), laid out layer by layer.  Named parameters are views.  That layout is what makes the
distributed pieces simple and fast on NVSwitch: an optimizer shard is a byte range, a gradient
reduce-scatter is one collective (or one peer-memory kernel) over the whole buffer, and the rollout
engine consumes the very same working weights the trainer updates (no copy, no re-layout).

QKV and gate/up projections are stored fused ([q;k;v] rows, [gate;up] rows); ``hf_views`` exposes the
un-fused HF tensors as zero-copy row slices, ``load_hf_state_dict`` accepts HF-named tensors.
Reference for the HF naming and fused/unfused conversions: ``verl/utils/model.py``,
``verl/workers/engine/fsdp/utils.py:90-123`` (MoE unfuse), ``verl/models/mcore/weight_converter.py``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterator, Optional

import torch

from .config import ModelConfig

__all__ = ["ParamSpec", "build_param_specs", "FlatParams", "ALIGN"]

ALIGN = 128  # elements; keeps every view 256-byte aligned in bf16 and shard boundaries TMA friendly


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    init: str = "normal"  # normal | ones | zeros
    decay: bool = True
    layer: int = -1  # -1: embedding/pre, num_layers: final norm/head

    @property
    def numel(self) -> int:
        return int(math.prod(self.shape))


def build_param_specs(cfg: ModelConfig, value_head: bool = False) -> list[ParamSpec]:
    h = cfg.hidden_size
    L = cfg.num_hidden_layers
    specs = []
    if cfg.has_embedding:
        specs.append(ParamSpec("embed_tokens.weight", (cfg.vocab_size, h), "normal", True, -1))
    for i in range(L):
        p = f"layers.{i}."
        specs.append(ParamSpec(p + "input_layernorm.weight", (h,), "ones", False, i))
        specs.append(ParamSpec(p + "self_attn.qkv_proj.weight", (cfg.qkv_size, h), "normal", True, i))
        if cfg.attention_bias:
            specs.append(ParamSpec(p + "self_attn.qkv_proj.bias", (cfg.qkv_size,), "zeros", False, i))
        if cfg.qk_norm:
            specs.append(ParamSpec(p + "self_attn.q_norm.weight", (cfg.head_dim,), "ones", False, i))
            specs.append(ParamSpec(p + "self_attn.k_norm.weight", (cfg.head_dim,), "ones", False, i))
        specs.append(ParamSpec(p + "self_attn.o_proj.weight", (h, cfg.q_size), "normal", True, i))
        specs.append(ParamSpec(p + "post_attention_layernorm.weight", (h,), "ones", False, i))
        if cfg.is_moe:
            E, ie = cfg.num_experts, cfg.moe_intermediate_size
            El = cfg.num_local_experts or E  # expert-parallel shards store their own experts only; the router is replicated
            specs.append(ParamSpec(p + "mlp.gate.weight", (E, h), "normal", True, i))
            specs.append(ParamSpec(p + "mlp.experts.gate_up_proj", (El, 2 * ie, h), "normal", True, i))
            specs.append(ParamSpec(p + "mlp.experts.down_proj", (El, h, ie), "normal", True, i))
            if cfg.shared_expert_intermediate_size:
                se = cfg.shared_expert_intermediate_size
                specs.append(ParamSpec(p + "mlp.shared_expert.gate_up_proj.weight", (2 * se, h), "normal", True, i))
                specs.append(ParamSpec(p + "mlp.shared_expert.down_proj.weight", (h, se), "normal", True, i))
                # scalar gate stored with 8 rows (row 0 is the gate) so the GEMM's N % 8 == 0 rule holds
                specs.append(ParamSpec(p + "mlp.shared_expert_gate.weight", (8, h), "normal", True, i))
        else:
            specs.append(ParamSpec(p + "mlp.gate_up_proj.weight", (2 * cfg.intermediate_size, h), "normal", True, i))
            specs.append(ParamSpec(p + "mlp.down_proj.weight", (h, cfg.intermediate_size), "normal", True, i))
    if not cfg.has_head:
        return specs
    specs.append(ParamSpec("norm.weight", (h,), "ones", False, L))
    if value_head:
        # scalar head stored with 8 rows (row 0 is the value) so the GEMM's N % 8 == 0 rule holds
        specs.append(ParamSpec("v_head.weight", (8, h), "normal", True, L))
    elif not cfg.tie_word_embeddings:
        specs.append(ParamSpec("lm_head.weight", (cfg.head_vocab_size or cfg.vocab_size, h), "normal", True, L))
    return specs


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatParams:
    """Named views over one flat working buffer (+ optional fp32 main-grad buffer)."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", value_head: bool = False,
                 with_main_grad: bool = False, pad_to: int = 1, buffer: Optional[torch.Tensor] = None,
                 grad_buffer: Optional[torch.Tensor] = None):
        assert not getattr(cfg, "is_generic", False), (
            f"model_type={cfg.model_type!r} has no hand-scheduled parameter layout: use verl_b200.models.make_flat_params "
            f"(library-module storage, models/generic.py)")
        self.cfg = cfg
        self.dtype = dtype
        self.value_head = value_head
        self.specs = build_param_specs(cfg, value_head)
        self.offsets: dict[str, int] = {}
        # An expert-parallel shard keeps its own experts in a tail region [dense_numel, numel): that region is local to the
        # rank (never reduced or gathered over the data-parallel group), the region in front of it is replicated.
        ep_shard = cfg.is_moe and cfg.num_local_experts > 0
        is_local = lambda s: ep_shard and ".mlp.experts." in s.name
        off = 0
        for s in self.specs:
            if not is_local(s):
                self.offsets[s.name] = off
                off += _round_up(s.numel, ALIGN)
        self.dense_numel = _round_up(off, ALIGN * max(1, pad_to))
        off = self.dense_numel
        for s in self.specs:
            if is_local(s):
                self.offsets[s.name] = off
                off += _round_up(s.numel, ALIGN)
        self.numel = off if ep_shard else self.dense_numel
        self.flat = buffer if buffer is not None else torch.zeros(self.numel, dtype=dtype, device=device)
        assert self.flat.numel() == self.numel
        self.main_grad: Optional[torch.Tensor] = None
        self.views: dict[str, torch.Tensor] = {}
        for s in self.specs:
            o = self.offsets[s.name]
            self.views[s.name] = self.flat[o : o + s.numel].view(*s.shape)
        if with_main_grad:
            self.attach_main_grad(grad_buffer)

    # ------------------------------------------------------------------ gradients
    def attach_main_grad(self, grad_buffer: Optional[torch.Tensor] = None) -> None:
        self.main_grad = grad_buffer if grad_buffer is not None else torch.zeros(
            self.numel, dtype=torch.float32, device=self.flat.device)
        for s in self.specs:
            o = self.offsets[s.name]
            self.views[s.name].main_grad = self.main_grad[o : o + s.numel].view(*s.shape)

    def detach_main_grad(self) -> None:
        self.main_grad = None
        for v in self.views.values():
            if hasattr(v, "main_grad"):
                del v.main_grad

    def zero_grad(self) -> None:
        if self.main_grad is not None:
            self.main_grad.zero_()

    # ------------------------------------------------------------------ access
    def __getitem__(self, name: str) -> torch.Tensor:
        return self.views[name]

    def layer(self, i: int) -> dict[str, torch.Tensor]:
        p = f"layers.{i}."
        return {k[len(p):]: v for k, v in self.views.items() if k.startswith(p)}

    def layer_range(self, i: int) -> tuple[int, int]:
        """[start, end) element range of layer i in the flat buffer (-1: embeddings, L: norm/head)."""
        names = [s for s in self.specs if s.layer == i and self.offsets[s.name] < self.dense_numel]
        start = self.offsets[names[0].name]
        last = names[-1]
        return start, self.offsets[last.name] + _round_up(last.numel, ALIGN)

    def decay_mask_ranges(self) -> list[tuple[int, int, bool]]:
        """(start, end, weight_decay?) ranges covering the flat buffer in order."""
        out = []
        for s in sorted(self.specs, key=lambda s: self.offsets[s.name]):
            o = self.offsets[s.name]
            out.append((o, o + _round_up(s.numel, ALIGN), s.decay))
        return out

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.views["embed_tokens.weight"] if "lm_head.weight" not in self.views else self.views["lm_head.weight"]

    # ------------------------------------------------------------------ init
    def init_weights(self, seed: int = 0, std: Optional[float] = None) -> None:
        std = std if std is not None else self.cfg.initializer_range
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)
        for s in self.specs:
            v = self.views[s.name]
            if s.init == "ones":
                v.fill_(1.0)
            elif s.init == "zeros":
                v.zero_()
            else:
                if v.is_cuda:
                    g = torch.Generator(device=v.device)
                    g.manual_seed(seed + self.offsets[s.name] % 1000003)
                    v.copy_(torch.empty(v.shape, device=v.device, dtype=torch.float32).normal_(0, std, generator=g))
                else:
                    v.copy_(torch.empty(v.shape, dtype=torch.float32).normal_(0, std, generator=gen))

    # ------------------------------------------------------------------ HF interchange
    def hf_views(self, prefix: str = "model.") -> Iterator[tuple[str, torch.Tensor]]:
        """HF-named tensors as zero-copy views of the fused storage."""
        cfg = self.cfg
        q, kv = cfg.q_size, cfg.kv_size
        mixtral, phi3 = cfg.model_type == "mixtral", cfg.model_type == "phi3"
        for s in self.specs:
            v = self.views[s.name]
            n = s.name
            if n == "lm_head.weight":
                yield "lm_head.weight", v
            elif n == "v_head.weight":
                yield "v_head.weight", v[:1]
            elif phi3 and (n.endswith("self_attn.qkv_proj.weight") or n.endswith("mlp.gate_up_proj.weight")):
                yield prefix + n, v                      # Phi-3 checkpoints store these projections fused, in the same order
            elif mixtral and n.endswith("mlp.gate.weight"):
                yield prefix + n.replace("mlp.gate.weight", "block_sparse_moe.gate.weight"), v
            elif mixtral and n.endswith("mlp.experts.gate_up_proj"):
                base = n[: -len("mlp.experts.gate_up_proj")] + "block_sparse_moe.experts."
                ie = cfg.moe_intermediate_size
                for e in range(cfg.num_experts):
                    yield f"{prefix}{base}{e}.w1.weight", v[e, :ie]   # gate
                    yield f"{prefix}{base}{e}.w3.weight", v[e, ie:]   # up
            elif mixtral and n.endswith("mlp.experts.down_proj"):
                base = n[: -len("mlp.experts.down_proj")] + "block_sparse_moe.experts."
                for e in range(cfg.num_experts):
                    yield f"{prefix}{base}{e}.w2.weight", v[e]
            elif n.endswith("self_attn.qkv_proj.weight") or n.endswith("self_attn.qkv_proj.bias"):
                base, kind = n.rsplit("qkv_proj.", 1)
                yield f"{prefix}{base}q_proj.{kind}", v[:q]
                yield f"{prefix}{base}k_proj.{kind}", v[q : q + kv]
                yield f"{prefix}{base}v_proj.{kind}", v[q + kv :]
            elif n.endswith("mlp.shared_expert_gate.weight"):
                yield prefix + n, v[:1]
            elif n.endswith("mlp.shared_expert.gate_up_proj.weight"):
                base = n[: -len("gate_up_proj.weight")]
                se = cfg.shared_expert_intermediate_size
                yield f"{prefix}{base}gate_proj.weight", v[:se]
                yield f"{prefix}{base}up_proj.weight", v[se:]
            elif n.endswith("mlp.gate_up_proj.weight"):
                base = n[: -len("gate_up_proj.weight")]
                I = cfg.intermediate_size
                yield f"{prefix}{base}gate_proj.weight", v[:I]
                yield f"{prefix}{base}up_proj.weight", v[I:]
            elif n.endswith("mlp.experts.gate_up_proj"):
                base = n[: -len("gate_up_proj")]
                ie = cfg.moe_intermediate_size
                for e in range(cfg.num_experts):
                    yield f"{prefix}{base}{e}.gate_proj.weight", v[e, :ie]
                    yield f"{prefix}{base}{e}.up_proj.weight", v[e, ie:]
            elif n.endswith("mlp.experts.down_proj"):
                base = n[: -len("down_proj")]
                for e in range(cfg.num_experts):
                    yield f"{prefix}{base}{e}.down_proj.weight", v[e]
            else:
                yield prefix + n, v
        if cfg.tie_word_embeddings and not self.value_head:
            yield "lm_head.weight", self.views["embed_tokens.weight"]

    def hf_state_dict(self, clone: bool = False) -> dict[str, torch.Tensor]:
        return {k: (v.clone() if clone else v) for k, v in self.hf_views()}

    def load_hf_state_dict(self, sd: dict[str, torch.Tensor], strict: bool = True) -> list[str]:
        """Copy HF-named tensors into the fused storage. Returns the list of missing names."""
        missing = []
        for name, view in self.hf_views():
            if name in sd:
                view.copy_(sd[name].to(view.dtype))
            elif name == "lm_head.weight" and self.cfg.tie_word_embeddings:
                continue
            else:
                missing.append(name)
        if strict and missing:
            raise KeyError(f"missing tensors: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
        return missing

    def copy_from(self, other: "FlatParams") -> None:
        self.flat.copy_(other.flat.to(self.flat.dtype))

    def named_parameters(self) -> Iterator[tuple[str, torch.Tensor]]:
        return iter(self.views.items())
