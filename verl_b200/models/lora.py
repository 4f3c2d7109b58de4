"""Low-rank adapters on the linear projections.

For every target weight ``W0 [out, in]`` the adapter holds ``A [r, in]`` (random) and ``B [out, r]`` (zero) and the model
computes with the merged weight ``W0 + (alpha / r) * B A``. Forward, input gradients and the rollout engine therefore run
at full speed on ordinary weights; only the adapter gradients are extra work (two skinny GEMMs per projection, see
``DecoderModel._wgrad``), and only the adapters have optimizer state. After every optimizer step ``merge`` recomputes the
working weights from the frozen base copy.

Parity target: the LoRA path of ``verl/workers/engine/fsdp/transformer_impl.py:320`` (peft ``LoraConfig``: ``lora_rank``,
``lora_alpha``, ``target_modules``), ``verl/utils/fsdp_utils.py:645-1100`` (collect / merge), merged-weight export :1040.
"""

from __future__ import annotations

import json
import math
import os
from typing import Optional

import torch

from ..ops import functional as F
from .weights import ALIGN, FlatParams

__all__ = ["LoRAParams", "DEFAULT_TARGETS"]

DEFAULT_TARGETS = ("self_attn.qkv_proj.weight", "self_attn.o_proj.weight", "mlp.gate_up_proj.weight", "mlp.down_proj.weight")
_HF_ALIASES = {"q_proj": "self_attn.qkv_proj.weight", "k_proj": "self_attn.qkv_proj.weight", "v_proj": "self_attn.qkv_proj.weight",
               "o_proj": "self_attn.o_proj.weight", "gate_proj": "mlp.gate_up_proj.weight", "up_proj": "mlp.gate_up_proj.weight",
               "down_proj": "mlp.down_proj.weight"}


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class LoRAParams:
    """Flat storage of all adapters with the interface the engine's optimizer expects (``flat``, ``numel``, ``offsets``,
    ``views``, ``main_grad``, ``attach_main_grad`` ...)."""

    def __init__(self, base: FlatParams, rank: int, alpha: float, target_modules=None, pad_to: int = 1, seed: int = 0):
        assert rank % 8 == 0 and rank > 0, "lora_rank must be a positive multiple of 8 (16-byte rows for the tensor-core GEMMs)"
        self.base, self.rank, self.alpha = base, int(rank), float(alpha)
        self.scale = self.alpha / self.rank
        self.dtype = base.flat.dtype
        tm = target_modules
        if tm in (None, "all-linear", ["all-linear"]):
            wanted = set(DEFAULT_TARGETS)
        else:
            wanted = {_HF_ALIASES.get(t, t) for t in ([tm] if isinstance(tm, str) else list(tm))}
        self.targets = [n for n, v in base.views.items() if v.dim() == 2 and any(n.endswith(w) for w in wanted)]
        self.offsets: dict[str, int] = {}
        shapes = {}
        off = 0
        for n in self.targets:
            out_f, in_f = base.views[n].shape
            for suffix, shape in (("lora_A", (self.rank, in_f)), ("lora_B", (out_f, self.rank))):
                key = f"{n}.{suffix}"
                self.offsets[key] = off
                shapes[key] = shape
                off += _round_up(shape[0] * shape[1], ALIGN)
        self.numel = _round_up(max(off, ALIGN), ALIGN * max(1, pad_to))
        self.flat = torch.zeros(self.numel, dtype=self.dtype, device=base.flat.device)
        self.views = {k: self.flat[o : o + shapes[k][0] * shapes[k][1]].view(*shapes[k]) for k, o in self.offsets.items()}
        self.main_grad: Optional[torch.Tensor] = None
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for n in self.targets:
            a = self.views[f"{n}.lora_A"]
            bound = 1.0 / math.sqrt(a.shape[1])
            a.copy_((torch.rand(a.shape, generator=gen) * 2 - 1) * bound * math.sqrt(3.0))  # kaiming-uniform, B stays zero
            base.views[n].lora = (a, self.views[f"{n}.lora_B"], self.scale)
        self.base0 = base.flat.clone()  # frozen base weights: the working buffer holds the merged weights

    # ---- gradient buffer (same contract as FlatParams)
    def attach_main_grad(self, grad_buffer: Optional[torch.Tensor] = None) -> None:
        self.main_grad = grad_buffer if grad_buffer is not None else torch.zeros(self.numel, dtype=torch.float32, device=self.flat.device)
        for k, o in self.offsets.items():
            v = self.views[k]
            v.main_grad = self.main_grad[o : o + v.numel()].view(*v.shape)

    def detach_main_grad(self) -> None:
        self.main_grad = None
        for v in self.views.values():
            if hasattr(v, "main_grad"):
                del v.main_grad

    def zero_grad(self) -> None:
        if self.main_grad is not None:
            self.main_grad.zero_()

    def decay_mask_ranges(self):
        return [(0, self.numel, True)]

    # ---- merge
    @torch.no_grad()
    def merge(self) -> None:
        """working weight <- frozen base + scale * B A for every target."""
        b0 = self.base0
        for n in self.targets:
            w = self.base.views[n]
            o = self.base.offsets[n]
            A, B = self.views[f"{n}.lora_A"], self.views[f"{n}.lora_B"]
            delta = F.gemm(B, A, b_mn=True, out_f32=True)  # [out, r] @ [r, in]
            w.copy_((b0[o : o + w.numel()].view_as(w).float() + self.scale * delta).to(w.dtype))

    # ---- adapter checkpoint in the peft layout
    def save_adapter(self, path: str, base_model_name: str = "") -> None:
        os.makedirs(path, exist_ok=True)
        torch.save({k: v.detach().cpu() for k, v in self.views.items()}, os.path.join(path, "adapter_model.pt"))
        with open(os.path.join(path, "adapter_config.json"), "w") as f:
            json.dump({"peft_type": "LORA", "r": self.rank, "lora_alpha": self.alpha, "target_modules": sorted({t.split(".")[-2] for t in self.targets}),
                       "base_model_name_or_path": base_model_name, "fused_projections": True}, f, indent=1)
        with open(os.path.join(path, "lora_train_meta.json"), "w") as f:
            json.dump({"r": self.rank, "lora_alpha": self.alpha, "task_type": "CAUSAL_LM"}, f)

    def load_adapter(self, path: str) -> None:
        st = torch.load(os.path.join(path, "adapter_model.pt"), map_location="cpu", weights_only=False)
        for k, v in st.items():
            if k in self.views:
                self.views[k].copy_(v.to(self.views[k].dtype))
        self.merge()
