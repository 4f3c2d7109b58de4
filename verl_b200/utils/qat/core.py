"""Quantisation-aware training with NVFP4 weights (``w4a16``): the bf16 working weights of the linear layers are kept equal
to ``dequant(quant(master))`` (e2m1 values in 1x16 blocks, e4m3 block scales, one fp32 scale per tensor) while the fp32
master weights receive the gradients unchanged (straight-through estimator). Forward, backward and the colocated rollout
engine all read the same working buffer, so the policy is trained and sampled with exactly the weights a 4-bit deployment
would use.

Parity target: ``verl/utils/qat/core.py`` (``QATConfig`` :31), ``verl/utils/qat/linear.py:42-125`` (fake-quant kernel),
``verl/utils/qat/quantizer.py`` (scales).
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Optional

import torch

__all__ = ["QATConfig", "nvfp4_global_scale", "nvfp4_fake_quantize", "qat_target_names", "apply_qat_to_params"]

FP4_MAX, FP8_MAX = 6.0, 448.0


@dataclass
class QATConfig:
    enable: bool = False
    mode: str = "w4a16"
    group_size: int = 16
    ignore_patterns: list = field(default_factory=lambda: ["lm_head", "embed_tokens", "re:.*mlp.gate$"])
    activation_observer: str = "static_minmax"
    quantization_config_path: Optional[str] = None

    @classmethod
    def from_any(cls, obj) -> "QATConfig":
        if obj is None:
            return cls()
        if isinstance(obj, cls):
            return obj
        get = obj.get if hasattr(obj, "get") else (lambda k, d=None: getattr(obj, k, d))
        c = cls()
        for k in ("enable", "mode", "group_size", "ignore_patterns", "activation_observer", "quantization_config_path"):
            v = get(k, None)
            if v is not None:
                setattr(c, k, list(v) if k == "ignore_patterns" else v)
        if get("enabled", None) is not None:
            c.enable = bool(get("enabled"))
        return c


def nvfp4_global_scale(x: torch.Tensor, group=None) -> float:
    """Per-tensor scale that lets the largest block scale use the whole e4m3 range. ``group``: the tensor is one shard of a
    weight split over a (tensor-parallel) group, whose members must agree on the scale (maximum over the group)."""
    amax = x.detach().abs().amax().float()
    if group is not None:
        import torch.distributed as dist

        amax = amax.clone()
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    return float(amax) / (FP4_MAX * FP8_MAX)


def _e2m1_round(a: torch.Tensor) -> torch.Tensor:
    out = torch.full_like(a, FP4_MAX)
    for bound, val, closed in ((5.0, 4.0, True), (3.5, 3.0, False), (2.5, 2.0, True), (1.75, 1.5, False), (1.25, 1.0, True),
                               (0.75, 0.5, False), (0.25, 0.0, True)):
        out = torch.where((a <= bound) if closed else (a < bound), torch.full_like(a, val), out)
    return out


def nvfp4_fake_quantize(x: torch.Tensor, global_scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dequant(quant(x))`` for a 2-D tensor whose row length is a multiple of 16. On a GPU (bf16) this is one kernel and
    ``out`` may be ``x`` itself."""
    assert x.dim() == 2 and x.shape[1] % 16 == 0
    gs = nvfp4_global_scale(x) if global_scale is None else float(global_scale)
    if x.is_cuda and x.dtype == torch.bfloat16:
        from ...ops import native

        out = torch.empty_like(x) if out is None else out
        native.ops().nvfp4_fake_quant_(x, out, gs)
        return out
    v = x.float().view(x.shape[0], -1, 16)
    amax = v.abs().amax(-1, keepdim=True)
    want = (amax / (FP4_MAX * max(gs, 1e-12))).clamp(max=FP8_MAX)
    scale = want.to(torch.float8_e4m3fn).float() * gs
    scale = torch.where(scale >= 1e-5, scale, torch.ones_like(scale))
    q = _e2m1_round(v.abs() / scale) * scale
    y = torch.where(v >= 0, q, -q).view_as(x).to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def _ignored(name: str, patterns: list) -> bool:
    for p in patterns:
        if p.startswith("re:"):
            if re.match(p[3:], name) or re.match(p[3:], name.rsplit(".weight", 1)[0]):
                return True
        elif p in name:
            return True
    return False


def qat_target_names(params, cfg: QATConfig) -> list[str]:
    """Linear weights (2-D or stacked expert weights, inner dimension a multiple of the group size) not matched by an
    ignore pattern; norms, biases, embeddings and the head stay in bf16."""
    out = []
    for name, v in params.views.items():
        if v.dim() < 2 or "norm" in name or name.endswith(".bias") or v.shape[-1] % cfg.group_size:
            continue
        if _ignored(name, cfg.ignore_patterns):
            continue
        out.append(name)
    return out


@torch.no_grad()
def apply_qat_to_params(params, cfg: QATConfig, names: Optional[list] = None, group=None) -> int:
    """Replace every target weight of ``params`` (a ``FlatParams``) by its fake-quantised value, in place. ``group``: the
    tensor-parallel group over which sharded weights agree on their per-tensor scale."""
    assert cfg.mode == "w4a16" and cfg.group_size == 16, "supported: NVFP4 weights (groups of 16), bf16 activations"
    names = qat_target_names(params, cfg) if names is None else names
    for n in names:
        w = params.views[n]
        w2 = w.view(-1, w.shape[-1])
        nvfp4_fake_quantize(w2, nvfp4_global_scale(w2, group) if group is not None else None, out=w2)
    return len(names)
