"""Packed NVFP4 export of quantisation-aware-trained weights.

Training keeps bf16 weights that already sit on the NVFP4 grid (``apply_qat_to_params``); an inference engine that runs
fp4 GEMMs wants them packed: two e2m1 codes per byte (even column in the low nibble), one fp8 (e4m3) scale per 16 columns
and one fp32 per-tensor scale, with ``w ~= code_value x block_scale x global_scale``. ``pack_nvfp4`` produces exactly that,
``unpack_nvfp4`` undoes it, and for a weight that is already on the grid ``unpack(pack(w)) == w`` bit for bit (checked in
the tests against ``nvfp4_fake_quantize``). ``QATWeightExporter`` walks a parameter set and emits, for every quantised
weight, ``<name>_packed`` (uint8), ``<name>_scale`` (float8_e4m3fn) and ``<name>_global_scale`` (fp32, 1 element); the
remaining tensors are passed through.

Parity target: ``verl/utils/modelopt/qat_weight_exporter.py`` (``QATWeightExporter`` :49-235, scale naming :260).
"""

from __future__ import annotations

from typing import Iterable, Iterator, Optional

import torch

from .core import FP4_MAX, FP8_MAX, QATConfig, _e2m1_round, nvfp4_global_scale, qat_target_names

__all__ = ["pack_nvfp4", "unpack_nvfp4", "QATWeightExporter"]

_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def pack_nvfp4(w: torch.Tensor, global_scale: Optional[float] = None):
    """``(packed uint8 [rows, cols / 2], block_scale float8_e4m3fn [rows, cols / 16], global_scale fp32 [1])``."""
    assert w.dim() == 2 and w.shape[1] % 16 == 0, "a 2-D weight whose row length is a multiple of 16"
    gs = nvfp4_global_scale(w) if global_scale is None else float(global_scale)
    v = w.detach().float().view(w.shape[0], -1, 16)
    amax = v.abs().amax(-1, keepdim=True)
    scale8 = (amax / (FP4_MAX * max(gs, 1e-12))).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
    scale = scale8.float() * gs
    scale = torch.where(scale >= 1e-5, scale, torch.ones_like(scale))   # an all-zero block: any scale, codes are 0
    mag = _e2m1_round(v.abs() / scale)
    code = torch.bucketize(mag, _E2M1_VALUES.to(mag.device)).to(torch.uint8)          # index of the magnitude, 0..7
    code = code | ((v < 0) & (mag > 0)).to(torch.uint8) * 8                            # sign bit; no negative zero
    code = code.view(w.shape[0], -1)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), scale8.view(w.shape[0], -1).contiguous(), torch.tensor([gs], dtype=torch.float32, device=w.device)


def unpack_nvfp4(packed: torch.Tensor, block_scale: torch.Tensor, global_scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    rows = packed.shape[0]
    code = torch.stack([packed & 0xF, packed >> 4], dim=-1).view(rows, -1).long()
    mag = _E2M1_VALUES.to(packed.device)[code & 7]
    val = torch.where((code & 8) > 0, -mag, mag).view(rows, -1, 16)
    scale = block_scale.float().view(rows, -1, 1) * float(global_scale.reshape(-1)[0])
    scale = torch.where(scale >= 1e-5, scale, torch.ones_like(scale))
    return (val * scale).view(rows, -1).to(dtype)


class QATWeightExporter:
    def __init__(self, config, tp_group=None):
        self.cfg = QATConfig.from_any(config)
        assert self.cfg.mode == "w4a16" and self.cfg.group_size == 16, "supported: NVFP4 weights (groups of 16), bf16 activations"
        self.tp_group = tp_group

    def export(self, params, names: Optional[Iterable[str]] = None) -> Iterator[tuple[str, torch.Tensor]]:
        """``(name, tensor)`` pairs of ``params`` (a ``FlatParams``): quantised weights as their three packed tensors, the
        rest unchanged. Stacked expert weights ``[E, N, K]`` are packed per expert with one per-tensor scale each."""
        targets = set(qat_target_names(params, self.cfg) if names is None else names)
        for name, w in params.views.items():
            if name not in targets:
                yield name, w
                continue
            if w.dim() == 2:
                p, s, g = pack_nvfp4(w, nvfp4_global_scale(w, self.tp_group))
            else:
                parts = [pack_nvfp4(w[e], nvfp4_global_scale(w[e], self.tp_group)) for e in range(w.shape[0])]
                p, s, g = (torch.stack([x[i] for x in parts]) for i in range(3))
            yield f"{name}_packed", p
            yield f"{name}_scale", s
            yield f"{name}_global_scale", g

    def quantization_config(self) -> dict:
        """What an inference engine needs to know to load the packed tensors."""
        return {"quant_method": "nvfp4", "format": "e2m1 pairs per byte, low nibble first", "group_size": 16,
                "scale_dtype": "float8_e4m3fn", "ignore": list(self.cfg.ignore_patterns)}
