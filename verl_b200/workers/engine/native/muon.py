"""Muon (momentum + Newton-Schulz orthogonalisation) on the engine's flat, range-sharded optimizer state.

The sharded optimizer owns byte ranges of the flat buffer, not whole matrices, while Muon's orthogonalisation needs whole
matrices. One step therefore runs as

1. momentum on the owned range (same buffer that holds Adam's first moment for the non-matrix parameters),
2. all-gather of the momentum-updated gradient into the (now idle) full-size fp32 gradient buffer,
3. every rank orthogonalises the matrices assigned to it (balanced by Newton-Schulz cost) and zeroes everything else,
4. reduce-scatter (sum) of that buffer: each rank receives the orthogonal updates of its own range,
5. decoupled weight decay + update on the fp32 master range; AdamW for embeddings, heads, norms, biases.

No matrix is orthogonalised twice and no optimizer state is replicated. Under tensor parallelism the flat buffer holds
this rank's shards and each shard is orthogonalised on its own (the "blockwise" mode of the reference's back-end).

Parity target: the Muon options of ``verl/workers/config/optimizer.py:154-224`` (``muon_momentum``, ``muon_nesterov``,
``muon_split_qkv``, ``muon_scale_mode``, ``muon_num_ns_steps``, ``muon_extra_scale_factor``,
``muon_match_adamw_update_rms``) and ``verl/utils/megatron/optimizer.py`` (``adamw_rms_match_scale_factor``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

__all__ = ["newton_schulz", "muon_scale_factor", "adamw_rms_match_scale_factor", "MuonPlan", "MuonMatrix", "NS_COEFFICIENTS"]

# quintic iteration X <- aX + (bA + cA^2)X with A = XX^T; the "quintic" set maximises the slope at zero so that five
# steps push every singular value into a band around one, "simple" is the classical cubic-convergent polynomial
NS_COEFFICIENTS = {
    "quintic": (3.4445, -4.7750, 2.0315),
    "simple": (15.0 / 8.0, -10.0 / 8.0, 3.0 / 8.0),
}


def newton_schulz(g: torch.Tensor, steps: int = 5, coefficient_type: str = "quintic", eps: float = 1e-7) -> torch.Tensor:
    """Approximate ``U V^T`` of ``g = U S V^T`` (the nearest semi-orthogonal matrix) by a matrix polynomial iteration.
    Runs in bf16 on a GPU (tensor cores) and in fp32 on the host; the result has the dtype of ``g``."""
    assert g.dim() == 2
    a, b, c = NS_COEFFICIENTS[coefficient_type]
    x = g.to(torch.bfloat16) if g.is_cuda else g.float()
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    x = x / (x.norm() + eps)          # spectral norm <= Frobenius norm = 1: inside the iteration's basin
    for _ in range(int(steps)):
        gram = x @ x.t()
        x = a * x + (b * gram + c * (gram @ gram)) @ x
    if transposed:
        x = x.t()
    return x.to(g.dtype)


def muon_scale_factor(rows: int, cols: int, mode: str = "spectral") -> float:
    """Factor that turns the orthogonalised gradient (singular values ~1, RMS ~ 1/sqrt(max(rows, cols))) into the update."""
    if mode == "spectral":
        return math.sqrt(max(rows, cols))          # unit RMS per element
    if mode == "shape_scaling":
        return math.sqrt(max(1.0, rows / cols))
    if mode == "unit_rms_norm":
        return math.sqrt(rows / cols)
    if mode in ("none", "identity"):
        return 1.0
    raise ValueError(f"unknown muon_scale_mode {mode!r} (spectral | shape_scaling | unit_rms_norm | none)")


def adamw_rms_match_scale_factor(beta1: float) -> float:
    """Extra factor under which a unit-RMS Muon update has the steady-state RMS of an AdamW update with ``beta1``."""
    return math.sqrt((1.0 - beta1) / (1.0 + beta1))


@dataclass
class MuonMatrix:
    offset: int     # first element in the flat buffer
    rows: int
    cols: int
    owner: int = 0  # rank (of the sharding group) that orthogonalises it

    @property
    def numel(self) -> int:
        return self.rows * self.cols

    @property
    def cost(self) -> float:
        m, n = min(self.rows, self.cols), max(self.rows, self.cols)
        return float(m) * m * (n + m)


class MuonPlan:
    """Which ranges of the flat buffer are Muon matrices, who orthogonalises which, and the matrix mask of a range."""

    def __init__(self, params, world: int = 1, split_qkv: bool = True, split_gate_up: bool = True):
        self.matrices: list[MuonMatrix] = []
        cfg = params.cfg
        for s in params.specs:
            if s.layer < 0 or s.layer >= cfg.num_hidden_layers or len(s.shape) < 2:
                continue  # embeddings, final norm, heads, 1-D parameters: AdamW
            if "shared_expert_gate" in s.name or "lora_" in s.name:
                continue  # a scalar gate stored in padded rows
            off = params.offsets[s.name]
            if off >= getattr(params, "dense_numel", params.numel):
                raise NotImplementedError("Muon on rank-local (expert-parallel) parameter regions")
            lead = int(math.prod(s.shape[:-2]))
            rows, cols = int(s.shape[-2]), int(s.shape[-1])
            native = not getattr(cfg, "is_generic", False)
            for e in range(lead):
                base = off + e * rows * cols
                if native and split_qkv and s.name.endswith("self_attn.qkv_proj.weight"):
                    q, kv = cfg.q_size, cfg.kv_size
                    parts = [(0, q), (q, kv), (q + kv, kv)]
                elif native and split_gate_up and ("gate_up_proj" in s.name):
                    parts = [(0, rows // 2), (rows // 2, rows // 2)]
                else:
                    parts = [(0, rows)]
                for r0, nr in parts:
                    self.matrices.append(MuonMatrix(base + r0 * cols, nr, cols))
        # longest-processing-time assignment: balanced Newton-Schulz work, identical on every rank
        load = [0.0] * max(1, world)
        for m in sorted(self.matrices, key=lambda m: (-m.cost, m.offset)):
            r = min(range(len(load)), key=lambda i: (load[i], i))
            m.owner = r
            load[r] += m.cost
        self.world = max(1, world)

    def mask(self, lo: int, hi: int, device) -> torch.Tensor:
        """bool [hi - lo]: True where the flat range [lo, hi) belongs to a Muon matrix."""
        out = torch.zeros(hi - lo, dtype=torch.bool, device=device)
        for m in self.matrices:
            a, b = max(lo, m.offset), min(hi, m.offset + m.numel)
            if a < b:
                out[a - lo : b - lo] = True
        return out

    def orthogonalise_owned(self, full: torch.Tensor, rank: int, steps: int, coefficient_type: str, scale_mode: str) -> None:
        """``full``: the gathered momentum buffer. On return it holds the scaled orthogonal updates of the matrices
        this rank owns and zeros everywhere else (ready to be summed over the group)."""
        mine = [m for m in self.matrices if m.owner == rank]
        outs = []
        for m in mine:
            x = full[m.offset : m.offset + m.numel].view(m.rows, m.cols)
            outs.append(newton_schulz(x, steps, coefficient_type) * muon_scale_factor(m.rows, m.cols, scale_mode))
        if self.world > 1:
            full.zero_()
        else:
            keep = self.mask(0, full.numel(), full.device)
            full.mul_(keep)  # only the matrix ranges carry an update
        for m, o in zip(mine, outs):
            full[m.offset : m.offset + m.numel].view(m.rows, m.cols).copy_(o)
