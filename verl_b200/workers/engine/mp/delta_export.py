"""Sparse export of what an optimizer step changed, from a tensor x pipeline x expert parallel shard, in the coordinates
of the HF-named full tensors.

After most RL steps only a fraction of the bf16 weights change bit pattern. Instead of re-assembling the full model for the
rollout side (``gather_full_params``), every rank compares its shard with the snapshot of the last export, turns the
positions of the changed elements into positions inside the *full* HF tensors by arithmetic on the shard layout (row /
column / expert slices; no full-size index buffer is ever built), and ships ``(tensor name, int64 positions, values)``
records. Replicated tensors are exported by tensor-parallel rank 0 of their stage only, so the union over the model-parallel
group covers every changed element exactly once. ``apply_hf_delta`` is the receiving side.

Parity target: ``verl/workers/engine/megatron/delta_export.py`` (``build_export_index`` :198, ``mcore_hf_delta_entry`` :361)
together with ``verl/checkpoint_engine/delta_checkpoint_engine.py``.
"""

from __future__ import annotations

import bisect
from typing import Iterable, Optional

import torch

from ....models.weights import FlatParams
from ....parallel.model_parallel import ShardMap

__all__ = ["ShardDeltaExporter", "apply_hf_delta", "full_positions"]


def _bits(t: torch.Tensor) -> torch.Tensor:
    v = t.detach().contiguous().view(-1)
    return v.view({1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[v.element_size()])


def full_positions(m: ShardMap, idx: torch.Tensor, local_shape: tuple, full_shape: tuple, tp: int, tp_rank: int, ep: int = 1,
                   ep_rank: int = 0) -> torch.Tensor:
    """Flat positions inside the FULL tensor of the flat positions ``idx`` of this rank's shard of it."""
    if m.kind == "experts":
        per_rank = int(torch.tensor(local_shape).prod())
        return idx + ep_rank * per_rank
    if m.kind == "rep" or tp == 1:
        return idx
    if m.kind == "cols":
        lc, fc = local_shape[1], full_shape[1]
        return (idx // lc) * fc + idx % lc + tp_rank * lc
    e_off = ep_rank * local_shape[0] if (ep > 1 and m.kind in ("expert_rows", "expert_cols")) else 0   # first expert held here
    if m.kind == "expert_cols":              # [E, rows, cols / tp]: the last dimension is cut
        lc, fc = local_shape[2], full_shape[2]
        return (idx // lc) * fc + idx % lc + tp_rank * lc + e_off * full_shape[1] * fc
    if m.kind == "expert_rows":              # [E, rows / tp (block-wise), cols]: per expert like ``rows``
        cols = local_shape[2]
        e, rem = idx // (local_shape[1] * cols), idx % (local_shape[1] * cols)
        row, c = rem // cols, rem % cols
        full_row = torch.empty_like(row)
        l0 = f0 = 0
        for b in m.blocks:
            w = b // tp
            sel = (row >= l0) & (row < l0 + w)
            full_row[sel] = row[sel] - l0 + f0 + tp_rank * w
            l0 += w
            f0 += b
        return ((e + e_off) * full_shape[1] + full_row) * cols + c
    inner = 1
    for d in local_shape[1:]:
        inner *= d
    row, rest = idx // inner, idx % inner
    full_row = torch.empty_like(row)
    l0 = f0 = 0
    for b in m.blocks:                       # stacked blocks (q | k | v, gate | up, vocabulary): each is cut into tp slices
        w = b // tp
        sel = (row >= l0) & (row < l0 + w)
        full_row[sel] = row[sel] - l0 + f0 + tp_rank * w
        l0 += w
        f0 += b
    return full_row * inner + rest


class ShardDeltaExporter:
    """Snapshot of one rank's shard + the layout tables that translate shard positions into HF tensor positions."""

    def __init__(self, engine):
        self.engine = engine
        topo = engine.topo
        self.tp, self.tp_rank, self.ep, self.ep_rank = topo.tp, topo.tp_rank, topo.ep, topo.ep_rank
        # layout of the full model (no storage): offsets of the full tensors and of the HF-named ranges inside them
        full = FlatParams(engine.full_arch, dtype=engine.params.flat.dtype, device="meta", value_head=engine.value_head)
        self._full_offsets, self._full_shapes = full.offsets, {n: tuple(v.shape) for n, v in full.views.items()}
        seen, ranges = set(), []
        for name, v in full.hf_views():
            key = (v.storage_offset(), v.numel())
            if key in seen:
                continue                      # a tied head is the embedding's range under a second name
            seen.add(key)
            ranges.append((v.storage_offset(), v.numel(), name))
        ranges.sort()
        self._starts = [r[0] for r in ranges]
        self._ranges = ranges
        self.snapshot = engine.params.flat.detach().clone()

    def resnapshot(self) -> None:
        self.snapshot.copy_(self.engine.params.flat)

    def export(self, update_snapshot: bool = True) -> list[tuple[str, torch.Tensor, torch.Tensor]]:
        """``(hf_name, positions int64, values)`` for everything that changed in this rank's shard since the snapshot."""
        eng, P = self.engine, self.engine.params
        out: dict[str, list] = {}
        for m in eng.maps:
            if m.full_name not in self._full_offsets:
                continue
            if m.kind == "rep" and self.tp > 1 and self.tp_rank != 0:
                continue                      # every tensor-parallel rank holds the same values: one exporter is enough
            if m.kind not in ("experts", "expert_rows", "expert_cols") and self.ep > 1 and self.ep_rank != 0:
                continue                      # everything but the experts is replicated over the expert-parallel group
            lo = P.offsets[m.local_name]
            view = P.views[m.local_name]
            n = view.numel()
            idx = torch.nonzero(_bits(P.flat[lo : lo + n]) != _bits(self.snapshot[lo : lo + n]), as_tuple=False).view(-1)
            if idx.numel() == 0:
                continue
            vals = P.flat[lo : lo + n][idx]
            pos = full_positions(m, idx, tuple(view.shape), self._full_shapes[m.full_name], self.tp, self.tp_rank, self.ep, self.ep_rank)
            pos = pos + self._full_offsets[m.full_name]
            order = torch.argsort(pos)
            pos, vals = pos[order], vals[order]
            # split the sorted positions at the borders of the HF-named ranges they fall into
            first = bisect.bisect_right(self._starts, int(pos[0])) - 1
            last = bisect.bisect_right(self._starts, int(pos[-1])) - 1
            for r in range(first, last + 1):
                start, numel, name = self._ranges[r]
                sel = (pos >= start) & (pos < start + numel)
                if bool(sel.any()):
                    out.setdefault(name, []).append((pos[sel] - start, vals[sel]))
        if update_snapshot:
            self.resnapshot()
        return [(name, torch.cat([p for p, _ in parts]), torch.cat([v for _, v in parts])) for name, parts in out.items()]

    def changed_fraction(self) -> float:
        changed = int((_bits(self.engine.params.flat) != _bits(self.snapshot)).sum())
        return changed / max(1, self.snapshot.numel())


def apply_hf_delta(state_dict: dict, records: Iterable[tuple[str, torch.Tensor, torch.Tensor]], strict: bool = True) -> int:
    """Write exported records into HF-named tensors (a state dict, or the views of a rollout-side parameter store).
    Returns the number of elements written."""
    n = 0
    for name, pos, vals in records:
        t: Optional[torch.Tensor] = state_dict.get(name)
        if t is None:
            if strict:
                raise KeyError(name)
            continue
        t.view(-1)[pos.to(t.device)] = vals.to(device=t.device, dtype=t.dtype)
        n += int(pos.numel())
    return n
