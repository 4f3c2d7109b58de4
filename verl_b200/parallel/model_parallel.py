"""Tensor x pipeline x data parallel layout for training (the "Megatron-style" engine builds on this).

Rank order: tensor-parallel fastest, then pipeline stage, then data-parallel replica:
``rank = (dp * PP + pp) * TP + tp``. Each rank stores and computes a *local shard model*
(``ModelConfig.local_shard``): 1/TP of the attention heads and of the MLP width, ``L / PP`` consecutive layers, the
embedding on the first stage and the final norm + head on the last one.

* tensor parallelism: column-parallel QKV / gate-up, row-parallel O / down; one all-reduce of the block output in the
  forward pass and one of the block-input gradient in the backward pass (hooks of ``DecoderModel.tp_reduce``); embedding,
  norms and head are replicated inside the TP group (their gradients come out identical on every TP rank);
* pipeline parallelism: stages hand the summed hidden stream [T, H] forward and its gradient backward with point-to-point
  messages; all ranks of a replica see the same micro-batches, so shapes are known on both sides;
* data parallelism: gradient mean + sharded optimizer over the DP group (the native engine's machinery).

``ShardMap`` records how every local tensor is cut out of the full (HF-layout) tensor; it drives weight loading, the merge
back to a full model and the train -> rollout reshard.

Parity target: ``verl/workers/engine/megatron/transformer_impl.py:272-282`` (``initialize_model_parallel``),
``verl/utils/megatron_utils.py`` and ``verl/models/mcore/util.py`` (layout / broadcast helpers).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..models.weights import FlatParams

__all__ = ["ModelParallelTopology", "ShardMap", "build_shard_map", "copy_full_to_local", "copy_local_to_full", "cat_dim", "EXPERT_KINDS"]


class ModelParallelTopology:
    """Process groups of a TP x PP x DP job. Every rank of the job must construct it (group creation is collective)."""

    def __init__(self, tp: int = 1, pp: int = 1, ranks: Optional[list[int]] = None, ep: int = 1, vpp: int = 1):
        self.world_ranks = list(ranks) if ranks is not None else list(range(dist.get_world_size() if dist.is_initialized() else 1))
        n = len(self.world_ranks)
        assert n % (tp * pp) == 0, f"world size {n} is not a multiple of tp*pp = {tp * pp}"
        self.tp, self.pp, self.dp = tp, pp, n // (tp * pp)
        # expert parallelism borrows the data-parallel dimension: the ranks of a data-parallel group split the experts
        # (with tp > 1 as well, every expert's width is additionally cut over the tensor-parallel group)
        assert ep == 1 or ep == self.dp, "expert parallelism: ep must equal the data-parallel size"
        self.ep = ep
        # interleaved (virtual) pipeline stages: every rank holds ``vpp`` model chunks; chunk v of stage s is block
        # v * pp + s of the layer stack, so a micro-batch visits the ranks of the pipeline group vpp times round
        assert vpp >= 1 and (vpp == 1 or pp > 1), "virtual pipeline stages need pipeline_model_parallel_size > 1"
        self.vpp = int(vpp)
        me = dist.get_rank() if dist.is_initialized() else 0
        self.index = self.world_ranks.index(me)
        self.tp_rank = self.index % tp
        self.pp_rank = (self.index // tp) % pp
        self.dp_rank = self.index // (tp * pp)
        self.tp_group = self.pp_group = self.dp_group = self.mp_group = None
        g = lambda d, p, t: self.world_ranks[(d * pp + p) * tp + t]
        if n > 1:
            for d in range(self.dp):
                for p in range(pp):
                    ranks_ = [g(d, p, t) for t in range(tp)]
                    grp = dist.new_group(ranks_) if tp > 1 else None
                    if d == self.dp_rank and p == self.pp_rank:
                        self.tp_group = grp
            for d in range(self.dp):
                for t in range(tp):
                    ranks_ = [g(d, p, t) for p in range(pp)]
                    grp = dist.new_group(ranks_) if pp > 1 else None
                    if d == self.dp_rank and t == self.tp_rank:
                        self.pp_group = grp
            for p in range(pp):
                for t in range(tp):
                    ranks_ = [g(d, p, t) for d in range(self.dp)]
                    grp = dist.new_group(ranks_)
                    if p == self.pp_rank and t == self.tp_rank:
                        self.dp_group = grp
            for d in range(self.dp):
                ranks_ = [g(d, p, t) for p in range(pp) for t in range(tp)]
                grp = dist.new_group(ranks_) if tp * pp > 1 else None
                if d == self.dp_rank:
                    self.mp_group = grp
        self.prev_rank = g(self.dp_rank, self.pp_rank - 1, self.tp_rank) if self.pp_rank > 0 else None
        self.next_rank = g(self.dp_rank, self.pp_rank + 1, self.tp_rank) if self.pp_rank < pp - 1 else None
        self.last_stage_rank = g(self.dp_rank, pp - 1, self.tp_rank)
        self.ring_prev = g(self.dp_rank, (self.pp_rank - 1) % pp, self.tp_rank)   # neighbours on the ring the chunks travel
        self.ring_next = g(self.dp_rank, (self.pp_rank + 1) % pp, self.tp_rank)
        self.ep_rank = self.dp_rank if ep > 1 else 0
        self.ep_group = self.dp_group if ep > 1 else None

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp - 1

    def layer_range(self, num_layers: int) -> tuple[int, int]:
        """Consecutive layers of this stage; earlier stages take the remainder."""
        base, rem = divmod(num_layers, self.pp)
        lo = self.pp_rank * base + min(self.pp_rank, rem)
        return lo, lo + base + (1 if self.pp_rank < rem else 0)

    def local_layers(self, num_layers: int) -> list[int]:
        """Index in the full model of every local layer, in local order (chunk by chunk with virtual stages)."""
        if self.vpp == 1:
            lo, hi = self.layer_range(num_layers)
            return list(range(lo, hi))
        assert num_layers % (self.pp * self.vpp) == 0, \
            f"{num_layers} layers do not split into {self.pp} x {self.vpp} equal blocks (pipeline x virtual stages)"
        blk = num_layers // (self.pp * self.vpp)
        return [(v * self.pp + self.pp_rank) * blk + j for v in range(self.vpp) for j in range(blk)]

    def local_config(self, cfg: ModelConfig, vocab_parallel: bool = True) -> ModelConfig:
        lo, hi = 0, len(self.local_layers(cfg.num_hidden_layers))
        return cfg.local_shard(tp=self.tp, num_layers=hi - lo, has_embedding=self.is_first_stage, has_head=self.is_last_stage,
                               ep=self.ep, vocab_parallel=vocab_parallel)


@dataclass
class ShardMap:
    local_name: str
    full_name: str
    # rep | rows | cols | experts (dim 0 cut over the expert-parallel group) | expert_rows / expert_cols (stacked expert
    # matrices [E, rows, cols] under tensor parallelism: dim 1 cut block-wise like ``rows``, dim 2 cut like ``cols``)
    kind: str
    blocks: tuple = ()     # rows / expert_rows: sizes of the stacked blocks of the FULL tensor, each block is cut into tp slices


def build_shard_map(full_cfg: ModelConfig, topo: ModelParallelTopology, value_head: bool = False,
                    vocab_parallel: bool = True) -> list[ShardMap]:
    """One entry per tensor of the local shard model, in the local parameter order."""
    from ..models.weights import build_param_specs

    layer_of = topo.local_layers(full_cfg.num_hidden_layers)
    local_cfg = topo.local_config(full_cfg, vocab_parallel and not value_head)
    out = []
    for spec in build_param_specs(local_cfg, value_head and topo.is_last_stage):
        name = spec.name
        full_name = name
        if name.startswith("layers."):
            i, rest = name.split(".", 2)[1:]
            full_name = f"layers.{layer_of[int(i)]}.{rest}"
        else:
            rest = name
        if name == "lm_head.weight" and local_cfg.head_vocab_size:
            out.append(ShardMap(name, full_name, "rows", (full_cfg.vocab_size,)))
        elif rest.startswith("mlp.experts.") and topo.ep > 1 and topo.tp == 1:
            out.append(ShardMap(name, full_name, "experts"))
        elif rest == "mlp.experts.gate_up_proj" and topo.tp > 1:
            out.append(ShardMap(name, full_name, "expert_rows", (full_cfg.moe_intermediate_size, full_cfg.moe_intermediate_size)))
        elif rest == "mlp.experts.down_proj" and topo.tp > 1:
            out.append(ShardMap(name, full_name, "expert_cols"))
        elif rest == "mlp.shared_expert.gate_up_proj.weight":
            out.append(ShardMap(name, full_name, "rows", (full_cfg.shared_expert_intermediate_size,) * 2))
        elif rest == "mlp.shared_expert.down_proj.weight":
            out.append(ShardMap(name, full_name, "cols"))
        elif rest.startswith("self_attn.qkv_proj"):
            out.append(ShardMap(name, full_name, "rows", (full_cfg.q_size, full_cfg.kv_size, full_cfg.kv_size)))
        elif rest.startswith("mlp.gate_up_proj"):
            out.append(ShardMap(name, full_name, "rows", (full_cfg.intermediate_size, full_cfg.intermediate_size)))
        elif rest in ("self_attn.o_proj.weight", "mlp.down_proj.weight"):
            out.append(ShardMap(name, full_name, "cols"))
        else:
            out.append(ShardMap(name, full_name, "rep"))
    return out


def _slices(m: ShardMap, full: torch.Tensor, tp: int, tp_rank: int, ep: int = 1, ep_rank: int = 0) -> list[torch.Tensor]:
    """Views of the full tensor that, concatenated along the sharded dimension, form the local tensor."""
    if m.kind in EXPERT_KINDS and ep > 1:     # dim 0 (experts) is cut over the expert-parallel group first
        n = full.shape[0] // ep
        full = full[ep_rank * n : (ep_rank + 1) * n]
    if m.kind == "experts":
        return [full]
    if m.kind == "rep" or tp == 1:
        return [full]
    if m.kind == "cols":
        w = full.shape[1] // tp
        return [full[:, tp_rank * w : (tp_rank + 1) * w]]
    if m.kind == "expert_cols":
        w = full.shape[2] // tp
        return [full[:, :, tp_rank * w : (tp_rank + 1) * w]]
    parts, off = [], 0
    for b in m.blocks:
        w = b // tp
        lo = off + tp_rank * w
        parts.append(full[:, lo : lo + w] if m.kind == "expert_rows" else full[lo : lo + w])
        off += b
    return parts


EXPERT_KINDS = ("experts", "expert_rows", "expert_cols")


def cat_dim(kind: str) -> int:
    """Dimension along which the views of ``_slices`` line up in the local tensor."""
    return {"cols": 1, "expert_rows": 1, "expert_cols": 2}.get(kind, 0)


@torch.no_grad()
def copy_full_to_local(full: FlatParams, local: FlatParams, maps: list[ShardMap], tp: int, tp_rank: int, ep: int = 1,
                       ep_rank: int = 0) -> None:
    for m in maps:
        if m.full_name not in full.views:
            continue  # e.g. lm_head of a tied model
        parts = _slices(m, full.views[m.full_name], tp, tp_rank, ep, ep_rank)
        src = parts[0] if len(parts) == 1 else torch.cat(parts, cat_dim(m.kind))
        local.views[m.local_name].copy_(src.to(local.views[m.local_name].dtype))


@torch.no_grad()
def copy_local_to_full(local: FlatParams, full: FlatParams, maps: list[ShardMap], tp: int, tp_rank: int, ep: int = 1,
                       ep_rank: int = 0) -> None:
    """Write this rank's shard into its place of a full-layout buffer (merge / reshard building block)."""
    for m in maps:
        if m.full_name not in full.views:
            continue
        src = local.views[m.local_name]
        parts = _slices(m, full.views[m.full_name], tp, tp_rank, ep, ep_rank)
        if len(parts) == 1:
            parts[0].copy_(src.to(parts[0].dtype))
            continue
        off, dim = 0, cat_dim(m.kind)
        for p in parts:
            n = p.shape[dim]
            p.copy_(src.narrow(dim, off, n).to(p.dtype))
            off += n
