"""Expert-parallel mixture-of-experts layer over peer memory (forward).

Rank ``r`` of an ``W``-rank group owns experts ``[r*E/W, (r+1)*E/W)``. One layer call:

1. route locally (softmax top-k kernel) and publish the per-expert counts into every peer's ``[W, E]`` table;
2. every rank derives the same global layout: expert ``e`` occupies a 128-row-aligned segment in its owner's buffer,
   ordered by source rank, so each (token, choice) pair has an (owner, row) address known without further messages;
3. **dispatch** = the permutation kernel stores each token copy directly into its owner's buffer (peer stores);
4. the owner runs the grouped tcgen05 GEMMs (gate/up -> SwiGLU -> down) over its segments;
5. **combine** = the un-permutation kernel reads the expert outputs from the owners' buffers (peer loads) and forms the
   routing-weighted sum.

Dispatch and combine are therefore the all-to-alls, fused with permutation and weighted sum, with no staging buffers and
no collective library call; peer barriers (bounded, status-reporting) separate the phases. Token copies beyond
``capacity_factor`` x the average load of a rank are dropped and counted.

Parity target: the expert-parallel token dispatcher of the reference's Megatron/vLLM back-ends (all-to-all dispatch,
grouped expert GEMM, all-to-all combine).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as F
from .symmetric import PeerBarrier, SymmetricBuffer

__all__ = ["ExpertParallelMoE"]


class ExpertParallelMoE:
    def __init__(self, num_experts: int, top_k: int, hidden: int, max_tokens: int, device, group=None, capacity_factor: float = 2.0,
                 norm_topk_prob: bool = True):
        self.group = group
        self.W, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert num_experts % self.W == 0
        self.E, self.k, self.H = num_experts, top_k, hidden
        self.E_local = num_experts // self.W
        self.norm = norm_topk_prob
        self.cap = (int(max_tokens * top_k * capacity_factor + 127) // 128 + self.E_local) * 128
        self.xp = SymmetricBuffer.allocate(self.cap * hidden, torch.bfloat16, device, group, zero=True)
        self.y = SymmetricBuffer.allocate(self.cap * hidden, torch.bfloat16, device, group, zero=True)
        self.table = SymmetricBuffer.allocate(self.W * num_experts, torch.int32, device, group, zero=True)
        self.xp_ptrs, self.y_ptrs, self.table_ptrs = (b.ptrs.to(device) for b in (self.xp, self.y, self.table))
        self.barrier = PeerBarrier(device, group)
        self.dropped = torch.zeros((), dtype=torch.int64, device=device)

    def _layout(self, idx: torch.Tensor):
        """(dest_rank, dest_row) [T*k] of this rank's token copies and (seg, tile_expert, num_mtiles) of the local experts."""
        dev = idx.device
        W, E, El, k = self.W, self.E, self.E_local, self.k
        counts_all = self.table.tensor.view(W, E).long()              # [source rank, expert]
        per_expert = counts_all.sum(0)
        pad = (per_expert + 127) // 128 * 128
        pad_l = pad.view(W, El)
        seg_owner = torch.zeros(W, El + 1, dtype=torch.int64, device=dev)
        seg_owner[:, 1:] = pad_l.cumsum(1)                            # segment starts inside each owner's buffer
        before = counts_all.cumsum(0) - counts_all                    # rows of earlier source ranks, per expert
        flat_e = idx.reshape(-1).long()
        order = torch.argsort(flat_e, stable=True)
        mine = counts_all[self.rank]
        first = mine.cumsum(0) - mine
        e_sorted = flat_e[order]
        within = torch.arange(flat_e.numel(), device=dev) - first[e_sorted]
        owner_sorted = torch.div(e_sorted, El, rounding_mode="floor")
        row_sorted = seg_owner[owner_sorted, e_sorted % El] + before[self.rank, e_sorted] + within
        over = row_sorted >= self.cap
        self.dropped += over.sum()
        row_sorted = torch.where(over, torch.full_like(row_sorted, -1), row_sorted)
        dest_rank = torch.empty(flat_e.numel(), dtype=torch.int32, device=dev)
        dest_row = torch.empty_like(dest_rank)
        dest_rank[order] = owner_sorted.int()
        dest_row[order] = row_sorted.int()
        seg = seg_owner[self.rank].clamp(max=self.cap)
        tiles = torch.arange(self.cap // 128, device=dev) * 128
        tile_expert = torch.searchsorted(seg[1:].contiguous(), tiles, right=True).clamp_(max=El - 1).int()
        return dest_rank, dest_row, seg.int(), tile_expert, (seg[El:] // 128).int()

    @torch.no_grad()
    def forward(self, h2: torch.Tensor, gate_weight: torch.Tensor, w_gate_up_local: torch.Tensor, w_down_local: torch.Tensor) -> torch.Tensor:
        ops = F._ops()
        T = h2.shape[0]
        logits = F.gemm(h2, gate_weight)
        w, idx, counts = ops.moe_route_topk(logits, self.k, self.norm)
        ops.moe_publish_counts_(counts, self.table_ptrs, self.rank)
        self.barrier()                                              # all count rows are in place
        dest_rank, dest_row, seg, tile_expert, num_mtiles = self._layout(idx)
        self.xp.tensor.zero_()                                      # padding rows must read as zero
        self.barrier()                                              # nobody writes into a buffer that is being cleared
        ops.moe_dispatch_peer_(h2, self.xp_ptrs, dest_rank, dest_row, self.k)
        self.barrier()                                              # all token copies have arrived
        xp = self.xp.tensor.view(self.cap, self.H)
        gu = ops.gemm_grouped_rows(xp, w_gate_up_local, False, tile_expert, num_mtiles)
        yv = ops.gemm_grouped_rows(F.swiglu(gu), w_down_local, False, tile_expert, num_mtiles)
        self.y.tensor.view(self.cap, self.H).copy_(yv)
        self.barrier()                                              # expert outputs are visible to the peers
        out = ops.moe_combine_peer(self.y_ptrs, dest_rank.view(T, self.k), dest_row.view(T, self.k), w, self.H, h2)
        self.barrier()                                              # buffers may be reused by the next layer
        return out
