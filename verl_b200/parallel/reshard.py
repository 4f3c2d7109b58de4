"""Train -> rollout weight reshard of the model-parallel engine over peer memory.

Every rank of a training replica holds a shard of the model (a tensor-parallel slice of a pipeline stage, or a block of
experts). The colocated rollout engine of every rank reads a *full* replica in the layout of the unsharded model. After an
optimizer step each rank stores its shards straight into their places of every rank's replica: one kernel
(``ops.scatter_copy_``) walks a table of 2-D copy jobs whose destinations are peer-mapped addresses, so the bytes cross
NVLink once, peer to peer, with no host bounce, no zero-padded full-size buffer and no collective. Two device-side
barriers bracket the stores (nobody overwrites a replica that a peer's rollout still reads; nobody samples before every
shard has landed).

Parity target: ``verl/utils/megatron_utils.py:1389-1531`` (``per_tensor_generator``: gather the TP / PP / EP shards of every
tensor for the rollout engine).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..models.weights import FlatParams
from .model_parallel import EXPERT_KINDS, _slices
from .symmetric import PeerBarrier, SymmetricBuffer, symmetric_available

__all__ = ["PeerReshard"]

BLOCK_BYTES = 16384  # bytes one thread block of the copy kernel moves


class PeerReshard:
    def __init__(self, engine, limit_s: float = 60.0):
        topo = engine.topo
        self.engine, self.limit_s = engine, float(limit_s)
        dev, dtype = engine.device, engine.dtype
        # the ranks that together hold one full model; peer-mapped buffers are bound to the default group, so the replica
        # has to span the whole job (TP x PP with one data-parallel replica, or experts split over all ranks)
        world = dist.get_world_size()
        span = topo.tp * topo.pp * (topo.ep if topo.ep > 1 else 1)
        if span != world:
            raise NotImplementedError(f"the training replica spans {span} of {world} ranks")
        probe = FlatParams(engine.full_arch, dtype=dtype, device="meta", value_head=engine.value_head)
        self.sym = SymmetricBuffer.allocate(probe.numel, dtype, dev, None)
        self.full = FlatParams(engine.full_arch, dtype=dtype, device=dev, value_head=engine.value_head, buffer=self.sym.tensor)
        self.barrier = PeerBarrier(dev, None)
        self.world = world
        self._build_jobs()

    @classmethod
    def try_create(cls, engine) -> Optional["PeerReshard"]:
        """The peer-memory reshard when this job can use it (GPUs with peer-mapped memory, replica = whole job, shard
        rows that are whole 16-byte units), else None: the caller keeps the collective formulation."""
        if engine.device.type != "cuda" or not symmetric_available():
            return None
        try:
            return cls(engine)
        except (NotImplementedError, AssertionError):
            return None

    def _build_jobs(self) -> None:
        eng, topo = self.engine, self.engine.topo
        esz = self.full.flat.element_size()
        base = self.full.flat.data_ptr()
        local = []  # (byte offset in the replica, src address, rows, row bytes, dst stride, src stride)
        for m in eng.maps:
            if m.full_name not in self.full.views:
                continue
            # one writer per tensor that several ranks hold identically
            if m.kind == "rep" and topo.tp > 1 and topo.tp_rank != 0:
                continue
            if m.kind not in EXPERT_KINDS and topo.ep > 1 and topo.ep_rank != 0:
                continue
            src = eng.params.views[m.local_name]
            assert src.is_contiguous()
            parts = _slices(m, self.full.views[m.full_name], topo.tp, topo.tp_rank, topo.ep, topo.ep_rank)
            if m.kind in ("expert_rows", "expert_cols") and topo.tp > 1:
                # stacked expert matrices [E, rows, cols] cut inside every expert: one job per expert and part
                E_l, rows_l, cols_l = src.shape
                r0 = 0
                for part in parts:
                    pr, pc = part.shape[1], part.shape[2]
                    for e in range(E_l):
                        off = part[e].data_ptr() - base
                        s_addr = src.data_ptr() + ((e * rows_l + r0) * cols_l) * esz
                        if m.kind == "expert_rows":   # pr whole rows of the expert: one contiguous run
                            local.append((off, s_addr, 1, pr * pc * esz, pr * pc * esz, pr * pc * esz))
                        else:                          # a column block of the expert's matrix
                            local.append((off, s_addr, pr, pc * esz, part.stride(1) * esz, cols_l * esz))
                    r0 += pr if m.kind == "expert_rows" else 0
                continue
            row0 = 0
            for part in parts:
                off = part.data_ptr() - base
                if part.is_contiguous():
                    n = part.shape[0] if (len(parts) > 1 and part.dim() > 0) else None
                    nbytes = part.numel() * esz
                    s_addr = src.data_ptr() + (row0 * (src.numel() // src.shape[0]) * esz if n is not None else 0)
                    local.append((off, s_addr, 1, nbytes, nbytes, nbytes))
                    row0 += n or 0
                else:  # a column block of a 2-D tensor
                    assert part.dim() == 2 and part.stride(1) == 1 and len(parts) == 1
                    rows, w = part.shape
                    local.append((off, src.data_ptr(), rows, w * esz, part.stride(0) * esz, w * esz))
        for off, s_addr, rows, rb, ds, ss in local:
            assert rb % 16 == 0 and off % 16 == 0 and s_addr % 16 == 0 and ds % 16 == 0 and ss % 16 == 0, "16-byte units"
        jobs, starts, nblk = [], [0], 0
        for r in range(self.world):
            peer = int(self.sym.ptrs[r])
            for off, s_addr, rows, rb, ds, ss in local:
                jobs.append((peer + off, s_addr, rows, rb, ds, ss))
                nblk += -(-(rows * rb) // BLOCK_BYTES)
                starts.append(nblk)
        dev = self.engine.device
        self.jobs = torch.tensor(jobs, dtype=torch.int64).view(-1, 6).to(dev)
        self.block_start = torch.tensor(starts, dtype=torch.int32).to(dev)
        self.total_blocks = nblk
        self.bytes_per_run = sum(rows * rb for _, _, rows, rb, _, _ in local) * self.world

    def run(self) -> None:
        """Collective over the job: every rank pushes its shards into every replica."""
        from ..ops import native

        self.barrier(limit_s=self.limit_s)
        if self.total_blocks:
            native.ops().scatter_copy_(self.jobs, self.block_start, self.total_blocks)
        self.barrier(limit_s=self.limit_s)
