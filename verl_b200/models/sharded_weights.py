"""Working weights sharded at rest and gathered one unit at a time (the ZeRO-3 / FULL_SHARD layout).

A *unit* is what one gather brings in: the embedding table, one decoder layer, or the final norm plus the head. Every
unit's run of the flat parameter buffer is cut into ``world`` equal slices (rounded up to whole 16 KB chunks, so that a
copy job of a GEMM's fetch warp never straddles two owners); rank r keeps slice r of every unit in one store. Two arenas
of the size of the largest unit hold the units currently in use: while the kernels of unit u run out of one arena, the
next unit is gathered into the other (a collective on a side stream). Gradients of a unit accumulate in an fp32 arena of
the same shape and are reduce-scattered into the rank's gradient shard as soon as the unit's backward is done, so a full
gradient buffer never exists.

The class offers the access paths of :class:`FlatParams` that the hand-scheduled decoder uses (``layer(i)``,
``params[name]``, ``lm_head_weight``, ``.main_grad`` on the weight views) and the three hooks the decoder calls around
every unit (``pre_layer_hook`` / ``post_layer_backward_hook``), which drive prefetch and gradient reduction.

Parity target: ``verl/workers/engine/fsdp/transformer_impl.py:372-454`` (FSDP wrap, mixed precision),
``verl/utils/fsdp_utils.py:573-613`` (``fully_shard`` per layer).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .weights import ALIGN, FlatParams, _round_up

__all__ = ["UnitShardedParams"]

CHUNK_BYTES = 16384


class UnitShardedParams:
    def __init__(self, template: FlatParams, group=None, device=None, dtype: Optional[torch.dtype] = None,
                 symmetric: bool = False):
        """``template``: a FlatParams of the same model (any device, ``meta`` included) that provides the layout."""
        self.cfg, self.value_head = template.cfg, template.value_head
        self.specs, self.offsets = template.specs, template.offsets
        self.numel = self.dense_numel = template.dense_numel
        assert template.numel == template.dense_numel, "rank-local (expert-parallel) parameters cannot be unit-sharded"
        self.dtype = dtype or template.dtype
        self.device = torch.device(device) if device is not None else template.flat.device
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        L = self.cfg.num_hidden_layers
        esz = torch.empty((), dtype=self.dtype).element_size()
        chunk = CHUNK_BYTES // esz
        self.units: list[int] = sorted({s.layer for s in self.specs})          # -1, 0 .. L-1, L
        self.unit_range: dict[int, tuple[int, int]] = {u: template.layer_range(u) for u in self.units}
        self.slice_elems = {u: _round_up(-(-(hi - lo) // self.world), chunk) for u, (lo, hi) in self.unit_range.items()}
        self.store_off, off = {}, 0
        for u in self.units:
            self.store_off[u] = off
            off += self.slice_elems[u]
        self.owned_numel = off
        self.sym = self._peer_barrier = None
        self._fetch: Optional[dict] = None          # a gather in progress on the fetch warps of the running GEMMs
        self._flops_seen = 0.0                      # GEMM work since the current unit was entered
        self._flops_last = 0.0                      # ... of the unit before it (the budget of the next gather)
        if symmetric:
            # peer-mapped store: units are gathered by the GEMM kernels themselves (``ops.gemm_fetch``), no collective
            from ..parallel.symmetric import PeerBarrier, SymmetricBuffer

            self.sym = SymmetricBuffer.allocate(off, self.dtype, self.device, group)
            self.store = self.sym.tensor
            self._peer_barrier = PeerBarrier(self.device, group)
            self._esz = esz
        else:
            self.store = torch.zeros(off, dtype=self.dtype, device=self.device)
        self.flat = self.store                                                  # what this rank holds (dtype / size queries)
        cap = max(self.world * n for n in self.slice_elems.values())
        self.arenas = [torch.zeros(cap, dtype=self.dtype, device=self.device) for _ in range(2)]
        self.grad_arenas: list[Optional[torch.Tensor]] = [None, None]
        self.resident: list[Optional[int]] = [None, None]
        self._views: list[dict[str, torch.Tensor]] = [{}, {}]
        self._last_slot = 1
        self._pending: dict[int, object] = {}                                   # slot -> event of a gather in flight
        self._side = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.main_grad = None                                                   # FlatParams compatibility (never a full buffer)
        self.grad_shard: Optional[torch.Tensor] = None                          # fp32 [owned_numel]: sum over ranks, this rank's slices
        self._grads_on = False
        self._names_of = {u: [s for s in self.specs if s.layer == u] for u in self.units}
        self.gather_count = self.reduce_count = self.flush_count = 0
        self._phase = "forward"
        self._touched = [False, False]

    # ------------------------------------------------------------------ construction helpers
    def owned_index_ranges(self) -> list[tuple[int, int, int]]:
        """(flat_lo, flat_hi, store_offset) of this rank's part of every unit (empty parts are left out)."""
        out = []
        for u in self.units:
            lo, hi = self.unit_range[u]
            a = min(lo + self.rank * self.slice_elems[u], hi)
            b = min(a + self.slice_elems[u], hi)
            if b > a:
                out.append((a, b, self.store_off[u]))
        return out

    def load_from_full(self, full_flat: torch.Tensor) -> None:
        """Keep this rank's slices of a full flat buffer (layout of the template)."""
        self.store.zero_()
        for a, b, so in self.owned_index_ranges():
            self.store[so : so + (b - a)].copy_(full_flat[a:b])
        self.invalidate()

    def materialize_full(self, out: Optional[FlatParams] = None) -> FlatParams:
        """All units gathered into one full-layout FlatParams (what the rollout engine and HF export read). Collective."""
        if out is None:
            out = FlatParams(self.cfg, dtype=self.dtype, device=self.device, value_head=self.value_head, pad_to=self.world)
        self.invalidate()
        for u in self.units:
            lo, hi = self.unit_range[u]
            out.flat[lo:hi].copy_(self._gather_into(u, self.arenas[0])[: hi - lo])
        return out

    # ------------------------------------------------------------------ gathers
    def _gather_into(self, u: int, arena: torch.Tensor) -> torch.Tensor:
        se = self.slice_elems[u]
        src = self.store[self.store_off[u] : self.store_off[u] + se]
        dst = arena[: self.world * se]
        if self.world == 1:
            dst.copy_(src)
        elif self.device.type == "cuda":
            dist.all_gather_into_tensor(dst, src, group=self.group)
        else:
            dist.all_gather([dst[i * se : (i + 1) * se] for i in range(self.world)], src.contiguous(), group=self.group)
        self.gather_count += 1
        return dst

    def invalidate(self) -> None:
        """After the store changed (optimizer step, checkpoint load): gathered copies are stale. With a peer-mapped store
        this is also the point where every rank waits for the others' stores to be final before anyone reads them."""
        self._wait_all()
        self._fetch = None
        self.resident = [None, None]
        self._views = [{}, {}]
        if self._peer_barrier is not None:
            self._peer_barrier()

    # ------------------------------------------------------------------ gathers carried by the GEMM kernels
    def _start_fetch(self, u: int, slot: int) -> None:
        se = self.slice_elems[u]
        slice_bytes = se * self._esz
        cps = slice_bytes // CHUNK_BYTES                 # chunks per slice
        # this rank's own slice is one device-to-device copy away; the fetch warps bring the other ranks' slices
        self.arenas[slot][self.rank * se : (self.rank + 1) * se].copy_(self.store[self.store_off[u] : self.store_off[u] + se])
        todo = [iv for iv in ((0, self.rank * cps), ((self.rank + 1) * cps, self.world * cps)) if iv[1] > iv[0]]
        self._fetch = dict(unit=u, slot=slot, todo=todo, chunks=(self.world - 1) * cps, slice_bytes=slice_bytes,
                           total=self.world * slice_bytes, src=self.sym.ptrs + self.store_off[u] * self._esz,
                           budget=0.8 * max(self._flops_last, 1.0))
        from ..ops import functional as F

        F.set_fetch_rider(self)

    def take(self, flops: float):
        """Asked by every large GEMM (``ops.functional.gemm``): the share of the pending gather that this GEMM carries,
        in proportion to its work against the work of the previous unit, so the gather ends before the unit does."""
        self._flops_seen += flops
        f = self._fetch
        if f is None or not f["todo"]:
            return None
        n = max(1, int(f["chunks"] * flops / f["budget"]) + 1)
        c0, hi = f["todo"][0]
        c1 = min(hi, c0 + n)
        if c1 >= hi:
            f["todo"].pop(0)
        else:
            f["todo"][0] = (c1, hi)
        return f["src"], self.arenas[f["slot"]], f["total"], f["slice_bytes"], c0, c1

    def _finish_fetch(self) -> None:
        """The unit is needed now: whatever the GEMMs so far did not carry rides on small GEMMs of its own."""
        f = self._fetch
        if f is not None and f["todo"]:
            from ..ops import native

            if not hasattr(self, "_dummy"):
                self._dummy = (torch.zeros(128, 64, dtype=torch.bfloat16, device=self.device),
                               torch.zeros(128, 64, dtype=torch.bfloat16, device=self.device),
                               torch.zeros(128, 128, dtype=torch.bfloat16, device=self.device))
            a, b, d = self._dummy
            for c0, c1 in f["todo"]:
                native.ops().gemm_fetch(a, b, None, d, False, False, False, False, f["src"], self.arenas[f["slot"]], f["total"],
                                        f["slice_bytes"], c0, c1, -1, None, 2.0)
                self.flush_count += 1
            f["todo"] = []
        self._fetch = None

    def _wait_all(self) -> None:
        for slot, ev in list(self._pending.items()):
            torch.cuda.current_stream(self.device).wait_event(ev)
        self._pending.clear()

    def _build_views(self, slot: int, u: int) -> None:
        lo, _ = self.unit_range[u]
        views = {}
        for s in self._names_of[u]:
            o = self.offsets[s.name] - lo
            v = self.arenas[slot][o : o + s.numel].view(*s.shape)
            if self._grads_on:
                g = self.grad_arenas[slot]
                v.main_grad = g[o : o + s.numel].view(*s.shape)
            views[s.name] = v
        self._views[slot] = views

    def _slot_of(self, u: int) -> Optional[int]:
        for slot in (0, 1):
            if self.resident[slot] == u:
                return slot
        return None

    def _retarget(self, slot: int) -> None:
        """Before an arena takes another unit: wait for a gather still in flight into it and fold gradients that the
        unit it held has collected but not reduced yet (a tied embedding table collects some at the head, long before
        its own backward)."""
        if slot in self._pending:
            torch.cuda.current_stream(self.device).wait_event(self._pending.pop(slot))
        if self._grads_on and self._touched[slot]:
            self._reduce_slot(slot)

    def acquire(self, u: int) -> int:
        """Make unit ``u`` resident (gathering it now unless a prefetch already did) and return its arena slot."""
        slot = self._slot_of(u)
        if self._fetch is not None and (slot is None or self._fetch["unit"] == u):
            self._finish_fetch()  # the arena it fills is about to be used, or to be given to another unit
        if slot is None:
            slot = 1 - self._last_slot
            self._retarget(slot)
            if self.sym is not None:
                self._start_fetch(u, slot)
                self._finish_fetch()
                self.gather_count += 1
            else:
                self._gather_into(u, self.arenas[slot])
            self.resident[slot] = u
            self._build_views(slot, u)
        elif slot in self._pending:
            torch.cuda.current_stream(self.device).wait_event(self._pending.pop(slot))
        if slot != self._last_slot:
            self._flops_last, self._flops_seen = self._flops_seen, 0.0
        self._last_slot = slot
        if self._grads_on and self._phase == "backward":
            self._touched[slot] = True  # views with gradient targets are about to be handed out
        return slot

    def prefetch(self, u: int) -> None:
        """Start gathering unit ``u`` into the arena that the current unit does not use (side stream on a GPU; the
        collective order is the same on every rank because every rank walks the units in the same order)."""
        if u not in self.unit_range or self._slot_of(u) is not None:
            return
        slot = 1 - self._last_slot
        if slot in self._pending or (self._grads_on and self._touched[slot]):
            return  # busy, or its gradients still wait for their reduction: the gather happens at acquire time
        if self.sym is not None:
            if self._fetch is not None:
                return
            self._start_fetch(u, slot)      # same stream as the GEMMs that carry it: no events needed
            self.gather_count += 1
        elif self._side is None:
            self._gather_into(u, self.arenas[slot])
        else:
            # kernels already queued on the compute stream may still read the arena that is about to be overwritten
            self._side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._side):
                self._gather_into(u, self.arenas[slot])
                ev = torch.cuda.Event()
                ev.record(self._side)
            self._pending[slot] = ev
        self.resident[slot] = u
        self._build_views(slot, u)

    # ------------------------------------------------------------------ decoder hooks
    def pre_layer_hook(self, u: int, phase: str) -> None:
        self._phase = phase
        self.acquire(u)
        L = self.cfg.num_hidden_layers
        nxt = u + 1 if phase == "forward" else u - 1
        if -1 <= nxt <= L:
            self.prefetch(nxt)

    def post_layer_backward_hook(self, u: int) -> None:
        """Unit ``u``'s backward is complete: fold its gradients into this rank's shard (sum over ranks)."""
        slot = self._slot_of(u)
        if self._grads_on and slot is not None and self._touched[slot]:
            self._reduce_slot(slot)

    def _reduce_slot(self, slot: int) -> None:
        u = self.resident[slot]
        se = self.slice_elems[u]
        g = self.grad_arenas[slot][: self.world * se]
        tgt = self.grad_shard[self.store_off[u] : self.store_off[u] + se]
        if self.world == 1:
            tgt.add_(g)
        elif self.device.type == "cuda":
            tmp = torch.empty_like(tgt)
            dist.reduce_scatter_tensor(tmp, g, op=dist.ReduceOp.SUM, group=self.group)
            tgt.add_(tmp)
        else:
            dist.all_reduce(g, group=self.group)
            tgt.add_(g[self.rank * se : (self.rank + 1) * se])
        g.zero_()
        self._touched[slot] = False
        self.reduce_count += 1

    # ------------------------------------------------------------------ gradients
    def attach_main_grad(self, grad_buffer=None) -> None:
        cap = self.arenas[0].numel()
        self.grad_arenas = [torch.zeros(cap, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.grad_shard = torch.zeros(self.owned_numel, dtype=torch.float32, device=self.device)
        self._grads_on = True
        self._touched = [False, False]
        for slot in (0, 1):
            if self.resident[slot] is not None:
                self._build_views(slot, self.resident[slot])

    def detach_main_grad(self) -> None:
        self.grad_arenas = [None, None]
        self.grad_shard = None
        self._grads_on = False
        for slot in (0, 1):
            if self.resident[slot] is not None:
                self._build_views(slot, self.resident[slot])

    def zero_grad(self) -> None:
        if self._grads_on:
            self.grad_shard.zero_()
            for g in self.grad_arenas:
                g.zero_()
            self._touched = [False, False]

    # ------------------------------------------------------------------ access (FlatParams surface used by the decoder)
    def _unit_of(self, name: str) -> int:
        for s in self.specs:
            if s.name == name:
                return s.layer
        raise KeyError(name)

    def __getitem__(self, name: str) -> torch.Tensor:
        u = self._unit_of(name)
        return self._views[self.acquire(u)][name]

    def layer(self, i: int) -> dict[str, torch.Tensor]:
        slot = self.acquire(i)
        p = f"layers.{i}."
        return {k[len(p):]: v for k, v in self._views[slot].items() if k.startswith(p)}

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self["lm_head.weight" if "lm_head.weight" in self.offsets else "embed_tokens.weight"]

    def layer_range(self, i: int) -> tuple[int, int]:
        return self.unit_range[i]

    def decay_mask_ranges(self):
        out = []
        for s in sorted(self.specs, key=lambda s: self.offsets[s.name]):
            o = self.offsets[s.name]
            out.append((o, o + _round_up(s.numel, ALIGN), s.decay))
        return out

    def hf_state_dict(self, clone: bool = False):
        return self.materialize_full().hf_state_dict(clone=clone)

    def hf_views(self, prefix: str = "model."):
        return self.materialize_full().hf_views(prefix)
