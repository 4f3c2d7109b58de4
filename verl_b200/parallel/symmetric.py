"""Symmetric (peer-mapped) device buffers for in-kernel NVLink communication.

Every rank allocates the same-sized buffer, exchanges handles once (``torch.distributed._symmetric_memory``
rendezvous over the bootstrap process group) and from then on holds a table of device addresses — one per peer —
that the fused kernels dereference directly (peer loads / stores over NVLink 5 through the NVSwitch), plus, when
the fabric supports it, a multicast address for ``multimem`` instructions.  A per-rank signal pad of uint32 slots
carries the epoch flags of :func:`peer_barrier`.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

__all__ = ["SymmetricBuffer", "PeerBarrier", "symmetric_available", "ShardedRange", "PeerShardedLinear", "FusedRowParallelLinear",
           "PeerAllToAll", "PeerShare"]


def symmetric_available() -> bool:
    if not (torch.cuda.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
        return False
    try:
        from torch.distributed import _symmetric_memory  # noqa: F401

        return True
    except Exception:
        return False


@dataclass
class SymmetricBuffer:
    tensor: torch.Tensor          # this rank's buffer
    ptrs: torch.Tensor            # int64 CPU tensor [world]: device address of every rank's buffer
    multicast_ptr: int            # 0 when no multicast mapping exists
    handle: object

    @classmethod
    def allocate(cls, numel: int, dtype: torch.dtype, device, group=None, zero: bool = True) -> "SymmetricBuffer":
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        t = symm_mem.empty(numel, dtype=dtype, device=device)
        if zero:
            t.zero_()
        h = symm_mem.rendezvous(t, group)
        ptrs = torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64)
        mc = 0
        try:
            mc = int(h.multicast_ptr) if h.has_multicast_support(h.device.type if hasattr(h.device, "type") else "cuda", torch.cuda.current_device()) else 0
        except Exception:
            try:
                mc = int(h.multicast_ptr or 0)
            except Exception:
                mc = 0
        return cls(tensor=t, ptrs=ptrs, multicast_ptr=mc, handle=h)


class PeerBarrier:
    """Cross-GPU barrier on the current stream: monotonically increasing epochs through symmetric signal pads."""

    def __init__(self, device, group=None, slots: int = 64):
        self.buf = SymmetricBuffer.allocate(slots, torch.int32, device, group, zero=True)
        self.rank = dist.get_rank(group)
        self.epoch = 0
        dist.barrier(group)  # pads are zero everywhere before the first device-side epoch is written

    def __call__(self, limit_s: float = 20.0, poison: Optional[torch.Tensor] = None) -> None:
        """``poison``: an fp32 device scalar that receives +inf if the wait runs out (see ``peer_barrier_kernel``)."""
        from ..ops import native

        self.epoch += 1
        native.ops().peer_barrier(self.buf.ptrs, self.rank, self.epoch, float(limit_s), poison)


class FusedRowParallelLinear:
    """Row-parallel (K-sharded) linear whose all-reduce runs inside the GEMM epilogue over peer memory.

    Owns the peer-visible partial buffer (two halves, alternating per call), the flags and the call counter of one
    tensor-parallel group. Large calls (prefill) reduce inside the GEMM epilogue tile by tile; decode-sized calls (few
    output tiles, deep K) run the GEMM K-split over all SMs and fold the splits in the kernel that performs the all-reduce. Every rank of the group must issue the same sequence of calls; the result is bitwise
    identical on all ranks. ``max_rows`` bounds ``M`` of a call (rows of the activation)."""

    def __init__(self, max_rows: int, n: int, device, group=None, limit_s: float = 20.0):
        self.limit_s = float(limit_s)
        self.group = group
        # large calls on more than two ranks: GEMM + library all-reduce unless a form is asked for by name (``two_shot=``)
        self.library_for_large = os.environ.get("VERL_B200_LARGE_ALLREDUCE", "library") == "library"
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.n, self.max_rows = int(n), int(max_rows)
        self.buf_elems = self.max_rows * self.n
        self.part = SymmetricBuffer.allocate(2 * self.buf_elems, torch.bfloat16, device, group, zero=False)
        tiles = ((self.max_rows + 127) // 128) * ((self.n + 127) // 128)
        chunks = (self.buf_elems + 2047) // 2048  # flags of the decode-sized path (one per 2048 output elements)
        self.flags = SymmetricBuffer.allocate(max(4 * tiles, chunks), torch.int32, device, group, zero=True)
        # decode-sized calls run the GEMM K-split over all SMs and fold the splits inside the all-reduce kernel
        self.splitk_ws = torch.empty(8 * self.buf_elems, dtype=torch.float32, device=device) if self.max_rows <= 1024 else None
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # flags are zero everywhere before anyone publishes epoch 1

    def __call__(self, a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 b_mn: bool = False, scatter_rows: int = 0, two_shot: Optional[bool] = None):
        """``b_mn``: ``b`` is stored [K, N] (the input gradient of a column-parallel layer: ``dY_r @ W_r`` summed over ranks).
        ``scatter_rows`` > 0: reduce-scatter instead of all-reduce: returns this rank's ``[scatter_rows, N]`` slice of the
        sum (rows ``rank * scatter_rows ...``; zero where the slice runs past the input's rows); every rank must own a row.
        ``two_shot``: reduce this rank's share of the rows in the epilogue, then all-gather the shares (see ``_two_shot``);
        ``None`` picks it for large calls on more than two ranks."""
        from ..ops import native

        assert a.shape[0] <= self.max_rows and (b.shape[1] if b_mn else b.shape[0]) == self.n
        M = a.shape[0]
        if two_shot is None and self.world > 2 and M > 1024 and scatter_rows == 0 and self.library_for_large:
            # measured at 8 ranks (8192 x 3584 x 2368): GEMM + the library's in-switch all-reduce 0.37 - 0.42 ms, the
            # reduce-scatter epilogue + all-gather 0.83 ms, the one-kernel form 1.02 ms: the in-kernel forms pull with plain
            # peer loads and pay their latency per tile, the switch reduces in flight
            from ..ops import functional as F

            y = F.gemm(a, b, out=out, b_mn=bool(b_mn))
            dist.all_reduce(y, group=self.group)
            if bias is not None:
                y.add_(bias)
            return y
        if two_shot and scatter_rows == 0 and M >= self.world * self.world:
            return self._two_shot(a, b, bias, out, b_mn)
        return native.ops().gemm_allreduce(a, b, bias, self.part.ptrs, self.flags.ptrs, self.epoch, self.buf_elems, self.rank, self.limit_s, out,
                                           self.splitk_ws, bool(b_mn), int(scatter_rows))

    def _two_shot(self, a, b, bias, out, b_mn):
        """All-reduce as reduce-scatter + all-gather. The one-kernel form has every rank pull the same tile from every peer:
        (world - 1) x the output crosses each rank's link, which at 8 ranks costs more than the GEMM. Here a rank pulls and
        sums only its ``1 / world`` of the rows inside the GEMM epilogue, and the bf16 shares are then exchanged by one
        all-gather (in-switch multicast where the library uses it): 2 x (world - 1) / world of the output per link."""
        from ..ops import native

        M = a.shape[0]
        rows = -(-M // self.world)
        mine = native.ops().gemm_allreduce(a, b, bias, self.part.ptrs, self.flags.ptrs, self.epoch, self.buf_elems, self.rank,
                                           self.limit_s, None, None, bool(b_mn), rows)
        direct = out is not None and rows * self.world == M and out.is_contiguous()
        full = out if direct else torch.empty(rows * self.world, self.n, dtype=mine.dtype, device=mine.device)
        dist.all_gather_into_tensor(full, mine, group=self.group)
        if direct:
            return out
        if out is not None:
            out.copy_(full[:M])
            return out
        return full[:M]


class PeerShare:
    """All-gather of a few 32-bit words per rank over peer memory in one kernel whose call counter lives on the device, so it
    can sit inside a captured CUDA graph (the tensor-parallel rollout ranks each sample half of the batch and share the
    tokens and log-probs). ``cap``: words one rank may contribute per call."""

    def __init__(self, cap: int, device, group=None, limit_s: float = 20.0):
        self.cap, self.limit_s = int(cap), float(limit_s)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.buf = SymmetricBuffer.allocate(2 * self.world * self.cap, torch.int32, device, group, zero=True)
        self.flags = SymmetricBuffer.allocate(max(self.world, 16), torch.int32, device, group, zero=True)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # flags are zero everywhere before anyone publishes call 1

    def __call__(self, src: torch.Tensor) -> torch.Tensor:
        """``src`` int32 [n] (n <= cap, the same n on every rank) -> int32 [world, n]."""
        from ..ops import native

        out = torch.empty(self.world, src.numel(), dtype=torch.int32, device=src.device)
        native.ops().peer_share_(self.buf.ptrs, self.flags.ptrs, self.epoch, src, out, self.cap, self.rank, self.limit_s)
        return out


class PeerAllToAll:
    """The head <-> sequence exchange of Ulysses sequence parallelism over peer memory. One copy kernel stores every block
    straight from the (strided) source into its place in the destination rank's peer-mapped buffer, 16 KB per thread
    block, so the pack pass in front of a collective all-to-all disappears and the bytes cross NVLink once; two
    device-side barriers bracket the stores (nobody overwrites a buffer its owner still reads; nobody reads before every
    block has landed). The result is copied out of the buffer, which the next exchange reuses.

    Parity target: ``verl/utils/ulysses.py:137-195`` (``all_to_all_tensor`` behind ``gather_seq_scatter_heads`` /
    ``gather_heads_scatter_seq``)."""

    BLOCK = 16384

    def __init__(self, device, group=None, limit_s: float = 30.0):
        self.device, self.group, self.limit_s = device, group, float(limit_s)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.buf: Optional[SymmetricBuffer] = None
        self.cap_bytes = 0
        self.barrier = PeerBarrier(device, group)

    def _ensure(self, nbytes: int) -> None:
        if nbytes > self.cap_bytes:  # every rank of the group sees the same sizes, so they re-allocate together
            self.cap_bytes = max(2 * self.cap_bytes, -(-nbytes // (1 << 20)) * (1 << 20))
            self.buf = SymmetricBuffer.allocate(self.cap_bytes, torch.uint8, self.device, self.group, zero=False)

    def _run(self, jobs: list, out_bytes: int) -> torch.Tensor:
        from ..ops import native

        starts, n = [0], 0
        for _, _, rows, rb, _, _ in jobs:
            n += -(-(rows * rb) // self.BLOCK)
            starts.append(n)
        for dst, src, rows, rb, ds, ss in jobs:
            assert dst % 16 == 0 and src % 16 == 0 and rb % 16 == 0 and ds % 16 == 0 and ss % 16 == 0, "16-byte units"
        self.barrier(limit_s=self.limit_s)
        if n:
            j = torch.tensor(jobs, dtype=torch.int64).view(-1, 6).to(self.device)
            b = torch.tensor(starts, dtype=torch.int32).to(self.device)
            native.ops().scatter_copy_(j, b, n)
        self.barrier(limit_s=self.limit_s)
        return self.buf.tensor[:out_bytes]

    def exchange_rows(self, x: torch.Tensor, rows: list) -> torch.Tensor:
        """Variable-size row exchange (token dispatch of expert parallelism): ``rows[s][d]`` = rows that rank s sends to
        rank d, known to every rank. ``x`` holds this rank's rows for rank 0, then for rank 1, ...; returns the rows this
        rank receives, ordered by source rank. Every block is stored straight into its final place of the receiver's
        buffer (offset = the rows that lower-ranked sources send to the same receiver)."""
        W, me = self.world, self.rank
        assert x.dim() == 2 and x.is_contiguous()
        row_bytes = x.shape[1] * x.element_size()
        total_in = sum(rows[s][me] for s in range(W))
        most = max(sum(rows[s][d] for s in range(W)) for d in range(W))   # the same on every rank: they re-allocate together
        self._ensure(max(1, most) * row_bytes)
        jobs, src_row = [], 0
        for d in range(W):
            n = rows[me][d]
            if n:
                dst_row = sum(rows[s][d] for s in range(me))
                jobs.append((int(self.buf.ptrs[d]) + dst_row * row_bytes, x.data_ptr() + src_row * row_bytes, 1, n * row_bytes,
                             n * row_bytes, n * row_bytes))
            src_row += n
        return self._run(jobs, total_in * row_bytes).view(x.dtype).view(total_in, x.shape[1]).clone()

    def seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """[T/size, heads, hd] (my tokens, all heads) -> [T, heads/size, hd] (all tokens, my heads)."""
        tl, h, d = x.shape
        W, esz = self.world, x.element_size()
        hs = h // W
        assert x.stride(2) == 1 and x.stride(1) == d
        row, blk = hs * d * esz, tl * hs * d * esz
        self._ensure(W * blk)
        jobs = [(int(self.buf.ptrs[j]) + self.rank * blk, x.data_ptr() + j * row, tl, row, row, x.stride(0) * esz) for j in range(W)]
        return self._run(jobs, W * blk).view(x.dtype).view(W * tl, hs, d).clone()

    def heads_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        """[T, heads/size, hd] -> [T/size, heads, hd]: every block lands in its final place (column block of the row)."""
        t, hs, d = x.shape
        W, esz = self.world, x.element_size()
        tl = t // W
        assert x.is_contiguous()
        row = hs * d * esz
        self._ensure(tl * W * row)
        jobs = [(int(self.buf.ptrs[j]) + self.rank * row, x.data_ptr() + j * tl * row, tl, row, W * row, row) for j in range(W)]
        return self._run(jobs, tl * W * row).view(x.dtype).view(tl, W * hs, d).clone()


FETCH_CHUNK = 16384  # bytes per copy job of a GEMM's fetch warp (``FETCH_CHUNK`` in gemm_tcgen05.cu)


class ShardedRange:
    """A run of bytes kept in equal slices on the ranks of a group (1 / world of it per GPU, in peer-mapped memory) that
    GEMM kernels gather into a local arena while they compute (``ops.gemm_fetch``): the parameter all-gather of a fully
    sharded layout, carried by the fetch warps of the kernels that run anyway.

    ``slice_bytes`` is rounded up to whole 16 KB chunks so that a chunk never straddles two owners; rank r holds bytes
    [r * slice_bytes, (r + 1) * slice_bytes) of the range (the tail of the last slice is padding)."""

    def __init__(self, total_bytes: int, device, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert total_bytes % 16 == 0, "ranges are copied 16 bytes at a time"
        self.total_bytes = int(total_bytes)
        per = -(-self.total_bytes // self.world)
        self.slice_bytes = -(-per // FETCH_CHUNK) * FETCH_CHUNK
        self.num_chunks = -(-self.total_bytes // FETCH_CHUNK)
        self.buf = SymmetricBuffer.allocate(self.slice_bytes, torch.uint8, device, group, zero=True)
        self.slice = self.buf.tensor                      # this rank's bytes of the range
        self._barrier = PeerBarrier(device, group)

    @property
    def owned(self) -> tuple[int, int]:
        """[lo, hi) byte range of the whole that this rank stores."""
        lo = min(self.rank * self.slice_bytes, self.total_bytes)
        return lo, min(lo + self.slice_bytes, self.total_bytes)

    def store_from_full(self, full_bytes: torch.Tensor) -> None:
        """Keep this rank's slice of a full copy (uint8 view of ``total_bytes`` bytes)."""
        lo, hi = self.owned
        self.slice[: hi - lo].copy_(full_bytes[lo:hi])

    def barrier(self) -> None:
        """After an update of the slices: nobody gathers bytes that their owner is still writing."""
        self._barrier()


class PeerShardedLinear:
    """Linear layer whose weight [N, K] is stored in equal slices on the ranks of a group (1 / world of the bytes per GPU)
    and gathered by the very GEMM that consumes it: an extra warp in every CTA copies the weight, 16 KB at a time and in
    the order the tiles need it, from its owners' memory over NVLink into a local arena; a tile starts as soon as the
    rows it reads have landed, and every remote byte crosses the link once. Every rank computes the full ``x @ W^T``
    for its own tokens. This is the parameter all-gather of a fully sharded layout fused into the consuming GEMM.

    Call ``barrier()`` (or any collective) after a weight update so that no rank reads bytes that a peer is still
    writing. The arena holds the gathered weight until the next call; ``gathered`` exposes it (valid after a call)."""

    def __init__(self, n: int, k: int, device, group=None, dtype=torch.bfloat16, limit_s: float = 5.0):
        assert dtype == torch.bfloat16 and k % 8 == 0
        self.n, self.k, self.limit_s = int(n), int(k), float(limit_s)
        self.range = ShardedRange(self.n * self.k * 2, device, group)
        self.rank, self.world = self.range.rank, self.range.world
        self.arena = torch.empty(self.range.total_bytes, dtype=torch.uint8, device=device)
        self.gathered = self.arena.view(torch.bfloat16).view(self.n, self.k)
        self.panels = torch.zeros((self.n + 127) // 128, dtype=torch.int32, device=device)

    def load_full(self, weight: torch.Tensor) -> None:
        """Shard a full [N, K] weight (every rank passes the same values; each keeps its slice)."""
        self.range.store_from_full(weight.contiguous().view(-1).view(torch.uint8))

    def barrier(self) -> None:
        self.range.barrier()

    def __call__(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        from ..ops import native

        assert x.shape[-1] == self.k
        r = self.range
        return native.ops().gemm_fetch(x, self.gathered, bias, out, False, False, False, False, r.buf.ptrs, self.arena,
                                       r.total_bytes, r.slice_bytes, 0, r.num_chunks, 0, self.panels, self.limit_s)
