"""Decoder-only transformer with hand-scheduled forward and backward passes.

The model runs on packed ("remove-padding") token streams: ``input_ids`` / ``positions`` are 1-D over the
concatenation of all sequences of a micro-batch and ``cu_seqlens`` marks the boundaries, so no FLOP is
spent on padding.  The backward pass is written out explicitly instead of being traced by autograd:

* the set of saved activations is chosen by hand (layer input, rotated QKV, attention output + LSE,
  post-attention residual, gate/up pre-activation); norms and SwiGLU outputs are recomputed because
  they are memory-bound and cheaper to redo than to keep in HBM;
* ``recompute="full"`` keeps only each layer's input pair and replays the layer in backward;
* weight gradients are accumulated by the wgrad GEMM straight into the fp32 ``main_grad`` buffer;
* per-layer hooks let a sharded runtime gather parameters before a layer and reduce gradients after it.

The same code runs in fp32 on CPU (through the functional fallbacks), which is what the CPU/gloo
configuration and the numerics tests use.  Reference semantics: HF Llama/Qwen2/Qwen3(-MoE) modelling as
used by ``verl/workers/engine/fsdp/transformer_impl.py:1122-1564`` (packed inputs, labels rolled by one,
log-prob / entropy from the LM head).
"""

from __future__ import annotations

import os

import math
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch

from ..ops import functional as F
from .config import ModelConfig
from .weights import FlatParams

__all__ = ["PackedBatch", "DecoderModel", "RouterReplay", "ExpertParallelGroup", "UlyssesSequenceParallel", "ContextParallel",
           "TensorSequenceParallel"]


@dataclass
class PackedBatch:
    """A micro-batch of packed sequences."""

    input_ids: torch.Tensor  # [T] int64
    positions: torch.Tensor  # [T] int32/int64
    cu_seqlens: torch.Tensor  # [B+1] int32 (device) ...
    max_seqlen: int
    cu_seqlens_cpu: Optional[torch.Tensor] = None  # host copy (avoids syncs in fallbacks)
    # Shared-prefix batches: sequences of one group have the same prompt. The token stream then holds the prompt ONCE per
    # group followed by the members' responses; every token-wise op (norms, projections, MLP, head) runs on that
    # de-duplicated stream. Only attention needs whole sequences: ``expand_index`` [T_e] gathers the stream into the
    # per-member (prompt + response) layout that ``cu_seqlens`` describes, ``collapse_index`` [T] picks one representative of
    # every stream token back out of it.
    expand_index: Optional[torch.Tensor] = None
    collapse_index: Optional[torch.Tensor] = None

    @property
    def num_tokens(self) -> int:
        return int(self.input_ids.shape[0])

    @classmethod
    def from_lengths(cls, input_ids: torch.Tensor, lengths: list[int], device=None) -> "PackedBatch":
        device = device if device is not None else input_ids.device
        cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(torch.tensor(lengths, dtype=torch.int32), 0)
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths]) if lengths else torch.zeros(0, dtype=torch.int32)
        return cls(input_ids=input_ids.to(device), positions=pos.to(device), cu_seqlens=cu.to(device),
                   max_seqlen=max(lengths) if lengths else 0, cu_seqlens_cpu=cu)


class _Anchor(torch.autograd.Function):
    """Autograd bridge: forward returns the model outputs, backward runs the hand-written backward."""

    @staticmethod
    def forward(ctx, anchor, model, state, *outs):
        ctx.model = model
        ctx.state = state
        return tuple(o.detach() for o in outs)

    @staticmethod
    def backward(ctx, *grads):
        ctx.model._backward(ctx.state, grads)
        ctx.state = None
        dev = ctx.model.device
        ctx.model = None
        return (torch.zeros((), device=dev), None, None) + tuple(None for _ in grads)


class TensorParallelShard:
    """Inference-time tensor parallelism over *views* of the replicated weights: rank ``r`` of ``size`` uses its heads'
    rows of the fused QKV weight and its rows of gate/up (column-parallel, three plus two narrow GEMMs writing into one
    activation buffer) and the matching K-slices of ``o_proj`` / ``down_proj`` (row-parallel). Nothing is copied: a
    weight update of the full replica is visible to the shard at once. ``row_linear(a, w_kslice, bias)`` must return the
    sum over ranks (on GPUs: the GEMM whose epilogue all-reduces over peer memory)."""

    def __init__(self, rank: int, size: int, row_linear: Callable):
        self.rank, self.size, self.row_linear = int(rank), int(size), row_linear

    def rows(self, total: int) -> slice:
        per = total // self.size
        return slice(self.rank * per, (self.rank + 1) * per)


class UlyssesSequenceParallel:
    """Sequence parallelism over ``size`` ranks that hold the same micro-batch: every rank runs the token-wise layers on a
    contiguous 1/size slice of the packed token stream; around attention an all-to-all trades the sequence split for a
    head split (each rank attends over whole sequences with 1/size of the heads) and back.

    Parity target: ``verl/utils/ulysses.py:137-195`` (``gather_seq_scatter_heads`` / ``gather_heads_scatter_seq``) and
    ``verl/models/transformers/monkey_patch.py:87-155``."""

    def __init__(self, group, rank: int, size: int):
        self.group, self.rank, self.size = group, int(rank), int(size)
        self._peer = None  # PeerAllToAll, created at the first exchange on GPUs with peer-mapped memory

    def _peer_exchange(self, x: torch.Tensor):
        """The peer-memory exchange for this group, or None (CPU, one rank, no peer-mapped memory, VERL_B200_PEER_ULYSSES=0):
        the collective formulation is used then. Every rank of the group takes the same branch."""
        if self._peer is None:
            import os

            self._peer = False
            if x.is_cuda and self.size > 1 and os.environ.get("VERL_B200_PEER_ULYSSES", "1") != "0":
                from ..parallel.symmetric import PeerAllToAll, symmetric_available

                if symmetric_available():
                    try:
                        self._peer = PeerAllToAll(x.device, self.group)
                    except Exception:  # no peer mapping for this group: stay on the collective
                        self._peer = False
        return self._peer or None

    def local_slice(self, total: int) -> slice:
        assert total % self.size == 0, "the packed stream must be padded to a multiple of the sequence-parallel size"
        n = total // self.size
        return slice(self.rank * n, (self.rank + 1) * n)

    def pad_multiple(self) -> int:
        """The packed stream is padded to a multiple of this many tokens."""
        return self.size

    def local_rows(self, total: int, device=None):
        """Stream positions of this rank's rows, in local order (a slice here; an index tensor for split layouts)."""
        return self.local_slice(total)

    def local_of(self, positions: torch.Tensor, total: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(mask of the stream ``positions`` this rank holds, their local row numbers)."""
        sl = self.local_slice(total)
        mine = (positions >= sl.start) & (positions < sl.stop)
        return mine, positions[mine] - sl.start

    def seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """[T/size, heads, hd] (my tokens, all heads) -> [T, heads/size, hd] (all tokens, my heads)."""
        import torch.distributed as dist

        tl, h, d = x.shape
        hs = h // self.size
        peer = self._peer_exchange(x)
        if peer is not None and x.stride(2) == 1 and x.stride(1) == d and (hs * d * x.element_size()) % 16 == 0 and \
                (x.stride(0) * x.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0:
            return peer.seq_to_heads(x)
        send = x.view(tl, self.size, hs, d).permute(1, 0, 2, 3).contiguous()  # [size, tl, hs, d]: block j goes to rank j
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)                  # block i came from rank i: its tokens, my heads
        return recv.view(self.size * tl, hs, d)

    def heads_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        """[T, heads/size, hd] -> [T/size, heads, hd] (inverse of ``seq_to_heads``)."""
        import torch.distributed as dist

        t, hs, d = x.shape
        tl = t // self.size
        peer = self._peer_exchange(x)
        if peer is not None and x.is_contiguous() and (hs * d * x.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0:
            return peer.heads_to_seq(x)
        send = x.view(self.size, tl, hs, d).contiguous()                      # block j: rank j's tokens, my heads
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)                  # block i: my tokens, rank i's heads
        return recv.permute(1, 0, 2, 3).reshape(tl, self.size * hs, d)


class ContextParallel(UlyssesSequenceParallel):
    """Context parallelism over ``size`` ranks that hold the same micro-batch: like sequence parallelism every rank runs
    the token-wise layers on a contiguous 1/size slice of the packed token stream, but around attention the KEYS AND
    VALUES are all-gathered (all tokens, all heads) and every rank attends with its own queries; in the backward the
    key / value gradients are reduce-scattered back to the owners of the tokens. Unlike the head exchange this puts no
    divisibility constraint on the number of key/value heads (grouped-query models with few KV heads, long contexts).

    Parity target: Megatron context parallelism as configured by ``verl/workers/config/engine.py``
    (``context_parallel_size``) with the zigzag (load-balanced) and contiguous token splits of
    ``verl/models/mcore/util.py:62-211``."""

    def __init__(self, group, rank: int, size: int, zigzag: bool = True):
        super().__init__(group, rank, size)
        # zigzag: the stream is cut into 2 * size chunks and rank i holds chunks i and 2 * size - 1 - i, which evens out the
        # causal attention work (late tokens see more keys than early ones); contiguous: rank i holds the i-th 1/size
        self.zigzag = bool(zigzag) and size > 1

    def pad_multiple(self) -> int:
        return 2 * self.size if self.zigzag else self.size

    def chunks(self, total: int) -> list[tuple[int, int]]:
        """[start, stop) stream ranges of this rank's rows, in local order."""
        if not self.zigzag:
            sl = self.local_slice(total)
            return [(sl.start, sl.stop)]
        assert total % (2 * self.size) == 0, "the packed stream must be padded to a multiple of twice the context-parallel size"
        c = total // (2 * self.size)
        a, b = self.rank, 2 * self.size - 1 - self.rank
        return [(a * c, (a + 1) * c), (b * c, (b + 1) * c)]

    def local_rows(self, total: int, device=None):
        if not self.zigzag:
            return self.local_slice(total)
        return torch.cat([torch.arange(lo, hi, device=device) for lo, hi in self.chunks(total)])

    def local_of(self, positions: torch.Tensor, total: int) -> tuple[torch.Tensor, torch.Tensor]:
        if not self.zigzag:
            return super().local_of(positions, total)
        mine = torch.zeros_like(positions, dtype=torch.bool)
        local = torch.zeros_like(positions)
        off = 0
        for lo, hi in self.chunks(total):
            sel = (positions >= lo) & (positions < hi)
            mine |= sel
            local = torch.where(sel, positions - lo + off, local)
            off += hi - lo
        return mine, local[mine]

    def _stream_order(self, total: int, device) -> Optional[torch.Tensor]:
        """Row of the rank-major gathered tensor that holds stream chunk j, for every j (None: already in order)."""
        if not self.zigzag:
            return None
        c = total // (2 * self.size)
        src = []
        for j in range(2 * self.size):
            r, half = (j, 0) if j < self.size else (2 * self.size - 1 - j, 1)
            src.append(torch.arange((2 * r + half) * c, (2 * r + half + 1) * c, device=device))
        return torch.cat(src)

    def gather_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """[T/size, ...] of every rank -> [T, ...] in stream order."""
        import torch.distributed as dist

        x = x.contiguous()
        out = torch.empty(self.size * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x, group=self.group)
        else:
            dist.all_gather(list(out.chunk(self.size, 0)), x, group=self.group)
        order = self._stream_order(out.shape[0], x.device)
        return out if order is None else out.index_select(0, order)

    def scatter_sum(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of every rank's [T, ...] contribution, this rank's [T/size, ...] rows of it."""
        import torch.distributed as dist

        order = self._stream_order(x.shape[0], x.device)
        if order is not None:            # back to the rank-major layout the collective scatters
            rank_major = torch.empty_like(x)
            rank_major.index_copy_(0, order, x)
            x = rank_major
        x = x.contiguous()
        n = x.shape[0] // self.size
        if x.is_cuda:
            out = torch.empty(n, *x.shape[1:], dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, x, group=self.group)
            return out
        dist.all_reduce(x, group=self.group)
        return x[self.rank * n : (self.rank + 1) * n].clone()


class TensorSequenceParallel:
    """Sequence parallelism inside a tensor-parallel group (Megatron style): the residual stream, the norms and everything
    else that is token-wise live on a 1 / size slice of the (padded) token stream; an all-gather in front of every
    column-parallel projection and a reduce-scatter behind every row-parallel one replace the all-reduce of plain tensor
    parallelism (same bytes on the wire, 1 / size of the activation memory between the blocks).

    Parity target: Megatron sequence parallelism as enabled by ``verl/workers/config/engine.py`` (``McoreEngineConfig``:
    on whenever tensor parallelism is) and ``verl/utils/megatron/sequence_parallel.py:29`` (padding)."""

    def __init__(self, group, rank: int, size: int):
        self.group, self.rank, self.size = group, int(rank), int(size)

    def local_rows(self, total: int) -> int:
        return (int(total) + self.size - 1) // self.size

    def slice(self, x: torch.Tensor) -> torch.Tensor:
        """Rows of this rank out of a full [T, ...] tensor (zero rows where the padded stream runs past T)."""
        n = self.local_rows(x.shape[0])
        lo = self.rank * n
        part = x[lo : lo + n]
        if part.shape[0] == n:
            return part.contiguous()
        out = torch.zeros(n, *x.shape[1:], dtype=x.dtype, device=x.device)
        out[: part.shape[0]] = part
        return out

    def gather(self, x_local: torch.Tensor, total: int) -> torch.Tensor:
        import torch.distributed as dist

        n = x_local.shape[0]
        full = torch.empty(n * self.size, *x_local.shape[1:], dtype=x_local.dtype, device=x_local.device)
        if x_local.is_cuda:
            dist.all_gather_into_tensor(full, x_local.contiguous(), group=self.group)
        else:
            dist.all_gather(list(full.split(n)), x_local.contiguous(), group=self.group)
        return full[:total]

    def scatter_sum(self, x_full: torch.Tensor) -> torch.Tensor:
        """Sum of every rank's [T, H] over the group, of which this rank keeps its rows."""
        import torch.distributed as dist

        T = x_full.shape[0]
        n = self.local_rows(T)
        if n * self.size != T:
            pad = torch.zeros(n * self.size - T, *x_full.shape[1:], dtype=x_full.dtype, device=x_full.device)
            x_full = torch.cat([x_full, pad])
        if x_full.is_cuda:
            out = torch.empty(n, *x_full.shape[1:], dtype=x_full.dtype, device=x_full.device)
            dist.reduce_scatter_tensor(out, x_full.contiguous(), group=self.group)
            return out
        x_full = x_full.contiguous().clone()
        dist.all_reduce(x_full, group=self.group)  # gloo has no reduce-scatter
        return x_full[self.rank * n : (self.rank + 1) * n].contiguous()


class ExpertParallelGroup:
    """Expert parallelism for training: ``size`` data-parallel ranks (each with its own tokens) store ``E / size`` experts
    each. A layer sends every routed token copy to the owner of its expert, runs the owner's experts, and sends the
    results back along the same path; the backward pass retraces it (the gradient of an exchange is the reverse
    exchange). Expert parameters therefore receive gradient contributions from the tokens of all ranks and are never
    reduced over the data-parallel group.

    Parity target: Megatron's token dispatcher used through ``verl/workers/engine/megatron/transformer_impl.py``
    (``expert_model_parallel_size``) and ``verl/models/mcore/model_forward.py``."""

    def __init__(self, group, rank: int, size: int):
        self.group, self.rank, self.size = group, int(rank), int(size)
        self._peer = None  # PeerAllToAll, created at the first exchange on GPUs with peer-mapped memory

    def _peer_exchange(self, x: torch.Tensor):
        """The peer-memory row exchange for this group, or None (CPU, no peer-mapped memory, VERL_B200_PEER_EP=0): the
        collective formulation is used then. Every rank of the group takes the same branch."""
        if self._peer is None:
            import os

            self._peer = False
            if x.is_cuda and self.size > 1 and os.environ.get("VERL_B200_PEER_EP", "1") != "0":
                from ..parallel.symmetric import PeerAllToAll, symmetric_available

                if symmetric_available():
                    try:
                        self._peer = PeerAllToAll(x.device, self.group)
                    except Exception:
                        self._peer = False
        return self._peer or None

    def gather_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """``counts`` [size, E_local] (copies this rank sends to each (owner, local expert)) of every rank:
        [source rank, owner, E_local], the same tensor on all ranks."""
        import torch.distributed as dist

        send = counts.contiguous()
        out = torch.empty(self.size, *send.shape, dtype=send.dtype, device=send.device)
        if send.is_cuda:
            dist.all_gather_into_tensor(out, send, group=self.group)
        else:
            dist.all_gather(list(out.unbind(0)), send, group=self.group)
        return out

    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """``counts`` [size, E_local]: copies this rank sends to each (owner, local expert). Returns the same matrix seen
        from the receiving side: row s = copies arriving from rank s per local expert."""
        import torch.distributed as dist

        send = counts.contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv

    def exchange_rows(self, x: torch.Tensor, in_splits: list, out_splits: list, rows: Optional[list] = None) -> torch.Tensor:
        """Rows of ``x`` go to the ranks in blocks of ``in_splits``; returns the ``sum(out_splits)`` rows received.
        ``rows[s][d]`` (rows rank s sends to rank d in THIS exchange, known to all ranks) enables the peer-memory path: one
        copy kernel stores every block into its place of the receiver's buffer, no collective."""
        import torch.distributed as dist

        if rows is not None and x.dim() == 2 and (x.shape[1] * x.element_size()) % 16 == 0:
            peer = self._peer_exchange(x)
            if peer is not None:
                return peer.exchange_rows(x.contiguous(), rows)
        out = torch.empty(sum(out_splits), *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=self.group)
        return out


class RouterReplay:
    """Expert choices of a token stream, per mixture-of-experts layer. ``record``: every router writes the experts it picked
    (``store[layer]`` = [T, k]); ``replay``: every router takes its experts from the store and only recomputes their
    weights from its own logits. Replaying the routing that produced the behaviour log-probs keeps the policy-gradient
    ratio free of routing flips between the two passes.

    Parity target: ``verl/utils/megatron/router_replay_utils.py`` and ``router_replay_patch.py`` (modes R2 / R3)."""

    def __init__(self, mode: str, store: Optional[dict] = None):
        assert mode in ("record", "replay")
        self.mode, self.store = mode, ({} if store is None else store)

    @classmethod
    def from_tokens(cls, routed: torch.Tensor, moe_layers: list) -> "RouterReplay":
        """``routed`` [T, n_moe_layers, k] -> replay object."""
        return cls("replay", {l: routed[:, j].contiguous() for j, l in enumerate(moe_layers)})

    def stacked(self, moe_layers: list) -> torch.Tensor:
        return torch.stack([self.store[l] for l in moe_layers], dim=1)


class DecoderModel:
    def __init__(self, cfg: ModelConfig, params: FlatParams, recompute: str = "none", max_positions: int = 0,
                 pre_layer_hook: Optional[Callable[[int, str], None]] = None,
                 post_layer_backward_hook: Optional[Callable[[int], None]] = None):
        assert recompute in ("none", "full", "auto")
        assert not cfg.is_generic, (f"model_type={cfg.model_type!r} has no hand-scheduled decoder: it runs through "
                                    f"verl_b200.models.generic (training engine and its cache-based rollout)")
        self.keep_layers_fn: Optional[Callable[[int], int]] = None
        self.tp: Optional[TensorParallelShard] = None  # set by the rollout engine; forward-only
        self.fp8_weights: Optional[dict] = None         # data_ptr of a bf16 weight -> (e4m3 copy, block scales)
        self.offloader = None                           # ActivationOffloader: inputs of recomputed layers live on the host
        self.etp_sum = None                             # all-reduce over the tensor-parallel group (experts cut over it)
        self.chunk = None                               # (lo, hi, first, last): the model chunk the next pass runs (virtual stages)
        # tensor-parallel training (this model is one shard: 1/tp of heads and MLP width): ``reduce(x)`` must sum x over the
        # tensor-parallel group in place. Forward: after the row-parallel o_proj / down_proj. Backward: on the input
        # gradients of the column-parallel qkv_proj / gate_up_proj.
        self.tp_reduce: Optional[Callable[[torch.Tensor], torch.Tensor]] = None
        # tensor-parallel training on GPUs: ``tp_linear_sum(x, w, b_mn)`` = (x @ w^T, or x @ w with b_mn) summed over the
        # tensor-parallel group by ONE kernel (GEMM with the all-reduce in its epilogue over peer memory); replaces the
        # GEMM + collective pairs behind the row-parallel projections and in the input gradients of the column-parallel ones
        self.tp_linear_sum: Optional[Callable[..., torch.Tensor]] = None
        self.stats_hook: Optional[Callable[[str, torch.Tensor], None]] = None  # called with (name, tensor) per layer output
        self.vocab_parallel = None                          # (group, first vocabulary row) of a vocabulary-parallel LM head
        self.mlp_tile_tokens = 0                            # > 0: sequence-tiled dense MLP (tokens per tile)
        self.router_replay: Optional[RouterReplay] = None   # record / replay the experts every router picks
        self._layer_idx = 0
        self.tsp: Optional[TensorSequenceParallel] = None   # token-sliced residual stream inside a tensor-parallel group
        self.ep: Optional[ExpertParallelGroup] = None       # expert parallelism (this model stores E / size experts)
        self.sp: Optional[UlyssesSequenceParallel] = None  # sequence parallelism (token-wise layers on a slice of the stream)
        self.cfg = cfg
        self.params = params
        self.recompute = recompute
        self.pre_layer_hook = pre_layer_hook
        self.post_layer_backward_hook = post_layer_backward_hook
        self.kv_hook: Optional[Callable[[int, torch.Tensor, torch.Tensor], None]] = None  # prefill: receives rotated K, V
        self.prefix_kv: Optional[Callable[[int], tuple]] = None  # prefill: (cached K, cached V, cached length per sequence) of a layer
        self.device = params.flat.device
        self._rope_len = 0
        self._cos = self._sin = None
        self._ensure_rope(max_positions or min(cfg.max_position_embeddings, 8192))
        self._anchor = torch.zeros((), device=self.device, requires_grad=True)

    # ------------------------------------------------------------------------------------ helpers
    def _ensure_rope(self, n: int) -> None:
        if n > self._rope_len:
            self._rope_len = int(2 ** math.ceil(math.log2(max(n, 16))))
            self._cos, self._sin = F.rope_table(self._rope_len, self.cfg.head_dim, self.cfg.rope_theta, self.device, self.cfg.rope_scaling,
                                                 self.cfg.max_position_embeddings)

    def _wgrad(self, w: torch.Tensor, dy: torch.Tensor, x: torch.Tensor) -> None:
        lora = getattr(w, "lora", None)
        if lora is not None:
            # the weight in use is W0 + s * B A (merged): its own gradient is never formed; the adapter gradients are
            #   dB += s * dy^T (x A^T)   [out, r]        dA += s * (dy B)^T x   [r, in]
            A, B, scale = lora
            if getattr(A, "main_grad", None) is None:
                return
            u = F.gemm(x, A)
            F.gemm(dy, u * scale, out=B.main_grad, a_mn=True, b_mn=True, out_f32=True, accumulate=True)
            t = F.gemm(dy, B, b_mn=True)
            F.gemm(t * scale, x, out=A.main_grad, a_mn=True, b_mn=True, out_f32=True, accumulate=True)
            return
        mg = getattr(w, "main_grad", None)
        if mg is None:
            return
        F.gemm(dy, x, out=mg, a_mn=True, b_mn=True, out_f32=True, accumulate=True)

    @staticmethod
    def _cu_cpu(batch: PackedBatch) -> torch.Tensor:
        if batch.cu_seqlens_cpu is None:
            batch.cu_seqlens_cpu = batch.cu_seqlens.cpu()
        return batch.cu_seqlens_cpu

    # ------------------------------------------------------------------------------------ attention block
    def _attn_fwd(self, W, h1, batch: PackedBatch, S: Optional[dict], layer_idx: int = -1):
        cfg = self.cfg
        T = h1.shape[0]
        nh, nkv, hd, Q, KV = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.q_size, cfg.kv_size
        if self.tp is not None:
            assert S is None, "tensor-parallel shards are forward-only"
            qkv = self.qkv_tp(W, h1)
            nh, nkv, Q, KV = nh // self.tp.size, nkv // self.tp.size, Q // self.tp.size, KV // self.tp.size
        else:
            qkv = self._lin(W, "self_attn.qkv_proj.weight", h1, S)
        q = qkv[:, :Q].view(T, nh, hd)
        k = qkv[:, Q : Q + KV].view(T, nkv, hd)
        v = qkv[:, Q + KV :].view(T, nkv, hd)
        if cfg.qk_norm:
            qp, kp = q.reshape(T * nh, hd).contiguous(), k.reshape(T * nkv, hd).contiguous()
            qn, _, rq = F.rms_norm(qp, W["self_attn.q_norm.weight"], cfg.rms_norm_eps)
            kn, _, rk = F.rms_norm(kp, W["self_attn.k_norm.weight"], cfg.rms_norm_eps)
            q.copy_(qn.view(T, nh, hd))
            k.copy_(kn.view(T, nkv, hd))
            if S is not None:
                S.update(q_pre=qp, k_pre=kp, rstd_q=rq, rstd_k=rk)
        pos = batch.positions if self.sp is None else batch.positions[self.sp.local_rows(batch.num_tokens, batch.positions.device)]
        F.apply_rope_(q, pos, self._cos, self._sin)
        F.apply_rope_(k, pos, self._cos, self._sin)
        if self.kv_hook is not None:
            self.kv_hook(layer_idx, k, v)
        native_ok = q.is_cuda and F._ATTN_IMPL["fwd"] is not None and hd in (64, 128)
        cu = batch.cu_seqlens if native_ok else self._cu_cpu(batch)
        if isinstance(self.sp, ContextParallel):
            assert batch.expand_index is None, "context parallelism and shared-prefix packing are exclusive"
            kf, vf = self.sp.gather_tokens(k), self.sp.gather_tokens(v)
            spans, cu_cpu, qc, row = self.sp.chunks(batch.num_tokens), self._cu_cpu(batch), q.contiguous(), 0
            parts = []
            for lo, hi in spans:         # one or two contiguous runs of stream positions
                parts.append(F.attention_query_slice(qc[row : row + hi - lo], kf, vf, cu_cpu, lo))
                row += hi - lo
            attn2, lse = torch.cat(parts, 0).reshape(T, Q), None
            if S is not None:
                S.update(qkv=qkv, attn=attn2, lse=None, cp_full=(kf, vf, spans))
        elif self.sp is not None:
            assert batch.expand_index is None, "sequence parallelism and shared-prefix packing are exclusive"
            qf, kf, vf = self.sp.seq_to_heads(q.contiguous()), self.sp.seq_to_heads(k.contiguous()), self.sp.seq_to_heads(v.contiguous())
            attn_f, lse = F.attention_varlen(qf, kf, vf, cu, batch.max_seqlen)
            attn2 = self.sp.heads_to_seq(attn_f.contiguous()).reshape(T, Q)
            if S is not None:
                S.update(qkv=qkv, attn=attn2, lse=lse, sp_full=(qf, kf, vf, attn_f))
        elif batch.expand_index is not None:
            ex = batch.expand_index
            qe, ke, ve = q.index_select(0, ex), k.index_select(0, ex), v.index_select(0, ex)
            attn_e, lse = F.attention_varlen(qe, ke, ve, cu, batch.max_seqlen)
            attn2 = attn_e.index_select(0, batch.collapse_index).reshape(T, Q)
            if S is not None:
                S.update(qkv=qkv, attn=attn2, lse=lse, attn_e=attn_e)
        elif self.prefix_kv is not None:
            # prefill behind a prefix-cache hit: the batch holds the uncached tail of every prompt
            assert S is None, "cached prefixes are a forward-only (rollout) feature"
            kp, vp, plens = self.prefix_kv(layer_idx)
            attn2, lse = F.attention_with_prefix(q.contiguous(), k.contiguous(), v.contiguous(), kp, vp, self._cu_cpu(batch), plens).reshape(T, Q), None
        else:
            attn, lse = F.attention_varlen(q, k, v, cu, batch.max_seqlen)
            attn2 = attn.reshape(T, Q)
            if S is not None:
                S.update(qkv=qkv, attn=attn2, lse=lse)
        if self.tp is not None:
            return self.tp.row_linear(attn2, W["self_attn.o_proj.weight"][:, self.tp.rows(cfg.q_size)], None)
        if self.tp_linear_sum is not None and W.get("self_attn.o_proj.bias") is None:
            return self.tp_linear_sum(attn2, W["self_attn.o_proj.weight"], False)
        o = self._lin(W, "self_attn.o_proj.weight", attn2, S)
        return self.tp_reduce(o) if self.tp_reduce is not None else o

    def qkv_tp(self, W, h1: torch.Tensor) -> torch.Tensor:
        """[T, (Q + 2 KV) / size]: this rank's q | k | v columns."""
        cfg, tp = self.cfg, self.tp
        Q, KV = cfg.q_size, cfg.kv_size
        Ql, KVl = Q // tp.size, KV // tp.size
        w, b = W["self_attn.qkv_proj.weight"], W.get("self_attn.qkv_proj.bias")
        return F.gemm_row_ranges(h1, w, b, [(tp.rank * Ql, Ql), (Q + tp.rank * KVl, KVl), (Q + KV + tp.rank * KVl, KVl)])

    def mlp_tp(self, W, h2: torch.Tensor) -> torch.Tensor:
        cfg, tp = self.cfg, self.tp
        I = cfg.intermediate_size
        Il = I // tp.size
        w = W["mlp.gate_up_proj.weight"]
        gu = F.gemm_row_ranges(h2, w, W.get("mlp.gate_up_proj.bias"), [(tp.rank * Il, Il), (I + tp.rank * Il, Il)])
        return tp.row_linear(F.swiglu(gu), W["mlp.down_proj.weight"][:, tp.rows(I)], None)

    def _attn_bwd(self, W, g_o, h1, batch: PackedBatch, S: dict):
        cfg = self.cfg
        T = g_o.shape[0]
        nh, nkv, hd, Q, KV = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.q_size, cfg.kv_size
        qkv, attn2, lse = S["qkv"], S["attn"], S["lse"]
        g_attn = F.gemm(g_o, W["self_attn.o_proj.weight"], b_mn=True)
        self._wgrad(W["self_attn.o_proj.weight"], g_o, attn2)
        q = qkv[:, :Q].view(T, nh, hd)
        k = qkv[:, Q : Q + KV].view(T, nkv, hd)
        v = qkv[:, Q + KV :].view(T, nkv, hd)
        cu = batch.cu_seqlens if q.is_cuda and F._ATTN_IMPL["bwd"] is not None and lse is not None else self._cu_cpu(batch)
        if isinstance(self.sp, ContextParallel):
            kf, vf, spans = S["cp_full"]
            ga, qc, cu_cpu, row = g_attn.view(T, nh, hd), q.contiguous(), self._cu_cpu(batch), 0
            dqs, dk_f, dv_f = [], 0, 0
            for lo, hi in spans:
                a, b, c = F.attention_query_slice_bwd(ga[row : row + hi - lo], qc[row : row + hi - lo], kf, vf, cu_cpu, lo)
                dqs.append(a)
                dk_f, dv_f = dk_f + b, dv_f + c
                row += hi - lo
            dq = torch.cat(dqs, 0)
            # every rank's queries contribute to the gradients of all the keys / values they saw
            dk, dv = self.sp.scatter_sum(dk_f.float()).to(q.dtype), self.sp.scatter_sum(dv_f.float()).to(q.dtype)
        elif self.sp is not None:
            qf, kf, vf, attn_f = S["sp_full"]
            g_f = self.sp.seq_to_heads(g_attn.view(T, nh, hd).contiguous())
            dq_f, dk_f, dv_f = F.attention_varlen_bwd(g_f, qf, kf, vf, attn_f, lse, cu, batch.max_seqlen)
            dq, dk, dv = (self.sp.heads_to_seq(t.contiguous()) for t in (dq_f, dk_f, dv_f))
        elif batch.expand_index is not None:
            # gradients of the per-member layout: only the representative copies carry an output gradient; the prompt's
            # key/value gradients are the sums over all members of its group
            ex, col = batch.expand_index, batch.collapse_index
            attn_e = S["attn_e"]
            g_e = torch.zeros_like(attn_e)
            g_e.index_copy_(0, col, g_attn.view(T, nh, hd))
            dq_e, dk_e, dv_e = F.attention_varlen_bwd(g_e, q.index_select(0, ex), k.index_select(0, ex), v.index_select(0, ex),
                                                      attn_e, lse, cu, batch.max_seqlen)
            dq = torch.zeros(T, nh, hd, dtype=torch.float32, device=q.device).index_add_(0, ex, dq_e.float()).to(q.dtype)
            dk = torch.zeros(T, nkv, hd, dtype=torch.float32, device=q.device).index_add_(0, ex, dk_e.float()).to(q.dtype)
            dv = torch.zeros(T, nkv, hd, dtype=torch.float32, device=q.device).index_add_(0, ex, dv_e.float()).to(q.dtype)
        else:
            dq, dk, dv = F.attention_varlen_bwd(g_attn.view(T, nh, hd), q, k, v, attn2.view(T, nh, hd), lse, cu,
                                                batch.max_seqlen)
        g_qkv = torch.empty_like(qkv)
        gq = g_qkv[:, :Q].view(T, nh, hd)
        gk = g_qkv[:, Q : Q + KV].view(T, nkv, hd)
        gq.copy_(dq)
        gk.copy_(dk)
        g_qkv[:, Q + KV :].view(T, nkv, hd).copy_(dv)
        pos = batch.positions if self.sp is None else batch.positions[self.sp.local_rows(batch.num_tokens, batch.positions.device)]
        F.apply_rope_(gq, pos, self._cos, self._sin, backward=True)
        F.apply_rope_(gk, pos, self._cos, self._sin, backward=True)
        if cfg.qk_norm:
            wq, wk = W["self_attn.q_norm.weight"], W["self_attn.k_norm.weight"]
            dqp = F.rms_norm_bwd(gq.reshape(T * nh, hd).contiguous(), S["q_pre"], wq, S["rstd_q"], None,
                                 self._grad_of(wq), True)
            dkp = F.rms_norm_bwd(gk.reshape(T * nkv, hd).contiguous(), S["k_pre"], wk, S["rstd_k"], None,
                                 self._grad_of(wk), True)
            gq.copy_(dqp.view(T, nh, hd))
            gk.copy_(dkp.view(T, nkv, hd))
        if self.tp_linear_sum is not None:
            g_h1 = self.tp_linear_sum(g_qkv, W["self_attn.qkv_proj.weight"], True)
        else:
            g_h1 = F.gemm(g_qkv, W["self_attn.qkv_proj.weight"], b_mn=True)
            if self.tp_reduce is not None:
                g_h1 = self.tp_reduce(g_h1)
        self._wgrad(W["self_attn.qkv_proj.weight"], g_qkv, h1)
        b = W.get("self_attn.qkv_proj.bias")
        if b is not None and getattr(b, "main_grad", None) is not None:
            b.main_grad.add_(g_qkv.float().sum(0))
        return g_h1

    def _lin(self, W, name: str, x: torch.Tensor, S: Optional[dict] = None) -> torch.Tensor:
        """``x @ W[name]^T (+ bias)``; forward-only calls use the fp8 copy of the weight when one is installed."""
        w = W[name]
        b = W.get(name[: -len("weight")] + "bias")
        if S is None and self.fp8_weights is not None:
            q = self.fp8_weights.get(w.data_ptr())
            if q is not None:
                return F.linear_fp8(x, q[0], q[1], b)
        return F.gemm(x, w, b)

    def quantize_linear_weights_fp8(self) -> int:
        """(Re)build e4m3 copies with 1x128 block scales of every dense projection (rollout precision of the MoE
        recipe; call after each weight update). Returns the bytes held by the copies."""
        self.fp8_weights = {}
        total = 0
        names = ("self_attn.qkv_proj.weight", "self_attn.o_proj.weight", "mlp.gate_up_proj.weight", "mlp.down_proj.weight")
        for i in range(self.cfg.num_hidden_layers):
            W = self.params.layer(i)
            for n in names:
                if n in W and W[n].dim() == 2 and W[n].shape[1] % 128 == 0:
                    q, sc = F.fp8_quantize_1x128(W[n])
                    self.fp8_weights[W[n].data_ptr()] = (q, sc)
                    total += q.numel() + sc.numel() * 4
            for n in ("mlp.experts.gate_up_proj", "mlp.experts.down_proj"):  # stacked expert matrices [E, N, K] -> [E * N, K]
                if n in W and W[n].shape[-1] % 128 == 0:
                    q, sc = F.fp8_quantize_1x128(W[n].reshape(-1, W[n].shape[-1]))
                    self.fp8_weights[W[n].data_ptr()] = (q, sc)
                    total += q.numel() + sc.numel() * 4
        return total

    def _grad_of(self, w: torch.Tensor) -> torch.Tensor:
        mg = getattr(w, "main_grad", None)
        return mg if mg is not None else torch.zeros_like(w, dtype=torch.float32)

    # ------------------------------------------------------------------------------------ MLP blocks
    def _mlp_fwd(self, W, h2, S: Optional[dict]):
        if self.cfg.is_moe:
            return self._moe_fwd(W, h2, S)
        if self.tp is not None:
            assert S is None, "tensor-parallel shards are forward-only"
            return self.mlp_tp(W, h2)
        tile = self.mlp_tile_tokens
        if tile and h2.shape[0] > tile and self.fp8_weights is None:
            # sequence-tiled MLP: the [tokens, 2 * intermediate] activation exists for one tile at a time and is recomputed
            # tile by tile in the backward pass (nothing of it is saved)
            d = torch.empty(h2.shape[0], W["mlp.down_proj.weight"].shape[0], dtype=h2.dtype, device=h2.device)
            for s0 in range(0, h2.shape[0], tile):
                gu = F.gemm(h2[s0 : s0 + tile], W["mlp.gate_up_proj.weight"])
                F.gemm(F.swiglu(gu), W["mlp.down_proj.weight"], out=d[s0 : s0 + tile])
            if S is not None:
                S["gu"] = None
            return self.tp_reduce(d) if self.tp_reduce is not None else d
        if S is None and W.get("mlp.gate_up_proj.bias") is None and self.fp8_weights is None:
            # forward-only passes and the first pass of a recomputed layer: the activation runs in the epilogue of the
            # up-projection and the pre-activation is never written. (A layer that keeps its pre-activation runs the two
            # kernels: the epilogue that writes both measured slower than GEMM + activation, 4.36 vs 3.60 ms at 16k tokens.)
            act, gu = F.gemm_swiglu(h2, W["mlp.gate_up_proj.weight"], want_gate_up=False)
        else:
            gu = self._lin(W, "mlp.gate_up_proj.weight", h2, S)
            act = F.swiglu(gu)
        if S is not None:
            S["gu"] = gu
        if self.tp_linear_sum is not None and W.get("mlp.down_proj.bias") is None:
            return self.tp_linear_sum(act, W["mlp.down_proj.weight"], False)
        d = self._lin(W, "mlp.down_proj.weight", act, S)
        return self.tp_reduce(d) if self.tp_reduce is not None else d

    def _mlp_bwd(self, W, g_d, h2, S: dict):
        if self.cfg.is_moe:
            return self._moe_bwd(W, g_d, h2, S)
        gu = S["gu"]
        if gu is None:  # sequence-tiled: recompute gate_up per tile, accumulate the weight gradients tile by tile
            tile = self.mlp_tile_tokens
            g_h2 = torch.empty_like(h2)
            for s0 in range(0, h2.shape[0], tile):
                sl = slice(s0, s0 + tile)
                gu_t = F.gemm(h2[sl], W["mlp.gate_up_proj.weight"])
                g_act = F.gemm(g_d[sl], W["mlp.down_proj.weight"], b_mn=True)
                self._wgrad(W["mlp.down_proj.weight"], g_d[sl], F.swiglu(gu_t))
                g_gu = F.swiglu_bwd(g_act, gu_t)
                F.gemm(g_gu, W["mlp.gate_up_proj.weight"], b_mn=True, out=g_h2[sl])
                self._wgrad(W["mlp.gate_up_proj.weight"], g_gu, h2[sl])
            return self.tp_reduce(g_h2) if self.tp_reduce is not None else g_h2
        act = F.swiglu(gu)
        g_act = F.gemm(g_d, W["mlp.down_proj.weight"], b_mn=True)
        self._wgrad(W["mlp.down_proj.weight"], g_d, act)
        g_gu = F.swiglu_bwd(g_act, gu)
        if self.tp_linear_sum is not None:
            g_h2 = self.tp_linear_sum(g_gu, W["mlp.gate_up_proj.weight"], True)
        else:
            g_h2 = F.gemm(g_gu, W["mlp.gate_up_proj.weight"], b_mn=True)
            if self.tp_reduce is not None:
                g_h2 = self.tp_reduce(g_h2)
        self._wgrad(W["mlp.gate_up_proj.weight"], g_gu, h2)
        return g_h2

    # -- mixture of experts: softmax router, top-k, tokens grouped by expert ------------------------
    def _route(self, logits: torch.Tensor, idx: Optional[torch.Tensor] = None):
        """Softmax over experts, top-k, optional renormalisation. With ``idx`` given the selection is taken as is and
        only the weights are (differentiably) recomputed, so that forward and backward agree on exact ties."""
        cfg = self.cfg
        probs = torch.softmax(logits.float(), dim=-1)
        if idx is None:
            if logits.is_cuda and logits.dtype == torch.bfloat16 and cfg.num_experts <= 1024:
                idx = F._ops().moe_route_topk(logits, cfg.num_experts_per_tok, bool(cfg.norm_topk_prob))[1].long()
            else:
                idx = torch.topk(probs, cfg.num_experts_per_tok, dim=-1).indices
        w = probs.gather(-1, idx.long())
        if cfg.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        return w, idx

    def _routing(self, logits: torch.Tensor):
        """(weights fp32 [T, k], experts int64 [T, k], per-expert counts) with record / replay of the choice."""
        cfg, rr = self.cfg, self.router_replay
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        if rr is not None and rr.mode == "replay":
            w, idx = self._route(logits, idx=rr.store[self._layer_idx].to(logits.device).long())
            return w, idx, torch.bincount(idx.reshape(-1), minlength=E).int()
        if logits.is_cuda and logits.dtype == torch.bfloat16 and E <= 1024:
            w, idx, counts = F._ops().moe_route_topk(logits, k, bool(cfg.norm_topk_prob))
            idx = idx.long()
        else:
            w, idx = self._route(logits)
            counts = torch.bincount(idx.reshape(-1), minlength=E).int()
        if rr is not None:
            rr.store[self._layer_idx] = idx.detach().clone()
        return w, idx, counts

    # -- device path: router, expert-grouped layout and grouped tcgen05 GEMMs; no host synchronisation anywhere --------
    @staticmethod
    def _moe_plan(idx: torch.Tensor, counts: torch.Tensor, T: int, k: int, E: int) -> dict:
        """Expert-grouped row layout in which every expert's rows start at a multiple of 128 (padding rows are zero).
        ``slot[t, j]`` = row of the j-th expert copy of token t; ``src[row]`` = source token or -1 for padding."""
        dev = idx.device
        flat_e = idx.reshape(-1).long()
        order = torch.argsort(flat_e, stable=True)
        cnt = counts.long()
        seg = torch.zeros(E + 1, dtype=torch.int64, device=dev)
        seg[1:] = ((cnt + 127) // 128 * 128).cumsum(0)
        first = cnt.cumsum(0) - cnt
        e_sorted = flat_e[order]
        slot_sorted = seg[e_sorted] + (torch.arange(T * k, device=dev) - first[e_sorted])
        cap = ((T * k + 127) // 128 + E) * 128  # upper bound of the padded row count, known without reading `counts`
        slot = torch.empty(T * k, dtype=torch.int32, device=dev)
        slot[order] = slot_sorted.int()
        src = torch.full((cap,), -1, dtype=torch.int32, device=dev)
        src[slot_sorted] = torch.div(order, k, rounding_mode="floor").int()
        tiles = torch.arange(cap // 128, device=dev) * 128
        tile_expert = torch.searchsorted(seg[1:].contiguous(), tiles, right=True).clamp_(max=E - 1).int()
        return dict(slot=slot.view(T, k), src=src, seg=seg.int(), tile_expert=tile_expert,
                    num_mtiles=(seg[E:] // 128).int(), cap=cap)

    def _moe_fwd_native(self, W, h2, S: Optional[dict]):
        cfg = self.cfg
        ops = F._ops()
        T, H = h2.shape
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        logits = F.gemm(h2, W["mlp.gate.weight"])
        w, idx, counts = self._routing(logits)
        w = w.float().contiguous()
        plan = self._moe_plan(idx, counts, T, k, E)
        xp = ops.moe_gather_rows(h2, plan["src"], None)
        Wgu, Wd = W["mlp.experts.gate_up_proj"], W["mlp.experts.down_proj"]
        q_gu = self.fp8_weights.get(Wgu.data_ptr()) if (S is None and self.fp8_weights is not None) else None
        q_d = self.fp8_weights.get(Wd.data_ptr()) if (S is None and self.fp8_weights is not None) else None
        if q_gu is not None and q_d is not None:  # forward-only with fp8 expert copies installed (rollout precision)
            gu = F.linear_fp8_grouped(xp, q_gu[0], q_gu[1], Wgu.shape[1], plan["tile_expert"], plan["num_mtiles"])
            y = F.linear_fp8_grouped(F.swiglu(gu), q_d[0], q_d[1], Wd.shape[1], plan["tile_expert"], plan["num_mtiles"])
        else:
            gu = ops.gemm_grouped_rows(xp, Wgu, False, plan["tile_expert"], plan["num_mtiles"])
            y = ops.gemm_grouped_rows(F.swiglu(gu), Wd, False, plan["tile_expert"], plan["num_mtiles"])
        out = ops.moe_combine(y, plan["slot"], w)
        if S is not None:
            S.update(moe=dict(native=True, logits=logits, w=w, idx=idx, plan=plan, gu=gu, y=y))
        return out

    def _moe_bwd_native(self, W, g_d, h2, S: dict):
        cfg = self.cfg
        ops = F._ops()
        M = S["moe"]
        plan, w, gu, y = M["plan"], M["w"], M["gu"], M["y"]
        T, H = h2.shape
        k = cfg.num_experts_per_tok
        g_d = g_d.contiguous()
        g_w = self._etp_sum(ops.moe_combine_bwd_w(g_d, y, plan["slot"]))   # y holds this rank's part of every expert output
        w_rows = torch.zeros(plan["cap"], dtype=torch.float32, device=h2.device)
        w_rows[plan["slot"].reshape(-1).long()] = w.reshape(-1)
        g_y = ops.moe_gather_rows(g_d, plan["src"], w_rows)
        Wgu, Wd = W["mlp.experts.gate_up_proj"], W["mlp.experts.down_proj"]
        act = F.swiglu(gu)
        g_act = ops.gemm_grouped_rows(g_y, Wd, True, plan["tile_expert"], plan["num_mtiles"])
        if getattr(Wd, "main_grad", None) is not None:
            ops.gemm_grouped_wgrad_(g_y, act, Wd.main_grad, plan["seg"], True)
        g_gu = F.swiglu_bwd(g_act, gu)
        g_xp = ops.gemm_grouped_rows(g_gu, Wgu, True, plan["tile_expert"], plan["num_mtiles"])
        if getattr(Wgu, "main_grad", None) is not None:
            xp = ops.moe_gather_rows(h2, plan["src"], None)
            ops.gemm_grouped_wgrad_(g_gu, xp, Wgu.main_grad, plan["seg"], True)
        g_h2 = self._etp_sum(ops.moe_combine(g_xp, plan["slot"], None).float())
        with torch.enable_grad():
            lg = M["logits"].detach().float().requires_grad_(True)
            wr, _ = self._route(lg, idx=M["idx"])
            (g_logits,) = torch.autograd.grad(wr, lg, g_w)
        g_logits = g_logits.to(h2.dtype)
        g_h2 += F.gemm(g_logits, W["mlp.gate.weight"], b_mn=True).float()
        self._wgrad(W["mlp.gate.weight"], g_logits, h2)
        return g_h2.to(h2.dtype)

    def _moe_native_ok(self, h2) -> bool:
        c = self.cfg
        return (h2.is_cuda and h2.dtype == torch.bfloat16 and c.num_experts <= 1024 and c.hidden_size % 64 == 0
                and c.moe_intermediate_size % 64 == 0 and os.environ.get("VERL_B200_MOE_NATIVE", "1") != "0")

    # -- expert-parallel path: token copies travel to the owner of their expert and back -------------------------------
    def _experts_apply(self, W, x, counts: list, S: Optional[dict]):
        """Rows of ``x`` sorted by local expert (``counts`` rows each) through gate_up -> SwiGLU -> down."""
        Wgu, Wd = W["mlp.experts.gate_up_proj"], W["mlp.experts.down_proj"]
        gu = torch.empty(x.shape[0], Wgu.shape[1], dtype=x.dtype, device=x.device)
        y = torch.empty(x.shape[0], Wd.shape[1], dtype=x.dtype, device=x.device)
        s0 = 0
        for e, n in enumerate(counts):
            if n:
                F.gemm(x[s0 : s0 + n], Wgu[e], out=gu[s0 : s0 + n])
                F.gemm(F.swiglu(gu[s0 : s0 + n]), Wd[e], out=y[s0 : s0 + n])
                s0 += n
        if S is not None:
            S["gu"] = gu
        return y

    def _experts_apply_bwd(self, W, g_y, x, gu, counts: list):
        Wgu, Wd = W["mlp.experts.gate_up_proj"], W["mlp.experts.down_proj"]
        g_x = torch.empty_like(x)
        s0 = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            sl = slice(s0, s0 + n)
            g_act = F.gemm(g_y[sl], Wd[e], b_mn=True)
            mg = getattr(Wd, "main_grad", None)
            if mg is not None:
                F.gemm(g_y[sl], F.swiglu(gu[sl]), out=mg[e], a_mn=True, b_mn=True, out_f32=True, accumulate=True)
            g_gu = F.swiglu_bwd(g_act, gu[sl])
            F.gemm(g_gu, Wgu[e], b_mn=True, out=g_x[sl])
            mg = getattr(Wgu, "main_grad", None)
            if mg is not None:
                F.gemm(g_gu, x[sl], out=mg[e], a_mn=True, b_mn=True, out_f32=True, accumulate=True)
            s0 += n
        return g_x

    def _moe_fwd_ep(self, W, h2, S: Optional[dict]):
        cfg, ep = self.cfg, self.ep
        T, H = h2.shape
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        El = E // ep.size
        logits = F.gemm(h2, W["mlp.gate.weight"])
        w, idx, counts = self._routing(logits)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)          # copies sorted by global expert = by (owner, local expert)
        tok = torch.div(order, k, rounding_mode="floor")
        send_counts = counts.long().view(ep.size, El)
        all_counts = ep.gather_counts(send_counts)          # [source rank, owner, local expert], the same on every rank
        recv_counts = all_counts[:, ep.rank]                 # [source rank, local expert]
        host = all_counts.cpu()                              # the one host read of the layer: every split size of the exchange
        both = torch.stack([host[ep.rank], host[:, ep.rank]])
        in_splits, out_splits = both[0].sum(1).tolist(), both[1].sum(1).tolist()
        rows_fwd = host.sum(-1).tolist()                     # rows_fwd[s][d]: token copies rank s sends to rank d
        rows_back = [list(r) for r in zip(*rows_fwd)]        # the way back: what d received from s returns to s
        x_recv = ep.exchange_rows(h2[tok], in_splits, out_splits, rows_fwd)
        # received rows are grouped by source rank, then local expert: regroup by local expert
        eid = torch.repeat_interleave(torch.arange(El, device=h2.device).repeat(ep.size), recv_counts.reshape(-1).to(h2.device))
        perm = torch.argsort(eid, stable=True)
        local_counts = both[1].sum(0).tolist()
        St = {} if S is not None else None
        x_sorted = x_recv[perm]
        y_sorted = self._experts_apply(W, x_sorted, local_counts, St)
        y_recv = torch.empty_like(y_sorted)
        y_recv[perm] = y_sorted
        y_send = ep.exchange_rows(y_recv, out_splits, in_splits, rows_back)  # back to the ranks of the tokens, in `order`
        wp = w.reshape(-1)[order].to(h2.dtype)
        out = torch.zeros(T, H, dtype=torch.float32, device=h2.device)
        out.index_add_(0, tok, (y_send * wp.unsqueeze(-1)).float())
        if S is not None:
            S.update(moe=dict(ep=True, logits=logits, idx=idx, order=order, tok=tok, wp=wp, y=y_send, perm=perm, x=x_sorted,
                              gu=St["gu"], counts=local_counts, in_splits=in_splits, out_splits=out_splits, rows_fwd=rows_fwd,
                              rows_back=rows_back))
        return out.to(h2.dtype)

    def _moe_bwd_ep(self, W, g_d, h2, S: dict):
        cfg, ep = self.cfg, self.ep
        M = S["moe"]
        order, tok, wp, perm = M["order"], M["tok"], M["wp"], M["perm"]
        k = cfg.num_experts_per_tok
        T, H = h2.shape
        g_dp = g_d[tok]
        g_wp = self._etp_sum((g_dp.float() * M["y"].float()).sum(-1))
        g_y_recv = ep.exchange_rows((g_dp * wp.unsqueeze(-1)).contiguous(), M["in_splits"], M["out_splits"], M.get("rows_fwd"))
        g_x_sorted = self._experts_apply_bwd(W, g_y_recv[perm].contiguous(), M["x"], M["gu"], M["counts"])
        g_x_recv = torch.empty_like(g_x_sorted)
        g_x_recv[perm] = g_x_sorted
        g_x_send = ep.exchange_rows(g_x_recv, M["out_splits"], M["in_splits"], M.get("rows_back"))
        g_h2 = torch.zeros(T, H, dtype=torch.float32, device=h2.device)
        g_h2.index_add_(0, tok, g_x_send.float())
        g_h2 = self._etp_sum(g_h2)  # the experts' part is a partial sum when their width is cut over the tensor-parallel group
        g_w = torch.empty(T * k, dtype=torch.float32, device=h2.device)
        g_w[order] = g_wp
        with torch.enable_grad():
            lg = M["logits"].detach().float().requires_grad_(True)
            wr, _ = self._route(lg, idx=M["idx"])
            (g_logits,) = torch.autograd.grad(wr, lg, g_w.view(T, k))
        g_logits = g_logits.to(h2.dtype)
        g_h2 += F.gemm(g_logits, W["mlp.gate.weight"], b_mn=True).float()
        self._wgrad(W["mlp.gate.weight"], g_logits, h2)
        return g_h2.to(h2.dtype)

    # -- shared expert (Qwen2-MoE): a dense SwiGLU MLP applied to every token, scaled by sigmoid(h . w_gate) -------------
    def _shared_expert_fwd(self, W, h2, S: Optional[dict]):
        gu = F.gemm(h2, W["mlp.shared_expert.gate_up_proj.weight"])
        y = F.gemm(F.swiglu(gu), W["mlp.shared_expert.down_proj.weight"])
        z = F.gemm(h2, W["mlp.shared_expert_gate.weight"])[:, 0].float()
        sg = torch.sigmoid(z)
        if S is not None:
            S["shared"] = dict(gu=gu, y=y, sg=sg)
        return (y.float() * sg.unsqueeze(-1)).to(h2.dtype)

    def _shared_expert_bwd(self, W, g_d, h2, S: dict):
        Sh = S["shared"]
        gu, y, sg = Sh["gu"], Sh["y"], Sh["sg"]
        Wgu, Wd, Wg = W["mlp.shared_expert.gate_up_proj.weight"], W["mlp.shared_expert.down_proj.weight"], W["mlp.shared_expert_gate.weight"]
        g_y = (g_d.float() * sg.unsqueeze(-1)).to(h2.dtype)
        g_z = self._etp_sum((g_d.float() * y.float()).sum(-1)) * sg * (1.0 - sg)
        g_act = F.gemm(g_y, Wd, b_mn=True)
        self._wgrad(Wd, g_y, F.swiglu(gu))
        g_gu = F.swiglu_bwd(g_act, gu)
        g_h2 = self._etp_sum(F.gemm(g_gu, Wgu, b_mn=True).float())
        self._wgrad(Wgu, g_gu, h2)
        dl = torch.zeros(h2.shape[0], Wg.shape[0], dtype=h2.dtype, device=h2.device)
        dl[:, 0] = g_z.to(h2.dtype)
        g_h2 += F.gemm(dl, Wg, b_mn=True).float()
        self._wgrad(Wg, dl, h2)
        return g_h2

    def _etp_sum(self, t: torch.Tensor) -> torch.Tensor:
        """Sum over the tensor-parallel group when the experts' intermediate width is cut over it (``etp_sum`` is set by the
        model-parallel engine for mixture-of-experts models with tp > 1), else the tensor itself."""
        return self.etp_sum(t) if self.etp_sum is not None else t

    def _moe_fwd(self, W, h2, S: Optional[dict]):
        out = self._moe_routed_fwd(W, h2, S)
        if self.cfg.shared_expert_intermediate_size:
            out = out + self._shared_expert_fwd(W, h2, S)
        return self._etp_sum(out.contiguous()) if self.etp_sum is not None else out

    def _moe_bwd(self, W, g_d, h2, S: dict):
        g_h2 = self._moe_routed_bwd(W, g_d, h2, S)
        if self.cfg.shared_expert_intermediate_size:
            g_h2 = (g_h2.float() + self._shared_expert_bwd(W, g_d.contiguous(), h2, S)).to(h2.dtype)
        return g_h2

    def _moe_routed_fwd(self, W, h2, S: Optional[dict]):
        if self.ep is not None:
            return self._moe_fwd_ep(W, h2, S)
        if self._moe_native_ok(h2):
            return self._moe_fwd_native(W, h2, S)
        cfg = self.cfg
        T, H = h2.shape
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        logits = F.gemm(h2, W["mlp.gate.weight"])
        w, idx, counts = self._routing(logits)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = torch.div(order, k, rounding_mode="floor")
        counts = counts.tolist()
        xp = h2[tok]
        Wgu, Wd = W["mlp.experts.gate_up_proj"], W["mlp.experts.down_proj"]
        gu = torch.empty(T * k, Wgu.shape[1], dtype=h2.dtype, device=h2.device)
        y = torch.empty(T * k, H, dtype=h2.dtype, device=h2.device)
        s0 = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            F.gemm(xp[s0 : s0 + n], Wgu[e], out=gu[s0 : s0 + n])
            F.gemm(F.swiglu(gu[s0 : s0 + n]), Wd[e], out=y[s0 : s0 + n])
            s0 += n
        wp = w.reshape(-1)[order].to(h2.dtype)
        out = torch.zeros(T, H, dtype=torch.float32, device=h2.device)
        out.index_add_(0, tok, (y * wp.unsqueeze(-1)).float())
        if S is not None:
            S.update(moe=dict(logits=logits, idx=idx, order=order, tok=tok, counts=counts, gu=gu, y=y, wp=wp))
        return out.to(h2.dtype)

    def _moe_routed_bwd(self, W, g_d, h2, S: dict):
        if S["moe"].get("ep"):
            return self._moe_bwd_ep(W, g_d, h2, S)
        if S["moe"].get("native"):
            return self._moe_bwd_native(W, g_d, h2, S)
        cfg = self.cfg
        M = S["moe"]
        order, tok, counts, gu, y, wp = M["order"], M["tok"], M["counts"], M["gu"], M["y"], M["wp"]
        k = cfg.num_experts_per_tok
        T, H = h2.shape
        g_dp = g_d[tok]
        g_wp = self._etp_sum((g_dp.float() * y.float()).sum(-1))  # d loss / d routing weight, permuted order
        g_y = (g_dp * wp.unsqueeze(-1)).contiguous()
        Wgu, Wd = W["mlp.experts.gate_up_proj"], W["mlp.experts.down_proj"]
        xp = h2[tok]
        g_xp = torch.empty_like(xp)
        s0 = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            sl = slice(s0, s0 + n)
            act = F.swiglu(gu[sl])
            g_act = F.gemm(g_y[sl], Wd[e], b_mn=True)
            mg = getattr(Wd, "main_grad", None)
            if mg is not None:
                F.gemm(g_y[sl], act, out=mg[e], a_mn=True, b_mn=True, out_f32=True, accumulate=True)
            g_gu = F.swiglu_bwd(g_act, gu[sl])
            F.gemm(g_gu, Wgu[e], b_mn=True, out=g_xp[sl])
            mg = getattr(Wgu, "main_grad", None)
            if mg is not None:
                F.gemm(g_gu, xp[sl], out=mg[e], a_mn=True, b_mn=True, out_f32=True, accumulate=True)
            s0 += n
        g_h2 = torch.zeros(T, H, dtype=torch.float32, device=h2.device)
        g_h2.index_add_(0, tok, g_xp.float())
        g_h2 = self._etp_sum(g_h2)  # the experts' part is a partial sum; the router's part below is whole on every rank
        # router: differentiate softmax/top-k/normalise on the small [T, E] problem with autograd
        g_w = torch.empty(T * k, dtype=torch.float32, device=h2.device)
        g_w[order] = g_wp
        with torch.enable_grad():
            lg = M["logits"].detach().float().requires_grad_(True)
            w, _ = self._route(lg, idx=M["idx"])
            (g_logits,) = torch.autograd.grad(w, lg, g_w.view(T, k))
        g_logits = g_logits.to(h2.dtype)
        g_h2 += F.gemm(g_logits, W["mlp.gate.weight"], b_mn=True).float()
        self._wgrad(W["mlp.gate.weight"], g_logits, h2)
        return g_h2.to(h2.dtype)

    # ------------------------------------------------------------------------------------ layer
    def _layer_fwd(self, i: int, a, r, batch: PackedBatch, S: Optional[dict]):
        if self.pre_layer_hook is not None:
            self.pre_layer_hook(i, "forward")
        W = self.params.layer(i)
        self._layer_idx = i
        eps = self.cfg.rms_norm_eps
        h1, x, rstd1 = F.rms_norm(a, W["input_layernorm.weight"], eps, residual=r)
        tsp, T = self.tsp, batch.num_tokens
        # sequence parallelism: the projections see every token (gathered), their row-parallel outputs come back
        # reduce-scattered (``tp_reduce``), norms and residuals stay on this rank's slice
        o = self._attn_fwd(W, h1 if tsp is None else tsp.gather(h1, T), batch, S, i)
        h2, x2, rstd2 = F.rms_norm(o, W["post_attention_layernorm.weight"], eps, residual=x)
        d = self._mlp_fwd(W, h2 if tsp is None else tsp.gather(h2, T), S)
        if self.stats_hook is not None:  # precision debugging: per-layer tensor statistics
            self.stats_hook(f"layers.{i}.attn_out", o)
            self.stats_hook(f"layers.{i}.mlp_out", d)
        if S is not None:
            S.update(x=x, rstd1=rstd1, x2=x2, rstd2=rstd2)
        return d, x2

    def _layer_bwd(self, i: int, g_d, g_x2, batch: PackedBatch, S: dict):
        if self.pre_layer_hook is not None:
            self.pre_layer_hook(i, "backward")
        W = self.params.layer(i)
        eps = self.cfg.rms_norm_eps
        w1, w2 = W["input_layernorm.weight"], W["post_attention_layernorm.weight"]
        tsp, T = self.tsp, batch.num_tokens
        full = (lambda t: t) if tsp is None else (lambda t: tsp.gather(t, T))  # gradient of a reduce-scatter = all-gather
        h2 = F.rms_norm(S["x2"], w2, eps)[0]
        g_h2 = self._mlp_bwd(W, full(g_d), full(h2), S)
        g_x2t = F.rms_norm_bwd(g_h2, S["x2"], w2, S["rstd2"], g_x2, self._grad_of(w2), True)
        h1 = F.rms_norm(S["x"], w1, eps)[0]
        g_h1 = self._attn_bwd(W, full(g_x2t), full(h1), batch, S)
        g_x = F.rms_norm_bwd(g_h1, S["x"], w1, S["rstd1"], g_x2t, self._grad_of(w1), True)
        if self.post_layer_backward_hook is not None:
            self.post_layer_backward_hook(i)
        return g_x

    # ------------------------------------------------------------------------------------ trunk
    def _first_kept_layer(self, num_tokens: int) -> int:
        """Layers ``[0, k)`` are recomputed in the backward pass, layers ``[k, L)`` keep their activations.
        ``recompute``: ``none`` -> k = 0, ``full`` -> k = L, ``auto`` -> as many kept layers as ``keep_layers_fn``
        (set by the engine from the free device memory and the size of the micro-batch) allows."""
        L = self.cfg.num_hidden_layers
        if self.recompute == "full":
            return L
        if self.recompute == "auto":
            keep = self.keep_layers_fn(num_tokens) if self.keep_layers_fn is not None else 0
            return L - max(0, min(L, int(keep)))
        return 0

    def activation_bytes_per_layer(self, num_tokens: int) -> int:
        """Bytes one kept layer pins until its backward: qkv, attention output, gate_up and the two residual streams."""
        c = self.cfg
        inter = c.moe_intermediate_size * c.num_experts_per_tok if c.is_moe else c.intermediate_size
        per_tok = (c.q_size + 2 * c.kv_size) + c.q_size + 2 * inter + 2 * c.hidden_size
        return int(num_tokens) * per_tok * self.params.flat.element_size() + int(num_tokens) * (c.num_attention_heads + 2) * 4

    def _trunk_fwd(self, batch: PackedBatch, save: bool, stage_input: Optional[torch.Tensor] = None):
        cfg = self.cfg
        self._ensure_rope(batch.max_seqlen + 1)
        if self.pre_layer_hook is not None:
            self.pre_layer_hook(-1, "forward")
        # model chunk (interleaved pipeline stages): layers [lo, hi) of this model; the embedding belongs to the first chunk
        # and the final norm + head to the last one
        lo, hi, c_first, c_last = self.chunk if self.chunk is not None else (0, cfg.num_hidden_layers, True, True)
        use_embed = cfg.has_embedding and c_first
        if use_embed:
            ids = batch.input_ids if self.sp is None else batch.input_ids[self.sp.local_rows(batch.num_tokens, batch.input_ids.device)]
            a = F.embedding(ids, self.params["embed_tokens.weight"])
            if self.tsp is not None:
                a = self.tsp.slice(a)
        else:
            a = stage_input  # hidden stream handed over by the previous pipeline stage
            assert a is not None, "a pipeline stage without embedding needs stage_input"
        r = None
        saved: list[Any] = []
        keep_from = self._first_kept_layer(batch.num_tokens) if save else 0
        for i in range(lo, hi):
            if save and i < keep_from:  # only the layer input is kept; the layer runs again in the backward pass
                saved.append(self.offloader.offload(i, (a, r)) if self.offloader is not None else (a, r))
                a, r = self._layer_fwd(i, a, r, batch, None)
            else:
                S = {} if save else None
                a, r = self._layer_fwd(i, a, r, batch, S)
                if save:
                    saved.append(S)
        if self.pre_layer_hook is not None:
            self.pre_layer_hook(cfg.num_hidden_layers, "forward")
        span = (lo, hi, use_embed)
        if not (cfg.has_head and c_last):
            # stage boundary: the next stage continues from the summed stream (its first norm sees residual None)
            out = a if r is None else a + r
            return out, (dict(batch=batch, layers=saved, boundary=True, span=span) if save else None)
        hN, xN, rstdN = F.rms_norm(a, self.params["norm.weight"], cfg.rms_norm_eps, residual=r)
        if self.tsp is not None:
            hN = self.tsp.gather(hN, batch.num_tokens)  # the heads see every token
        state = dict(batch=batch, layers=saved, xN=xN, rstdN=rstdN, hN=hN, span=span) if save else None
        return hN, state

    def _trunk_bwd(self, state: dict, g_hN: torch.Tensor) -> Optional[torch.Tensor]:
        """Backward through this model's layers. ``g_hN``: gradient of the head input (last stage) or of the boundary
        stream (other stages). Returns the gradient of ``stage_input`` when the model has no embedding, else None."""
        cfg = self.cfg
        batch = state["batch"]
        if state.get("boundary"):
            g = g_hN
        else:
            wn = self.params["norm.weight"]
            if self.tsp is not None:
                g_hN = self.tsp.slice(g_hN)  # every rank of the group holds the same head-input gradient
            g = F.rms_norm_bwd(g_hN, state["xN"], wn, state["rstdN"], None, self._grad_of(wn), True)
        if self.post_layer_backward_hook is not None:
            self.post_layer_backward_hook(cfg.num_hidden_layers)
        g_d = g_x2 = g
        lo, hi, use_embed = state.get("span") or (0, cfg.num_hidden_layers, cfg.has_embedding)
        for i in reversed(range(lo, hi)):
            S = state["layers"][i - lo]
            if self.offloader is not None and not isinstance(S, (tuple, dict)):
                nxt = state["layers"][i - lo - 1] if i > lo else None
                if nxt is not None and not isinstance(nxt, (tuple, dict)):
                    self.offloader.prefetch(nxt)  # the previous layer's input travels back while this layer computes
                S = self.offloader.wait(S)
            if isinstance(S, tuple):
                a, r = S
                S = {}
                self._layer_fwd(i, a, r, batch, S)
            g = self._layer_bwd(i, g_d, g_x2, batch, S)
            state["layers"][i - lo] = None
            g_d = g_x2 = g
        if not use_embed:
            if self.post_layer_backward_hook is not None:
                self.post_layer_backward_hook(-1)
            return g
        emb = self.params["embed_tokens.weight"]
        if getattr(emb, "main_grad", None) is not None:
            if self.pre_layer_hook is not None:
                self.pre_layer_hook(-1, "backward")
            ids = batch.input_ids if self.sp is None else batch.input_ids[self.sp.local_rows(batch.num_tokens, batch.input_ids.device)]
            if self.tsp is not None:
                ids = self.tsp.slice(ids)  # padding rows carry a zero gradient
            F.embedding_bwd_(ids, g, emb.main_grad)
        if self.post_layer_backward_hook is not None:
            self.post_layer_backward_hook(-1)

    # ------------------------------------------------------------------------------------ heads
    def forward_logprobs(self, batch: PackedBatch, labels: torch.Tensor, temperature: float = 1.0,
                         need_grad: Optional[bool] = None, positions: Optional[torch.Tensor] = None,
                         stage_input: Optional[torch.Tensor] = None, position_labels: Optional[torch.Tensor] = None):
        """(log_probs, entropy) per packed position of ``labels`` (fp32 [T]); differentiable when grads are on.
        With ``positions`` (int64, increasing) the LM head runs only on those packed positions (the ones whose next
        token is a response token) and the outputs have ``len(positions)`` entries."""
        need_grad = torch.is_grad_enabled() if need_grad is None else need_grad
        with torch.no_grad():
            hN, state = self._trunk_fwd(batch, save=need_grad, stage_input=stage_input)
            if positions is not None:
                # ``position_labels``: one label per entry of ``positions`` (a shared last prompt token predicts a different
                # first response token for every member of its group, so positions may repeat)
                hS = hN.index_select(0, positions)
                labels = position_labels if position_labels is not None else labels.index_select(0, positions)
            else:
                hS = hN
            if self.vocab_parallel is not None:
                grp, v0 = self.vocab_parallel
                lp, ent, lse = F.lmhead_logprob_entropy_vocab_parallel(hS, self.params.lm_head_weight, labels, temperature, v0, grp)
            else:
                lp, ent, lse = F.lmhead_logprob_entropy(hS, self.params.lm_head_weight, labels, temperature)
        if not need_grad:
            return lp, ent
        state.update(kind="lm", labels=labels, temperature=temperature, lse=lse, ent=ent, positions=positions, hS=hS)
        self.last_state = state  # after backward: last_state["g_input"] is the gradient of stage_input
        return _Anchor.apply(self._anchor, self, state, lp, ent)

    def forward_values(self, batch: PackedBatch, need_grad: Optional[bool] = None,
                       stage_input: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Scalar value per packed position (fp32 [T]) from the value head."""
        need_grad = torch.is_grad_enabled() if need_grad is None else need_grad
        with torch.no_grad():
            hN, state = self._trunk_fwd(batch, save=need_grad, stage_input=stage_input)
            vals = F.gemm(hN, self.params["v_head.weight"])[:, 0].float()
        if not need_grad:
            return vals
        state.update(kind="value")
        self.last_state = state
        return _Anchor.apply(self._anchor, self, state, vals)[0]

    def forward_hidden(self, batch: PackedBatch) -> torch.Tensor:
        with torch.no_grad():
            return self._trunk_fwd(batch, save=False)[0]

    def forward_logits(self, batch: PackedBatch) -> torch.Tensor:
        with torch.no_grad():
            return F.gemm(self._trunk_fwd(batch, save=False)[0], self.params.lm_head_weight)

    # ------------------------------------------------------------------------------------ pipeline stages
    @torch.no_grad()
    def forward_stage(self, batch: PackedBatch, stage_input: Optional[torch.Tensor] = None, save: bool = True):
        """A stage (or model chunk) without head: returns (boundary stream [T, H], state for ``backward_stage``)."""
        assert not self.cfg.has_head or (self.chunk is not None and not self.chunk[3])
        return self._trunk_fwd(batch, save=save, stage_input=stage_input)

    @torch.no_grad()
    def backward_stage(self, state: dict, g_out: torch.Tensor) -> Optional[torch.Tensor]:
        """Backward of ``forward_stage``; returns the gradient of its ``stage_input`` (None on the first stage)."""
        return self._trunk_bwd(state, g_out)

    @torch.no_grad()
    def _backward(self, state: dict, grads) -> None:
        hN = state["hN"]
        if self.pre_layer_hook is not None:  # the head's unit is the first one the backward pass touches
            self.pre_layer_hook(self.cfg.num_hidden_layers, "backward")
        if state["kind"] == "lm":
            g_lp, g_ent = grads
            if g_lp is None:
                g_lp = torch.zeros_like(state["lse"])
            head = self.params.lm_head_weight
            g_hS = F.lmhead_backward(state["hS"], head, state["labels"], state["temperature"], state["lse"], state["ent"],
                                     g_lp.float(), g_ent.float() if g_ent is not None else None, getattr(head, "main_grad", None),
                                     vocab_start=self.vocab_parallel[1] if self.vocab_parallel is not None else 0)
            if self.vocab_parallel is not None:  # every rank holds the contribution of its vocabulary slice
                import torch.distributed as dist

                g_hS = g_hS.float()
                dist.all_reduce(g_hS, group=self.vocab_parallel[0])
                g_hS = g_hS.to(hN.dtype)
            if state.get("positions") is not None:
                g_hN = torch.zeros(hN.shape, dtype=torch.float32, device=hN.device)
                g_hN.index_add_(0, state["positions"], g_hS.float())  # positions may repeat (shared prefixes)
                g_hN = g_hN.to(hN.dtype)
            else:
                g_hN = g_hS
            state["hS"] = None
            state["g_input"] = self._trunk_bwd(state, g_hN)  # gradient of stage_input (pipeline stages after the first)
            return
        else:
            (g_v,) = grads
            wv = self.params["v_head.weight"]
            dl = torch.zeros(hN.shape[0], wv.shape[0], dtype=hN.dtype, device=hN.device)
            dl[:, 0] = g_v.to(hN.dtype)
            g_hN = F.gemm(dl, wv, b_mn=True)
            self._wgrad(wv, dl, hN)
        state["g_input"] = self._trunk_bwd(state, g_hN)
