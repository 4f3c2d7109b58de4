"""Tensor x pipeline x data parallel training engine (``strategy=megatron``).

Every rank trains the local shard model of ``ModelParallelTopology.local_config`` with the native engine's machinery
(flat buffers, hand-written backward, sharded optimizer over the data-parallel group). What this class adds:

* the tensor-parallel all-reduces inside the layer (``DecoderModel.tp_reduce``);
* the pipeline schedule: all micro-batches flow forward through the stages (hidden stream [T, H] sent with
  point-to-point messages), the last stage evaluates the loss, then the gradients flow back in the same order. Model
  outputs and the loss are broadcast from the last stage so that every rank of a replica returns the same result;
* a gradient norm that counts tensor-parallel-replicated parameters once and sums over the model-parallel group;
* weights initialised / loaded in the full HuggingFace layout and cut into shards with ``ShardMap`` (identical on every
  data-parallel replica), and the reverse gather for checkpoints and for handing weights to a rollout engine.

Parity target: ``verl/workers/engine/megatron/transformer_impl.py`` (engine class, ``forward_backward_batch`` with the
pipeline schedule, ``get_per_tensor_param`` export) and ``verl/utils/megatron_utils.py``.
"""

from __future__ import annotations

import os
from typing import Callable, Generator, Optional

import torch
import torch.distributed as dist

from ....ops import functional as F

from ....models.weights import FlatParams
from ....parallel.model_parallel import ModelParallelTopology, build_shard_map, copy_full_to_local, copy_local_to_full
from ....utils.distributed import get_data_parallel_group, set_data_parallel_group
from ..base import EngineRegistry
from ..native.engine import NativeEngine, pack_padded_batch

__all__ = ["ModelParallelEngine", "ModelParallelEngineWithLMHead", "ModelParallelEngineWithValueHead"]

_TOPOLOGIES: dict = {}


def get_topology(tp: int, pp: int, ep: int = 1, vpp: int = 1) -> ModelParallelTopology:
    """One topology (set of process groups) per (tp, pp, ep) and process: actor, critic and reference engines share it."""
    key = (tp, pp, ep, vpp)
    if key not in _TOPOLOGIES:
        _TOPOLOGIES[key] = ModelParallelTopology(tp, pp, ep=ep, vpp=vpp)
    return _TOPOLOGIES[key]


class ModelParallelEngine(NativeEngine):
    def __init__(self, model_config, engine_config, optimizer_config=None, checkpoint_config=None, **kwargs):
        super().__init__(model_config, engine_config, optimizer_config, checkpoint_config, **kwargs)
        g = lambda k, d: int(getattr(engine_config, k, None) or d)
        self.tp_size = g("tensor_model_parallel_size", 1)
        self.pp_size = g("pipeline_model_parallel_size", 1)
        self.ep_size = g("expert_model_parallel_size", 1) if self.arch.is_moe else 1
        self.vpp_size = g("virtual_pipeline_model_parallel_size", 1)
        self.full_arch = self.arch
        if g("context_parallel_size", 1) > 1 and self.pp_size > 1:
            raise NotImplementedError("context parallelism is combined with tensor and data parallelism; pipeline stages "
                                      "exchange whole token streams (use pipeline_model_parallel_size=1 with it)")
        if self.arch.is_generic:
            raise NotImplementedError(f"model_type={self.arch.model_type!r} runs as a library module: tensor / pipeline / expert "
                                      f"parallel training covers the natively supported families; use the data-parallel engine "
                                      f"(strategy fsdp) with its sharded optimizer for this one")

    # ------------------------------------------------------------------------------------ setup
    def initialize(self) -> None:
        if self._initialized:
            return
        self.topo = get_topology(self.tp_size, self.pp_size, self.ep_size, self.vpp_size)
        if self.full_arch.is_moe and self.tp_size > 1:
            # experts under tensor parallelism: every expert's intermediate width is cut over the tensor-parallel ranks
            # (expert tensor parallelism, the reference's default ``expert_tensor_parallel_size = tensor_model_parallel_size``)
            etp = getattr(self.engine_config, "expert_tensor_parallel_size", None)
            if etp is not None and int(etp) != self.tp_size:
                raise NotImplementedError(f"expert_tensor_parallel_size={etp}: experts are cut over the whole tensor-parallel group "
                                          f"({self.tp_size}); leave it unset or set it to the tensor-parallel size")
            # (with expert_model_parallel_size > 1 as well: whole experts over the data-parallel ranks, their width over tp)
        if self.full_arch.tie_word_embeddings and self.pp_size > 1:
            raise NotImplementedError("pipeline parallelism with tied input/output embeddings needs the embedding shared between "
                                      "the first and the last stage; use pipeline_model_parallel_size=1 for this model")
        # vocabulary-parallel LM head (each tensor-parallel rank holds V / tp rows; the fused log-prob kernel runs per slice)
        vp = bool(getattr(self.engine_config, "vocab_parallel_head", True)) and not self.value_head
        self.arch = self.topo.local_config(self.full_arch, vocab_parallel=vp)
        self.maps = build_shard_map(self.full_arch, self.topo, self.value_head, vocab_parallel=vp)
        outer = get_data_parallel_group()
        set_data_parallel_group(self.topo.dp_group)
        try:
            object.__setattr__(self.engine_config, "fused_comm", False) if hasattr(self.engine_config, "fused_comm") else None
            super().initialize()
        finally:
            set_data_parallel_group(outer)
        if self.arch.head_vocab_size:
            self.model.vocab_parallel = (self.topo.tp_group, self.topo.tp_rank * self.arch.head_vocab_size)
        if self.topo.ep > 1:
            from ....models.decoder import ExpertParallelGroup

            self.model.ep = ExpertParallelGroup(self.topo.ep_group, self.topo.ep_rank, self.topo.ep)
        if self.topo.tp > 1:
            grp = self.topo.tp_group

            def reduce(x: torch.Tensor) -> torch.Tensor:
                dist.all_reduce(x, group=grp)
                return x

            self.model.tp_reduce = reduce
            if self.full_arch.is_moe:
                self.model.etp_sum = reduce
            self.fused_tp_collectives = False
            # (mixture-of-experts blocks keep the whole token stream on every tensor-parallel rank: their routed tokens are
            # not a token slice; sequence parallelism is therefore a dense-model option and is left off for them)
            want_sp = bool(getattr(self.engine_config, "sequence_parallel", False)) and not self.full_arch.is_moe
            use_sp = want_sp and self.cp_size == 1
            fused = None
            if self.device.type == "cuda" and dist.get_world_size() == self.topo.tp and os.environ.get("VERL_B200_FUSED_TP", "1") != "0":
                # one kernel per row-parallel projection / column-parallel input gradient: GEMM with the all-reduce (or, with
                # sequence parallelism, the reduce-scatter over token rows) in its epilogue over peer memory. Peer-mapped
                # buffers are bound to the default group: the tensor-parallel group has to be the whole job; other layouts
                # keep GEMM + NCCL.
                from ....parallel.symmetric import FusedRowParallelLinear, symmetric_available

                if symmetric_available():
                    rows = int(getattr(self.engine_config, "max_token_len_per_gpu", 0) or 0) or 16384
                    rows = max(rows, int(getattr(self.engine_config, "infer_max_token_len_per_gpu", 0) or 0))
                    fused = FusedRowParallelLinear(rows, self.full_arch.hidden_size, self.device, None)
                    self.fused_tp_collectives = True
            if fused is not None and not use_sp:
                def linear_sum(x: torch.Tensor, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
                    if x.shape[0] > fused.max_rows:  # a micro-batch beyond the planned size: GEMM + collective
                        return reduce(F.gemm(x, w, b_mn=b_mn))
                    return fused(x.contiguous(), w, None, None, b_mn)

                self.model.tp_linear_sum = linear_sum
            if use_sp:
                # (with context parallelism the stream is already token-sliced over the context-parallel block, and the
                # tensor-parallel group keeps the plain all-reduce form)
                # token-sliced residual stream: reduce-scatter behind the row-parallel projections, all-gather in front of
                # the column-parallel ones
                from ....models.decoder import TensorSequenceParallel

                self.model.tsp = TensorSequenceParallel(grp, self.topo.tp_rank, self.topo.tp)
                self.model.tp_reduce = self.model.tsp.scatter_sum
                if fused is not None:
                    tsp, W = self.model.tsp, self.topo.tp

                    def linear_scatter(x: torch.Tensor, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
                        T = x.shape[0]
                        n = tsp.local_rows(T)
                        if T > fused.max_rows or n * (W - 1) >= T:  # too large for the buffers, or a rank without rows
                            return tsp.scatter_sum(F.gemm(x, w, b_mn=b_mn))
                        return fused(x.contiguous(), w, None, None, b_mn, scatter_rows=n)

                    self.model.tp_linear_sum = linear_scatter
        # replicated-parameter mask for the gradient norm (embedding, norms, head, biases of row-parallel layers)
        self._rep_ranges = [(self.params.offsets[m.local_name], self.params.views[m.local_name].numel())
                            for m in self.maps if m.kind == "rep"]

    def _load_or_init(self, seed: int) -> None:
        """Build (or load) the full model on the host with the same seed everywhere and keep this rank's shard."""
        mc = self.model_config
        path = getattr(mc, "local_path", None) or getattr(mc, "path", None)
        load = bool(getattr(mc, "load_weights", True)) and path and os.path.isdir(str(path))
        # random init happens on the device (per-tensor seeded generators: identical on every rank, and fast for 8B+
        # models); checkpoints are read on the host
        full = FlatParams(self.full_arch, dtype=torch.float32 if self.dtype == torch.float32 else torch.bfloat16,
                          device="cpu" if load else self.device, value_head=self.value_head)
        if load:
            from ....utils.model import load_hf_weights_into

            load_hf_weights_into(full, path)
        else:
            full.init_weights(seed=seed)
        copy_full_to_local(full, self.params, self.maps, self.topo.tp, self.topo.tp_rank, self.topo.ep, self.topo.ep_rank)
        del full

    def _qat_scale_group(self):
        topo = getattr(self, "topo", None)
        return topo.tp_group if topo is not None and topo.tp > 1 else None

    # ------------------------------------------------------------------------------------ topology facts for the worker
    def get_data_parallel_size(self) -> int:
        return self.topo.dp

    def get_data_parallel_rank(self) -> int:
        return self.topo.dp_rank

    def is_collection_rank(self) -> bool:
        """The rank of a replica whose outputs the controller keeps (all ranks return identical outputs)."""
        return self.topo.tp_rank == 0 and self.topo.is_last_stage

    # ------------------------------------------------------------------------------------ pipeline schedule
    def _stage_recv(self, T: int) -> torch.Tensor:
        x = torch.empty(T, self.full_arch.hidden_size, dtype=self.dtype, device=self.device)
        dist.recv(x, src=self.topo.prev_rank)
        return x

    # ---- point-to-point helpers of the pipeline (shapes are known on both sides: every rank of a replica sees the batch)
    def _hidden_buf(self, T: int) -> torch.Tensor:
        return torch.empty(T, self.full_arch.hidden_size, dtype=self.dtype, device=self.device)

    def _exchange(self, send: Optional[torch.Tensor], dst: Optional[int], recv_T: Optional[int], src: Optional[int]) -> Optional[torch.Tensor]:
        """One batched point-to-point step: optionally send ``send`` to ``dst`` and/or receive a [recv_T, H] tensor from
        ``src``. Issuing both directions as one batch is what keeps neighbouring stages, which talk to each other in both
        directions during the steady state, from waiting on each other."""
        ops, out = [], None
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), dst))
        if recv_T is not None:
            out = self._hidden_buf(recv_T)
            ops.append(dist.P2POp(dist.irecv, out, src))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return out

    def _run_micro_batches(self, mbs: list[dict], R: int, temperature: float, calc_entropy: bool, loss_function, forward_only: bool):
        """Pipeline schedule. Training uses one-forward-one-backward (1F1B): stage s runs ``P - 1 - s`` warm-up forwards,
        then alternates a forward with the backward of its oldest micro-batch in flight, then drains, so a stage never holds
        the activations of more than ``P - s`` micro-batches (the all-forward-then-all-backward order holds all of them;
        ``pipeline_schedule=gpipe`` selects it). Forward-only passes stream the micro-batches through the stages."""
        topo = self.topo
        if topo.pp == 1:
            return super()._run_micro_batches(mbs, R, temperature, calc_entropy, loss_function, forward_only)
        if topo.vpp > 1:
            return self._run_interleaved(mbs, R, temperature, calc_entropy, loss_function, forward_only)
        need_grad = not forward_only and loss_function is not None
        first, last = topo.is_first_stage, topo.is_last_stage
        packed = [pack_padded_batch(mb["input_ids"], mb["attention_mask"], mb.get("position_ids"), R) for mb in mbs]
        tsp = self.model.tsp
        Ts = [p[0].num_tokens if tsp is None else tsp.local_rows(p[0].num_tokens) for p in packed]  # rows of a boundary tensor
        M = len(mbs)
        rows: list[int] = [r for mb in mbs for r in mb["_rows"]]
        losses, metrics = [], {}
        head_out: list = [None] * M
        inflight: list = []  # (state, loss, index) of forwards whose backward has not run yet, oldest first

        def forward(i: int, x_in):
            batch, labels, resp_index, resp_valid = packed[i]
            if not last:
                x_out, st = self.model.forward_stage(batch, x_in, save=need_grad)
                inflight.append((st, None, i))
                return x_out
            out = self._head_outputs(batch, labels, resp_index, resp_valid, temperature, calc_entropy, need_grad, x_in)
            st = getattr(self.model, "last_state", None) if need_grad else None
            loss = None
            if loss_function is not None:
                loss, m = loss_function(model_output=out, data=mbs[i], dp_group=None)
                losses.append(loss.detach())
                for k, v in m.items():
                    metrics.setdefault(k, []).append(v)
            inflight.append((st, loss, i))
            head_out[i] = {k: v.detach() for k, v in out.items()}
            return None

        def backward(g_out):
            st, loss, _ = inflight.pop(0)
            if last:
                loss.backward()
                return st.get("g_input")
            return self.model.backward_stage(st, g_out)

        schedule = str(getattr(self.engine_config, "pipeline_schedule", "1f1b") or "1f1b").lower()
        if not need_grad or schedule == "gpipe":
            for i in range(M):
                x_in = None if first else self._exchange(None, None, Ts[i], topo.prev_rank)
                x_out = forward(i, x_in)
                if not last:
                    self._exchange(x_out, topo.next_rank, None, None)
            if need_grad:
                for i in range(M):
                    g_out = None if last else self._exchange(None, None, Ts[i], topo.next_rank)
                    g_in = backward(g_out)
                    if not first:
                        self._exchange(g_in, topo.prev_rank, None, None)
            else:
                inflight.clear()
        else:
            warm = min(topo.pp - 1 - topo.pp_rank, M)
            steady = M - warm
            nf = 0  # forwards issued
            x_in = None if first or M == 0 else self._exchange(None, None, Ts[0], topo.prev_rank)
            for _ in range(warm):
                x_out = forward(nf, x_in)
                nf += 1
                nxt = Ts[nf] if (nf < M and not first) else None
                # the last stage has no warm-up, so x_out is never None here
                self._exchange(x_out, topo.next_rank, None, None)
                x_in = self._exchange(None, None, nxt, topo.prev_rank) if nxt is not None else None
            for k in range(steady):
                x_out = forward(nf, x_in)
                nf += 1
                oldest = inflight[0][2]
                g_out = None if last else self._exchange(x_out, topo.next_rank, Ts[oldest], topo.next_rank)
                g_in = backward(g_out)
                more = nf < M
                if first:
                    x_in = None
                else:
                    x_in = self._exchange(g_in, topo.prev_rank, Ts[nf] if more else None, topo.prev_rank)
            while inflight:
                oldest = inflight[0][2]
                g_out = None if last else self._exchange(None, None, Ts[oldest], topo.next_rank)
                g_in = backward(g_out)
                if not first:
                    self._exchange(g_in, topo.prev_rank, None, None)
        # every stage returns the outputs of the last stage
        outs: dict[str, list] = {}
        for i in range(M):
            out = self._broadcast_outputs(head_out[i], packed[i][3].shape, calc_entropy or need_grad)
            for k, v in out.items():
                outs.setdefault(k, []).append(v.detach())
        # the loss and its metrics live on the last stage: share them inside the pipeline group
        losses, metrics = self._broadcast_loss(losses, metrics, M, loss_function is not None)
        return outs, rows, losses, metrics

    def _run_interleaved(self, mbs: list[dict], R: int, temperature: float, calc_entropy: bool, loss_function, forward_only: bool):
        """Interleaved (virtual) pipeline stages: every rank holds V model chunks and a micro-batch travels V times round
        the ring of P ranks. The schedule is breadth-first and in lockstep: with W = max(M, P), rank s runs chunk v of
        micro-batch i at step v * W + i + s (the backward pass mirrors it), so the start-up bubble is P - 1 steps of a
        1 / V model chunk instead of a whole stage. After every step a rank sends what it produced to the next rank of
        the ring and receives what the previous rank produced, both in ONE batched point-to-point call whose partner calls
        are the neighbours' calls of the same step: no rank ever waits on a call of another step, whatever M, P and V are.
        A value that arrives before its consumer's step waits in a buffer. All chunk states are kept until their backward."""
        topo = self.topo
        P, V, s_rank, M = topo.pp, topo.vpp, topo.pp_rank, len(mbs)
        need_grad = not forward_only and loss_function is not None
        packed = [pack_padded_batch(mb["input_ids"], mb["attention_mask"], mb.get("position_ids"), R) for mb in mbs]
        assert self.model.tsp is None, "virtual pipeline stages are not combined with sequence parallelism"
        Ts = [p[0].num_tokens for p in packed]
        rows: list[int] = [r for mb in mbs for r in mb["_rows"]]
        blk = self.arch.num_hidden_layers // V
        W = max(M, P)
        losses, metrics = [], {}
        head_out: list = [None] * M
        states: dict = {}

        def item_at(rank: int, t: int, backward: bool):
            """(v, i) that ``rank`` works on at step ``t``, or None."""
            k = t - (P - 1 - rank if backward else rank)
            if k < 0:
                return None
            v, i = divmod(k, W)
            if v >= V or i >= M:
                return None
            return (V - 1 - v if backward else v), i

        def is_entry(rank, v):
            return rank == 0 and v == 0

        def is_exit(rank, v):
            return rank == P - 1 and v == V - 1

        steps = (V - 1) * W + M + P - 1
        inbox: dict = {}
        prev_r, next_r = (s_rank - 1) % P, (s_rank + 1) % P
        # ---- forward
        for t in range(steps):
            mine = item_at(s_rank, t, False)
            send = None
            if mine is not None:
                v, i = mine
                self.model.chunk = (v * blk, (v + 1) * blk, v == 0, v == V - 1)
                batch, labels, resp_index, resp_valid = packed[i]
                x_in = None if is_entry(s_rank, v) else inbox.pop((v, i))
                if is_exit(s_rank, v):
                    out = self._head_outputs(batch, labels, resp_index, resp_valid, temperature, calc_entropy, need_grad, x_in)
                    st = getattr(self.model, "last_state", None) if need_grad else None
                    loss = None
                    if loss_function is not None:
                        loss, m = loss_function(model_output=out, data=mbs[i], dp_group=None)
                        losses.append(loss.detach())
                        for k_, v_ in m.items():
                            metrics.setdefault(k_, []).append(v_)
                    states[(v, i)] = (st, loss)
                    head_out[i] = {k_: v_.detach() for k_, v_ in out.items()}
                else:
                    send, st = self.model.forward_stage(batch, x_in, save=need_grad)
                    states[(v, i)] = (st, None)
            # what the previous rank of the ring produced in this step is the input of one of my later items
            theirs = item_at(prev_r, t, False)
            recv_key = None
            if theirs is not None and not is_exit(prev_r, theirs[0]):
                recv_key = (theirs[0] + 1, theirs[1]) if prev_r == P - 1 else theirs
            got = self._exchange(send, topo.ring_next if send is not None else None,
                                 Ts[recv_key[1]] if recv_key is not None else None, topo.ring_prev if recv_key is not None else None)
            if recv_key is not None:
                inbox[recv_key] = got
        # ---- backward
        if need_grad:
            for t in range(steps):
                mine = item_at(s_rank, t, True)
                send = None
                if mine is not None:
                    v, i = mine
                    st, loss = states.pop((v, i))
                    if is_exit(s_rank, v):
                        loss.backward()
                        g_in = st.get("g_input")
                    else:
                        g_in = self.model.backward_stage(st, inbox.pop(("g", v, i)))
                    send = None if is_entry(s_rank, v) else g_in
                theirs = item_at(next_r, t, True)
                recv_key = None
                if theirs is not None and not is_entry(next_r, theirs[0]):
                    recv_key = ("g", theirs[0] - 1, theirs[1]) if next_r == 0 else ("g", theirs[0], theirs[1])
                got = self._exchange(send, topo.ring_prev if send is not None else None,
                                     Ts[recv_key[2]] if recv_key is not None else None, topo.ring_next if recv_key is not None else None)
                if recv_key is not None:
                    inbox[recv_key] = got
        states.clear()
        self.model.chunk = None
        outs: dict[str, list] = {}
        for i in range(M):
            out = self._broadcast_outputs(head_out[i], packed[i][3].shape, calc_entropy or need_grad)
            for k_, v_ in out.items():
                outs.setdefault(k_, []).append(v_.detach())
        losses, metrics = self._broadcast_loss(losses, metrics, M, loss_function is not None)
        return outs, rows, losses, metrics

    def _head_outputs(self, batch, labels, resp_index, resp_valid, temperature, calc_entropy, need_grad, x_in) -> dict:
        positions = resp_index[resp_valid]
        lp, ent = self.model.forward_logprobs(batch, labels, temperature, need_grad=need_grad, positions=positions, stage_input=x_in)
        out = {"log_probs": torch.zeros(resp_valid.shape, dtype=lp.dtype, device=lp.device).masked_scatter(resp_valid, lp)}
        if calc_entropy or need_grad:
            out["entropy"] = torch.zeros(resp_valid.shape, dtype=ent.dtype, device=ent.device).masked_scatter(resp_valid, ent)
        return out

    def _broadcast_outputs(self, out: Optional[dict], shape, with_entropy: bool) -> dict:
        keys = ["log_probs"] + (["entropy"] if with_entropy else [])
        res = {}
        for k in keys:
            t = out[k].detach().float().contiguous() if out is not None else torch.empty(shape, dtype=torch.float32, device=self.device)
            dist.broadcast(t, src=self.topo.last_stage_rank, group=self.topo.pp_group)
            res[k] = out[k] if out is not None else t
        return res

    def _broadcast_loss(self, losses: list, metrics: dict, n_mb: int, has_loss: bool):
        if not has_loss:
            return losses, metrics
        box = [(torch.stack(losses).cpu(), metrics) if self.topo.is_last_stage else None]
        dist.broadcast_object_list(box, src=self.topo.last_stage_rank, group=self.topo.pp_group)
        l, m = box[0]
        return ([x.to(self.device) for x in l] if not self.topo.is_last_stage else losses), m

    def _forward_micro(self, mb: dict, R: int, temperature: float, calc_entropy: bool, need_grad: bool) -> dict:
        assert self.topo.pp == 1
        return super()._forward_micro(mb, R, temperature, calc_entropy, need_grad)

    # ------------------------------------------------------------------------------------ optimizer
    def _partial_grad_ranges(self) -> list:
        """(offset, numel) of replicated tensors whose gradient is a partial sum on every tensor-parallel rank: the
        per-head q / k norms (each rank sees its own heads)."""
        if getattr(self, "_partial_ranges", None) is None:
            partial = ("self_attn.q_norm.weight", "self_attn.k_norm.weight")
            if self.model.tsp is not None:  # token-wise parameters see this rank's tokens only
                partial += ("layernorm.weight", "norm.weight", "embed_tokens.weight")
            names = [m.local_name for m in self.maps if m.kind == "rep" and m.local_name.endswith(partial)]
            self._partial_ranges = [(self.params.offsets[n], self.params.views[n].numel()) for n in names]
        return self._partial_ranges

    def _complete_partial_grads(self) -> None:
        if self.topo.tp == 1 or self.tparams.main_grad is None:
            return
        ranges = self._partial_grad_ranges()
        if not ranges:
            return
        mg = self.tparams.main_grad
        buf = torch.cat([mg[o : o + n] for o, n in ranges])
        dist.all_reduce(buf, group=self.topo.tp_group)
        off = 0
        for o, n in ranges:
            mg[o : o + n].copy_(buf[off : off + n])
            off += n

    def _global_sumsq_correction(self) -> None:
        """``ctrl[0]`` holds the sum of squares of this rank's gradient shard over its DP group. Turn it into the model's
        global value: replicated tensors are counted on tensor-parallel rank 0 only, then summed over TP x PP."""
        if self.topo.tp * self.topo.pp == 1:
            return
        if self.topo.tp > 1 and self.topo.tp_rank != 0:
            sl_lo, sl_hi = self.shard_lo, self.shard_lo + self.shard_numel
            dup = torch.zeros((), dtype=torch.float32, device=self.device)
            for off, n in self._rep_ranges:
                a, b = max(off, sl_lo), min(off + n, sl_hi)
                if a < b:
                    dup += self.grad_shard[a - sl_lo : b - sl_lo].float().pow(2).sum()
            dist.all_reduce(dup, group=self.topo.dp_group) if self.topo.dp > 1 else None
            self.ctrl[0] -= dup
        dist.all_reduce(self.ctrl[:1], group=self.topo.mp_group)

    # ------------------------------------------------------------------------------------ weights out
    def gather_full_params(self, dtype=None) -> FlatParams:
        """The full model assembled on every rank of the replica (host of the train -> rollout reshard and of merged
        checkpoints): each rank writes its shard into a zeroed full-layout buffer, the buffers are summed over the
        model-parallel group, replicated tensors are divided by their multiplicity. Expert-parallel shards are gathered
        over the expert-parallel group. Without tensor / pipeline parallelism the buffer is built in ``dtype`` directly."""
        dtype = dtype or self.dtype
        topo = self.topo
        work = torch.float32 if topo.mp_group is not None else dtype
        full = FlatParams(self.full_arch, dtype=work, device=self.device, value_head=self.value_head)
        copy_local_to_full(self.params, full, self.maps, topo.tp, topo.tp_rank, topo.ep, topo.ep_rank)
        if topo.mp_group is not None:
            if topo.tp > 1 and topo.tp_rank != 0:  # replicated tensors are contributed by tp rank 0 only
                for m in self.maps:
                    if m.kind == "rep" and m.full_name in full.views:
                        full.views[m.full_name].zero_()
            dist.all_reduce(full.flat, group=topo.mp_group)
        if topo.ep > 1:
            from ....parallel.model_parallel import EXPERT_KINDS

            for m in self.maps:
                if m.kind in EXPERT_KINDS:
                    dst = full.views[m.full_name]
                    n = dst.shape[0] // topo.ep     # this replica's experts, already whole (summed over its tensor-parallel ranks)
                    src = dst[topo.ep_rank * n : (topo.ep_rank + 1) * n].clone()
                    if self.device.type == "cuda":
                        dist.all_gather_into_tensor(dst, src, group=topo.ep_group)
                    else:
                        dist.all_gather(list(dst.chunk(topo.ep)), src, group=topo.ep_group)
        if dtype != work:
            out = FlatParams(self.full_arch, dtype=dtype, device=self.device, value_head=self.value_head)
            out.flat.copy_(full.flat.to(dtype))
            return out
        return full

    def get_per_tensor_param(self, **kwargs) -> Generator[tuple[str, torch.Tensor], None, None]:
        full = self.gather_full_params()
        yield from full.hf_views()

    def export_hf_delta(self, update_snapshot: bool = True):
        """What changed in this rank's shard since the previous call (or since the first call, which takes the snapshot), as
        ``(hf_name, positions, values)`` records in full-tensor coordinates: the sparse alternative to
        ``gather_full_params`` for keeping a remote copy of the weights current (``delta_export.py``)."""
        if getattr(self, "_delta_exporter", None) is None:
            from .delta_export import ShardDeltaExporter

            self._delta_exporter = ShardDeltaExporter(self)
            return []
        return self._delta_exporter.export(update_snapshot)

    # ------------------------------------------------------------------------------------ checkpoint (layout schema v2)
    @property
    def global_rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else 0

    def _ckpt_manager(self):
        if getattr(self, "_ckpt_mgr", None) is None:
            from ....utils.checkpoint.megatron_checkpoint_manager import MegatronCheckpointManager

            self._ckpt_mgr = MegatronCheckpointManager(self, checkpoint_config=self.checkpoint_config,
                                                       role="critic" if self.value_head else "actor")
        return self._ckpt_mgr

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None, **kwargs) -> None:
        """One directory per model-parallel rank under ``model|optimizer|extra/dist_ckpt`` plus a manifest
        (``utils/checkpoint/megatron_checkpoint_manager.py``); old checkpoints rotate as in the data-parallel engine."""
        self._ckpt_manager().save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)
        self._rotate_checkpoints(local_path, max_ckpt_to_keep)

    def load_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, del_local_after_load: bool = False, **kwargs) -> None:
        if local_path is None:
            return
        self._ckpt_manager().load_checkpoint(local_path, hdfs_path, del_local_after_load)
        if self.qat.enable:
            self._apply_qat()

    def optimizer_state(self) -> dict:
        """This rank's optimizer shard: fp32 masters, Adam moments, step counters."""
        return {"master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(),
                "step": self.opt_step_count, "sched_step": self.sched_step, "shard_lo": self.shard_lo, "shard_numel": self.shard_numel}

    def load_optimizer_state(self, st: dict) -> None:
        assert st["shard_lo"] == self.shard_lo and st["master"].numel() == self.master.numel(), "optimizer shard layout mismatch"
        self.master.copy_(st["master"])
        self.exp_avg.copy_(st["exp_avg"])
        self.exp_avg_sq.copy_(st["exp_avg_sq"])
        self.opt_step_count, self.sched_step = int(st["step"]), int(st["sched_step"])
        # the working weights follow the masters (identical to what was saved, up to the bf16 cast)
        self._scatter_owned(self.master.to(self.device), self.tparams.flat)
        self._publish_shard()

    def reset_master_from_params(self) -> None:
        """Model weights were loaded without optimizer state: the fp32 masters restart from them."""
        self.master.copy_(self._owned(self.tparams.flat).float())

    def local_named_tensors(self):
        """(full-model name of the shard, local tensor) pairs: what the model-parallel checkpoint layout stores."""
        for m in self.maps:
            yield m.full_name, self.params.views[m.local_name]

    def shard_meta(self) -> dict:
        """full-model name -> (kind, blocks) of every local tensor: how the merger places a shard in the whole tensor."""
        return {m.full_name: (m.kind, tuple(m.blocks)) for m in self.maps}

    def load_local_named_tensors(self, tensors: dict) -> None:
        for m in self.maps:
            if m.full_name in tensors:
                self.params.views[m.local_name].copy_(tensors[m.full_name].to(self.dtype))


@EngineRegistry.register(model_type="language_model", backend=["megatron", "mp", "mindspeed"], device=["cuda", "cpu"])
class ModelParallelEngineWithLMHead(ModelParallelEngine):
    value_head = False


@EngineRegistry.register(model_type="value_model", backend=["megatron", "mp", "mindspeed"], device=["cuda", "cpu"])
class ModelParallelEngineWithValueHead(ModelParallelEngine):
    """Critic: the last stage ends in a scalar head; ``model_output`` carries ``values`` [b, R]."""

    value_head = True

    def _head_outputs(self, batch, labels, resp_index, resp_valid, temperature, calc_entropy, need_grad, x_in) -> dict:
        vals = self.model.forward_values(batch, need_grad=need_grad, stage_input=x_in)
        zero = torch.zeros((), dtype=vals.dtype, device=vals.device)
        return {"values": torch.where(resp_valid, vals[resp_index], zero)}

    def _forward_micro(self, mb: dict, R: int, temperature: float, calc_entropy: bool, need_grad: bool) -> dict:
        batch, labels, resp_index, resp_valid = pack_padded_batch(mb["input_ids"], mb["attention_mask"], mb.get("position_ids"), R)
        return self._head_outputs(batch, labels, resp_index, resp_valid, temperature, calc_entropy, need_grad, None)

    def _broadcast_outputs(self, out, shape, with_entropy: bool) -> dict:
        t = out["values"].detach().float().contiguous() if out is not None else torch.empty(shape, dtype=torch.float32, device=self.device)
        dist.broadcast(t, src=self.topo.last_stage_rank, group=self.topo.pp_group)
        return {"values": out["values"] if out is not None else t}


