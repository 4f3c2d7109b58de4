"""Sharded data-parallel training engine on the native sm_100a kernels.

Memory plan per GPU (sized for 180 GB HBM3e):

* bf16 working parameters in one flat buffer (``zero_stage=2``: full replica, shared in place with the
  rollout engine; no parameter gather anywhere in forward/backward),
* fp32 main-gradient flat buffer that the wgrad GEMMs accumulate into across micro-batches,
* this rank's 1/W shard of the fp32 master weights and Adam moments.

One optimizer step = reduce-scatter of the main-grad buffer (fp32, mean over data-parallel ranks) ->
global grad-norm (one scalar all-reduce) -> fused AdamW on the shard, which also writes the new bf16
values into the working buffer -> all-gather of the working buffer.  With ``fused_comm`` and symmetric
memory available the reduce-scatter/AdamW/all-gather run as peer-memory kernels
(:mod:`verl_b200.parallel.fused_optim`); otherwise the same steps use NCCL (GPU) or gloo (CPU).

On CPU the engine runs the same code in fp32 over gloo, which is the oracle configuration.

Parity target: ``verl/workers/engine/fsdp/transformer_impl.py`` (``FSDPEngine`` :87-1117: initialise,
``forward_backward_batch`` :700-753, ``optimizer_step`` :764-810 with clip + non-finite skip,
``get_per_tensor_param`` :954-1038, value-head variant :1567-1617) and the checkpoint file layout of
``verl/utils/checkpoint/fsdp_checkpoint_manager.py:213-417``.
"""

from __future__ import annotations

import json
import logging
import math
import os
from typing import Any, Callable, Generator, Optional

import torch
import torch.distributed as dist

from ....models.config import ModelConfig
from ....models.decoder import DecoderModel, PackedBatch
from ....models.weights import ALIGN, FlatParams
from ....ops import functional as F
from ....ops import native
from ....utils.device import get_device_name
from ...config.optimizer import lr_at_step
from ..base import BaseEngine, EngineRegistry

logger = logging.getLogger(__name__)


def _host_has_room(nbytes: int) -> bool:
    """Whether ``nbytes`` of page-locked host memory can be taken with a wide margin (twice the size plus 16 GB must be
    available, within the container's memory limit when there is one)."""
    try:
        import psutil

        avail = psutil.virtual_memory().available
        for path in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
            try:
                raw = open(path).read().strip()
                if raw.isdigit():
                    used_path = path.replace("memory.max", "memory.current").replace("limit_in_bytes", "usage_in_bytes")
                    avail = min(avail, int(raw) - int(open(used_path).read().strip()))
            except OSError:
                pass
        return avail > 2 * nbytes + (16 << 30)
    except Exception:
        return False

__all__ = ["NativeEngine", "NativeEngineWithLMHead", "NativeEngineWithValueHead", "pack_padded_batch",
           "collate_multi_modal_inputs"]


def pack_padded_batch(input_ids: torch.Tensor, attention_mask: torch.Tensor, position_ids: Optional[torch.Tensor],
                      response_length: int, lens_list: Optional[list] = None):
    """Remove padding from a [b, P+R] batch (left-padded prompt, right-padded response).

    Returns ``(packed_batch, labels, resp_index, resp_valid)`` where ``labels[t]`` is the next token of packed
    position ``t`` and ``resp_index`` [b, R] are the packed positions whose outputs predict the response
    tokens (column ``P-1+j`` of each row), valid where ``resp_valid``.
    """
    b, L = input_ids.shape
    mask = attention_mask.bool()
    if lens_list is None:  # (callers that know the row lengths on the host pass them: no device synchronisation here)
        lens_list = mask.sum(-1).tolist()
    lens_list = [int(x) for x in lens_list]
    ids = input_ids[mask]
    labels = torch.roll(input_ids, shifts=-1, dims=1)[mask]
    if position_ids is None:
        pos = (torch.cumsum(mask.to(torch.int32), -1) - 1)[mask]
    else:
        pos = position_ids[mask]
    cu = torch.zeros(b + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens_list, dtype=torch.int32), 0)
    batch = PackedBatch(input_ids=ids.contiguous(), positions=pos.to(torch.int32).contiguous(),
                        cu_seqlens=cu.to(input_ids.device), max_seqlen=max(lens_list) if lens_list else 0,
                        cu_seqlens_cpu=cu)
    flat_index = (torch.cumsum(mask.reshape(-1).to(torch.int64), 0) - 1).view(b, L)
    P = L - response_length
    resp_index = flat_index[:, P - 1 : L - 1]
    resp_valid = mask[:, P:]
    return batch, labels.contiguous(), resp_index, resp_valid


def collate_multi_modal_inputs(rows, device=None) -> dict:
    """One dict of tensors for a micro-batch from its rows' processor outputs (``pixel_values``, ``image_grid_thw``,
    ``pixel_values_videos``, ...): every key is concatenated along its first dimension in row order; rows without
    images contribute nothing. Parity target: the reference's ``multi_modal_inputs`` handling in
    ``verl/workers/utils/padding.py`` / ``verl/utils/model.py`` (``extract_multi_modal_inputs``)."""
    out: dict[str, list] = {}
    for r in rows:
        if not r:
            continue
        for k, v in r.items():
            if isinstance(v, torch.Tensor):
                out.setdefault(k, []).append(v)
    return {k: torch.cat(v, 0).to(device) if device is not None else torch.cat(v, 0) for k, v in out.items()}


def prompt_group_ids(input_ids: torch.Tensor, attention_mask: torch.Tensor, response_length: int) -> list[int]:
    """Group id per row: consecutive rows with an identical (left-padded) prompt belong to one group."""
    P = input_ids.shape[1] - response_length
    if input_ids.shape[0] <= 1:
        return [0] * input_ids.shape[0]
    same = (input_ids[1:, :P] == input_ids[:-1, :P]).all(-1) & (attention_mask[1:, :P] == attention_mask[:-1, :P]).all(-1)
    gid = torch.cat([torch.zeros(1, dtype=torch.int64, device=same.device), (~same).to(torch.int64).cumsum(0)])
    return gid.tolist()


def _ranges(segments: list) -> "np.ndarray":
    """Concatenation of ``arange(start, start + n)`` over ``(start, n)`` pairs, built with two array operations."""
    import numpy as np

    if not segments:
        return np.zeros(0, dtype=np.int64)
    seg = np.asarray(segments, dtype=np.int64).reshape(-1, 2)
    starts, lens = seg[:, 0], seg[:, 1]
    total = int(lens.sum())
    if total == 0:
        return np.zeros(0, dtype=np.int64)
    first = np.concatenate([[0], np.cumsum(lens)[:-1]])
    return np.repeat(starts - first, lens) + np.arange(total, dtype=np.int64)


def pack_shared_prefix_batch(input_ids: torch.Tensor, attention_mask: torch.Tensor, position_ids: Optional[torch.Tensor],
                             response_length: int, gids: list[int], plen: Optional[list] = None, rlen: Optional[list] = None):
    """Packing with the prompt of every group stored once (see ``PackedBatch.expand_index``).

    Returns ``(packed_batch, positions_sel, labels_sel, resp_valid)``: ``positions_sel[n]`` is the stream position whose
    output predicts the n-th valid response token (row-major over ``resp_valid``) and ``labels_sel[n]`` that token.
    ``plen`` / ``rlen``: valid prompt / response tokens per row when the caller already has them on the host (saves the
    device synchronisation that reading them from the mask costs). The index arrays are built on the host from a handful
    of (start, length) segments per row and copied over once each."""
    b, L = input_ids.shape
    P = L - response_length
    dev = input_ids.device
    mask = attention_mask.bool()
    if plen is None or rlen is None:
        plen = mask[:, :P].sum(-1).tolist()
        rlen = mask[:, P:].sum(-1).tolist()
    src, expand, collapse, pos_sel, lab_src, lens_e = [], [], [], [], [], []
    t_d = t_e = 0
    i = 0
    while i < b:
        j = i
        while j + 1 < b and gids[j + 1] == gids[i]:
            j += 1
        p = int(plen[i])
        prompt_lo = t_d
        src.append((i * L + P - p, p))                 # the leader's prompt tokens
        collapse.append((t_e, p))                      # represented by the leader's copy
        t_d += p
        for m in range(i, j + 1):
            r = int(rlen[m])
            src.append((m * L + P, r))
            expand.append((prompt_lo, p))
            expand.append((t_d, r))
            collapse.append((t_e + p, r))
            if r > 0:
                pos_sel.append((prompt_lo + p - 1, 1))
                pos_sel.append((t_d, r - 1))
                lab_src.append((m * L + P, r))
            lens_e.append(p + r)
            t_d += r
            t_e += p + r
        i = j + 1
    to_dev = lambda segs: torch.from_numpy(_ranges(segs)).to(dev, non_blocking=True)
    src_t, lab_t = to_dev(src), to_dev(lab_src)
    flat_ids = input_ids.reshape(-1)
    ids_d = flat_ids[src_t]
    if position_ids is None:
        pos_full = (torch.cumsum(mask.to(torch.int32), -1) - 1).reshape(-1)
    else:
        pos_full = position_ids.reshape(-1)
    cu = torch.zeros(len(lens_e) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens_e, dtype=torch.int32), 0)
    batch = PackedBatch(input_ids=ids_d.contiguous(), positions=pos_full[src_t].to(torch.int32).contiguous(), cu_seqlens=cu.to(dev),
                        max_seqlen=max(lens_e) if lens_e else 0, cu_seqlens_cpu=cu, expand_index=to_dev(expand), collapse_index=to_dev(collapse))
    return batch, to_dev(pos_sel), flat_ids[lab_t].contiguous(), mask[:, P:]


class NativeEngine(BaseEngine):
    value_head = False

    def __init__(self, model_config, engine_config, optimizer_config=None, checkpoint_config=None, **kwargs):
        self.model_config = model_config
        self.engine_config = engine_config
        self.optimizer_config = optimizer_config
        self.checkpoint_config = checkpoint_config
        self.arch: ModelConfig = model_config.arch if hasattr(model_config, "arch") else model_config
        self.device_name = get_device_name()
        self.forward_only = bool(getattr(engine_config, "forward_only", False)) or optimizer_config is None
        self.opt_step_count = 0
        self.sched_step = 0
        self._initialized = False
        self.muon = None
        self._shared_params: Optional[FlatParams] = kwargs.get("shared_params")

    # ------------------------------------------------------------------------------------ setup
    def initialize(self) -> None:
        if self._initialized:
            return
        from ....utils.distributed import get_data_parallel_group

        self.group = get_data_parallel_group()  # None = the default (world) group
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self._src0 = dist.get_global_rank(self.group, 0) if (self.group is not None and dist.is_initialized()) else 0
        # Hybrid sharding (``fsdp_size`` = s, 0 < s < data-parallel size): optimizer state and gradient shards are split over
        # blocks of s consecutive ranks and replicated across the blocks; gradients are reduce-scattered inside a block and
        # all-reduced between the blocks. Default: one block = the whole data-parallel group.
        self.sh_group, self.sh_rank, self.sh_world = self.group, self.rank, self.world
        self.rep_group, self.rep_rank, self.rep_world = None, 0, 1
        fs = int(getattr(self.engine_config, "fsdp_size", -1) or -1)
        if 0 < fs < self.world:
            assert self.world % fs == 0, "fsdp_size must divide the data-parallel size"
            pool = dist.get_process_group_ranks(self.group if self.group is not None else dist.group.WORLD)
            for b0 in range(0, self.world, fs):          # collective: every rank creates every group, in the same order
                g = dist.new_group(pool[b0 : b0 + fs])
                if b0 <= self.rank < b0 + fs:
                    self.sh_group, self.sh_rank, self.sh_world = g, self.rank - b0, fs
            for r0 in range(fs):
                g = dist.new_group(pool[r0::fs])
                if self.rank % fs == r0:
                    self.rep_group, self.rep_rank, self.rep_world = g, self.rank // fs, self.world // fs
        if self.device_name == "cuda":
            self.device = torch.device("cuda", torch.cuda.current_device())
            self.dtype = torch.bfloat16
            native.load()
        else:
            self.device = torch.device("cpu")
            self.dtype = torch.float32
        ec = self.engine_config
        seed = int(getattr(ec, "seed", 42))
        self.fused_comm = False
        self.peer_barrier_timeout_s = float(getattr(ec, "peer_barrier_timeout_s", 120.0) or 120.0)
        self._sym_params = self._sym_grads = self._peer_barrier = None
        if self._shared_params is not None:
            self.params = self._shared_params
        else:
            want_fused = (bool(getattr(ec, "fused_comm", True)) and not self.forward_only and self.device.type == "cuda"
                          and not self.arch.is_generic
                          and str(getattr(self.optimizer_config, "optimizer", "AdamW") or "AdamW").lower() != "muon"
                          and not int(getattr(self.model_config, "lora_rank", 0) or 0)
                          and self.world > 1 and self.group is None  # symmetric buffers are bound to the world group
                          and self.rep_world == 1
                          and int(getattr(ec, "zero_stage", 2) or 2) != 3  # sharded working weights have their own peer-memory path
                          and os.environ.get("VERL_B200_FUSED_COMM", "1") != "0")
            buf = None
            if want_fused:
                from ....parallel.symmetric import PeerBarrier, SymmetricBuffer, symmetric_available

                if symmetric_available():
                    probe = FlatParams(self.arch, dtype=self.dtype, device="meta", value_head=self.value_head, pad_to=self.sh_world)
                    self._sym_params = SymmetricBuffer.allocate(probe.numel, self.dtype, self.device)
                    self._sym_grads = SymmetricBuffer.allocate(probe.numel, torch.float32, self.device)
                    self._peer_barrier = PeerBarrier(self.device)
                    buf = self._sym_params.tensor
                    self.fused_comm = True
            if self.arch.is_generic:
                # an architecture without a hand-scheduled decoder: a library module whose parameters live in the flat buffer
                from ....models.generic import ModuleFlatParams

                self.params = ModuleFlatParams(self.arch, dtype=self.dtype, device=self.device, value_head=self.value_head,
                                               pad_to=self.sh_world, seed=seed,
                                               attn_implementation=getattr(self.model_config, "attn_implementation", None))
            else:
                self.params = FlatParams(self.arch, dtype=self.dtype, device=self.device, value_head=self.value_head,
                                         pad_to=self.sh_world, buffer=buf)
            self._load_or_init(seed)
        # gradient checkpointing: "auto" keeps the activations of as many trailing layers as free memory allows and
        # recomputes the rest (all of them when memory is short, none when everything fits)
        recompute = "none" if not getattr(ec, "enable_gradient_checkpointing", True) else \
            str(os.environ.get("VERL_B200_RECOMPUTE", getattr(ec, "recompute_granularity", None) or "auto"))
        if self.arch.is_generic:
            from ....models.generic import GenericCausalLM

            assert int(getattr(self.model_config, "lora_rank", 0) or 0) == 0 and int(getattr(ec, "ulysses_sequence_parallel_size", 1) or 1) == 1, \
                "LoRA and sequence parallelism need one of the natively supported model families"
            self.model = GenericCausalLM(self.arch, self.params, recompute=recompute)
        else:
            self.model = DecoderModel(self.arch, self.params, recompute=recompute)
        self.model.keep_layers_fn = self._layers_that_fit
        tm = getattr(self.model_config, "tiled_mlp", None) or {}
        if (tm.get("enabled") if hasattr(tm, "get") else getattr(tm, "enabled", False)):
            shards = int((tm.get("num_shards") if hasattr(tm, "get") else getattr(tm, "num_shards", 4)) or 4)
            budget = int(getattr(ec, "max_token_len_per_gpu", 0) or 8192)
            self.model.mlp_tile_tokens = max(128, -(-budget // shards) // 128 * 128)
        # trainable parameters: the whole model, or low-rank adapters on a frozen base (``model.lora_rank`` > 0)
        self.tparams = self.params
        self.lora = None
        lora_rank = int(getattr(self.model_config, "lora_rank", 0) or 0)
        if lora_rank > 0 and not self.forward_only:
            from ....models.lora import LoRAParams

            assert not self.fused_comm, "LoRA uses the collective-library optimizer path (set fused_comm=false)"
            self.lora = LoRAParams(self.params, lora_rank, float(getattr(self.model_config, "lora_alpha", 16) or 16),
                                   getattr(self.model_config, "target_modules", None), pad_to=self.sh_world, seed=seed)
            self.tparams = self.lora
        # Ulysses sequence parallelism: blocks of ``sp`` consecutive ranks work on the same micro-batches
        self.sp_size = int(getattr(ec, "ulysses_sequence_parallel_size", 1) or 1)
        self.cp_size = int(getattr(ec, "context_parallel_size", 1) or 1)
        assert self.sp_size == 1 or self.cp_size == 1, "Ulysses sequence parallelism and context parallelism are exclusive"
        if self.cp_size > 1:
            # same placement and micro-batch handling as Ulysses (a block of ranks shares its micro-batches and splits their
            # tokens); only the exchange around attention differs
            assert not self.arch.is_generic, "context parallelism needs one of the natively supported model families"
            self.sp_size = self.cp_size
        self.sp_group, self.sp_rank = None, 0
        self._dcp_scheduler, self._dcp = None, {}
        if self.sp_size > 1:
            assert self.world % self.sp_size == 0 and not self.value_head, "sequence parallel size must divide the data-parallel world"
            assert self.cp_size > 1 or self.arch.num_key_value_heads % self.sp_size == 0, "sequence parallel size must divide the KV heads"
            from ....models.decoder import ContextParallel, UlyssesSequenceParallel

            pool = dist.get_process_group_ranks(self.group if self.group is not None else dist.group.WORLD)
            if self.group is None:
                for g0 in range(0, self.world, self.sp_size):  # collective: every rank creates every group, in the same order
                    grp = dist.new_group(pool[g0 : g0 + self.sp_size])
                    if g0 <= self.rank < g0 + self.sp_size:
                        self.sp_group, self.sp_rank = grp, self.rank - g0
            else:
                # the data-parallel group is itself a sub-group (model-parallel engines): other ranks of the job build
                # different groups at this point, so only the members of a block take part in creating it
                g0 = self.rank // self.sp_size * self.sp_size
                self.sp_group = dist.new_group(pool[g0 : g0 + self.sp_size], use_local_synchronization=True)
                self.sp_rank = self.rank - g0
            if self.cp_size > 1:
                mode = str(getattr(ec, "context_parallel_mode", "zigzag") or "zigzag")
                assert mode in ("zigzag", "contiguous"), f"context_parallel_mode {mode!r}"
                self.model.sp = ContextParallel(self.sp_group, self.sp_rank, self.sp_size, zigzag=(mode == "zigzag"))
                if bool(getattr(ec, "dynamic_context_parallel", False)):
                    # a group size per row: one ContextParallel object (and process group) per power-of-two size and aligned
                    # window of the block; the scheduler says which one a micro-batch uses on this rank
                    from ....utils.dynamic_cp_scheduler import DynamicCPScheduler

                    C = self.sp_size
                    self._dcp_scheduler = DynamicCPScheduler(int(getattr(ec, "max_seqlen_per_dp_cp_rank", 4096)), C)
                    self._dcp = {C: (self.model.sp, self.sp_group, self.sp_rank), 1: (None, None, 0)}
                    size = C // 2
                    while size >= 2:
                        if self.group is None:   # collective creation: every rank walks every block and window
                            for g0 in range(0, self.world, size):
                                grp = dist.new_group(pool[g0 : g0 + size])
                                if g0 <= self.rank < g0 + size:
                                    self._dcp[size] = (ContextParallel(grp, self.rank - g0, size, zigzag=(mode == "zigzag")), grp, self.rank - g0)
                        else:
                            g0 = self.rank // size * size
                            grp = dist.new_group(pool[g0 : g0 + size], use_local_synchronization=True)
                            self._dcp[size] = (ContextParallel(grp, self.rank - g0, size, zigzag=(mode == "zigzag")), grp, self.rank - g0)
                        size //= 2
            else:
                self.model.sp = UlyssesSequenceParallel(self.sp_group, self.sp_rank, self.sp_size)
        # the block of ranks that holds the same rows (with dynamic context parallelism ``sp_size`` / ``sp_group`` / ``sp_rank``
        # follow the group of the micro-batch at hand; the block itself does not change)
        self._blk_size, self._blk_rank = self.sp_size, self.sp_rank
        # shared-prompt packing of GRPO groups (same results, fewer tokens through every projection and MLP)
        self._share_prefix = (bool(getattr(ec, "use_prefix_grouper", True)) and os.environ.get("VERL_B200_SHARE_PREFIX", "1") != "0"
                              and self.sp_size == 1 and not self.arch.is_generic)
        if bool(getattr(ec, "enable_activation_offload", False)) and not self.forward_only:
            from ....utils.activation_offload import ActivationOffloader

            self.model.offloader = ActivationOffloader(self.device)
        # zero_stage=3: the bf16 working weights are sharded too (per unit: embedding, each layer, head) and gathered unit by
        # unit around their use; gradients are reduce-scattered per unit as the backward pass leaves it
        self.zero3 = int(getattr(ec, "zero_stage", 2) or 2) == 3 and self._shared_params is None
        if self.zero3:
            self._shard_working_weights()
        # The replicated region [0, dense_numel) is optimised in equal shards over the data-parallel group; a rank-local tail
        # region (the experts of an expert-parallel shard) is optimised whole by its owner.
        self.dense_numel = int(getattr(self.tparams, "dense_numel", self.tparams.numel))
        self.local_numel = self.tparams.numel - self.dense_numel
        self.shard_numel = self.dense_numel // self.sh_world
        self.shard_lo = self.sh_rank * self.shard_numel
        if self.zero3:  # this rank's slices of every unit, contiguous in its own store
            self.dense_numel = self.shard_numel = self.tparams.owned_numel
            self.local_numel = self.shard_lo = 0
        assert self.local_numel == 0 or (self.world > 1 and not self.fused_comm and self.lora is None and self.rep_world == 1)
        # The fp32 gradient buffer only lives from optimizer_zero_grad() to the end of optimizer_step(), so its
        # memory (4 bytes/param) is available to the rollout KV cache in between.
        self.lazy_grad = bool(getattr(ec, "lazy_grad_buffer", self.device.type == "cuda")) and not self.fused_comm
        if not self.forward_only:
            opt_name = str(getattr(self.optimizer_config, "optimizer", "AdamW") or "AdamW")
            if opt_name.lower() not in ("adamw", "adam", "fusedadam", "fused_adamw", "muon"):
                raise NotImplementedError(f"optimizer {opt_name!r}: this engine implements the sharded fused AdamW "
                                          f"(decoupled weight decay; weight_decay=0 gives Adam) and Muon")
            self.muon = None
            if opt_name.lower() == "muon":
                from .muon import MuonPlan

                assert self.lora is None and not self.fused_comm and self.local_numel == 0 and self.rep_world == 1, \
                    "Muon runs on the full-parameter, collective-library optimizer path without hybrid sharding"
                self.muon = MuonPlan(self.tparams, world=self.sh_world,
                                     split_qkv=bool(getattr(self.optimizer_config, "muon_split_qkv", True)))
                self._muon_mask = self.muon.mask(self.shard_lo, self.shard_lo + self.shard_numel, self.device)
            self.master = self._owned(self.tparams.flat).float()
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)
            self._setup_optimizer_offload()
            self.grad_shard = None
            self.ctrl = torch.zeros(4, dtype=torch.float32, device=self.device)
            if not self.lazy_grad:
                self._alloc_grads()
        # quantisation-aware training: working weights = fake-quantised master weights (master stays full precision)
        from ....utils.qat import QATConfig

        self.qat = QATConfig.from_any(getattr(ec, "qat", None))
        self._qat_names = None
        if self.qat.enable and self._shared_params is None:
            assert self.lora is None, "QAT and LoRA are exclusive"
            self._apply_qat()
        self._setup_param_offload()
        self._initialized = True

    def _shard_working_weights(self) -> None:
        """Replace the full working buffer by this rank's slices (``UnitShardedParams``) and hook the decoder's unit
        boundaries to its prefetch / gradient-reduction logic. The full buffer exists once, during initialisation."""
        from ....models.sharded_weights import UnitShardedParams

        assert not self.arch.is_generic and self.lora is None and self.rep_world == 1 and not self.fused_comm, \
            "zero_stage=3 supports the hand-scheduled model families without LoRA, hybrid sharding or the peer-memory optimizer"
        assert self.sp_size == 1 and not getattr(self.arch, "num_local_experts", 0), \
            "zero_stage=3 does not combine with sequence / context / expert parallelism"
        assert str(getattr(self.optimizer_config, "optimizer", "AdamW") or "AdamW").lower() != "muon", "zero_stage=3 runs AdamW"
        full = self.params
        # on GPUs with peer-mapped memory the units are gathered by the GEMM kernels themselves (fetch warps), else by a
        # collective on a side stream
        fused = False
        if self.device.type == "cuda" and self.world > 1 and self.group is None and os.environ.get("VERL_B200_ZERO3_FUSED", "1") != "0":
            from ....parallel.symmetric import symmetric_available

            fused = symmetric_available() and bool(getattr(self.engine_config, "fused_comm", True))
        self.zero3_fused_gather = fused
        sharded = UnitShardedParams(full, group=self.sh_group, device=self.device, dtype=self.dtype, symmetric=fused)
        sharded.load_from_full(full.flat)
        self.params = self.tparams = sharded
        self.model.params = sharded
        self.model.pre_layer_hook = sharded.pre_layer_hook
        self.model.post_layer_backward_hook = sharded.post_layer_backward_hook
        del full
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def gather_full_params(self, out: Optional[FlatParams] = None, dtype=None) -> FlatParams:
        """The whole model in the full flat layout on this rank (collective when the weights are sharded): what the
        colocated rollout engine, the reference policy's initial copy and merged exports read."""
        if self.zero3:
            return self.params.materialize_full(out)
        if out is not None:
            out.flat.copy_(self.params.flat)
            return out
        return self.params

    def _load_or_init(self, seed: int) -> None:
        mc = self.model_config
        path = getattr(mc, "local_path", None) or getattr(mc, "path", None)
        load = bool(getattr(mc, "load_weights", True)) and path and os.path.isdir(str(path))
        if load and self.rank == 0:
            from ....utils.model import load_hf_weights_into

            load_hf_weights_into(self.params, path)
        elif not load:
            self.params.init_weights(seed=seed)
        if self.world > 1:
            dist.broadcast(self.params.flat, src=self._src0, group=self.group)

    def _layers_that_fit(self, num_tokens: int) -> int:
        """How many layers can keep their activations for a micro-batch of ``num_tokens`` packed tokens: 60 % of what is
        free now (driver-free plus the allocator's cached-but-unused blocks), the rest stays for the LM-head chunks,
        attention workspaces and the gradient buffers that appear later in the step."""
        per_layer = self.model.activation_bytes_per_layer(num_tokens)
        if self.device.type != "cuda":
            return self.arch.num_hidden_layers
        free, _ = torch.cuda.mem_get_info(self.device)
        free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        if self.lazy_grad and getattr(self.tparams, "main_grad", None) is None:
            free -= self.tparams.numel * 4  # the fp32 gradient buffer is allocated on the first backward
        keep = int(0.6 * max(0, free) // max(1, per_layer))
        if getattr(self.model, "ep", None) is not None:
            # expert-parallel layers exchange tokens in forward, recompute and backward: every rank must make the same choice
            t = torch.tensor([keep], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.model.ep.group)
            keep = int(t.item())
        self.last_kept_layers = keep
        return keep


    # ------------------------------------------------------------------------------------ host offload
    _offloaded_states: tuple = ()  # names of the optimizer tensors that live in host memory

    def _setup_optimizer_offload(self) -> None:
        """``optimizer_offload``: the Adam moments live in pinned host memory and pass through the GPU in chunks during
        the optimizer step (copy in, fused AdamW, copy out on three streams, so both directions of the host link and the
        update kernel overlap). ``param_offload`` of a trainable engine adds the fp32 master weights. The memory goes to
        activations: with the moments of a 7B model on the host a single GPU keeps every layer's activations instead of
        recomputing most layers. Parity target: ``verl/utils/fsdp_utils.py`` (``offload_fsdp_optimizer`` /
        ``load_fsdp_optimizer``: whole-state copies before and after the step)."""
        ec = self.engine_config
        self._offloaded_states: tuple = ()
        self._stage: dict = {}
        if not bool(getattr(ec, "optimizer_offload", False)):
            return
        if self.muon is not None or self.fused_comm or self.zero3 or self.lora is not None or self.local_numel:
            logger.warning("optimizer_offload is implemented for the plain sharded AdamW path; keeping the optimizer state on the device")
            return
        which = str(getattr(ec, "optimizer_offload_states", "moments") or "moments")
        assert which in ("moments", "exp_avg", "exp_avg_sq"), f"optimizer_offload_states={which!r}"
        names = ["exp_avg", "exp_avg_sq"] if which == "moments" else [which]
        qat = getattr(ec, "qat", None) or {}
        if bool(getattr(ec, "param_offload", False)) and not bool(qat.get("enable", False) if hasattr(qat, "get") else getattr(qat, "enable", False)):
            names.append("master")
        cuda = self.device.type == "cuda"
        if cuda and not _host_has_room(sum(getattr(self, nm).numel() * 4 for nm in names)):
            logger.warning("optimizer_offload: not enough free host memory for the optimizer state; keeping it on the device")
            return
        host = {}
        try:
            for nm in names:
                t = getattr(self, nm)
                host[nm] = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=cuda)
                host[nm].copy_(t)
        except RuntimeError as e:  # page-locking that much memory was refused
            logger.warning("optimizer_offload: %s; keeping the optimizer state on the device", e)
            return
        for nm in names:
            setattr(self, nm, host[nm])
        del t, host
        self._offloaded_states = tuple(names)
        self.offload_chunk_elems = int(os.environ.get("VERL_B200_OFFLOAD_CHUNK", 32 << 20))
        if cuda:
            torch.cuda.empty_cache()
            self._offload_streams = (torch.cuda.Stream(self.device), torch.cuda.Stream(self.device))
            c = min(self.offload_chunk_elems, max(1, self.master.numel()))
            self._stage = {nm: [torch.empty(c, dtype=torch.float32, device=self.device) for _ in range(2)] for nm in names}

    def _offload_sync(self) -> None:
        """Host copies of the offloaded state are complete (before anything on the host reads them)."""
        if self._offloaded_states and self.device.type == "cuda":
            self._offload_streams[1].synchronize()

    def _streamed_adamw(self, own: slice, dst: Optional[slice], lr: float, coef: Optional[float] = None) -> None:
        """AdamW over the owned range ``own`` with part of the state on the host: chunk by chunk, two staging buffers per
        offloaded tensor. ``dst``: where the bf16 working weights of the range go (device path; the kernel writes them)."""
        oc = self.optimizer_config
        b1, b2 = float(oc.betas[0]), float(oc.betas[1])
        names, C = self._offloaded_states, self.offload_chunk_elems
        cuda = self.device.type == "cuda"
        if cuda:
            ops = native.ops()
            cur = torch.cuda.current_stream(self.device)
            s_in, s_out = self._offload_streams
            s_in.wait_stream(s_out)  # the previous step's copies to the host are complete before its staging buffers are reused
            s_in.wait_stream(cur)
            out_done: list = [None, None]
        for ci, lo in enumerate(range(own.start, own.stop, C)):
            hi = min(lo + C, own.stop)
            k, b = hi - lo, ci % 2
            part = {nm: getattr(self, nm)[lo:hi] for nm in ("master", "exp_avg", "exp_avg_sq")}
            if not cuda:
                g = self.grad_shard[lo:hi] * coef
                part["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                part["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1, bc2 = 1 - b1 ** self.opt_step_count, 1 - b2 ** self.opt_step_count
                part["master"].mul_(1 - lr * oc.weight_decay)
                part["master"].addcdiv_(part["exp_avg"], (part["exp_avg_sq"].sqrt() / math.sqrt(bc2)).add_(oc.eps), value=-lr / bc1)
                continue
            with torch.cuda.stream(s_in):
                if out_done[b] is not None:
                    s_in.wait_event(out_done[b])
                for nm in names:
                    self._stage[nm][b][:k].copy_(part[nm], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            dev = {nm: (self._stage[nm][b][:k] if nm in names else part[nm]) for nm in part}
            d0 = dst.start + (lo - own.start)
            ops.adamw_(dev["master"], self.grad_shard[lo:hi], dev["exp_avg"], dev["exp_avg_sq"], self.tparams.flat[d0 : d0 + k],
                       self.ctrl, lr, b1, b2, float(oc.eps), float(oc.weight_decay), self.opt_step_count, 1.0, False)
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for nm in names:
                    part[nm].copy_(self._stage[nm][b][:k], non_blocking=True)
                out_done[b] = torch.cuda.Event()
                out_done[b].record(s_out)

    def _setup_param_offload(self) -> None:
        """``param_offload`` of a forward-only engine (the reference policy): the working weights wait in pinned host memory
        and occupy the device only inside ``eval_mode()``. The parameter views stay valid: the buffer's storage is emptied
        and refilled in place. Parity target: ``verl/utils/fsdp_utils.py`` (``offload_fsdp_model_to_cpu`` /
        ``load_fsdp_model_to_gpu``)."""
        self._param_host = None
        if not (self.forward_only and bool(getattr(self.engine_config, "param_offload", False)) and self.device.type == "cuda"):
            return
        if self._shared_params is not None or self.arch.is_generic:
            return  # weights that another engine owns stay where their owner keeps them
        if not _host_has_room(self.params.flat.numel() * self.params.flat.element_size()):
            logger.warning("param_offload: not enough free host memory for the weights; keeping them on the device")
            return
        try:
            self._param_host = torch.empty(self.params.flat.shape, dtype=self.params.flat.dtype, device="cpu", pin_memory=True)
        except RuntimeError as e:
            logger.warning("param_offload: %s; keeping the weights on the device", e)
            self._param_host = None
            return
        self._param_resident = True
        self._param_dirty = True  # the device copy holds values the host copy has not seen

    def _enter_mode(self, mode: str, **kwargs) -> None:
        if getattr(self, "_param_host", None) is not None and not self._param_resident:
            flat = self.params.flat
            flat.untyped_storage().resize_(self._param_host.numel() * self._param_host.element_size())
            flat.copy_(self._param_host, non_blocking=True)
            self._param_resident = True

    def _exit_mode(self, mode: str, **kwargs) -> None:
        if getattr(self, "_param_host", None) is not None and self._param_resident:
            if self._param_dirty:
                self._param_host.copy_(self.params.flat)
                self._param_dirty = False
            torch.cuda.current_stream(self.device).synchronize()
            self.params.flat.untyped_storage().resize_(0)
            self._param_resident = False

    def mark_params_changed(self) -> None:
        """The device weights were overwritten from outside (a checkpoint, a weight hand-over): the host copy is stale."""
        if getattr(self, "_param_host", None) is not None:
            assert self._param_resident, "write the weights inside eval_mode(): they are on the host now"
            self._param_dirty = True

    # ------------------------------------------------------------------------------------ topology
    def get_data_parallel_size(self) -> int:
        return self.world

    def get_data_parallel_rank(self) -> int:
        return self.rank

    def get_data_parallel_group(self):
        return self.group

    # ------------------------------------------------------------------------------------ batching
    def _micro_batches(self, data: dict, forward_only: bool) -> list[dict]:
        ec = self.engine_config
        ids = data["input_ids"]
        n = ids.shape[0]
        dyn = bool(data.get("use_dynamic_bsz", getattr(ec, "use_dynamic_bsz", False)))
        if self._dcp_scheduler is not None:
            return self._dynamic_cp_micro_batches(data)
        share = self._share_prefix and "responses" in data and not self.value_head
        gids_all = prompt_group_ids(ids, data["attention_mask"], data["responses"].shape[1]) if share else None
        if share and len(set(gids_all)) == len(gids_all):
            share, gids_all = False, None  # no two rows share a prompt
        if share:
            # whole groups per micro-batch, in order, under the token budget counted on the de-duplicated stream
            P = ids.shape[1] - data["responses"].shape[1]
            pl = data["attention_mask"][:, :P].sum(-1).tolist()
            rl = data["attention_mask"][:, P:].sum(-1).tolist()
            budget = int(data.get("max_token_len_per_gpu") or (ec.infer_max_token_len_per_gpu if forward_only else ec.max_token_len_per_gpu)) \
                if dyn else None
            cap_rows = None if dyn else int(data.get("micro_batch_size_per_gpu") or (ec.infer_micro_batch_size_per_gpu if forward_only
                                                                                    else ec.micro_batch_size_per_gpu) or n)
            parts, cur, cur_tok = [], [], 0
            i = 0
            while i < n:
                j = i
                while j + 1 < n and gids_all[j + 1] == gids_all[i]:
                    j += 1
                rows_g = list(range(i, j + 1))
                tok_g = pl[i] + sum(rl[i : j + 1])
                full = (budget is not None and cur and cur_tok + tok_g > budget) or (cap_rows is not None and cur and len(cur) + len(rows_g) > cap_rows)
                if full:
                    parts.append(cur)
                    cur, cur_tok = [], 0
                cur += rows_g
                cur_tok += tok_g
                i = j + 1
            if cur:
                parts.append(cur)
        elif dyn:
            budget = int(data.get("max_token_len_per_gpu") or (ec.infer_max_token_len_per_gpu if forward_only
                                                               else ec.max_token_len_per_gpu))
            from ....utils.seqlen_balancing import get_seqlen_balanced_partitions

            lens = data["attention_mask"].sum(-1).tolist()
            k = max(1, min(n, math.ceil(sum(lens) / budget)))
            parts = get_seqlen_balanced_partitions(lens, k, equal_size=False)
        else:
            mb = data.get("micro_batch_size_per_gpu") or (ec.infer_micro_batch_size_per_gpu if forward_only
                                                          else ec.micro_batch_size_per_gpu) or n
            parts = [list(range(s, min(n, s + int(mb)))) for s in range(0, n, int(mb))]
        if getattr(self.model, "ep", None) is not None:
            # every rank of an expert-parallel group must run the same number of micro-batches (each one is a round of
            # collectives): split the largest parts until the counts agree
            t = torch.tensor([len(parts)], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.model.ep.group)
            assert n >= int(t.item()), "fewer rows than micro-batches on another rank of the expert-parallel group"
            while len(parts) < int(t.item()):
                j = max(range(len(parts)), key=lambda i: len(parts[i]))
                big = parts.pop(j)
                parts[j:j] = [big[: len(big) // 2], big[len(big) // 2 :]]
        out = []
        for p in parts:
            idx = torch.tensor(p, dtype=torch.int64, device=ids.device)
            mb = {k: (v[idx] if isinstance(v, torch.Tensor) and v.dim() > 0 and v.shape[0] == n else v)
                  for k, v in data.items()} | {"_rows": p} | ({"_gids": [gids_all[r] for r in p]} if share else {})
            if share:      # lengths already read for the split: the packing of each micro-batch reuses them
                mb["_plen"], mb["_rlen"] = [pl[r] for r in p], [rl[r] for r in p]
            elif dyn:
                mb["_lens"] = [lens[r] for r in p]
            if mb.get("multi_modal_inputs") is not None:   # per-row processor outputs (vision-language models)
                mb["multi_modal_inputs"] = [data["multi_modal_inputs"][r] for r in p]
            out.append(mb)
        return out

    def _dynamic_cp_micro_batches(self, data: dict) -> list[dict]:
        """Micro-batches of dynamic context parallelism: the scheduler packs the block's rows (every rank of the block holds
        all of them) into micro-batches of per-row groups; this rank keeps the ones it takes part in. ``_dcp`` = size of the
        group that works on the micro-batch, ``_dcp_leader`` = this rank reports the group's outputs to the block."""
        ids = data["input_ids"]
        n = ids.shape[0]
        lens = [int(x) for x in data["attention_mask"].sum(-1).tolist()]
        plan = self._dcp_scheduler.schedule(lens)
        self.last_dcp_plan = plan
        out = []
        for ranks in plan:
            a = ranks[self._blk_rank]
            if not a.rows:
                continue
            idx = torch.tensor(a.rows, dtype=torch.int64, device=ids.device)
            mb = {k: (v[idx] if isinstance(v, torch.Tensor) and v.dim() > 0 and v.shape[0] == n else v) for k, v in data.items()}
            mb.update(_rows=list(a.rows), _dcp=a.size, _dcp_leader=self._blk_rank == a.start, _lens=[lens[r] for r in a.rows])
            out.append(mb)
        return out

    def forward_backward_batch(self, data, loss_function: Optional[Callable] = None, forward_only: bool = False) -> dict:
        """``data``: dict-like with padded ``input_ids``/``attention_mask``/``position_ids`` [b, P+R], ``responses``
        [b, R] and whatever the loss function needs.  Returns ``{"model_output": {...}, "loss": ..., "metrics": ...}``
        with per-row outputs restored to the input order."""
        data = dict(data.items()) if not isinstance(data, dict) else data
        data = {k: (v.to(self.device, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in data.items()}
        R = data["responses"].shape[1]
        n = data["input_ids"].shape[0]
        temperature = float(data.get("temperature", 1.0))
        calc_entropy = bool(data.get("calculate_entropy", False))
        # global normalisation constants for agg_loss
        if loss_function is not None and not forward_only:
            mask = data.get("response_mask", data["attention_mask"][:, -R:])
            tok = mask.sum().float()
            seqs = torch.tensor(float(n), device=self.device)
            if self.world > 1:
                pack = torch.stack([tok, seqs])
                dist.all_reduce(pack, group=self.group)
                tok, seqs = pack[0] / self._blk_size, pack[1] / self._blk_size  # the ranks of a sequence-parallel block hold the same rows
            data["global_batch_info"] = dict(dp_size=self.world, batch_num_tokens=tok, global_batch_size=seqs,
                                             loss_scale_factor=data.get("loss_scale_factor"))
        mbs = self._micro_batches(data, forward_only)
        outs, rows, losses, metrics = self._run_micro_batches(mbs, R, temperature, calc_entropy, loss_function, forward_only)
        if self._dcp_scheduler is not None:
            self.sp_size = self._blk_size      # back to the block: what other code sees between passes
            self.model.sp, self.sp_group, self.sp_rank = self._dcp[self._blk_size]
            model_output = self._dynamic_cp_collect(mbs, outs, n, R, calc_entropy or not forward_only)
        else:
            inv = torch.empty(n, dtype=torch.int64, device=self.device)
            inv[torch.tensor(rows, dtype=torch.int64, device=self.device)] = torch.arange(n, device=self.device)
            model_output = {k: torch.cat(v, 0)[inv] for k, v in outs.items()}
        result = {"model_output": model_output, "metrics": metrics}
        if losses:
            result["loss"] = torch.stack(losses).sum()
        return result

    def _dynamic_cp_collect(self, mbs: list[dict], outs: dict, n: int, R: int, with_entropy: bool) -> dict:
        """Per-row outputs of the whole block on every rank of it: each group's first rank writes the rows its group worked
        on into a zeroed [n, R] tensor, the block sums them (every row was computed by exactly one group)."""
        keys = ["log_probs"] + (["entropy"] if with_entropy else [])
        full = {k: torch.zeros(n, R, dtype=torch.float32, device=self.device) for k in keys}
        for i, mb in enumerate(mbs):
            if not mb["_dcp_leader"]:
                continue
            idx = torch.tensor(mb["_rows"], dtype=torch.int64, device=self.device)
            for k in keys:
                full[k][idx] = outs[k][i].float()
        stacked = torch.stack([full[k] for k in keys])
        dist.all_reduce(stacked, group=self._dcp[self._dcp_scheduler.cp_size][1])
        return {k: stacked[j] for j, k in enumerate(keys)}

    def _run_micro_batches(self, mbs: list[dict], R: int, temperature: float, calc_entropy: bool, loss_function, forward_only: bool):
        """Forward (+ loss + backward) of every micro-batch; model-parallel engines override this with their schedule."""
        outs: dict[str, list] = {}
        rows: list[int] = []
        losses, metrics = [], {}
        for mb in mbs:
            out = self._forward_micro(mb, R, temperature, calc_entropy, need_grad=not forward_only)
            rows.extend(mb["_rows"])
            if loss_function is not None:
                loss, m = loss_function(model_output=out, data=mb, dp_group=None)
                if not forward_only:
                    loss.backward()
                losses.append(loss.detach())
                for k, v in m.items():
                    metrics.setdefault(k, []).append(v)
            for k, v in out.items():
                outs.setdefault(k, []).append(v.detach())
        return outs, rows, losses, metrics

    def _forward_micro(self, mb: dict, R: int, temperature: float, calc_entropy: bool, need_grad: bool) -> dict:
        if "_dcp" in mb:
            # dynamic context parallelism: this micro-batch runs in the group the scheduler chose for its rows (the decoder
            # reads ``model.sp`` in the forward pass and in the backward pass that follows before the next micro-batch)
            self.model.sp, self.sp_group, self.sp_rank = self._dcp[mb["_dcp"]]
            self.sp_size = mb["_dcp"]
        gids = mb.get("_gids")
        replay_or_record = self.arch.is_moe and (mb.get("routed_experts") is not None or (bool(mb.get("record_routing", False)) and not need_grad))
        shared = (gids is not None and len(set(gids)) < len(gids) and self.model.tp is None and self.sp_size == 1
                  and not replay_or_record)
        if shared:
            # members of a group share their prompt: it is embedded, projected and fed through the MLPs once
            batch, positions, position_labels, resp_valid = pack_shared_prefix_batch(
                mb["input_ids"], mb["attention_mask"], mb.get("position_ids"), R, gids, mb.get("_plen"), mb.get("_rlen"))
            labels = None
        else:
            lens = mb.get("_lens")
            if lens is None and mb.get("_plen") is not None:
                lens = [a + b for a, b in zip(mb["_plen"], mb["_rlen"])]
            batch, labels, resp_index, resp_valid = pack_padded_batch(mb["input_ids"], mb["attention_mask"],
                                                                      mb.get("position_ids"), R, lens)
            # the LM head (a third of a 7B forward's head+tail work at vocabulary 152k) runs only where a response token is
            # predicted: prompt positions never enter a loss or a returned log-prob
            if self.sp_size > 1:
                return self._forward_micro_sp(batch, labels, resp_index, resp_valid, temperature, calc_entropy, need_grad)
            positions = resp_index[resp_valid]
            position_labels = None
        # router replay (mixture-of-experts): take every router's expert choice from the batch, or record it for the batch
        replay = mb.get("routed_experts") if self.arch.is_moe else None
        record = bool(mb.get("record_routing", False)) and self.arch.is_moe and not need_grad
        self.model.router_replay = None
        if replay is not None or record:
            from ....models.decoder import RouterReplay

            gids = None  # the stored choices are laid out per row: no shared-prefix packing for this micro-batch
            moe_layers = list(range(self.arch.num_hidden_layers))
            mask = mb["attention_mask"].bool()
            self.model.router_replay = (RouterReplay.from_tokens(replay[mask], moe_layers) if replay is not None
                                        else RouterReplay("record"))
        extra = {}
        if mb.get("multi_modal_inputs") is not None:
            assert self.arch.is_multimodal, "multi_modal_inputs need a vision-language architecture"
            extra["mm_inputs"] = collate_multi_modal_inputs(mb["multi_modal_inputs"], self.device)
        lp, ent = self.model.forward_logprobs(batch, labels, temperature, need_grad=need_grad, positions=positions,
                                              position_labels=position_labels, **extra)
        out = {"log_probs": torch.zeros(resp_valid.shape, dtype=lp.dtype, device=lp.device).masked_scatter(resp_valid, lp)}
        if calc_entropy or need_grad:
            out["entropy"] = torch.zeros(resp_valid.shape, dtype=ent.dtype, device=ent.device).masked_scatter(resp_valid, ent)
        if record:
            routed = self.model.router_replay.stacked(moe_layers)  # [T, layers, k]
            full = torch.zeros(*mask.shape, *routed.shape[1:], dtype=torch.int32, device=routed.device)
            full[mask] = routed.int()
            out["routed_experts"] = full
            self.model.router_replay = None
        return out

    def _forward_micro_sp(self, batch, labels, resp_index, resp_valid, temperature, calc_entropy, need_grad) -> dict:
        """Sequence-parallel micro-batch: this rank evaluates the head on the response positions inside its slice of the
        (padded) token stream; the [b, R] outputs are completed by a sum over the block. Gradients flow only into the
        locally computed entries, which is exactly this rank's share of the block's loss."""
        sp, T = self.model.sp.pad_multiple(), batch.num_tokens
        pad = (-T) % sp
        if pad:
            dev = batch.input_ids.device
            ids = torch.cat([batch.input_ids, batch.input_ids.new_zeros(pad)])
            pos = torch.cat([batch.positions, torch.arange(pad, dtype=batch.positions.dtype, device=dev)])
            cu_cpu = torch.cat([batch.cu_seqlens_cpu, torch.tensor([T + pad], dtype=torch.int32)])
            batch = PackedBatch(input_ids=ids, positions=pos, cu_seqlens=cu_cpu.to(dev), max_seqlen=max(batch.max_seqlen, pad),
                                cu_seqlens_cpu=cu_cpu)
            labels = torch.cat([labels, labels.new_zeros(pad)])
        positions = resp_index[resp_valid]
        mine, local_pos = self.model.sp.local_of(positions, batch.num_tokens)
        lp, ent = self.model.forward_logprobs(batch, labels, temperature, need_grad=need_grad, positions=local_pos,
                                              position_labels=labels[positions[mine]])
        flat_idx = resp_valid.reshape(-1).nonzero().squeeze(-1)[mine]
        n_out = resp_valid.numel()

        def complete(local: torch.Tensor) -> torch.Tensor:
            part = torch.zeros(n_out, dtype=local.dtype, device=local.device).index_copy(0, flat_idx, local)
            total = part.detach().clone()
            dist.all_reduce(total, group=self.sp_group)
            return (part + (total - part.detach())).view(resp_valid.shape)

        out = {"log_probs": complete(lp)}
        if calc_entropy or need_grad:
            out["entropy"] = complete(ent)
        return out

    # ------------------------------------------------------------------------------------ optimizer
    def _owned(self, flat: torch.Tensor) -> torch.Tensor:
        """Copy of the elements of a full-layout buffer that this rank optimises: its shard of the replicated region
        followed by the rank-local region."""
        sl = flat[self.shard_lo : self.shard_lo + self.shard_numel]
        return torch.cat([sl, flat[self.dense_numel :]]) if self.local_numel else sl.clone()

    def _scatter_owned(self, owned: torch.Tensor, flat: torch.Tensor) -> None:
        flat[self.shard_lo : self.shard_lo + self.shard_numel].copy_(owned[: self.shard_numel].to(flat.dtype))
        if self.local_numel:
            flat[self.dense_numel :].copy_(owned[self.shard_numel :].to(flat.dtype))

    def _alloc_grads(self) -> None:
        if self.zero3:
            self.tparams.attach_main_grad()
            self.grad_shard = self.tparams.grad_shard
            return
        self.tparams.attach_main_grad(self._sym_grads.tensor if self.fused_comm else None)
        sl = slice(self.shard_lo, self.shard_lo + self.shard_numel)
        self.grad_shard = self.tparams.main_grad[sl] if self.sh_world == 1 else \
            torch.zeros(self.master.numel(), dtype=torch.float32, device=self.device)

    def _complete_partial_grads(self) -> None:
        """Hook for model-parallel engines: gradients of replicated parameters that every rank of a model-parallel group
        computed from its own part of the work (heads, tokens) are summed over that group before the optimizer sees them."""
        return None

    def _global_sumsq_correction(self) -> None:
        """Hook for model-parallel engines: ``ctrl[0]`` (sum of squared gradients over the data-parallel group) becomes
        the sum over the whole model."""
        return None

    def optimizer_zero_grad(self) -> None:
        if self.forward_only:
            return
        if self.zero3:
            if self.tparams.grad_shard is None:
                self._alloc_grads()
            else:
                self.tparams.zero_grad()
            return
        if self.tparams.main_grad is None:
            self._alloc_grads()
        else:
            self.tparams.zero_grad()

    def optimizer_step(self) -> float:
        """Gradient mean over DP ranks, global-norm clip, AdamW on this rank's shard, publish new bf16 weights.
        A non-finite gradient norm skips the update. Returns the gradient norm."""
        oc = self.optimizer_config
        W = self.world
        mg = self.tparams.main_grad
        sl = slice(self.shard_lo, self.shard_lo + self.shard_numel)
        self._complete_partial_grads()
        if self.fused_comm:
            return self._fused_optimizer_step()
        D, n_sh = self.dense_numel, self.shard_numel
        if self.zero3:
            # every unit's gradient was reduce-scattered (sum) when the backward pass left it; the mean is one scale away
            if W > 1:
                self.grad_shard.mul_(1.0 / W)
        elif W > 1:
            if self.device.type == "cuda":
                if self.sh_world > 1:
                    dist.reduce_scatter_tensor(self.grad_shard[:n_sh], mg[:D], op=dist.ReduceOp.AVG, group=self.sh_group)
                if self.rep_world > 1:  # mean over the replicas of this shard
                    dist.all_reduce(self.grad_shard[:n_sh], op=dist.ReduceOp.AVG, group=self.rep_group)
            else:  # gloo has no reduce-scatter: all-reduce over everyone and keep this rank's slice
                dist.all_reduce(mg[:D], group=self.group)
                if self.sh_world > 1:
                    self.grad_shard[:n_sh].copy_(mg[sl]).div_(W)
                else:
                    mg[:D].div_(W)
            if self.local_numel:
                # rank-local parameters already hold the sum over every rank's tokens; 1/W makes it the same global mean
                torch.mul(mg[D:], 1.0 / W, out=self.grad_shard[n_sh:])
        self.ctrl.zero_()
        lr = self.lr_override if getattr(self, "lr_override", None) is not None else lr_at_step(oc, self.sched_step)
        self.opt_step_count += 1
        if self.muon is not None:
            norm = self._muon_update(lr)
        elif self.device.type == "cuda":
            ops = native.ops()
            ops.sumsq_(self.grad_shard, self.ctrl)
            if self.sh_world > 1:  # replicas hold identical shards: the norm is a sum over one block
                dist.all_reduce(self.ctrl[:1], group=self.sh_group)
            self._global_sumsq_correction()
            ops.clip_coef_(self.ctrl, float(oc.clip_grad))
            for own, dst in ((slice(0, n_sh), sl), (slice(n_sh, n_sh + self.local_numel), slice(D, D + self.local_numel))):
                if own.stop > own.start and self._offloaded_states:
                    self._streamed_adamw(own, dst, lr)
                elif own.stop > own.start:
                    ops.adamw_(self.master[own], self.grad_shard[own], self.exp_avg[own], self.exp_avg_sq[own], self.tparams.flat[dst],
                               self.ctrl, lr, float(oc.betas[0]), float(oc.betas[1]), float(oc.eps), float(oc.weight_decay),
                               self.opt_step_count, 1.0, False)
            norm = self.ctrl[3]
        else:
            ss = self.grad_shard.double().pow(2).sum()
            if self.sh_world > 1:
                dist.all_reduce(ss, group=self.sh_group)
            self.ctrl[0] = ss.float()
            self._global_sumsq_correction()
            ss = self.ctrl[0].double()
            norm = ss.sqrt().float()
            if torch.isfinite(norm):
                coef = min(1.0, float(oc.clip_grad) / (float(norm) + 1e-6)) if oc.clip_grad and oc.clip_grad > 0 else 1.0
                if self._offloaded_states:  # the chunk walk of the offloaded optimizer, with host arithmetic
                    self._streamed_adamw(slice(0, self.master.numel()), None, lr, coef=coef)
                    self._scatter_owned(self.master, self.tparams.flat)
                    coef = None
            if torch.isfinite(norm) and coef is not None:
                g = self.grad_shard * coef
                b1, b2 = oc.betas
                self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
                self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1 = 1 - b1 ** self.opt_step_count
                bc2 = 1 - b2 ** self.opt_step_count
                self.master.mul_(1 - lr * oc.weight_decay)
                denom = (self.exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(oc.eps)
                self.master.addcdiv_(self.exp_avg, denom, value=-lr / bc1)
                self._scatter_owned(self.master, self.tparams.flat)
        self._publish_shard()
        if self.lora is not None:
            self.lora.merge()  # the working weights (shared with the rollout engine) follow the adapters
        if self.qat.enable:
            self._apply_qat()  # fresh bf16 casts of the master weights -> their NVFP4 values
        norm = float(norm)
        if not math.isfinite(norm):
            self.opt_step_count -= 1  # a skipped step does not advance the bias correction
        if self.lazy_grad:
            self.tparams.detach_main_grad()
            self.grad_shard = None
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
        return norm

    def _muon_update(self, lr: float) -> torch.Tensor:
        """Muon on the matrix ranges and AdamW on the rest of this rank's range (``muon.py`` has the step's plan). Expects
        the mean gradient of the owned range in ``grad_shard``; returns the global gradient norm."""
        oc, n_sh, W = self.optimizer_config, self.shard_numel, self.sh_world
        g, mask = self.grad_shard, self._muon_mask
        ss = g.double().pow(2).sum() if self.device.type == "cpu" else g.float().pow(2).sum()
        if W > 1:
            dist.all_reduce(ss, group=self.sh_group)
        self.ctrl[0] = ss.float()
        self._global_sumsq_correction()
        norm = self.ctrl[0].double().sqrt().float()
        if not bool(torch.isfinite(norm)):
            return norm  # skipped step: state and weights stay as they are
        coef = min(1.0, float(oc.clip_grad) / (float(norm) + 1e-6)) if oc.clip_grad and oc.clip_grad > 0 else 1.0
        if coef != 1.0:
            g.mul_(coef)
        b1, b2 = float(oc.betas[0]), float(oc.betas[1])
        mu, nesterov = float(oc.muon_momentum), bool(oc.muon_nesterov)
        # second moment (used on the AdamW ranges only), then one buffer for both kinds of first moment
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        self.exp_avg.mul_(torch.where(mask, mu, b1)).add_(g * torch.where(mask, 1.0, 1 - b1))
        u = torch.where(mask, g + mu * self.exp_avg if nesterov else self.exp_avg, torch.zeros((), device=g.device))
        # whole matrices for the orthogonalisation: gather into the idle full-size gradient buffer
        mg = self.tparams.main_grad
        full = mg[: self.dense_numel]
        if W > 1:
            if self.device.type == "cuda":
                dist.all_gather_into_tensor(full, u.contiguous(), group=self.sh_group)
            else:
                dist.all_gather([full[i * n_sh : (i + 1) * n_sh] for i in range(W)], u.contiguous(), group=self.sh_group)
        else:
            full.copy_(u)
        self.muon.orthogonalise_owned(full, self.sh_rank, int(oc.muon_num_ns_steps), str(oc.muon_coefficient_type),
                                      str(oc.muon_scale_mode))
        if W > 1:
            if self.device.type == "cuda":
                upd = torch.empty_like(u)
                dist.reduce_scatter_tensor(upd, full, op=dist.ReduceOp.SUM, group=self.sh_group)
            else:
                dist.all_reduce(full, group=self.sh_group)
                upd = full[self.shard_lo : self.shard_lo + n_sh]
        else:
            upd = full[self.shard_lo : self.shard_lo + n_sh]
        bc1, bc2 = 1 - b1 ** self.opt_step_count, 1 - b2 ** self.opt_step_count
        denom = (self.exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(float(oc.eps))
        step = torch.where(mask, upd * (lr * oc.muon_update_scale), self.exp_avg / denom * (lr / bc1))
        self.master.mul_(1 - lr * float(oc.weight_decay)).sub_(step)
        self._scatter_owned(self.master, self.tparams.flat)
        return norm

    def _fused_optimizer_step(self) -> float:
        """Peer-memory path: barrier -> reduce-scatter+mean+sumsq kernel (peer loads of this rank's shard of every
        gradient buffer) -> scalar norm all-reduce -> AdamW + all-gather kernel (stores the new bf16 weights into every
        rank's working buffer) -> barrier."""
        oc = self.optimizer_config
        ops = native.ops()
        use_mc = os.environ.get("VERL_B200_MULTIMEM", "0") == "1"
        lr = self.lr_override if getattr(self, "lr_override", None) is not None else lr_at_step(oc, self.sched_step)
        self.opt_step_count += 1
        # The barrier's wait is bounded. If it runs out on this rank (a straggler further behind than the limit), the
        # kernel poisons the squared-norm accumulator with +inf; the sum over ranks below spreads that to every rank,
        # the straggler included once it arrives, so the AdamW kernel takes its non-finite branch everywhere: optimizer
        # state stays untouched and the old weights are republished. Only then does the host read the status and raise.
        self.ctrl.zero_()
        self._peer_barrier(limit_s=self.peer_barrier_timeout_s, poison=self.ctrl[:1])
        ops.rs_sumsq_(self._sym_grads.ptrs, self._sym_grads.multicast_ptr if use_mc else 0, self.grad_shard, self.shard_lo,
                      self.rank, 1.0 / self.world, self.ctrl)
        dist.all_reduce(self.ctrl[:1], group=self.group)
        ops.clip_coef_(self.ctrl, float(oc.clip_grad))
        ops.adamw_allgather_(self.master, self.grad_shard, self.exp_avg, self.exp_avg_sq, self._sym_params.ptrs,
                             self._sym_params.multicast_ptr if use_mc else 0, self.shard_lo, self.rank, self.ctrl, lr,
                             float(oc.betas[0]), float(oc.betas[1]), float(oc.eps), float(oc.weight_decay), self.opt_step_count)
        self._peer_barrier(limit_s=self.peer_barrier_timeout_s)
        norm = float(self.ctrl[3])
        code = int(ops.comm_status())
        if code != 0:
            self.opt_step_count -= 1
            raise RuntimeError(f"peer barrier timed out after {self.peer_barrier_timeout_s:.0f} s (status {code}): a rank did not "
                               f"reach the optimizer step; the update was skipped on every rank, optimizer state is unchanged")
        if not math.isfinite(norm):
            self.opt_step_count -= 1  # skipped step (non-finite gradient here, or a barrier that ran out on a peer)
        if self.qat.enable:
            self._apply_qat()
        return norm

    def _qat_scale_group(self):
        """Group over which sharded weights agree on their per-tensor quantisation scale (tensor-parallel engines)."""
        return None

    def _apply_qat(self) -> None:
        from ....utils.qat import apply_qat_to_params, qat_target_names

        if self._qat_names is None:
            self._qat_names = qat_target_names(self.params, self.qat)
        apply_qat_to_params(self.params, self.qat, self._qat_names, group=self._qat_scale_group())

    def _publish_shard(self) -> None:
        """All-gather this rank's updated slice of the working weights into every replica."""
        if self.zero3:
            self.tparams.invalidate()  # gathered copies of the old weights are stale; the store itself was updated in place
            return
        if self.sh_world == 1:
            return
        sl = slice(self.shard_lo, self.shard_lo + self.shard_numel)
        dense = self.tparams.flat[: self.dense_numel]
        if self.device.type == "cuda":
            dist.all_gather_into_tensor(dense, dense[sl].clone(), group=self.sh_group)
        else:
            parts = [dense[i * self.shard_numel : (i + 1) * self.shard_numel] for i in range(self.sh_world)]
            dist.all_gather(parts, dense[sl].clone(), group=self.sh_group)

    def lr_scheduler_step(self) -> float:
        self.sched_step += 1
        return lr_at_step(self.optimizer_config, self.sched_step)

    # ------------------------------------------------------------------------------------ weights
    def get_per_tensor_param(self, **kwargs) -> Generator[tuple[str, torch.Tensor], None, None]:
        """HF-named views of the working weights (zero-copy; every rank holds the full replica)."""
        yield from self.params.hf_views()

    def to(self, device: str, model: bool = True, optimizer: bool = True, grad: bool = True) -> None:
        """Move optimizer state (and optionally gradients) between GPU and pinned host memory."""
        if self.forward_only or self.device.type != "cuda":
            return
        tgt = torch.device(device) if device != "cuda" else self.device
        if optimizer:
            for name in ("master", "exp_avg", "exp_avg_sq"):
                if name in self._offloaded_states:  # lives on the host for good (optimizer_offload)
                    continue
                t = getattr(self, name)
                if t.device != tgt:
                    setattr(self, name, t.to(tgt, non_blocking=True))
        torch.cuda.synchronize()

    # ------------------------------------------------------------------------------------ checkpoint
    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None, **kwargs) -> None:
        os.makedirs(local_path, exist_ok=True)
        if not self.forward_only:
            self._offload_sync()
        W, r = self.sh_world, self.sh_rank  # replicas of a block hold identical shards: block 0 writes, everyone reads
        if self.rep_rank != 0:
            if self.world > 1:
                dist.barrier(group=self.group)
            return
        contents = list(getattr(self.checkpoint_config, "save_contents", ["model", "optimizer", "extra"]) or [])
        sl = slice(self.shard_lo, self.shard_lo + self.shard_numel)
        # an HF export needs the whole model: gathering it is a collective, so every rank takes part before rank 0 writes
        self._full_for_export = self.gather_full_params() if "hf_model" in contents else None
        if "model" in contents:
            src = self.master if not self.forward_only else self._owned(self.tparams.flat).float()
            torch.save({"flat_shard": src.cpu(), "shard_lo": self.shard_lo, "numel": self.tparams.numel,
                        "shard_numel": self.shard_numel, "dense_numel": self.dense_numel, "local_numel": self.local_numel,
                        **({"layout": "unit_sharded", "ranges": self.tparams.owned_index_ranges(), "numel": self.tparams.numel}
                           if self.zero3 else {}),
                        "offsets": self.tparams.offsets}, os.path.join(local_path, f"model_world_size_{W}_rank_{r}.pt"))
        if "optimizer" in contents and not self.forward_only:
            torch.save({"exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(), "step": self.opt_step_count},
                       os.path.join(local_path, f"optim_world_size_{W}_rank_{r}.pt"))
        if "extra" in contents:
            torch.save({"sched_step": self.sched_step, "rng": torch.get_rng_state(),
                        "cuda_rng": torch.cuda.get_rng_state() if self.device.type == "cuda" else None},
                       os.path.join(local_path, f"extra_state_world_size_{W}_rank_{r}.pt"))
        if self.rank == 0:
            with open(os.path.join(local_path, "fsdp_config.json"), "w") as f:
                json.dump({"FSDP_version": 2, "world_size": W, "layout": "verl_b200.flat", "value_head": self.value_head,
                           "zero_stage": 3 if self.zero3 else 2}, f)
            hf_dir = os.path.join(local_path, "huggingface")
            self.arch.save_pretrained(hf_dir)
            if self.lora is not None:
                self.lora.save_adapter(os.path.join(local_path, "lora_adapter"), str(getattr(self.model_config, "path", "")))
            if "hf_model" in contents:
                from ....utils.model import save_hf_weights

                save_hf_weights(self._full_for_export, hf_dir)
        self._full_for_export = None
        if self.world > 1:
            dist.barrier(group=self.group)
        self._rotate_checkpoints(local_path, max_ckpt_to_keep)

    def _rotate_checkpoints(self, local_path: str, max_ckpt_to_keep: Optional[int]) -> None:
        """Keep at most ``max_ckpt_to_keep`` of the directories this engine has written (oldest removed first, by rank 0,
        after every rank has finished writing the new one). Parity target: ``verl/utils/checkpoint/checkpoint_manager.py``
        (``remove_previous_save_local_path``)."""
        saved = self.__dict__.setdefault("_saved_ckpt_paths", [])
        path = os.path.abspath(local_path)
        if path in saved:
            saved.remove(path)
        saved.append(path)
        if not max_ckpt_to_keep or int(max_ckpt_to_keep) <= 0:
            return
        while len(saved) > int(max_ckpt_to_keep):
            old = saved.pop(0)
            if self.rank == 0 and os.path.isdir(old):
                import shutil

                shutil.rmtree(old, ignore_errors=True)

    def _saved_world_size(self, local_path: str) -> Optional[int]:
        cfg_path = os.path.join(local_path, "fsdp_config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path) as f:
                return int(json.load(f).get("world_size", 0)) or None
        return None

    def _read_owned_range(self, local_path: str, prefix: str, keys: tuple, saved_world: int) -> dict:
        """Rebuild this rank's slice [shard_lo, shard_lo + shard_numel) of the replicated region from the shard files of a
        checkpoint written with another shard world size. Elements beyond the saved region are alignment padding (zero)."""
        lo, n = self.shard_lo, self.shard_numel
        out = {k: torch.zeros(n, dtype=torch.float32) for k in keys}
        meta = {}
        for r0 in range(saved_world):
            path = os.path.join(local_path, f"{prefix}_world_size_{saved_world}_rank_{r0}.pt")
            if not os.path.exists(path):
                raise FileNotFoundError(f"checkpoint shard {path} is missing (the checkpoint records shard world size {saved_world})")
            st = torch.load(path, map_location="cpu", weights_only=False)
            n0 = int(st[keys[0]].numel())
            lo0 = int(st["shard_lo"]) if "shard_lo" in st else r0 * n0
            if int(st.get("local_numel", 0) or 0) != 0:
                raise RuntimeError("a checkpoint with rank-local (expert-parallel) parameters can only be loaded with the shard "
                                   f"world size it was written with ({saved_world})")
            a, b = max(lo, lo0), min(lo + n, lo0 + n0)
            if a < b:
                for k in keys:
                    out[k][a - lo : b - lo].copy_(st[k][a - lo0 : b - lo0])
            meta = {k: v for k, v in st.items() if k not in keys}
        return {**meta, **out}

    def load_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, del_local_after_load: bool = False,
                        **kwargs) -> None:
        if local_path is None:
            return
        if getattr(self, "_param_host", None) is not None:  # weights offloaded to the host: make them resident, the load overwrites them
            self._enter_mode("eval")
            self._param_dirty = True
        self._offload_sync()
        W, r = self.sh_world, self.sh_rank
        contents = list(getattr(self.checkpoint_config, "load_contents", ["model", "optimizer", "extra"]) or [])
        if not os.path.isdir(local_path):
            raise FileNotFoundError(f"checkpoint directory {local_path} does not exist")
        saved_W = self._saved_world_size(local_path)

        def shard_file(prefix: str) -> Optional[str]:
            """This rank's file of the current layout, or None when the checkpoint was sharded differently."""
            path = os.path.join(local_path, f"{prefix}_world_size_{W}_rank_{r}.pt")
            if os.path.exists(path):
                return path
            if saved_W is None or saved_W == W:
                raise FileNotFoundError(
                    f"{path} is missing: load_contents asks for it and the checkpoint "
                    + (f"records shard world size {saved_W}" if saved_W else "has no fsdp_config.json naming its shard world size")
                    + f" (this engine shards over {W})")
            return None

        if "model" in contents:
            mp = shard_file("model")
            if mp is not None:
                st = torch.load(mp, map_location="cpu", weights_only=False)
                if (st.get("layout") == "unit_sharded") != self.zero3:
                    raise RuntimeError(f"checkpoint was written with zero_stage={3 if st.get('layout') == 'unit_sharded' else 2}, this engine "
                                       f"runs zero_stage={3 if self.zero3 else 2}: merge it to HF weights (model_merger) and load those")
                assert st["numel"] == self.tparams.numel and st["shard_lo"] == self.shard_lo, "checkpoint/model layout mismatch"
                owned = st["flat_shard"]
            else:
                if self.local_numel or self.zero3:
                    raise RuntimeError(f"rank-local or unit-sharded parameters: the checkpoint (shard world size {saved_W}) must be loaded "
                                       f"with {saved_W} shards")
                owned = self._read_owned_range(local_path, "model", ("flat_shard",), saved_W)["flat_shard"]
            if not self.forward_only:
                self.master.copy_(owned)
            self._scatter_owned(owned.to(self.device), self.tparams.flat)
            self._publish_shard()
            if self.lora is not None:
                self.lora.merge()
        if "optimizer" in contents and not self.forward_only:
            op = shard_file("optim")
            st = torch.load(op, map_location="cpu", weights_only=False) if op is not None else \
                self._read_owned_range(local_path, "optim", ("exp_avg", "exp_avg_sq"), saved_W)
            self.exp_avg.copy_(st["exp_avg"])
            self.exp_avg_sq.copy_(st["exp_avg_sq"])
            self.opt_step_count = int(st["step"])
        if "extra" in contents:
            ep = os.path.join(local_path, f"extra_state_world_size_{W}_rank_{r}.pt")
            if not os.path.exists(ep):
                if saved_W is None or saved_W == W:
                    raise FileNotFoundError(f"{ep} is missing although load_contents asks for the extra state")
                # another shard world size: the schedule position is shared by all ranks, random streams start afresh
                ep = os.path.join(local_path, f"extra_state_world_size_{saved_W}_rank_0.pt")
                if not os.path.exists(ep):
                    raise FileNotFoundError(f"{ep} is missing (the checkpoint records shard world size {saved_W})")
                self.sched_step = int(torch.load(ep, map_location="cpu", weights_only=False)["sched_step"])
            else:
                st = torch.load(ep, map_location="cpu", weights_only=False)
                self.sched_step = int(st["sched_step"])
                torch.set_rng_state(st["rng"])
                if st.get("cuda_rng") is not None and self.device.type == "cuda":
                    torch.cuda.set_rng_state(st["cuda_rng"])


@EngineRegistry.register(model_type="language_model", backend=["fsdp", "fsdp2", "native", "veomni", "torchtitan", "automodel"],
                         device=["cuda", "cpu"])
class NativeEngineWithLMHead(NativeEngine):
    value_head = False


@EngineRegistry.register(model_type="value_model", backend=["fsdp", "fsdp2", "native", "veomni", "torchtitan", "automodel"],
                         device=["cuda", "cpu"])
class NativeEngineWithValueHead(NativeEngine):
    """Same trunk with a scalar head; ``model_output`` carries ``values`` [b, R] aligned with the responses."""

    value_head = True

    def _forward_micro(self, mb: dict, R: int, temperature: float, calc_entropy: bool, need_grad: bool) -> dict:
        batch, labels, resp_index, resp_valid = pack_padded_batch(mb["input_ids"], mb["attention_mask"],
                                                                  mb.get("position_ids"), R)
        extra = {}
        if mb.get("multi_modal_inputs") is not None:
            extra["mm_inputs"] = collate_multi_modal_inputs(mb["multi_modal_inputs"], self.device)
        vals = self.model.forward_values(batch, need_grad=need_grad, **extra)
        return {"values": torch.where(resp_valid, vals[resp_index], torch.zeros((), dtype=vals.dtype, device=vals.device))}
