"""Worker roles: a generic training worker and the hybrid actor / rollout / reference worker.

In this framework the trainer and the rollout engine live in ONE process per GPU and share the bf16 working
weights in place, so "weight sync" after an optimizer step is a KV-cache reset, not a transfer.

Parity target: ``verl/workers/engine_workers.py`` (``TrainingWorker`` :76-448, ``ActorRolloutRefWorker``
:451-832).
"""

from __future__ import annotations

import os
import time
from functools import partial
from typing import Any, Callable, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..protocol import DataProto
from ..single_controller.base import Dispatch, Worker, make_nd_compute_dataproto_dispatch_fn, register
from ..utils import torch_functional as VF
from ..utils.config import omega_conf_to_dataclass
from ..utils.device import get_device_name, get_nccl_backend
from ..utils.distributed import initialize_global_process_group
from ..utils.flops_counter import FlopsCounter
from ..utils.profiler import DistProfilerExtension, log_gpu_memory_usage
from .config import (ActorConfig, CheckpointConfig, FSDPActorConfig, FSDPEngineConfig, HFModelConfig, OptimizerConfig,
                     RolloutConfig, TrainingWorkerConfig)
from .engine.base import EngineRegistry
from .engine.native import engine as _native_engine  # noqa: F401  (registers the engines)
from .engine.native import turbo as _turbo_engine  # noqa: F401  (registers the fsdp_turbo backend)
from .utils.losses import ppo_loss, sft_loss, value_loss

__all__ = ["TrainingWorker", "ActorRolloutRefWorker", "CriticWorker"]


def _reduce_metrics(metrics: dict) -> dict:
    out = {}
    for k, v in metrics.items():
        if isinstance(v, (list, tuple)):
            vals = [float(x.item() if torch.is_tensor(x) else x) for x in v]
            out[k] = float(np.mean(vals)) if vals else 0.0
        else:
            out[k] = float(v.item() if torch.is_tensor(v) else v)
    return out


class TrainingWorker(Worker, DistProfilerExtension):
    """One engine + a loss function; the building block for actor, critic, reference and SFT."""

    def __init__(self, config: TrainingWorkerConfig, **engine_kwargs):
        Worker.__init__(self)
        DistProfilerExtension.__init__(self, getattr(config, "profiler_config", None))
        self.config = config
        initialize_global_process_group()
        ec = config.engine_config
        self.engine = EngineRegistry.new(config.model_type, getattr(ec, "strategy", "fsdp"), model_config=config.model_config,
                                         engine_config=ec, optimizer_config=config.optimizer_config,
                                         checkpoint_config=config.checkpoint_config, **engine_kwargs)
        self.loss_fn: Optional[Callable] = None
        self.flops_counter = FlopsCounter(config.model_config.arch if hasattr(config.model_config, "arch") else config.model_config)
        self._register_dispatch_collect_info("train", dp_rank=self.rank, is_collect=True)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def to(self, device, model: bool = True, optimizer: bool = True, grad: bool = True):
        self.engine.to(device, model=model, optimizer=optimizer, grad=grad)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def set_loss_fn(self, loss_fn: Callable):
        self.loss_fn = loss_fn

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def reset(self):
        self.engine.initialize()

    # ------------------------------------------------------------------ helpers
    def _as_dict(self, data) -> dict:
        if isinstance(data, DataProto):
            d = {k: v for k, v in data.batch.items()}
            d.update(data.meta_info)
            if "multi_modal_inputs" in data.non_tensor_batch:   # per-row processor outputs of vision-language samples
                d["multi_modal_inputs"] = list(data.non_tensor_batch["multi_modal_inputs"])
            return d
        return dict(data.items()) if hasattr(data, "items") else dict(data)

    def _postprocess(self, out: dict, tokens: int, seconds: float, forward_only: bool) -> dict:
        metrics = _reduce_metrics(out.get("metrics", {}))
        if "loss" in out:
            loss = out["loss"].detach().float().clone()
            if dist.is_initialized() and dist.get_world_size() > 1:
                from ..utils.distributed import get_data_parallel_group

                g = get_data_parallel_group()
                dist.all_reduce(loss, group=g)
                loss /= dist.get_world_size(g)
            metrics["loss"] = float(loss)
        if seconds > 0 and tokens > 0:
            est, promised = self.flops_counter.estimate_flops([tokens], seconds)
            mfu = est / promised
            metrics["perf/mfu"] = float(mfu / 3.0 if forward_only else mfu)
        if get_device_name() == "cuda":
            metrics["perf/max_memory_allocated_gb"] = torch.cuda.max_memory_allocated() / 1024**3
        return metrics

    # ------------------------------------------------------------------ compute
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def train_mini_batch(self, data: DataProto) -> DataProto:
        """Iterate mini-batches (``mini_batch_size`` rows on this rank, ``epochs`` passes); one optimizer step each."""
        return self._train_mini_batch(data)

    def _train_mini_batch(self, data: DataProto) -> DataProto:
        meta = data.meta_info
        mini = int(meta.get("mini_batch_size", len(data)))
        epochs = int(meta.get("epochs", 1))
        all_metrics: dict[str, list] = {}
        for mb in data.make_iterator(mini_batch_size=min(mini, len(data)), epochs=epochs, seed=meta.get("seed", 1),
                                     dataloader_kwargs={"shuffle": bool(meta.get("shuffle", False))}):
            m = self._train_batch(mb)
            for k, v in m.items():
                all_metrics.setdefault(k, []).append(v)
        return DataProto(meta_info={"metrics": all_metrics})

    def _train_batch(self, data: DataProto) -> dict:
        assert self.loss_fn is not None, "set_loss_fn must be called before training"
        t0 = time.time()
        tokens = int(data.batch["attention_mask"].sum())
        with self.engine.train_mode():
            out = self.engine.train_batch(self._as_dict(data), self.loss_fn)
        if get_device_name() == "cuda":
            torch.cuda.synchronize()
        return self._postprocess(out, tokens, time.time() - t0, forward_only=False)

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def train_batch(self, data: DataProto) -> DataProto:
        return DataProto(meta_info={"metrics": {k: [v] for k, v in self._train_batch(data).items()}})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def infer_batch(self, data: DataProto) -> DataProto:
        return self._infer_batch(data)

    def _infer_batch(self, data: DataProto) -> DataProto:
        t0 = time.time()
        with self.engine.eval_mode():
            out = self.engine.infer_batch(self._as_dict(data), None)
        tensors = {k: v.float() for k, v in out["model_output"].items()}
        return DataProto.from_dict(tensors=tensors, meta_info={"metrics": {}, "timing": time.time() - t0})

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None):
        self.engine.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False):
        self.engine.load_checkpoint(local_path, hdfs_path, del_local_after_load)


def _dp_world(engine=None) -> int:
    """Number of data-parallel replicas that split a global batch (model-parallel engines: world / (tp * pp))."""
    if engine is not None and hasattr(engine, "get_data_parallel_size") and getattr(engine, "_initialized", False):
        return int(engine.get_data_parallel_size())
    return dist.get_world_size() if dist.is_initialized() else 1


class CriticWorker(TrainingWorker):
    """Value model worker: ``compute_values`` and ``update_critic`` on top of :class:`TrainingWorker`."""

    def __init__(self, config, **kw):
        if not isinstance(config, TrainingWorkerConfig):
            critic = config
            mc = omega_conf_to_dataclass(critic.get("model"), HFModelConfig) if not isinstance(critic.get("model"), HFModelConfig) else critic.model
            if str(critic.get("strategy", "fsdp")) == "megatron":
                from .config import McoreEngineConfig

                ec = omega_conf_to_dataclass(critic.get("megatron") or critic.get("engine") or McoreEngineConfig(), McoreEngineConfig)
            else:
                ec = critic.get("fsdp_config") or critic.get("engine") or FSDPEngineConfig()
                ec = omega_conf_to_dataclass(ec, FSDPEngineConfig)
            object.__setattr__(ec, "micro_batch_size_per_gpu", critic.get("ppo_micro_batch_size_per_gpu"))
            object.__setattr__(ec, "infer_micro_batch_size_per_gpu", critic.get("forward_micro_batch_size_per_gpu") or critic.get("ppo_micro_batch_size_per_gpu"))
            # token-budgeted micro-batches for the update and for ``compute_values`` (``critic.use_dynamic_bsz``,
            # ``ppo_max_token_len_per_gpu``, ``forward_max_token_len_per_gpu``: verl/workers/config/critic.py)
            if critic.get("use_dynamic_bsz") is not None:
                object.__setattr__(ec, "use_dynamic_bsz", bool(critic.get("use_dynamic_bsz")))
            if critic.get("ppo_max_token_len_per_gpu"):
                object.__setattr__(ec, "max_token_len_per_gpu", int(critic.get("ppo_max_token_len_per_gpu")))
            fwd_budget = critic.get("forward_max_token_len_per_gpu") or critic.get("ppo_max_token_len_per_gpu")
            if fwd_budget:
                object.__setattr__(ec, "infer_max_token_len_per_gpu", int(fwd_budget))
            self.critic_config = critic
            config = TrainingWorkerConfig(model_type="value_model", model_config=mc, engine_config=ec,
                                          optimizer_config=omega_conf_to_dataclass(critic.get("optim"), OptimizerConfig),
                                          checkpoint_config=omega_conf_to_dataclass(critic.get("checkpoint"), CheckpointConfig))
        super().__init__(config, **kw)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        self.engine.initialize()
        self.loss_fn = partial(value_loss, getattr(self, "critic_config", None))

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def compute_values(self, data: DataProto) -> DataProto:
        return DataProto.from_dict(tensors={"values": self._infer_batch(data).batch["values"]})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def update_critic(self, data: DataProto) -> DataProto:
        cc = getattr(self, "critic_config", None)
        ws = _dp_world(self.engine)
        if cc is not None:
            data.meta_info.setdefault("mini_batch_size", max(1, cc.ppo_mini_batch_size * cc.get("rollout_n", 1) // ws))
            data.meta_info.setdefault("epochs", cc.ppo_epochs)
        return self._train_mini_batch(data)


class ActorRolloutRefWorker(Worker, DistProfilerExtension):
    """Actor (trainable policy), rollout engine and frozen reference policy on one GPU.

    ``role`` selects which parts exist: ``actor``, ``rollout``, ``ref``, ``actor_rollout``, ``actor_rollout_ref``."""

    def __init__(self, config, role: str = "actor_rollout_ref", distillation_config=None, **kwargs):
        Worker.__init__(self)
        DistProfilerExtension.__init__(self, None)
        self.config = config
        self.role = role
        # on-policy distillation: the actor's loss becomes task loss + distillation term (verl/workers/engine_workers.py:462-467)
        self.distillation_config = distillation_config
        self._is_actor = "actor" in role
        self._is_rollout = "rollout" in role
        self._is_ref = "ref" in role
        initialize_global_process_group()
        self.actor = self.ref = self.rollout = None
        self._register_dispatch_collect_info("train", dp_rank=self.rank, is_collect=True)
        self._register_dispatch_collect_info("rollout", dp_rank=self.rank, is_collect=True)

    # ------------------------------------------------------------------ bring-up
    def _model_config(self) -> HFModelConfig:
        m = self.config.model
        return m if isinstance(m, HFModelConfig) else omega_conf_to_dataclass(m, HFModelConfig)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        cfg = self.config
        mc = self._model_config()
        ws = dist.get_world_size() if dist.is_initialized() else 1
        if self._is_actor:
            if isinstance(cfg.actor, ActorConfig):
                ac = cfg.actor
            elif str(cfg.actor.get("strategy", "fsdp")) == "megatron":
                from .config import McoreActorConfig

                ac = omega_conf_to_dataclass(cfg.actor, McoreActorConfig)
            else:
                ac = omega_conf_to_dataclass(cfg.actor, FSDPActorConfig)
            self.actor_config = ac
            ec = ac.engine if ac.engine is not None else FSDPEngineConfig()
            for k_src, k_dst in (("ppo_micro_batch_size_per_gpu", "micro_batch_size_per_gpu"),
                                 ("ppo_max_token_len_per_gpu", "max_token_len_per_gpu"), ("use_dynamic_bsz", "use_dynamic_bsz")):
                v = ac.get(k_src)
                if v is not None:
                    object.__setattr__(ec, k_dst, v)
            rc = cfg.get("rollout") if hasattr(cfg, "get") else None
            infer_mb = (rc.get("log_prob_micro_batch_size_per_gpu") if rc is not None else None) or ac.get("ppo_infer_micro_batch_size_per_gpu") or ac.get("ppo_micro_batch_size_per_gpu")
            object.__setattr__(ec, "infer_micro_batch_size_per_gpu", infer_mb)
            if rc is not None and rc.get("log_prob_max_token_len_per_gpu"):
                object.__setattr__(ec, "infer_max_token_len_per_gpu", rc.get("log_prob_max_token_len_per_gpu"))
            object.__setattr__(ec, "enable_gradient_checkpointing", bool(mc.enable_gradient_checkpointing))
            sp_size = int(ac.get("ulysses_sequence_parallel_size", 1) or 1)
            if sp_size > 1 and hasattr(ec, "ulysses_sequence_parallel_size"):
                object.__setattr__(ec, "ulysses_sequence_parallel_size", sp_size)
            tw = TrainingWorkerConfig(model_type="language_model", model_config=mc, engine_config=ec,
                                      optimizer_config=ac.optim, checkpoint_config=ac.checkpoint)
            self.actor = EngineRegistry.new("language_model", getattr(ec, "strategy", "fsdp"), model_config=mc, engine_config=ec,
                                            optimizer_config=ac.optim, checkpoint_config=ac.checkpoint)
            self.actor.initialize()
            self.actor_loss = partial(ppo_loss, ac)
            dc = self.distillation_config
            if dc is not None and bool(dc.get("enabled", False) if hasattr(dc, "get") else getattr(dc, "enabled", False)):
                from ..trainer.distillation.losses import (DistillationConfig, DistillationLossConfig, distillation_ppo_loss,
                                                           get_distillation_loss_settings)

                if not isinstance(dc, DistillationConfig):
                    lc = dc.get("distillation_loss") or {}
                    known = DistillationLossConfig.__dataclass_fields__
                    dc = DistillationConfig(enabled=True, teacher_key=str(dc.get("teacher_key", "data_source")),
                                            distillation_loss=DistillationLossConfig(**{k: v for k, v in dict(lc).items() if k in known}))
                if get_distillation_loss_settings(dc.distillation_loss.loss_mode).use_topk:
                    raise NotImplementedError(
                        "distillation_loss.loss_mode=forward_kl_topk needs the student's log-probs on the teacher's top-k ids, "
                        "which this engine's fused LM-head kernel does not return; use one of the sampled-token estimators "
                        "(k1, k2, k3, abs, mse, low_var_kl)")
                self.distillation_config = dc
                self.actor_loss = partial(distillation_ppo_loss, ac, dc)
            # the ranks of a sequence-parallel block see the same prompts: they split the generation work among them
            self._sp_replica = getattr(self.actor, "sp_size", 1) > 1
        if self._is_ref:
            rcfg = cfg.get("ref") if hasattr(cfg, "get") else None
            rec = FSDPEngineConfig(forward_only=True)
            if rcfg is not None:
                mb = rcfg.get("log_prob_micro_batch_size_per_gpu")
                object.__setattr__(rec, "infer_micro_batch_size_per_gpu", mb)
                object.__setattr__(rec, "use_dynamic_bsz", bool(rcfg.get("log_prob_use_dynamic_bsz", False)))
                if rcfg.get("log_prob_max_token_len_per_gpu"):
                    object.__setattr__(rec, "infer_max_token_len_per_gpu", rcfg.get("log_prob_max_token_len_per_gpu"))
                rfc = rcfg.get("fsdp_config")
                if rfc is not None and bool(rfc.get("param_offload", False) if hasattr(rfc, "get") else getattr(rfc, "param_offload", False)):
                    object.__setattr__(rec, "param_offload", True)
            if self.actor is not None and getattr(self.actor, "topo", None) is not None:  # same model-parallel layout as the actor
                from .config import McoreEngineConfig

                mrec = McoreEngineConfig(tensor_model_parallel_size=self.actor.tp_size, pipeline_model_parallel_size=self.actor.pp_size,
                                         expert_model_parallel_size=getattr(self.actor, "ep_size", 1), forward_only=True)
                for k in ("infer_micro_batch_size_per_gpu", "use_dynamic_bsz", "infer_max_token_len_per_gpu"):
                    object.__setattr__(mrec, k, getattr(rec, k))
                self.ref = EngineRegistry.new("language_model", "megatron", model_config=mc, engine_config=mrec, optimizer_config=None)
            else:
                self.ref = EngineRegistry.new("language_model", "fsdp", model_config=mc, engine_config=rec, optimizer_config=None)
            self.ref.initialize()
            if self.actor is not None:  # the reference policy starts as an exact copy of the actor
                if getattr(self.actor, "zero3", False):
                    self.actor.gather_full_params(out=self.ref.params)
                else:
                    self.ref.params.flat.copy_(self.actor.params.flat)
        if self._is_rollout:
            from .rollout.native.engine import RolloutEngine

            rc = cfg.rollout if isinstance(cfg.rollout, RolloutConfig) else omega_conf_to_dataclass(cfg.rollout, RolloutConfig)
            self.rollout_config = rc
            src = self.actor if self.actor is not None else self.ref
            topo = getattr(src, "topo", None) if src is not None else None
            self._mp_actor = topo is not None and topo.tp * topo.pp > 1
            self._regather = (topo is not None and (self._mp_actor or topo.ep > 1)) or bool(getattr(src, "zero3", False))
            if self._regather:
                # the trainer holds a shard of the model (1/(tp*pp) of it, or 1/ep of the experts): the rollout engine gets a
                # full replica that update_weights() re-assembles from the shards after every optimizer step; with tensor /
                # pipeline parallelism the trainer's data-parallel group = the replicas
                from ..utils.distributed import set_data_parallel_group

                self._mp_engine = src
                # shards go peer to peer into every rank's replica when the job allows it (parallel/reshard.py), else the
                # replica is assembled with collectives
                self._reshard = None
                if getattr(src, "topo", None) is not None and os.environ.get("VERL_B200_PEER_RESHARD", "1") != "0":
                    from ..parallel.reshard import PeerReshard

                    self._reshard = PeerReshard.try_create(src)
                if self._reshard is not None:
                    self.rollout_params = self._reshard.full
                    self._reshard.run()
                else:
                    self.rollout_params = src.gather_full_params()
                if self._mp_actor:
                    set_data_parallel_group(topo.dp_group)

                class _Holder:
                    params = self.rollout_params

                src = _Holder()
            if src is None:  # rollout-only rank: a forward-only engine holds the weights that weight sync overwrites
                self.rollout_weights = EngineRegistry.new("language_model", "fsdp", model_config=mc,
                                                          engine_config=FSDPEngineConfig(forward_only=True), optimizer_config=None)
                self.rollout_weights.initialize()
                src = self.rollout_weights
            arch = mc.arch
            max_len = rc.max_model_len or (rc.prompt_length + rc.response_length)
            # rollout tensor parallelism: consecutive ranks form a group that serves the union of its members' prompts;
            # every member shards the replicated weights in place, so the train -> rollout reshard moves no bytes
            from ..utils.distributed import get_data_parallel_group

            pool = None if getattr(self, "_mp_actor", False) else get_data_parallel_group()  # ranks that run this kind of worker
            pool_ranks = dist.get_process_group_ranks(pool if pool is not None else dist.group.WORLD) if ws > 1 else [0]
            n_pool, me = len(pool_ranks), (pool_ranks.index(dist.get_rank()) if ws > 1 else 0)
            tp = int(rc.tensor_model_parallel_size or 1)
            tp = tp if (n_pool > 1 and tp > 1 and n_pool % tp == 0 and not arch.is_moe and not arch.is_generic
                        and arch.num_key_value_heads % tp == 0) else 1
            self.rollout_tp, self.rollout_tp_group = tp, None
            if tp > 1:  # only the members take part in creating their group
                g0 = me // tp * tp
                self.rollout_tp_group = dist.new_group(pool_ranks[g0 : g0 + tp], use_local_synchronization=True)
            if arch.is_generic:
                # no hand-scheduled decoder for this family: sampling runs on the library module with its key/value cache
                from ..models.generic import GenericRolloutEngine as RolloutEngine

            self.rollout = RolloutEngine(arch, src.params, max_num_seqs=rc.max_num_seqs * tp, tp_group=self.rollout_tp_group,
                                         record_routing=(self._router_replay_mode() == "R3"),
                                         enable_prefix_caching=bool(rc.get("enable_prefix_caching", False)),
                                         quantization=(rc.get("quantization") if tp == 1 else None),
                                         max_num_batched_tokens=rc.max_num_batched_tokens, max_model_len=max_len + 1,
                                         block_size=rc.block_size, gpu_memory_utilization=rc.gpu_memory_utilization,
                                         use_cuda_graph=not rc.enforce_eager, sync_interval=rc.sync_interval,
                                         seed=1234 + (me // tp if tp > 1 else self.rank), num_blocks=rc.engine_kwargs.get("num_blocks"),
                                         valid_vocab_size=rc.engine_kwargs.get("valid_vocab_size", 0))
            if rc.free_cache_engine:
                self.rollout.release_kv_cache()
            prom = rc.prometheus or {}
            self._rollout_metrics = None
            if (prom.get("enable") if hasattr(prom, "get") else getattr(prom, "enable", False)):
                from .rollout.metrics import RolloutMetricsExporter

                port = (prom.get("port") if hasattr(prom, "get") else getattr(prom, "port", None))
                self._rollout_metrics = RolloutMetricsExporter(replica=str(self.rank), port=(int(port) + self.rank) if port else None)

    # ------------------------------------------------------------------ rollout
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("rollout"))
    def generate_sequences(self, prompts: DataProto) -> DataProto:
        """Token-in / token-out generation for a batch of left-padded prompts."""
        from .rollout.native.engine import SamplingParams

        rc = self.rollout_config
        t0 = time.time()
        prompts = self._dev(prompts)
        self.rollout.resume_kv_cache()
        ids = prompts.batch["input_ids"]
        mask = prompts.batch["attention_mask"].bool()
        dev = ids.device
        meta = prompts.meta_info
        do_sample = meta.get("do_sample", rc.do_sample)
        validate = meta.get("validate", False)
        src = rc.val_kwargs if validate else rc
        sp = SamplingParams(temperature=float(meta.get("temperature", src.temperature)) if do_sample else 0.0,
                            top_p=float(meta.get("top_p", src.top_p)), top_k=int(meta.get("top_k", src.top_k)),
                            max_tokens=int(meta.get("response_length", rc.response_length)), ignore_eos=rc.ignore_eos,
                            logprobs=True)
        ids_cpu, mask_cpu = ids.cpu(), mask.cpu()
        plist = [ids_cpu[i][mask_cpu[i]].tolist() for i in range(ids.shape[0])]
        if getattr(self, "_mp_actor", False) or getattr(self, "_sp_replica", False):
            outs = self._generate_in_replica(plist, sp)
        elif getattr(self, "rollout_tp", 1) > 1:
            # the group generates the union of its members' prompts in lockstep; each member keeps its own slice
            parts: list = [None] * self.rollout_tp
            dist.all_gather_object(parts, plist, group=self.rollout_tp_group)
            me = dist.get_rank(self.rollout_tp_group)
            lo = sum(len(x) for x in parts[:me])
            outs = self.rollout.generate([p for part in parts for p in part], sp)[lo : lo + len(plist)]
        elif "multi_modal_inputs" in prompts.non_tensor_batch:
            # vision-language prompts: the placeholder tokens are in the prompt ids, the patches travel beside them
            outs = self.rollout.generate(plist, sp, mm_inputs=list(prompts.non_tensor_batch["multi_modal_inputs"]))
        else:
            outs = self.rollout.generate(plist, sp)
        R = sp.max_tokens
        pad = int(meta.get("pad_token_id", self.rollout.cfg.pad_token_id or 0))
        b = len(outs)
        resp = torch.full((b, R), pad, dtype=torch.int64)
        lps = torch.zeros(b, R, dtype=torch.float32)
        lens = torch.zeros(b, dtype=torch.int64)
        for i, o in enumerate(outs):
            n = len(o.token_ids)
            lens[i] = n
            resp[i, :n] = torch.tensor(o.token_ids, dtype=torch.int64)
            if o.log_probs is not None:
                lps[i, :n] = torch.tensor(o.log_probs, dtype=torch.float32)
        resp_mask = (torch.arange(R).unsqueeze(0) < lens.unsqueeze(1)).to(torch.int64)
        resp, lps, resp_mask = resp.to(dev), lps.to(dev), resp_mask.to(dev)
        full_ids = torch.cat([ids, resp], dim=1)
        full_mask = torch.cat([prompts.batch["attention_mask"], resp_mask.to(prompts.batch["attention_mask"].dtype)], dim=1)
        pos = VF.compute_position_id_with_mask(full_mask)
        if getattr(self, "_rollout_metrics", None) is not None:
            self._rollout_metrics.update(self.rollout)
        if rc.free_cache_engine:
            self.rollout.release_kv_cache()
        tensors = {"prompts": ids, "responses": resp, "input_ids": full_ids, "attention_mask": full_mask,
                   "position_ids": pos, "response_mask": resp_mask, "rollout_log_probs": lps}
        if outs and "routed_experts" in outs[0].extra_fields:
            # router replay from the rollout (R3): experts per position of the padded [b, P + R] layout; the last generated
            # token never went through the rollout model, its row stays zero (its output enters no loss)
            P_len = ids.shape[1]
            first = outs[0].extra_fields["routed_experts"]
            routed = torch.zeros(b, P_len + R, first.shape[1], first.shape[2], dtype=torch.int32)
            for i, o in enumerate(outs):
                re_ = o.extra_fields["routed_experts"].to(torch.int32)
                p_n = len(o.prompt_ids)
                routed[i, P_len - p_n : P_len - p_n + re_.shape[0]] = re_
            tensors["routed_experts"] = routed.to(dev)
        out = DataProto.from_dict(
            tensors=tensors,
            meta_info={"timing": {"generate_sequences": time.time() - t0},
                       "rollout_stats": dict(self.rollout.stats)})
        return out

    def _generate_in_replica(self, plist: list, sp) -> list:
        """All ranks of a model-parallel training replica hold the same prompts. Its rollout groups (``rollout_tp`` consecutive
        ranks each) take interleaved slices of them, generate, and the replica exchanges the results so that every rank
        ends up with the outputs of all prompts in the original order."""
        if getattr(self, "_sp_replica", False):
            eng = self.actor
            mp, me, group = eng.sp_size, eng.sp_rank, eng.sp_group
        else:
            topo = self._mp_engine.topo
            mp, group = topo.tp * topo.pp, topo.mp_group
            me = topo.pp_rank * topo.tp + topo.tp_rank      # position inside the replica
        tp = max(1, getattr(self, "rollout_tp", 1))
        groups = mp // tp
        mine = me // tp
        idx = list(range(mine, len(plist), groups))
        local = self.rollout.generate([plist[i] for i in idx], sp) if idx else []
        box = [None] * mp
        dist.all_gather_object(box, (mine, idx, local if me % tp == 0 else None), group=group)
        outs: list = [None] * len(plist)
        for g, ids_, res in box:
            if res is None:
                continue
            for i, o in zip(ids_, res):
                outs[i] = o
        return outs

    # ------------------------------------------------------------------ log-probs
    def _dev(self, data: DataProto) -> DataProto:
        eng = self.actor or self.ref
        if eng is not None and data.batch is not None and data.batch.device != eng.device:
            data = DataProto(batch=data.batch.to(eng.device), non_tensor_batch=data.non_tensor_batch, meta_info=data.meta_info)
        return data

    def _infer(self, engine, data: DataProto, calculate_entropy: bool, replay_routing: bool = True) -> dict:
        data = self._dev(data)
        d = {k: v for k, v in data.batch.items() if replay_routing or k != "routed_experts"}
        if "multi_modal_inputs" in data.non_tensor_batch:
            d["multi_modal_inputs"] = list(data.non_tensor_batch["multi_modal_inputs"])
        d.update({k: v for k, v in data.meta_info.items() if k in ("temperature", "micro_batch_size_per_gpu", "record_routing",
                                                                   "max_token_len_per_gpu", "use_dynamic_bsz")})
        d["calculate_entropy"] = calculate_entropy
        with engine.eval_mode():
            return engine.infer_batch(d, None)["model_output"]

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def compute_log_prob(self, data: DataProto) -> DataProto:
        # router replay (mixture-of-experts actors): "R2" records the experts chosen in this pass so that the policy update
        # replays them; "R3" replays the rollout engine's choices when the batch carries them (and records otherwise)
        record = self._router_replay_mode() in ("R2", "R3") and "routed_experts" not in data.batch.keys()
        if record:
            data.meta_info["record_routing"] = True
        out = self._infer(self.actor, data, calculate_entropy=True)
        tensors = {"old_log_probs": out["log_probs"].float(), "entropys": out["entropy"].float()}
        if record and "routed_experts" in out:
            tensors["routed_experts"] = out["routed_experts"].to(torch.int32)
        return DataProto.from_dict(tensors=tensors, meta_info={"temperature": data.meta_info.get("temperature", 1.0)})

    def _router_replay_mode(self) -> str:
        ac = getattr(self, "actor_config", None)
        for holder in (ac, getattr(ac, "megatron", None), getattr(ac, "engine", None)):
            rr = getattr(holder, "router_replay", None) if holder is not None else None
            if rr is None and hasattr(holder, "get"):
                rr = holder.get("router_replay")
            mode = (rr.get("mode") if hasattr(rr, "get") else getattr(rr, "mode", None)) if rr is not None else None
            if mode and mode != "disabled":
                return str(mode)
        return "disabled"

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def compute_ref_log_prob(self, data: DataProto) -> DataProto:
        out = self._infer(self.ref, data, calculate_entropy=False, replay_routing=False)  # the reference policy routes by itself
        return DataProto.from_dict(tensors={"ref_log_prob": out["log_probs"].float()})

    # ------------------------------------------------------------------ training
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def update_actor(self, data: DataProto) -> DataProto:
        ac = self.actor_config
        data = self._dev(data)
        ws = _dp_world(self.actor)
        n = len(data)
        mini = int(data.meta_info.get("mini_batch_size") or max(1, ac.ppo_mini_batch_size * ac.rollout_n // ws))
        mini = min(mini, n)
        metrics: dict[str, list] = {}
        t0 = time.time()
        for mb in data.make_iterator(mini_batch_size=mini, epochs=int(ac.ppo_epochs), seed=ac.data_loader_seed,
                                     dataloader_kwargs={"shuffle": bool(ac.shuffle)}):
            d = {k: v for k, v in mb.batch.items()}
            if "multi_modal_inputs" in mb.non_tensor_batch:
                d["multi_modal_inputs"] = list(mb.non_tensor_batch["multi_modal_inputs"])
            d.update(temperature=data.meta_info.get("temperature", 1.0), calculate_entropy=ac.entropy_coeff != 0,
                     loss_scale_factor=ac.loss_scale_factor)
            with self.actor.train_mode():
                out = self.actor.train_batch(d, self.actor_loss)
            m = _reduce_metrics(out.get("metrics", {}))
            m = {(k if k.startswith("actor/") else f"actor/{k}"): v for k, v in m.items()}
            for k, v in m.items():
                metrics.setdefault(k, []).append(v)
        metrics["timing_s/update_actor_worker"] = [time.time() - t0]
        return DataProto(meta_info={"metrics": metrics})

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def update_weights(self, global_steps: Optional[int] = None) -> dict:
        """Make the latest actor weights visible to the rollout engine. The engine reads the trainer's working
        buffer in place, so this only invalidates cached KV; returns the device time spent."""
        t0 = time.time()
        if getattr(self, "_regather", False) and self.rollout is not None:
            if getattr(self, "_reshard", None) is not None:
                self._reshard.run()                                          # peer stores straight into every replica
            elif getattr(self._mp_engine, "zero3", False):
                self._mp_engine.gather_full_params(out=self.rollout_params)  # unit by unit, straight into the replica
            else:
                fresh = self._mp_engine.gather_full_params()
                self.rollout_params.flat.copy_(fresh.flat)
                del fresh
        if self.rollout is not None:
            self.rollout.clear_kv_cache()
        if get_device_name() == "cuda":
            torch.cuda.synchronize()
        return {"timing_s/update_weights": time.time() - t0}

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None):
        self.actor.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False):
        self.actor.load_checkpoint(local_path, hdfs_path, del_local_after_load)
