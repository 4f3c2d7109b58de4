"""PPO / GRPO / REINFORCE++ / RLOO trainer: the single-controller dataflow.

The class keeps the reference's name although Ray is only one of the worker-group backends: the driver logic is
backend-agnostic and talks to worker groups through ``@register``-ed methods carrying ``DataProto`` batches.
Under ``torchrun`` the controller-replicated ``SPMDWorkerGroup`` keeps every batch on the GPU that produced it.

Parity target: ``verl/trainer/ppo/ray_trainer.py`` (``apply_kl_penalty`` :78, ``compute_response_mask`` :120,
``compute_advantage`` :187-282, ``RayPPOTrainer`` :286: ``_validate`` :596, ``init_workers`` :772,
``_save_checkpoint`` :983, ``_load_checkpoint`` :1052, ``_balance_batch`` :1182, ``fit`` :1405-1823).
"""

from __future__ import annotations

import json
import os
import time
import uuid
from collections import defaultdict
from copy import deepcopy
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import numpy as np
import torch
import torch.distributed as dist

from ...protocol import DataProto, pad_dataproto_to_divisor, unpad_dataproto
from ...single_controller.base import ClassWithInitArgs, ResourcePool
from ...utils import torch_functional as VF
from ...utils.checkpoint.checkpoint_manager import find_latest_ckpt_path, should_save_ckpt_esi
from ...utils.profiler import marked_timer
from ...utils.seqlen_balancing import calculate_workload, get_seqlen_balanced_partitions, log_seqlen_unbalance
from ...utils.tracking import Tracking, ValidationGenerationsLogger
from . import core_algos
from .core_algos import AdvantageEstimator, agg_loss
from .metric_utils import (compute_data_metrics, compute_throughout_metrics, compute_timing_metrics,
                           process_validation_metrics, reduce_metrics)
from .utils import Role, need_critic, need_reference_policy

__all__ = ["RayPPOTrainer", "ResourcePoolManager", "apply_kl_penalty", "compute_response_mask", "compute_advantage"]


@dataclass
class ResourcePoolManager:
    """Named resource pools and the role -> pool mapping."""

    resource_pool_spec: dict
    mapping: dict
    resource_pool_dict: dict = field(default_factory=dict)

    def create_resource_pool(self) -> None:
        for name, procs in self.resource_pool_spec.items():
            self.resource_pool_dict[name] = ResourcePool(process_on_nodes=list(procs), max_colocate_count=3)

    def get_resource_pool(self, role) -> ResourcePool:
        return self.resource_pool_dict[self.mapping[role]]

    def get_n_gpus(self) -> int:
        return sum(n for procs in self.resource_pool_spec.values() for n in procs)


class DataParallelView:
    """What a rank of a controller-replicated (SPMD) run needs to compute statistics over the *global* batch: gathers of
    per-sample tensors / arrays over the distinct data-parallel replicas, and the position of the local samples in the
    gathered batch. ``stride`` ranks in a row hold the same data (a model-parallel block); one of them is counted."""

    def __init__(self, group, stride: int = 1):
        self.group, self.stride = group, max(1, int(stride))
        self.rank = dist.get_rank(group) // self.stride
        self.world = dist.get_world_size(group) // self.stride
        self._sizes = None

    def _pick(self, parts: list) -> list:
        return parts[:: self.stride]

    def sizes(self, n: int) -> list[int]:
        if self._sizes is None:
            got = [None] * dist.get_world_size(self.group)
            dist.all_gather_object(got, int(n), group=self.group)
            self._sizes = self._pick(got)
        return self._sizes

    def tensor(self, t: torch.Tensor) -> torch.Tensor:
        sizes = self.sizes(t.shape[0])
        if len(set(sizes)) == 1:
            parts = [torch.empty_like(t) for _ in range(dist.get_world_size(self.group))]
            dist.all_gather(parts, t.contiguous(), group=self.group)
            return torch.cat(self._pick(parts), dim=0)
        got = [None] * dist.get_world_size(self.group)
        dist.all_gather_object(got, t.cpu(), group=self.group)
        return torch.cat([x.to(t.device) for x in self._pick(got)], dim=0)

    def array(self, a: np.ndarray) -> np.ndarray:
        got = [None] * dist.get_world_size(self.group)
        dist.all_gather_object(got, a, group=self.group)
        return np.concatenate(self._pick(got), axis=0)

    def local(self, t, n: int):
        lo = sum(self.sizes(n)[: self.rank])
        return t[lo : lo + n]

    def sum(self, *vals: float) -> list[float]:
        """Sums over the distinct replicas of a few host scalars."""
        t = torch.tensor([float(v) for v in vals], dtype=torch.float64)
        got = [None] * dist.get_world_size(self.group)
        dist.all_gather_object(got, t, group=self.group)
        return torch.stack(self._pick(got)).sum(0).tolist()


def apply_kl_penalty(data: DataProto, kl_ctrl, kl_penalty: str = "kl", dp: Optional[DataParallelView] = None):
    """token_level_rewards = token_level_scores - beta * KL(old || ref); updates the adaptive controller with the mean
    KL and the size of the *global* batch (``dp``: the other data-parallel ranks hold the rest of it)."""
    mask = data.batch["response_mask"]
    scores = data.batch["token_level_scores"]
    bsz = data.batch.batch_size[0]
    kld = core_algos.kl_penalty(data.batch["old_log_probs"], data.batch["ref_log_prob"], kl_penalty=kl_penalty) * mask
    beta = kl_ctrl.value
    data.batch["token_level_rewards"] = scores - beta * kld
    per_seq = VF.masked_mean(kld, mask=mask, axis=-1)
    if dp is not None and dp.world > 1:
        total, count = dp.sum(per_seq.sum().item(), bsz)
        current, bsz = total / max(count, 1.0), int(count)
    else:
        current = torch.mean(per_seq, dim=0).item()
    kl_ctrl.update(current_kl=current, n_steps=bsz)
    return data, {"actor/reward_kl_penalty": current, "actor/reward_kl_penalty_coeff": beta}


# estimators whose result depends on statistics of the whole batch (whitening, batch-size scaling): in a run where every
# rank holds a slice of the batch they are evaluated on the gathered batch, so the result does not depend on the
# data-parallel size
BATCH_WIDE_ESTIMATORS = ("gae", "reinforce_plus_plus", "reinforce_plus_plus_baseline", "gpg", "gdpo")


def compute_response_mask(data: DataProto) -> torch.Tensor:
    R = data.batch["responses"].size(1)
    return data.batch["attention_mask"][:, -R:]


def compute_advantage(data: DataProto, adv_estimator, gamma: float = 1.0, lam: float = 1.0, num_repeat: int = 1,
                      norm_adv_by_std_in_grpo: bool = True, config=None, dp: Optional[DataParallelView] = None) -> DataProto:
    """Fill ``advantages`` / ``returns`` with the configured estimator (device kernels for GAE and GRPO when the
    batch lives on a GPU). With ``dp`` (this rank holds a slice of the batch) the estimators of
    ``BATCH_WIDE_ESTIMATORS`` run on the gathered batch and the local rows are kept."""
    if "response_mask" not in data.batch.keys():
        data.batch["response_mask"] = compute_response_mask(data)
    name = adv_estimator.value if isinstance(adv_estimator, AdvantageEstimator) else str(adv_estimator)
    if dp is not None and dp.world > 1 and name in BATCH_WIDE_ESTIMATORS and not (config is not None and config.get("use_pf_ppo", False)):
        n = data.batch.batch_size[0]
        keys = [k for k in ("token_level_rewards", "response_mask", "values", "reward_baselines", "old_log_probs", "sum_pi_squared",
                            "rollout_is_weights", "prompts", "attention_mask") if k in data.batch.keys()]
        full = DataProto.from_dict(tensors={k: dp.tensor(data.batch[k]) for k in keys},
                                   non_tensors={k: dp.array(np.asarray(v)) for k, v in data.non_tensor_batch.items()
                                                if k == "uid" or (name == "gdpo" and np.asarray(v).dtype != object)})
        full = compute_advantage(full, adv_estimator, gamma, lam, num_repeat, norm_adv_by_std_in_grpo, config, dp=None)
        data.batch["advantages"] = dp.local(full.batch["advantages"], n).contiguous()
        data.batch["returns"] = dp.local(full.batch["returns"], n).contiguous()
        return data
    mask = data.batch["response_mask"]
    rewards = data.batch["token_level_rewards"]
    if name == "gae":
        if rewards.is_cuda:
            from ...ops import functional as OF

            adv, ret = OF.gae_advantage(rewards, data.batch["values"], mask, gamma, lam, whiten=True)
        else:
            adv, ret = core_algos.compute_gae_advantage_return(rewards, data.batch["values"], mask.to(rewards.dtype), gamma, lam)
        data.batch["advantages"], data.batch["returns"] = adv, ret
        if config is not None and config.get("use_pf_ppo", False):
            data = core_algos.compute_pf_ppo_reweight_data(data, config.pf_ppo.get("reweight_method"),
                                                           config.pf_ppo.get("weight_pow"))
        return data
    if name == "grpo" and rewards.is_cuda:
        from ...ops import functional as OF
        from ...utils.groupwise import as_torch_index

        g = as_torch_index(data.non_tensor_batch["uid"], device=rewards.device)
        adv, _ = OF.grpo_advantage(rewards, mask, g, int(g.max().item()) + 1, 1e-6, norm_adv_by_std_in_grpo)
        data.batch["advantages"], data.batch["returns"] = adv, adv
        return data
    fn = core_algos.get_adv_estimator_fn(name)
    kwargs: dict[str, Any] = dict(token_level_rewards=rewards, response_mask=mask.to(rewards.dtype), config=config)
    if "uid" in data.non_tensor_batch:
        kwargs["index"] = data.non_tensor_batch["uid"]
    if "reward_baselines" in data.batch.keys():
        kwargs["reward_baselines"] = data.batch["reward_baselines"]
    if name in ("grpo", "grpo_vectorized", "gdpo", "grpo_passk"):
        kwargs["norm_adv_by_std_in_grpo"] = norm_adv_by_std_in_grpo
    if name == "gdpo":
        kwargs["non_tensor_batch"] = data.non_tensor_batch
    if name in ("optimal_token_baseline", "tir_optimal_token_baseline"):
        kwargs["old_log_probs"] = data.batch["old_log_probs"]
        kwargs["sum_pi_squared"] = data.batch["sum_pi_squared"]
        if "rollout_is_weights" in data.batch.keys():
            kwargs["rollout_is_weights"] = data.batch["rollout_is_weights"]
    if name in ("reinforce_plus_plus", "remax"):
        kwargs.pop("index", None)
    adv, ret = fn(**kwargs)
    data.batch["advantages"], data.batch["returns"] = adv, ret
    return data


class RayPPOTrainer:
    def __init__(self, config, tokenizer=None, role_worker_mapping: Optional[dict] = None,
                 resource_pool_manager: Optional[ResourcePoolManager] = None, ray_worker_group_cls=None, processor=None,
                 reward_fn=None, val_reward_fn=None, train_dataset=None, val_dataset=None, collate_fn=None,
                 train_sampler=None, device_name: Optional[str] = None, worker_group_kwargs: Optional[dict] = None):
        self.config = config
        self.tokenizer = tokenizer
        self.processor = processor
        self.reward_fn = reward_fn
        self.val_reward_fn = val_reward_fn
        self.role_worker_mapping = role_worker_mapping or {}
        self.resource_pool_manager = resource_pool_manager
        if ray_worker_group_cls is None:
            from ...single_controller.local import SPMDWorkerGroup

            ray_worker_group_cls = SPMDWorkerGroup
        self.ray_worker_group_cls = ray_worker_group_cls
        self.worker_group_kwargs = worker_group_kwargs or {}
        self.spmd = bool(getattr(ray_worker_group_cls, "is_spmd", False))
        self.device_name = device_name or config.trainer.get("device", "cuda")
        self.use_reference_policy = need_reference_policy(config)
        self.use_critic = need_critic(config)
        self.use_rm = False
        self.ref_in_actor = False
        self.hybrid_engine = True
        self.global_steps = 0
        self.validation_generations_logger = ValidationGenerationsLogger(
            project_name=config.trainer.get("project_name", "verl_b200"), experiment_name=config.trainer.get("experiment_name", "run"))
        if config.algorithm.get("use_kl_in_reward", False):
            self.kl_ctrl_in_reward = core_algos.get_kl_controller(config.algorithm.kl_ctrl)
        self._create_dataloader(train_dataset, val_dataset, collate_fn, train_sampler)

    # ------------------------------------------------------------------------------------ data
    def _dp_rank_world(self):
        if self.spmd and dist.is_initialized():
            from ...utils.distributed import get_data_parallel_group

            g = get_data_parallel_group()
            mp = self._model_parallel_size()
            if mp > 1 and (g is None or str(self.config.actor_rollout_ref.actor.get("strategy", "fsdp")) != "megatron"):
                # replicas are blocks of tp*pp (or sequence-parallel) consecutive ranks
                return dist.get_rank(g) // mp, dist.get_world_size(g) // mp
            return dist.get_rank(g), dist.get_world_size(g)
        return 0, 1

    def _dp_view(self) -> Optional[DataParallelView]:
        """Access to the rest of the global batch when every rank drives its own slice (SPMD), else None."""
        if not (self.spmd and dist.is_initialized()):
            return None
        from ...utils.distributed import get_data_parallel_group

        g = get_data_parallel_group()
        mp = self._model_parallel_size()
        stride = mp if mp > 1 and (g is None or str(self.config.actor_rollout_ref.actor.get("strategy", "fsdp")) != "megatron") else 1
        view = DataParallelView(g, stride)
        return view if view.world > 1 else None

    def _model_parallel_size(self) -> int:
        a = self.config.actor_rollout_ref.actor
        if str(a.get("strategy", "fsdp")) != "megatron":
            # a sequence-parallel or context-parallel block shares its data
            fc = a.get("fsdp_config") or {}
            cp = int((fc.get("context_parallel_size", 1) if hasattr(fc, "get") else getattr(fc, "context_parallel_size", 1)) or 1)
            return max(int(a.get("ulysses_sequence_parallel_size", 1) or 1), cp)
        m = a.get("megatron") or {}
        return int(m.get("tensor_model_parallel_size", 1) or 1) * int(m.get("pipeline_model_parallel_size", 1) or 1)

    def _create_dataloader(self, train_dataset, val_dataset, collate_fn, train_sampler) -> None:
        from ...utils.dataset.rl_dataset import collate_fn as default_collate
        from ...utils.dataset.rl_dataset import create_rl_dataset, create_rl_sampler
        from ...utils.dataset.stateful import StatefulDataLoader

        cfg = self.config
        if train_dataset is None:
            train_dataset = create_rl_dataset(cfg.data.get("train_files"), cfg.data, self.tokenizer, self.processor, is_train=True)
        if val_dataset is None and cfg.data.get("val_files"):
            val_dataset = create_rl_dataset(cfg.data.get("val_files"), cfg.data, self.tokenizer, self.processor, is_train=False)
        self.train_dataset, self.val_dataset = train_dataset, val_dataset
        collate_fn = collate_fn or default_collate
        rank, world = self._dp_rank_world()
        gbs = int(cfg.data.get("gen_batch_size", cfg.data.train_batch_size))
        assert gbs % world == 0, f"train_batch_size {gbs} must be divisible by the data-parallel world {world}"
        if train_sampler is None:
            train_sampler = create_rl_sampler(cfg.data, train_dataset, rank=rank, world=world)
        self.train_dataloader = StatefulDataLoader(train_dataset, batch_size=gbs // world, sampler=train_sampler,
                                                   collate_fn=collate_fn, drop_last=True,
                                                   num_workers=int(cfg.data.get("dataloader_num_workers", 0)))
        self.val_dataloader = None
        if val_dataset is not None and len(val_dataset) > 0:
            vbs = cfg.data.get("val_batch_size") or len(val_dataset)
            self.val_dataloader = StatefulDataLoader(val_dataset, batch_size=int(vbs), shuffle=bool(cfg.data.get("validation_shuffle", False)),
                                                     collate_fn=collate_fn, drop_last=False)
        assert len(self.train_dataloader) >= 1, "Train dataloader is empty!"
        total = len(self.train_dataloader) * cfg.trainer.total_epochs
        if cfg.trainer.get("total_training_steps") is not None:
            total = int(cfg.trainer.total_training_steps)
        self.total_training_steps = total
        for path in ("actor_rollout_ref.actor.optim", "critic.optim"):
            node = cfg.select(path) if hasattr(cfg, "select") else None
            if node is not None:
                node["total_training_steps"] = total

    # ------------------------------------------------------------------------------------ workers
    def init_workers(self) -> None:
        """Create the worker groups (actor/rollout/ref fused in one worker per GPU; critic optional)."""
        cfg = self.config
        if self.resource_pool_manager is not None:
            self.resource_pool_manager.create_resource_pool()
        pool = (self.resource_pool_manager.get_resource_pool(Role.ActorRollout)
                if self.resource_pool_manager is not None and Role.ActorRollout in self.resource_pool_manager.mapping else None)
        role = "actor_rollout_ref" if self.use_reference_policy else "actor_rollout"
        actor_cls = self.role_worker_mapping.get(Role.ActorRollout) or self.role_worker_mapping.get(Role.ActorRolloutRef)
        if actor_cls is None:
            from ...workers.engine_workers import ActorRolloutRefWorker as actor_cls
        from .utils import need_teacher_policy

        extra = {"distillation_config": cfg.get("distillation")} if need_teacher_policy(cfg) else {}
        self.actor_rollout_wg = self.ray_worker_group_cls(pool, ClassWithInitArgs(actor_cls, config=cfg.actor_rollout_ref, role=role, **extra),
                                                          **self.worker_group_kwargs)
        self.actor_rollout_wg.init_model()
        self.teacher_server_manager = self._build_teachers() if need_teacher_policy(cfg) else None
        self.ref_policy_wg = self.actor_rollout_wg
        self.ref_in_actor = True
        self.critic_wg = None
        if self.use_critic:
            critic_cls = self.role_worker_mapping.get(Role.Critic)
            if critic_cls is None:
                from ...workers.engine_workers import CriticWorker as critic_cls
            cpool = (self.resource_pool_manager.get_resource_pool(Role.Critic)
                     if self.resource_pool_manager is not None and Role.Critic in self.resource_pool_manager.mapping else pool)
            self.critic_wg = self.ray_worker_group_cls(cpool, ClassWithInitArgs(critic_cls, config=cfg.critic), **self.worker_group_kwargs)
            self.critic_wg.init_model()
        self.async_rollout_mode = False

    def _build_teachers(self):
        """Teacher models of on-policy distillation, colocated with the trainer: one frozen decoder per entry of
        ``distillation.teacher_models`` (``model_path``: a checkpoint directory or a preset name; ``key``: the value of
        ``distillation.teacher_key`` this teacher serves, the first entry is the default). They answer with the log-prob of
        the sampled token (estimator losses) or their top-k (``forward_kl_topk``).
        Parity target: ``verl/trainer/ppo/ray_trainer.py:925-940`` and ``verl/experimental/teacher_loop/teacher_model.py``."""
        from ...experimental.teacher_loop import AsyncTeacherLLMServerManager, MultiTeacherModelManager, TeacherModelManager
        from ...models import FlatParams
        from ...models.config import ModelConfig, get_preset
        from ...models.decoder import DecoderModel
        from ...utils.device import get_device_name
        from ..distillation.losses import get_distillation_loss_settings

        dc = self.config.distillation
        lc = dc.get("distillation_loss") or {}
        topk = int(lc.get("topk", 32) or 32) if get_distillation_loss_settings(str(lc.get("loss_mode", "k3"))).use_topk else 0
        dev = torch.device("cuda", torch.cuda.current_device()) if get_device_name() == "cuda" else torch.device("cpu")
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        managers = {}
        for name, tc in (dc.get("teacher_models") or {}).items():
            path = tc.get("model_path")
            if not path:
                continue
            if os.path.isdir(str(path)):
                from ...utils.model import load_hf_weights_into

                arch = ModelConfig.from_pretrained(str(path))
                params = FlatParams(arch, dtype=dtype, device=dev)
                load_hf_weights_into(params, str(path))
            else:
                arch = get_preset(str(path))
                params = FlatParams(arch, dtype=dtype, device=dev)
                params.init_weights(seed=int(tc.get("seed", 1234)))
            n = max(1, int(tc.get("num_replicas", 1) or 1))
            managers[str(tc.get("key") or name)] = TeacherModelManager.from_models(str(tc.get("key") or name), [DecoderModel(arch, params)] * n, topk=topk)
        if not managers:
            raise ValueError("distillation.enabled needs at least one distillation.teacher_models.<name>.model_path")
        rc = self.config.actor_rollout_ref.rollout
        return AsyncTeacherLLMServerManager(MultiTeacherModelManager(managers), int(self.config.data.max_response_length),
                                            int(getattr(self.tokenizer, "pad_token_id", 0) or 0))

    def _fit_compute_teacher_logprobs(self, batch: DataProto) -> DataProto:
        """On-policy distillation: the teachers' record for every trajectory of the batch, unless the rollout side attached it
        already (the agent loop does, trajectory by trajectory)."""
        if self.teacher_server_manager is None or "teacher_logprobs" in batch.batch.keys():
            return batch
        import asyncio

        with marked_timer("teacher", self.timing_raw, color="purple"):
            ids, am = batch.batch["input_ids"].cpu(), batch.batch["attention_mask"].cpu().bool()
            P = ids.shape[1] - batch.batch["responses"].shape[1]
            key = str(self.config.distillation.get("teacher_key", "data_source"))
            routes = batch.non_tensor_batch.get(key)

            async def go():
                return await asyncio.gather(*[
                    self.teacher_server_manager.compute_teacher_logprobs(
                        f"t{self.global_steps}-{i}", ids[i, :P][am[i, :P]].tolist(), ids[i, P:][am[i, P:]].tolist(),
                        routing_key=None if routes is None else routes[i]) for i in range(len(batch))])

            loop = asyncio.new_event_loop()
            try:
                got = loop.run_until_complete(go())
            finally:
                loop.close()
            dev = batch.batch["input_ids"].device
            batch.batch["teacher_ids"] = torch.stack([g["teacher_ids"] for g in got]).to(dev)
            batch.batch["teacher_logprobs"] = torch.stack([g["teacher_logprobs"] for g in got]).to(dev)
        return batch

    # ------------------------------------------------------------------------------------ checkpoint
    def _save_checkpoint(self) -> None:
        cfg = self.config.trainer
        root = os.path.join(cfg.default_local_dir, f"global_step_{self.global_steps}")
        os.makedirs(root, exist_ok=True)
        self.actor_rollout_wg.save_checkpoint(os.path.join(root, "actor"), None, self.global_steps,
                                              cfg.get("max_actor_ckpt_to_keep"))
        if self.use_critic:
            self.critic_wg.save_checkpoint(os.path.join(root, "critic"), None, self.global_steps,
                                           cfg.get("max_critic_ckpt_to_keep"))
        rank, _ = self._dp_rank_world()
        torch.save(self.train_dataloader.state_dict(), os.path.join(root, f"data_rank{rank}.pt" if self.spmd and rank else "data.pt"))
        if rank == 0:
            with open(os.path.join(cfg.default_local_dir, "latest_checkpointed_iteration.txt"), "w") as f:
                f.write(str(self.global_steps))
            keep = cfg.get("max_actor_ckpt_to_keep")
            if keep:
                from ...utils.checkpoint.checkpoint_manager import rotate_checkpoints

                rotate_checkpoints(cfg.default_local_dir, int(keep))

    def _load_checkpoint(self) -> int:
        cfg = self.config.trainer
        mode = cfg.get("resume_mode", "auto")
        if mode == "disable":
            return 0
        folder = None
        if mode == "auto":
            folder = find_latest_ckpt_path(cfg.default_local_dir)
        elif mode == "resume_path":
            folder = cfg.get("resume_from_path")
            assert folder and "global_step_" in folder, "resume ckpt must specify the global_steps"
        if folder is None:
            if mode == "auto":
                print("Training from scratch")
            return 0
        print(f"Load from checkpoint folder: {folder}")
        self.global_steps = int(str(folder).split("global_step_")[-1])
        self.actor_rollout_wg.load_checkpoint(os.path.join(folder, "actor"), None, cfg.get("del_local_ckpt_after_load", False))
        if self.use_critic:
            self.critic_wg.load_checkpoint(os.path.join(folder, "critic"), None, cfg.get("del_local_ckpt_after_load", False))
        rank, _ = self._dp_rank_world()
        dpath = os.path.join(folder, f"data_rank{rank}.pt" if self.spmd and rank else "data.pt")
        if os.path.exists(dpath):
            self.train_dataloader.load_state_dict(torch.load(dpath, weights_only=False))
        return self.global_steps

    # ------------------------------------------------------------------------------------ helpers
    def _balance_batch(self, batch: DataProto, metrics: dict, logging_prefix: str = "global_seqlen") -> None:
        """Reorder so that equal-sized data-parallel chunks carry equal attention+linear workload."""
        world = self.actor_rollout_wg.world_size
        if world <= 1:
            return
        lens = batch.batch["attention_mask"].view(len(batch), -1).sum(-1)
        cost = calculate_workload(lens).tolist()
        parts = get_seqlen_balanced_partitions(cost, k_partitions=world, equal_size=True)
        for p in parts:
            p.sort(key=lambda i: cost[i])
        idx = torch.tensor([j for p in parts for j in p])
        batch.reorder(idx)
        metrics.update(log_seqlen_unbalance(lens.tolist(), parts, logging_prefix))

    def _get_gen_batch(self, batch: DataProto) -> DataProto:
        # kept on the training batch as well: what the reward needs, and the processor outputs of images / videos that the
        # log-prob and update passes feed to the vision tower again
        reward_keys = {"data_source", "reward_model", "extra_info", "uid", "multi_modal_inputs"} & set(batch.non_tensor_batch)
        pop_keys = [k for k in ("input_ids", "attention_mask", "position_ids") if k in batch.batch.keys()]
        non_pop = [k for k in batch.non_tensor_batch if k not in reward_keys]
        gen = batch.pop(batch_keys=pop_keys, non_tensor_batch_keys=non_pop)
        for k in reward_keys:
            gen.non_tensor_batch[k] = batch.non_tensor_batch[k]
        return gen

    def _compute_reward(self, batch: DataProto, fn) -> tuple[torch.Tensor, dict]:
        if "rm_scores" in batch.batch.keys():
            return batch.batch["rm_scores"], {}
        res = fn(batch, return_dict=True)
        if isinstance(res, dict):
            return res["reward_tensor"], res.get("reward_extra_info", {})
        return res, {}

    def _allreduce_metrics(self, metrics: dict) -> dict:
        """SPMD mode: every rank holds metrics of its shard; average them so all ranks log the global value."""
        _, world = self._dp_rank_world()
        if world <= 1 or not metrics:
            return metrics
        keys = sorted(k for k, v in metrics.items() if isinstance(v, (int, float, np.floating, np.integer)))
        dev = "cuda" if self.device_name == "cuda" and torch.cuda.is_available() else "cpu"
        t = torch.tensor([float(metrics[k]) for k in keys], dtype=torch.float64, device=dev)
        mx, mn = t.clone(), t.clone()
        from ...utils.distributed import get_data_parallel_group

        g = get_data_parallel_group()
        dist.all_reduce(t, group=g)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=g)
        dist.all_reduce(mn, op=dist.ReduceOp.MIN, group=g)
        out = dict(metrics)
        for i, k in enumerate(keys):
            leaf = k.split("/")[-1]
            out[k] = float(mx[i]) if leaf == "max" or k.startswith("timing_s/") or k == "perf/time_per_step" else \
                float(mn[i]) if leaf == "min" else float(t[i]) if k == "perf/total_num_tokens" else float(t[i] / world)
        return out

    # ------------------------------------------------------------------------------------ validation
    def _validate(self) -> dict:
        if self.val_dataloader is None or self.val_reward_fn is None:
            return {}
        rewards_all, sources, uids = [], [], []
        extra: dict[str, list] = defaultdict(list)
        n = int(self.config.actor_rollout_ref.rollout.val_kwargs.get("n", 1))
        for batch_dict in self.val_dataloader:
            batch = DataProto.from_single_dict(batch_dict)
            if "uid" not in batch.non_tensor_batch:
                batch.non_tensor_batch["uid"] = np.array([str(uuid.uuid4()) for _ in range(len(batch))], dtype=object)
            batch = batch.repeat(n, interleave=True)
            gen = self._get_gen_batch(batch)
            gen.meta_info = {"do_sample": bool(self.config.actor_rollout_ref.rollout.val_kwargs.get("do_sample", False)),
                             "validate": True, "global_steps": self.global_steps}
            gen = self._to_device(gen)
            padded, pad = pad_dataproto_to_divisor(gen, max(1, self.actor_rollout_wg.world_size))
            out = unpad_dataproto(self.actor_rollout_wg.generate_sequences(padded), pad)
            batch = batch.union(out)
            reward, info = self._compute_reward(batch, self.val_reward_fn)
            scores = reward.sum(-1).cpu().tolist()
            rewards_all.extend(scores)
            extra["reward"].extend(scores)
            for k, v in info.items():
                extra[k].extend(list(v))
            sources.extend(batch.non_tensor_batch.get("data_source", np.array(["unknown"] * len(scores), dtype=object)).tolist())
            uids.extend(batch.non_tensor_batch["uid"].tolist())
        stats = process_validation_metrics(sources, uids, dict(extra))
        out = {}
        for ds, by_var in stats.items():
            core = "acc" if "acc" in by_var else "reward"
            for var, ms in by_var.items():
                for name, val in ms.items():
                    sec = "val-core" if var == core and (name.startswith("mean@") or name.startswith("maj@") or name.startswith("best@")) else "val-aux"
                    out[f"{sec}/{ds}/{var}/{name}"] = val
        return out

    def _to_device(self, data: DataProto) -> DataProto:
        """Stage a host batch onto this rank's GPU (pinned host memory, asynchronous copy)."""
        if self.device_name != "cuda" or not torch.cuda.is_available() or not self.spmd or data.batch is None:
            return data
        dev = torch.device("cuda", torch.cuda.current_device())
        for k in list(data.batch.keys()):
            v = data.batch[k]
            if isinstance(v, torch.Tensor) and not v.is_cuda:
                data.batch[k] = v.pin_memory().to(dev, non_blocking=True)
        return data

    # ------------------------------------------------------------------------------------ main loop
    def fit(self) -> None:
        cfg = self.config
        rank, world = self._dp_rank_world()
        logger = Tracking(project_name=cfg.trainer.get("project_name", "verl_b200"),
                          experiment_name=cfg.trainer.get("experiment_name", "run"),
                          default_backend=cfg.trainer.get("logger", ["console"]) if rank == 0 else [],
                          config=cfg)
        self.global_steps = 0
        self._load_checkpoint()
        self.actor_rollout_wg.update_weights(self.global_steps)
        if self.val_reward_fn is not None and cfg.trainer.get("val_before_train", False):
            val = self._validate()
            if val:
                logger.log(data=val, step=self.global_steps)
            if cfg.trainer.get("val_only", False):
                return
        self.global_steps += 1
        self.logger, self.last_val_metrics = logger, None
        for epoch in range(cfg.trainer.total_epochs):
            for batch_dict in self.train_dataloader:
                self.epoch = epoch
                self._bind_step({}, {})
                self._fit_prepare_step()
                metrics, timing_raw = self.train_step(batch_dict)
                self._bind_step(metrics, timing_raw)
                self._fit_validate()
                self._fit_save_checkpoint()
                self._fit_postprocess_step()
                if self.is_last_step:
                    if self.last_val_metrics:
                        print(f"Final validation metrics: {self.last_val_metrics}")
                    return

    # ---------------------------------------------------------------- one step as a template of overridable phases
    # ``fit_step`` / ``train_step`` run the ``_fit_*`` methods below in order; a subclass changes one phase by overriding
    # one method (same names and ``batch -> batch`` shape as ``verl/experimental/separation/ray_trainer.py:341-760``).
    # The phases write to ``self.metrics`` and ``self.timing_raw``, which ``_bind_step`` points at the caller's dicts.

    def _bind_step(self, metrics: Optional[dict] = None, timing_raw: Optional[dict] = None) -> None:
        if metrics is not None or not hasattr(self, "metrics"):
            self.metrics = {} if metrics is None else metrics
        if timing_raw is not None or not hasattr(self, "timing_raw"):
            self.timing_raw = {} if timing_raw is None else timing_raw

    def train_step(self, batch_dict: dict) -> tuple[dict, dict]:
        """One PPO/GRPO step on one batch of prompts: rollout -> reward -> log-probs -> advantage -> updates."""
        metrics: dict[str, Any] = {}
        timing_raw: dict[str, float] = {}
        with marked_timer("step", timing_raw):
            batch = self.rollout_phase(batch_dict, metrics, timing_raw)
            batch = self.learn_phase(batch, metrics, timing_raw)
            self.sync_phase(batch, metrics, timing_raw)
        return self.finish_step(batch, metrics, timing_raw)

    def fit_step(self, batch_dict: Any = None) -> tuple[dict, dict]:
        """``train_step`` plus what ``fit`` does around it (validation, checkpoint, logging, step counter), as one call."""
        self._bind_step({}, {})
        self._fit_prepare_step()
        self._fit_start_profile()
        with marked_timer("step", self.timing_raw):
            batch = self._fit_get_batch(batch_dict)
            batch = self._fit_generate(batch)
            batch = self._fit_balance(batch)
            batch = self._fit_compute_reward(batch)
            batch = self._fit_compute_log_prob(batch)
            batch = self._fit_compute_ref_log_prob(batch)
            batch = self._fit_compute_critic(batch)
            batch = self._fit_compute_teacher_logprobs(batch)
            batch = self._fit_compute_advantage(batch)
            batch = self._fit_update_critic(batch)
            batch = self._fit_update_actor(batch)
            self._fit_update_weights()
            self._fit_dump_data(batch)
        self._fit_validate()
        self._fit_save_checkpoint()
        self._fit_stop_profile()
        self._fit_collect_metrics(batch)
        self._fit_experimental(batch)
        self._fit_postprocess_step()
        return self.metrics, self.timing_raw

    def rollout_phase(self, batch_dict: dict, metrics: dict, timing_raw: dict) -> DataProto:
        """Prompts -> n sampled responses per prompt, merged with the prompt-side fields."""
        self._bind_step(metrics, timing_raw)
        return self._fit_generate(self._fit_get_batch(batch_dict))

    def learn_phase(self, batch: DataProto, metrics: dict, timing_raw: dict) -> DataProto:
        """Reward -> old/ref log-probs (-> values) -> advantages -> critic/actor updates on a generated batch."""
        self._bind_step(metrics, timing_raw)
        for phase in (self._fit_balance, self._fit_compute_reward, self._fit_compute_log_prob, self._fit_compute_ref_log_prob,
                      self._fit_compute_critic, self._fit_compute_teacher_logprobs, self._fit_compute_advantage, self._fit_update_critic,
                      self._fit_update_actor):
            batch = phase(batch)
        return batch

    def sync_phase(self, batch: Optional[DataProto], metrics: dict, timing_raw: dict) -> None:
        """Make the rollout side see the freshly updated weights (in place when colocated)."""
        self._bind_step(metrics, timing_raw)
        self._fit_update_weights()
        self._fit_dump_data(batch)

    def finish_step(self, batch: DataProto, metrics: dict, timing_raw: dict) -> tuple[dict, dict]:
        self._bind_step(metrics, timing_raw)
        self._fit_collect_metrics(batch)
        return self.metrics, timing_raw

    def _fit_prepare_step(self) -> None:
        self.is_last_step = self.global_steps >= self.total_training_steps

    def _fit_start_profile(self, should_profiler: Optional[bool] = None) -> None:
        steps = (self.config.get("global_profiler") or {}).get("steps") or []
        self.curr_step_profile = bool(should_profiler) if should_profiler is not None else self.global_steps in steps
        if self.curr_step_profile and hasattr(self.actor_rollout_wg, "start_profile"):
            with marked_timer("start_profile", self.timing_raw):
                self.actor_rollout_wg.start_profile(profile_step=self.global_steps)

    def _fit_stop_profile(self, should_profiler: Optional[bool] = None) -> None:
        on = getattr(self, "curr_step_profile", False) if should_profiler is None else should_profiler
        if on and hasattr(self.actor_rollout_wg, "stop_profile"):
            with marked_timer("stop_profile", self.timing_raw):
                self.actor_rollout_wg.stop_profile()
        self.curr_step_profile = False

    def _fit_get_batch(self, batch_dict: dict) -> DataProto:
        rank, _ = self._dp_rank_world()
        batch = DataProto.from_single_dict(batch_dict)
        batch.meta_info["temperature"] = self.config.actor_rollout_ref.rollout.temperature
        if "uid" not in batch.non_tensor_batch:
            batch.non_tensor_batch["uid"] = np.array([f"{rank}-{self.global_steps}-{i}" for i in range(len(batch))], dtype=object)
        return batch

    def _fit_generate(self, batch: DataProto) -> DataProto:
        cfg, algo, timing_raw = self.config, self.config.algorithm, self.timing_raw
        rollout_cfg = cfg.actor_rollout_ref.rollout
        remax = str(algo.adv_estimator) in ("remax", "AdvantageEstimator.REMAX")
        gen_batch = self._get_gen_batch(batch)
        gen_batch.meta_info = {"global_steps": self.global_steps, "temperature": rollout_cfg.temperature}
        gen_batch = gen_batch.repeat(repeat_times=rollout_cfg.n, interleave=True)
        gen_batch = self._to_device(gen_batch)
        with marked_timer("gen", timing_raw, color="red"):
            from ...utils.skip import SkipManager

            if cfg.get("skip") and not SkipManager.skip_instances and SkipManager.config is None:
                SkipManager.init(cfg)
            SkipManager.set_step(self.global_steps)
            gen_out = SkipManager.annotate("rollout")(lambda prompts: self.actor_rollout_wg.generate_sequences(prompts))(gen_batch)
            timing_raw.update({f"gen/{k}": v for k, v in gen_out.meta_info.pop("timing", {}).items()})
            gen_out.meta_info.pop("rollout_stats", None)
        if remax:
            with marked_timer("gen_max", timing_raw, color="purple"):
                base = deepcopy(gen_batch)
                base.meta_info["do_sample"] = False
                base_out = self.actor_rollout_wg.generate_sequences(base)
                tmp = batch.repeat(rollout_cfg.n, interleave=True).union(base_out)
                rb, _ = self._compute_reward(tmp, self.reward_fn)
                batch.batch = None
                baseline = rb.sum(-1)
        batch = batch.repeat(repeat_times=rollout_cfg.n, interleave=True)
        batch = batch.union(gen_out)
        if remax:
            batch.batch["reward_baselines"] = baseline
        if "response_mask" not in batch.batch.keys():
            batch.batch["response_mask"] = compute_response_mask(batch)
        return batch

    def _fit_balance(self, batch: DataProto) -> DataProto:
        """Reorder the rows so every data-parallel rank gets about the same number of tokens; record the token counts."""
        if self.config.trainer.get("balance_batch", True) and not self.spmd:
            self._balance_batch(batch, self.metrics)
        batch.meta_info["global_token_num"] = torch.sum(batch.batch["attention_mask"], dim=-1).tolist()
        return batch

    def _fit_compute_reward(self, batch: DataProto) -> DataProto:
        with marked_timer("reward", self.timing_raw, color="yellow"):
            reward_tensor, reward_extra = self._compute_reward(batch, self.reward_fn)
            batch.batch["token_level_scores"] = reward_tensor
            for k, v in reward_extra.items():
                batch.non_tensor_batch[k] = np.asarray(v)
        return batch

    def _fit_compute_log_prob(self, batch: DataProto) -> DataProto:
        cfg, metrics = self.config, self.metrics
        with marked_timer("old_log_prob", self.timing_raw, color="blue"):
            old = self.actor_rollout_wg.compute_log_prob(batch)
            ent = old.batch["entropys"]
            metrics["actor/entropy"] = agg_loss(ent, batch.batch["response_mask"].to(ent.dtype),
                                                cfg.actor_rollout_ref.actor.get("loss_agg_mode", "token-mean")).item()
            old.batch.pop("entropys")
            batch = batch.union(old)
            if "rollout_log_probs" in batch.batch.keys():
                m = batch.batch["response_mask"].bool()
                diff = (torch.exp(batch.batch["rollout_log_probs"]) - torch.exp(batch.batch["old_log_probs"])).abs()
                sel = diff[m]
                if sel.numel():
                    metrics.update({"training/rollout_probs_diff_max": sel.max().item(),
                                    "training/rollout_probs_diff_mean": sel.mean().item()})
        return batch

    def _fit_compute_ref_log_prob(self, batch: DataProto) -> DataProto:
        if self.use_reference_policy:
            with marked_timer("ref", self.timing_raw, color="olive"):
                batch = batch.union(self.ref_policy_wg.compute_ref_log_prob(batch))
        return batch

    def _fit_compute_critic(self, batch: DataProto) -> DataProto:
        if self.use_critic:
            with marked_timer("values", self.timing_raw, color="cyan"):
                batch = batch.union(self.critic_wg.compute_values(batch))
        return batch

    def _fit_compute_advantage(self, batch: DataProto) -> DataProto:
        algo, metrics = self.config.algorithm, self.metrics
        with marked_timer("adv", self.timing_raw, color="brown"):
            if algo.get("use_kl_in_reward", False):
                batch, kl_m = apply_kl_penalty(batch, kl_ctrl=self.kl_ctrl_in_reward, kl_penalty=algo.get("kl_penalty", "kl"),
                                               dp=self._dp_view())
                metrics.update(kl_m)
            else:
                batch.batch["token_level_rewards"] = batch.batch["token_level_scores"]
            rc = algo.get("rollout_correction")
            if rc is not None and "rollout_log_probs" in batch.batch.keys() and (rc.get("rollout_is") or rc.get("rollout_rs")):
                from .rollout_corr_helper import compute_rollout_correction_and_add_to_batch

                batch, rc_m = compute_rollout_correction_and_add_to_batch(batch, rc)
                metrics.update(rc_m)
            batch = self._compute_advantage(batch, adv_estimator=algo.adv_estimator, gamma=algo.get("gamma", 1.0),
                                            lam=algo.get("lam", 1.0), num_repeat=self.config.actor_rollout_ref.rollout.n,
                                            norm_adv_by_std_in_grpo=algo.get("norm_adv_by_std_in_grpo", True), config=algo,
                                            dp=self._dp_view())
        return batch

    def _compute_advantage(self, batch: DataProto, **kw) -> DataProto:
        """Estimator dispatch; the replay-buffer trainers override it for sessions that produced several rows."""
        return compute_advantage(batch, **kw)

    def _fit_update_critic(self, batch: DataProto) -> DataProto:
        if self.use_critic:
            with marked_timer("update_critic", self.timing_raw, color="pink"):
                cout = self.critic_wg.update_critic(batch)
            self.metrics.update(reduce_metrics(cout.meta_info["metrics"]))
        return batch

    def _fit_update_actor(self, batch: DataProto) -> DataProto:
        if self.config.trainer.get("critic_warmup", 0) <= self.global_steps:
            with marked_timer("update_actor", self.timing_raw, color="red"):
                aout = self.actor_rollout_wg.update_actor(batch)
            self.metrics.update(reduce_metrics(aout.meta_info["metrics"]))
        return batch

    def _fit_update_weights(self) -> None:
        with marked_timer("update_weights", self.timing_raw, color="red"):
            res = self.actor_rollout_wg.update_weights(self.global_steps)
            res = res[0] if isinstance(res, list) else res
            self.metrics["timing_s/update_weights_worker"] = float((res or {}).get("timing_s/update_weights", 0.0))

    def _fit_dump_data(self, batch: Optional[DataProto]) -> None:
        if batch is not None and self.config.trainer.get("rollout_data_dir"):
            self._dump_generations(batch, self.config.trainer.rollout_data_dir)

    def _fit_validate(self) -> None:
        tf = self.config.trainer.get("test_freq", -1)
        if self.val_reward_fn is not None and tf and tf > 0 and (self.is_last_step or self.global_steps % tf == 0):
            with marked_timer("testing", self.timing_raw):
                self.last_val_metrics = self._validate()
            self.metrics.update(self.last_val_metrics)

    def _fit_save_checkpoint(self) -> None:
        cfg = self.config
        sf = cfg.trainer.get("save_freq", -1)
        esi = should_save_ckpt_esi(max_steps_duration=self.timing_raw.get("step", 0.0),
                                   redundant_time=cfg.trainer.get("esi_redundant_time", 0))
        if sf and sf > 0 and (self.is_last_step or self.global_steps % sf == 0 or esi):
            with marked_timer("save_checkpoint", self.timing_raw):
                self._save_checkpoint()

    def _fit_collect_metrics(self, batch: DataProto) -> None:
        metrics, timing_raw = self.metrics, self.timing_raw
        rank, world = self._dp_rank_world()
        n_gpus = self.resource_pool_manager.get_n_gpus() if self.resource_pool_manager is not None else world
        metrics.update(compute_data_metrics(batch=batch, use_critic=self.use_critic))
        metrics.update(compute_timing_metrics(batch=batch, timing_raw=timing_raw))
        metrics.update(compute_throughout_metrics(batch=batch, timing_raw=timing_raw, n_gpus=max(1, n_gpus if not self.spmd else 1)))
        reduced = self._allreduce_metrics(metrics)
        if reduced is not metrics:
            metrics.clear()
            metrics.update(reduced)
        if self.spmd and world > 1:
            metrics["perf/throughput"] = metrics["perf/total_num_tokens"] / (metrics["perf/time_per_step"] * world)
        self.last_batch = batch

    def _fit_experimental(self, batch: DataProto) -> None:
        """Hook for subclasses (curriculum samplers, extra dumps); nothing by default."""

    def _fit_postprocess_step(self) -> None:
        self.metrics["training/global_step"] = self.global_steps
        self.metrics["training/epoch"] = getattr(self, "epoch", 0)
        logger = getattr(self, "logger", None)
        if logger is not None:
            logger.log(data=self.metrics, step=self.global_steps)
        self.global_steps += 1

    def _dump_generations(self, batch: DataProto, dump_path: str) -> None:
        os.makedirs(dump_path, exist_ok=True)
        rank, _ = self._dp_rank_world()
        scores = batch.batch["token_level_scores"].sum(-1).cpu().tolist()
        ids_in = batch.batch["prompts"].cpu()
        ids_out = batch.batch["responses"].cpu()
        with open(os.path.join(dump_path, f"{self.global_steps}_rank{rank}.jsonl"), "w") as f:
            for i in range(len(batch)):
                rec = {"step": self.global_steps, "score": scores[i]}
                if self.tokenizer is not None:
                    rec["input"] = self.tokenizer.decode(ids_in[i], skip_special_tokens=True)
                    rec["output"] = self.tokenizer.decode(ids_out[i], skip_special_tokens=True)
                else:
                    rec["input_ids"] = ids_in[i].tolist()
                    rec["output_ids"] = ids_out[i].tolist()
                f.write(json.dumps(rec, ensure_ascii=False) + "\n")
