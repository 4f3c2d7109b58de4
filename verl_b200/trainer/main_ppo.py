"""Command-line entry point of the PPO-family trainers.

    python -m verl_b200.trainer.main_ppo key=value ...                       # one process: controller + workers
    torchrun --nproc-per-node 8 -m verl_b200.trainer.main_ppo key=value ...   # one process per GPU (SPMD controller)

Parity target: ``verl/trainer/main_ppo.py`` (:34-196) and ``main_ppo_v0.py`` (``TaskRunner.run`` :151-234).
"""

from __future__ import annotations

import os
import sys
from typing import Optional, Sequence

from ..utils.config import DictConfig, load_config, validate_config
from ..utils.device import auto_set_device, get_device_name
from .config import CONFIG_DIR
from .ppo.utils import Role, need_critic, need_reference_policy

__all__ = ["main", "run_ppo", "TaskRunner", "create_rl_dataset", "create_rl_sampler"]

from ..utils.dataset.rl_dataset import create_rl_dataset, create_rl_sampler  # noqa: E402  (re-exported like the reference)


def _select_worker_group(config):
    from ..single_controller.local import InProcessWorkerGroup, MultiprocessWorkerGroup, SPMDWorkerGroup

    kind = config.trainer.get("worker_group", "auto")
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    n = int(config.trainer.n_gpus_per_node) * int(config.trainer.nnodes)
    if kind == "auto":
        kind = "spmd" if (world_env > 1 or n == 1) else "multiprocess"
    if kind == "spmd":
        return SPMDWorkerGroup, {}
    if kind == "multiprocess":
        return MultiprocessWorkerGroup, {"device": get_device_name()}
    if kind == "inprocess":
        return InProcessWorkerGroup, {}
    if kind == "ray":
        from ..single_controller.ray import RayWorkerGroup

        return RayWorkerGroup, {}
    raise ValueError(f"unknown trainer.worker_group={kind}")


class TaskRunner:
    """Builds tokenizer, reward functions, datasets, resource pools and the trainer, then runs ``fit``."""

    def __init__(self):
        self.role_worker_mapping = {}
        self.mapping = {}

    def add_actor_rollout_worker(self, config):
        from ..workers.engine_workers import ActorRolloutRefWorker

        self.role_worker_mapping[Role.ActorRollout] = ActorRolloutRefWorker
        self.mapping[Role.ActorRollout] = "global_pool"
        return ActorRolloutRefWorker

    def add_critic_worker(self, config):
        from ..workers.engine_workers import CriticWorker

        self.role_worker_mapping[Role.Critic] = CriticWorker
        self.mapping[Role.Critic] = "global_pool"

    def init_resource_pool_mgr(self, config):
        from .ppo.ray_trainer import ResourcePoolManager

        spec = {"global_pool": [int(config.trainer.n_gpus_per_node)] * int(config.trainer.nnodes)}
        return ResourcePoolManager(resource_pool_spec=spec, mapping=self.mapping)

    def run(self, config):
        from ..utils.tokenizer import hf_tokenizer
        from .ppo.ray_trainer import RayPPOTrainer
        from .ppo.reward import load_reward_manager

        auto_set_device(config)
        validate_config(config, use_reference_policy=need_reference_policy(config), use_critic=need_critic(config))
        self.add_actor_rollout_worker(config)
        if need_critic(config):
            self.add_critic_worker(config)
        path = config.actor_rollout_ref.model.path
        # a model directory that holds only a configuration (random-initialised runs on token-level data) has no tokenizer
        has_tok = os.path.isdir(str(path)) and any(os.path.exists(os.path.join(str(path), f))
                                                   for f in ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "vocab.json"))
        tokenizer = hf_tokenizer(path, trust_remote_code=config.data.get("trust_remote_code", False)) if has_tok else None
        reward_fn = load_reward_manager(config, tokenizer, num_examine=0)
        val_reward_fn = load_reward_manager(config, tokenizer, num_examine=1)
        wg_cls, wg_kwargs = _select_worker_group(config)
        pool_mgr = self.init_resource_pool_mgr(config)
        if getattr(wg_cls, "is_spmd", False):
            from ..utils.distributed import initialize_global_process_group

            initialize_global_process_group()
        trainer_cls, v1, extra = RayPPOTrainer, False, {}
        in_process = wg_cls.__name__ in ("InProcessWorkerGroup", "SPMDWorkerGroup")
        use_v1 = bool(config.trainer.get("use_v1", True)) and in_process
        if use_v1:
            why = _v1_unsupported_reason(config)
            if why:
                import warnings

                warnings.warn(f"trainer.use_v1=true, but {why}: running the synchronous v0 trainer instead", stacklevel=2)
                use_v1 = False
        if use_v1:
            from .ppo.v1.trainer_base import get_trainer_cls

            v1cfg = config.trainer.get("v1") or {}
            mode = v1cfg.get("trainer_mode", "sync")
            trainer_cls, v1 = get_trainer_cls(mode), True
            if mode in ("separate_async", "separation", "one_step_off"):
                res = self._split_job(config, int(v1cfg.get("rollout_ranks", 0) or 0), tokenizer)
                if not hasattr(res, "T"):
                    return res  # this rank served rollout until the trainers finished
                extra["topology"] = res
        trainer = trainer_cls(config=config, tokenizer=tokenizer, role_worker_mapping=self.role_worker_mapping,
                              resource_pool_manager=pool_mgr, ray_worker_group_cls=wg_cls, reward_fn=reward_fn,
                              val_reward_fn=val_reward_fn, device_name=config.trainer.device, worker_group_kwargs=wg_kwargs,
                              **extra)
        if v1:
            trainer.init()
        else:
            trainer.init_workers()
        trainer.fit()
        return trainer


def _v1_unsupported_reason(config) -> Optional[str]:
    """The v1 (replay-buffer) trainers drive the native continuous-batching rollout engine step by step; a model family that
    samples through the library module's own cache has no such engine. Returns why v1 cannot run, or None."""
    try:
        from ..utils.config import omega_conf_to_dataclass
        from ..workers.config import HFModelConfig

        m = config.actor_rollout_ref.model
        mc = m if isinstance(m, HFModelConfig) else omega_conf_to_dataclass(m, HFModelConfig)
        if getattr(mc.arch, "is_generic", False):
            return f"model family '{mc.arch.model_type}' samples through the library module (no step-wise rollout engine)"
    except Exception:
        return None
    # a training replica that spans several ranks (sequence / context / tensor / pipeline parallel) shares one set of prompts
    # and exchanges the generated rows inside the replica; that exchange lives in the synchronous generate_sequences path
    a = config.actor_rollout_ref.actor
    fc = a.get("fsdp_config") or {}
    m = a.get("megatron") or {}
    span = max(int(a.get("ulysses_sequence_parallel_size", 1) or 1), int((fc.get("context_parallel_size", 1) if hasattr(fc, "get") else 1) or 1))
    if str(a.get("strategy", "fsdp")) == "megatron":
        span = max(span, int(m.get("tensor_model_parallel_size", 1) or 1) * int(m.get("pipeline_model_parallel_size", 1) or 1)
                   * int(m.get("context_parallel_size", 1) or 1))
    if span > 1:
        return f"the training replica spans {span} ranks (sequence / context / tensor / pipeline parallelism)"
    return None


def _split_job_impl(config, rollout_ranks: int, tokenizer):
    """separate_async: build the rank layout; rollout-only ranks serve until told to stop and return their stats,
    trainer ranks get the topology back."""
    from ..utils.distributed import set_data_parallel_group
    from ..workers.engine_workers import ActorRolloutRefWorker
    from .ppo.v1.trainer_separate_async import RolloutService, SeparateTopology

    topo = SeparateTopology(rollout_ranks)
    if topo.R == 0:
        return topo
    if not topo.is_rollout_rank:
        set_data_parallel_group(topo.trainer_group)
        return topo
    set_data_parallel_group(topo.rollout_group)
    worker = ActorRolloutRefWorker(config=config.actor_rollout_ref, role="rollout")
    worker.init_model()
    return RolloutService(config, worker, topo, tokenizer).run()


TaskRunner._split_job = staticmethod(_split_job_impl)


def run_ppo(config, task_runner_class=None):
    runner = (task_runner_class or TaskRunner)()
    return runner.run(config)


def main(argv: Optional[Sequence[str]] = None):
    argv = list(sys.argv[1:] if argv is None else argv)
    cfg_dir, cfg_name, overrides = CONFIG_DIR, "ppo_trainer", []
    for a in argv:
        if a.startswith("--config-path="):
            cfg_dir = a.split("=", 1)[1]
        elif a.startswith("--config-name="):
            cfg_name = a.split("=", 1)[1]
        else:
            overrides.append(a)
    config = load_config(cfg_dir, cfg_name, overrides)
    return run_ppo(config)


if __name__ == "__main__":
    main()
