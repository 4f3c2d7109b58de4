"""Pool and role tables of a disaggregated job: which roles exist and how many GPUs each pool gets.

Parity target: ``verl/experimental/separation/utils.py`` (``create_resource_pool_manager`` :22,
``create_role_worker_mapping`` :62).
"""

from __future__ import annotations

from ...trainer.ppo.ray_trainer import ResourcePoolManager
from ...trainer.ppo.utils import Role, need_critic, need_reference_policy

__all__ = ["create_resource_pool_manager", "create_role_worker_mapping"]


def _get(cfg, path: str, default=None):
    cur = cfg
    for k in path.split("."):
        cur = cur.get(k, None) if hasattr(cur, "get") else getattr(cur, k, None)
        if cur is None:
            return default
    return cur


def create_resource_pool_manager(config, roles: list) -> ResourcePoolManager:
    """Trainer pool (actor, critic, reference policy) sized by ``trainer.{nnodes,n_gpus_per_node}``; rollout pool sized by
    ``rollout.{nnodes,n_gpus_per_node}``; roles that do not exist in ``roles`` get no mapping."""
    spec, mapping = {}, {}
    train_roles = [r for r in roles if r in (Role.Actor, Role.ActorRollout, Role.ActorRolloutRef, Role.Critic, Role.RefPolicy, Role.RewardModel)]
    if train_roles:
        spec["trainer_pool"] = [int(_get(config, "trainer.n_gpus_per_node", 1))] * int(_get(config, "trainer.nnodes", 1))
        mapping.update({r: "trainer_pool" for r in train_roles})
    if Role.Rollout in roles:
        n = int(_get(config, "rollout.n_gpus_per_node", 0) or 0)
        assert n > 0, "a separate rollout pool needs rollout.n_gpus_per_node > 0"
        spec["rollout_pool"] = [n] * int(_get(config, "rollout.nnodes", 1))
        mapping[Role.Rollout] = "rollout_pool"
    return ResourcePoolManager(resource_pool_spec=spec, mapping=mapping)


def create_role_worker_mapping(config) -> dict:
    """Role -> worker class for the disaggregated trainer: detached actor (no colocated generation), a rollout-only
    service, plus critic / reference policy where the algorithm needs them."""
    from ...workers.engine_workers import ActorRolloutRefWorker, CriticWorker
    from .ray_trainer import DetachActorWorker, DetachRolloutService

    mapping = {Role.Actor: DetachActorWorker, Role.Rollout: DetachRolloutService}
    if need_critic(config):
        mapping[Role.Critic] = CriticWorker
    if need_reference_policy(config):
        mapping[Role.RefPolicy] = ActorRolloutRefWorker
    return mapping
