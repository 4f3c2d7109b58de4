"""Trainer roles. Parity target: ``verl/trainer/ppo/utils.py`` (``Role`` :27-72, ``need_reference_policy`` :75,
``need_critic`` :96)."""

from __future__ import annotations

import warnings
from enum import Enum

__all__ = ["Role", "need_reference_policy", "need_reward_model", "need_critic", "need_teacher_policy"]


class Role(Enum):
    Actor = 0
    Rollout = 1
    ActorRollout = 2
    Critic = 3
    RefPolicy = 4
    RewardModel = 5
    ActorRolloutRef = 6
    Env = 7
    TeacherModel = 8

    def __str__(self) -> str:
        return self._get_role_string()

    def _get_role_string(self) -> str:
        return {Role.Actor: "actor", Role.Rollout: "rollout", Role.ActorRollout: "actor_rollout", Role.Critic: "critic",
                Role.RefPolicy: "ref", Role.RewardModel: "rm", Role.ActorRolloutRef: "actor_rollout_ref", Role.Env: "env",
                Role.TeacherModel: "teacher"}.get(self, self.name.lower())

    @classmethod
    def from_string(cls, name: str) -> "Role":
        m = {"actor": cls.Actor, "rollout": cls.Rollout, "actor_rollout": cls.ActorRollout, "critic": cls.Critic,
             "ref": cls.RefPolicy, "rm": cls.RewardModel, "actor_rollout_ref": cls.ActorRolloutRef, "env": cls.Env,
             "teacher": cls.TeacherModel}
        if name.lower() not in m:
            raise ValueError(f"No Role found for string: {name}")
        return m[name.lower()]


def need_reference_policy(config) -> bool:
    """A frozen reference policy is needed for KL-in-reward or a KL loss term."""
    return bool(config.algorithm.get("use_kl_in_reward", False) or config.actor_rollout_ref.actor.get("use_kl_loss", False))


def need_reward_model(config) -> bool:
    rm = config.get("reward_model") or (config.get("reward") or {}).get("reward_model") or {}
    return bool(rm.get("enable", False))


def need_teacher_policy(config) -> bool:
    return bool((config.get("distillation") or {}).get("enabled", False))


def need_critic(config) -> bool:
    """The critic is needed for GAE unless explicitly disabled; group-baseline estimators never need it."""
    enable = config.critic.get("enable", None) if config.get("critic") is not None else False
    if enable is not None:
        return bool(enable)
    if config.algorithm.adv_estimator == "gae":
        return True
    warnings.warn("Disabled critic as algorithm.adv_estimator != gae. If it is not intended, please set critic.enable=True",
                  stacklevel=2)
    return False
