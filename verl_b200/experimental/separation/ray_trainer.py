"""Base of the trainers that keep the actor and the rollout engines in separate pools.

The split-job machinery (rank layout, prompt/sample queues, flat-buffer weight broadcast, rollout-only service) is
``verl_b200.trainer.ppo.v1.trainer_separate_async``; this class fixes the policy knobs that "separation" means in the
reference: no hybrid switching (pools never exchange GPUs) and weights pushed after every step. The step itself is the
template of ``_fit_*`` phases inherited from ``RayPPOTrainer`` (``fit_step``: prepare, profile, get batch, generate, reward,
log-probs, reference log-probs, values, advantage, critic update, actor update, weight hand-over, dump, validate, checkpoint,
metrics): a subclass changes one phase by overriding one method, as with the reference's class of the same name.

Parity target: ``verl/experimental/separation/{ray_trainer.py 763, engine_workers.py 169, utils.py 95}``.
"""

from __future__ import annotations

from ...trainer.ppo.v1.trainer_base import register_trainer
from ...trainer.ppo.v1.trainer_separate_async import PPOTrainerSeparateAsync, RolloutService, SeparateTopology  # noqa: F401

__all__ = ["SeparateRayPPOTrainer", "DetachActorWorker", "DetachRolloutService"]


@register_trainer("separation")
class SeparateRayPPOTrainer(PPOTrainerSeparateAsync):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.switch.enabled = False

    def _tc(self, key: str, default=None):
        if key == "parameter_sync_step":
            return 1
        if key == "hybrid_switch":
            return False
        return super()._tc(key, default)


DetachRolloutService = RolloutService


def DetachActorWorker(config, **kwargs):
    """Actor (+ref) worker of the trainer pool; it still owns an idle in-place rollout engine for validation."""
    from ...workers.engine_workers import ActorRolloutRefWorker

    return ActorRolloutRefWorker(config=config, role=kwargs.pop("role", "actor_rollout_ref"), **kwargs)
