"""One-step-off-policy training: while the trainer pool updates on batch ``k``, the rollout pool already generates
batch ``k+1`` with the weights of step ``k-1``; weights are broadcast after every step. Staleness is therefore
exactly one version, by construction rather than by filtering.

On a split job this is the separate-pool trainer with one batch of look-ahead, a sync every step and no dropping;
on a single pool generation and training cannot overlap and the schedule degenerates to: generate ``k+1`` (old
weights), train ``k``, hand weights over.

Parity target: ``verl/experimental/one_step_off_policy/{ray_trainer.py 408, main_ppo.py 129}``; docs
``docs/advance/one_step_off.md``.
"""

from __future__ import annotations

from ...trainer.ppo.v1.trainer_base import register_trainer
from ..separation.ray_trainer import SeparateRayPPOTrainer

__all__ = ["OneStepOffRayTrainer"]


@register_trainer("one_step_off")
class OneStepOffRayTrainer(SeparateRayPPOTrainer):
    def _tc(self, key: str, default=None):
        fixed = {"num_warmup_batches": 1, "max_off_policy_threshold": 1, "max_off_policy_strategy": "wait", "parameter_sync_step": 1}
        return fixed[key] if key in fixed else super()._tc(key, default)
