"""``sync`` mode: strictly on-policy. Each step submits exactly one batch of prompts, waits for all groups,
puts the engines to sleep while training, and hands weights over at the end of the step.

Parity target: ``verl/trainer/ppo/v1/trainer_sync.py:25-42`` (``on_step_end`` -> ``update_weights``,
``on_sample_end`` -> ``sleep_replicas``).
"""

from __future__ import annotations

from .trainer_base import PPOTrainer, register_trainer

__all__ = ["PPOTrainerSync"]


@register_trainer("sync")
class PPOTrainerSync(PPOTrainer):
    def on_sample_begin(self) -> None:
        self._each_server("wake_up")
        need = int(self.config.data.train_batch_size) - self.replay_buffer.inflight()
        if need > 0:
            self._submit_prompts(self._next_prompts(need))

    def on_sample_end(self) -> None:
        # DAPO over-provisioning may leave extra groups in flight: they belong to no later (on-policy) step
        self._each_server("abort_all_requests")
        for t in list(self._tasks):
            t.cancel()
        self._pump()
        self.replay_buffer.drain_inflight()
        self._each_server("resume_generation")
        self._each_server("sleep")

    def on_step_end(self, batch, metrics, timing_raw) -> None:
        self._push_weights(batch, metrics, timing_raw)
