"""``colocate_async`` mode: trainer and rollout share the GPUs, but rollout requests outlive training steps.

``num_warmup_batches`` extra batches of prompts are kept in flight. When a batch worth of groups is complete the
engines are paused (in-flight requests are aborted; the client keeps their partial outputs), training and the weight
hand-over run, and generation resumes from the partial outputs under the new weights with the remaining token
budget. Trajectories therefore span several weight versions, bounded by ``max_off_policy_threshold`` with strategy
``drop`` (evict and refill) or ``wait`` (stop admitting new prompts until the oldest group finishes).

Parity target: ``verl/trainer/ppo/v1/trainer_colocate_async.py:26-59``, ``verl/workers/rollout/llm_server.py:292-461``.
"""

from __future__ import annotations

from .trainer_base import PPOTrainer, register_trainer

__all__ = ["PPOTrainerColocateAsync"]


@register_trainer("colocate_async")
class PPOTrainerColocateAsync(PPOTrainer):
    fully_async_client = True

    def _target_inflight(self) -> int:
        return int(self.config.data.train_batch_size) * (1 + int(self._tc("num_warmup_batches", 1)))

    def _top_up(self) -> None:
        rb = self.replay_buffer
        if not rb.may_start_new_prompt(self.param_version):
            return
        backlog = rb.inflight() + rb.count("finished") + rb.count("failure")
        need = self._target_inflight() - backlog
        if need > 0:
            self._submit_prompts(self._next_prompts(need))

    def on_train_begin(self) -> None:
        self._each_server("wake_up")
        self._top_up()

    def on_sample_begin(self) -> None:
        self._each_server("resume_generation")
        self._top_up()

    def on_sample_end(self) -> None:
        self._each_server("abort_all_requests")  # partial outputs stay with the clients; nothing is lost
        self._pump()

    def on_step_end(self, batch, metrics, timing_raw) -> None:
        self._push_weights(batch, metrics, timing_raw)
