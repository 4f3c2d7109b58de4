"""``python -m verl_b200.experimental.fully_async_policy.fully_async_main <overrides>``: GRPO/PPO with a streaming
rollouter, a message queue and a trainer that synchronises weights every ``async_training.trigger_parameter_sync_step``
updates. Parity target: ``verl/experimental/fully_async_policy/fully_async_main.py``."""

from __future__ import annotations

import sys
from typing import Optional, Sequence

from ...trainer import main_ppo


class FullyAsyncTaskRunner(main_ppo.TaskRunner):
    def run(self, config):
        import verl_b200.trainer.ppo.v1.trainer_base as tb

        from .fully_async_trainer import FullyAsyncTrainer

        tb._TRAINERS["fully_async"] = FullyAsyncTrainer
        config.trainer["use_v1"] = True
        if config.trainer.get("v1") is None:
            config.trainer["v1"] = {}
        config.trainer["v1"]["trainer_mode"] = "fully_async"
        return super().run(config)


def main(argv: Optional[Sequence[str]] = None):
    from ...utils.config import load_config

    argv = list(sys.argv[1:] if argv is None else argv)
    config = load_config(main_ppo.CONFIG_DIR, "ppo_trainer", argv)
    return main_ppo.run_ppo(config, task_runner_class=FullyAsyncTaskRunner)


if __name__ == "__main__":
    main()
