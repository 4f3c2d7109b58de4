"""``python -m verl_b200.experimental.one_step_off_policy.main_ppo <overrides>`` (add ``trainer.v1.rollout_ranks=R`` under
``torchrun`` to dedicate the last R ranks to generation). Parity target:
``verl/experimental/one_step_off_policy/main_ppo.py``."""

from __future__ import annotations

import sys
from typing import Optional, Sequence

from ...trainer import main_ppo


class OneStepOffTaskRunner(main_ppo.TaskRunner):
    mode = "one_step_off"

    def run(self, config):
        from . import ray_trainer  # noqa: F401  (registers the mode)

        config.trainer["use_v1"] = True
        if config.trainer.get("v1") is None:
            config.trainer["v1"] = {}
        config.trainer["v1"]["trainer_mode"] = self.mode
        return super().run(config)


def main(argv: Optional[Sequence[str]] = None):
    from ...utils.config import load_config

    argv = list(sys.argv[1:] if argv is None else argv)
    return main_ppo.run_ppo(load_config(main_ppo.CONFIG_DIR, "ppo_trainer", argv), task_runner_class=OneStepOffTaskRunner)


if __name__ == "__main__":
    main()
