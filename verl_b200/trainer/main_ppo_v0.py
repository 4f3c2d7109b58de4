"""Entry point pinned to the synchronous (v0) trainer regardless of ``trainer.use_v1``.
Parity target: ``verl/trainer/main_ppo_v0.py:35-234``."""

from __future__ import annotations

import sys
from typing import Optional, Sequence

from . import main_ppo


def main(argv: Optional[Sequence[str]] = None):
    argv = list(sys.argv[1:] if argv is None else argv) + ["trainer.use_v1=false"]
    return main_ppo.main(argv)


if __name__ == "__main__":
    main()
