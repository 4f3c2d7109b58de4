from .skip_manager import SkipManager  # noqa: F401
from .rollout_skip import RolloutSkip  # noqa: F401
