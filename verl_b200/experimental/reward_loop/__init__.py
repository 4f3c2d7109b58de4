from .reward_loop import RewardLoopManager, RewardLoopWorker, migrate_legacy_reward_impl  # noqa: F401
from .reward_model import RewardModelManager, RewardModelServer  # noqa: F401
