from .base import RewardManagerBase  # noqa: F401
from .dapo import DAPORewardManager  # noqa: F401
from .gdpo import GDPORewardManager  # noqa: F401
from .limited import AsyncTokenBucket, RateLimitedRewardManager  # noqa: F401
from .naive import NaiveRewardManager  # noqa: F401
from .registry import get_reward_manager_cls, register  # noqa: F401
from .remote import RemoteRewardManager  # noqa: F401
