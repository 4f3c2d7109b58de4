from .abstract import AbstractRewardManager  # noqa: F401
from .naive import BatchRewardManager, DAPORewardManager, NaiveRewardManager, TokenRuleRewardManager  # noqa: F401
from .prime import PrimeRewardManager  # noqa: F401
from .registry import get_reward_manager_cls, register  # noqa: F401
