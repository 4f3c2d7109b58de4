from .replay_buffer import ReplayBuffer, ReplayBufferAsync  # noqa: F401
from .trainer_base import PPOTrainer, get_trainer_cls, register_trainer  # noqa: F401
