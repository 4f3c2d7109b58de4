from .checkpoint_manager import BaseCheckpointManager, find_latest_ckpt_path, should_save_ckpt_esi, rotate_checkpoints  # noqa: F401
