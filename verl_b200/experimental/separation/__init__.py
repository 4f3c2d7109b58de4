from .ray_trainer import SeparateRayPPOTrainer  # noqa: F401
