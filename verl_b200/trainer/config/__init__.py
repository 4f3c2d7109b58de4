from .algorithm import AlgoConfig, FilterGroupsConfig, KLControlConfig, RolloutCorrectionConfig  # noqa: F401
import os as _os

CONFIG_DIR = _os.path.dirname(_os.path.abspath(__file__))
