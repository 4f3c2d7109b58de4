from .config import ModelConfig, PRESETS, get_preset  # noqa: F401
from .weights import FlatParams, build_param_specs  # noqa: F401
from .decoder import DecoderModel, PackedBatch  # noqa: F401
