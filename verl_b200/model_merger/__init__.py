from .base_model_merger import BaseModelMerger, ModelMergerConfig  # noqa: F401
from .fsdp_model_merger import FSDPModelMerger  # noqa: F401
