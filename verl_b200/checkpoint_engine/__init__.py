from .base import (CheckpointEngine, CheckpointEngineManager, CheckpointEngineRegistry, ColocatedCheckpointEngine,  # noqa: F401
                   TensorMeta, bucketize, merge_weight_chunks, split_weight_chunks)
