from .vllm_rollout import VLLMRollout

__all__ = ["VLLMRollout"]
