"""Model source configuration. Parity target: ``verl/workers/config/model.py:71-261`` (``HFModelConfig``)."""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig

__all__ = ["HFModelConfig"]


@dataclass
class HFModelConfig(BaseConfig):
    _mutable_fields = {"hf_config_path", "tokenizer_path", "hf_config", "generation_config", "tokenizer", "processor",
                       "local_path", "architectures", "local_hf_config_path", "local_tokenizer_path", "arch"}
    path: str = "tiny-qwen2"  # local HF directory, or the name of a built-in architecture preset
    local_path: Optional[str] = None
    hf_config_path: Optional[str] = None
    tokenizer_path: Optional[str] = None
    use_shm: bool = False
    trust_remote_code: bool = False
    custom_chat_template: Optional[str] = None
    external_lib: Optional[str] = None
    override_config: dict = field(default_factory=dict)
    enable_gradient_checkpointing: bool = True
    enable_activation_offload: bool = False
    use_remove_padding: bool = True
    load_weights: bool = True  # False = random initialisation of the named architecture
    lora_rank: int = 0
    lora_alpha: int = 16
    target_modules: Any = "all-linear"
    exclude_modules: Optional[str] = None
    lora_adapter_path: Optional[str] = None
    use_liger: bool = False
    use_fused_kernels: bool = True
    fused_kernel_options: dict = field(default_factory=dict)
    tiled_mlp: dict = field(default_factory=dict)
    attn_implementation: str = "native"
    mtp: dict = field(default_factory=dict)
    arch: Any = None

    def __post_init__(self):
        from ...models.config import ModelConfig, get_preset

        if self.arch is None:
            p = self.local_path or self.path
            if p and os.path.isdir(p) and os.path.exists(os.path.join(p, "config.json")):
                arch = ModelConfig.from_pretrained(p)
            else:
                arch = get_preset(self.path)
            for k, v in (self.override_config or {}).items():
                if hasattr(arch, k):
                    setattr(arch, k, v)
            object.__setattr__(self, "arch", arch)

    def get_tokenizer(self):
        from ...utils.tokenizer import hf_tokenizer

        p = self.tokenizer_path or self.local_path or self.path
        return hf_tokenizer(p, trust_remote_code=self.trust_remote_code) if p and os.path.isdir(p) else None
