from .core import QATConfig, apply_qat_to_params, nvfp4_fake_quantize, nvfp4_global_scale, qat_target_names

__all__ = ["QATConfig", "apply_qat_to_params", "nvfp4_fake_quantize", "nvfp4_global_scale", "qat_target_names"]
