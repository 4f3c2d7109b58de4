from .losses import (DistillationConfig, DistillationLossConfig, DistillationLossSettings, distillation_loss,  # noqa: F401
                     get_distillation_loss_fn, get_distillation_loss_settings, is_distillation_enabled,
                     register_distillation_loss)
