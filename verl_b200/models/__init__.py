from .config import ModelConfig, PRESETS, get_preset  # noqa: F401
from .weights import FlatParams, build_param_specs  # noqa: F401
from .decoder import DecoderModel, PackedBatch  # noqa: F401


def make_flat_params(cfg: ModelConfig, **kw):
    """Flat parameter storage for ``cfg``: the hand-scheduled layout (``FlatParams``) for the natively supported families,
    the library module's parameters in one flat buffer (``generic.ModuleFlatParams``) for everything else."""
    if cfg.is_generic:
        from .generic import ModuleFlatParams

        kw.pop("with_main_grad", None)
        kw.pop("grad_buffer", None)
        return ModuleFlatParams(cfg, **kw)
    return FlatParams(cfg, **kw)
