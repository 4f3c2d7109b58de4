"""verl_b200: a Blackwell-native (sm_100a) HybridFlow RL post-training framework."""

__version__ = "0.1.0"

_LAZY = {
    "DataProto": "protocol",
    "DataProtoFuture": "protocol",
    "pad_dataproto_to_divisor": "protocol",
    "unpad_dataproto": "protocol",
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        return getattr(importlib.import_module(f"{__name__}.{_LAZY[name]}"), name)
    raise AttributeError(name)
