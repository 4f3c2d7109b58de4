"""Names of floating-point precisions as they appear in configs (``"bf16"``, ``"bfloat16"``, ``torch.bfloat16``, 16, ...).

Parity target: ``verl/utils/torch_dtypes.py`` (``PrecisionType``).
"""

from __future__ import annotations

import torch

__all__ = ["PrecisionType"]

_HALF = {"fp16", "float16", "half", "16", 16, torch.float16}
_BF16 = {"bf16", "bfloat16", torch.bfloat16}
_FP32 = {"fp32", "float32", "float", "32", 32, torch.float32}
_FP64 = {"fp64", "float64", "double", "64", 64, torch.float64}
_FP8 = {"fp8", "fp8_e4m3", "float8_e4m3fn", torch.float8_e4m3fn}


class PrecisionType:
    HALF, BFLOAT16, FLOAT, DOUBLE, FP8 = "16", "bf16", "32", "64", "fp8"

    @staticmethod
    def _key(p):
        return p.lower() if isinstance(p, str) else p

    @classmethod
    def supported_type(cls, precision) -> bool:
        k = cls._key(precision)
        return any(k in s for s in (_HALF, _BF16, _FP32, _FP64, _FP8))

    @classmethod
    def is_fp16(cls, precision) -> bool:
        return cls._key(precision) in _HALF

    @classmethod
    def is_bf16(cls, precision) -> bool:
        return cls._key(precision) in _BF16

    @classmethod
    def is_fp32(cls, precision) -> bool:
        return cls._key(precision) in _FP32

    @classmethod
    def to_dtype(cls, precision) -> torch.dtype:
        k = cls._key(precision)
        for names, dt in ((_HALF, torch.float16), (_BF16, torch.bfloat16), (_FP32, torch.float32), (_FP64, torch.float64),
                          (_FP8, torch.float8_e4m3fn)):
            if k in names:
                return dt
        raise RuntimeError(f"unexpected precision: {precision!r}")

    @classmethod
    def to_str(cls, precision) -> str:
        return {torch.float16: "fp16", torch.bfloat16: "bf16", torch.float32: "fp32", torch.float64: "fp64",
                torch.float8_e4m3fn: "fp8"}[cls.to_dtype(precision)]
