"""Typed metric accumulators: a value list plus how it is reduced (mean / sum / min / max), with the data-parallel rule
"average per gradient-accumulation slot over DP ranks first, then reduce" for mean/sum and "over everything" for
min/max. Parity target: ``verl/utils/metric/utils.py:61-163`` (``AggregationType``, ``Metric``) and ``reduce_metrics`` :27.
"""

from __future__ import annotations

from enum import Enum
from typing import Any, Optional, Union

import numpy as np
import torch

__all__ = ["AggregationType", "Metric", "reduce_metrics"]

_NUMERIC = (int, float, np.integer, np.floating, torch.Tensor, np.ndarray)


class AggregationType(Enum):
    MEAN = "mean"
    SUM = "sum"
    MIN = "min"
    MAX = "max"


_REDUCERS = {AggregationType.MEAN: np.mean, AggregationType.SUM: np.sum, AggregationType.MIN: np.min, AggregationType.MAX: np.max}


class Metric:
    def __init__(self, aggregation: Union[str, AggregationType], value=None) -> None:
        try:
            self.aggregation = AggregationType(aggregation) if not isinstance(aggregation, AggregationType) else aggregation
        except ValueError as e:
            raise ValueError(f"Unsupported aggregation type: {aggregation}") from e
        self.values: list = []
        if value is not None:
            (self.extend if isinstance(value, (list, tuple)) else self.append)(value)

    def append(self, value) -> None:
        if isinstance(value, Metric):
            return self.extend(value)
        if isinstance(value, torch.Tensor):
            if value.numel() != 1:
                raise ValueError("Only scalar tensors can be converted to float")
            value = value.detach().item()
        if not isinstance(value, _NUMERIC):
            raise ValueError(f"Unsupported value type: {type(value)}")
        self.values.append(value)

    def extend(self, values) -> None:
        if isinstance(values, Metric):
            if values.aggregation != self.aggregation:
                raise ValueError(f"Aggregation type mismatch: {self.aggregation} != {values.aggregation}")
            values = values.values
        for v in values:
            self.append(v)

    def aggregate(self) -> float:
        return float(_REDUCERS[self.aggregation](self.values))

    @classmethod
    def aggregate_dp(cls, metric_lists: list["Metric"]) -> float:
        if not metric_lists:
            raise ValueError("Cannot aggregate an empty list of metrics.")
        lens = [len(m.values) for m in metric_lists]
        if len(set(lens)) != 1:
            raise ValueError(f"All Metric instances must have the same number of values for dp aggregation: {lens}")
        arr = np.array([m.values for m in metric_lists], dtype=np.float64)  # [dp, accumulation slots]
        agg = metric_lists[0].aggregation
        if agg in (AggregationType.SUM, AggregationType.MEAN):
            return float(_REDUCERS[agg](arr.mean(axis=0)))
        return float(_REDUCERS[agg](arr.reshape(-1)))

    @classmethod
    def from_dict(cls, data: dict, aggregation) -> dict[str, "Metric"]:
        return {k: cls(aggregation, v) for k, v in data.items()}

    def init_list(self) -> "Metric":
        return Metric(self.aggregation)

    def __repr__(self) -> str:
        return f"Metric({self.aggregation.value}, {self.values})"


def reduce_metrics(metrics: dict[str, Any]) -> dict[str, float]:
    """Typed metrics reduce by their own rule; plain lists by name (``max``/``min`` in the key, else mean)."""
    from ...trainer.ppo.metric_utils import reduce_metrics as by_name

    typed = {k: v.aggregate() for k, v in metrics.items() if isinstance(v, Metric)}
    rest = by_name({k: v for k, v in metrics.items() if not isinstance(v, Metric)})
    return {**rest, **typed}
