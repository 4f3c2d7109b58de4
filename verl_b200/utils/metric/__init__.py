from .utils import AggregationType, Metric, reduce_metrics  # noqa: F401
