from .naive_rollout import NaiveRollout  # noqa: F401
