from .naive.naive_rollout import NaiveRollout  # noqa: F401
