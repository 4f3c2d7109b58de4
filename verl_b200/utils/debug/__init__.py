from .metrics import calculate_debug_metrics, calculate_log_prob_diff, calculate_token_list_diff, pearson_correlation_coefficient
from .trajectory_tracker import TrajectoryTracker, dump_data, get_trajectory_tracker

__all__ = ["calculate_debug_metrics", "calculate_log_prob_diff", "calculate_token_list_diff", "pearson_correlation_coefficient",
           "TrajectoryTracker", "dump_data", "get_trajectory_tracker"]
