from .aggregate_logger import (DecoratorLoggerBase, LocalLogger, concat_dict_to_str, log_with_rank, print_rank_0, print_with_rank,
                               print_with_rank_and_timer)

__all__ = ["LocalLogger", "DecoratorLoggerBase", "concat_dict_to_str", "print_rank_0", "print_with_rank",
           "print_with_rank_and_timer", "log_with_rank"]
