from .api import get_split_strategy, set_split_strategy_by_idx, set_split_strategy_by_size  # noqa: F401
