from .rank_zero import rank_zero_only  # noqa: F401
