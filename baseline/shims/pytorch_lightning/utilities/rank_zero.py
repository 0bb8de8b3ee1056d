import functools
import os


def _rank() -> int:
    for key in ("RANK", "LOCAL_RANK", "SLURM_PROCID"):
        if os.environ.get(key) is not None:
            return int(os.environ[key])
    return 0


def rank_zero_only(fn):
    @functools.wraps(fn)
    def wrapped(*args, **kwargs):
        if _rank() == 0:
            return fn(*args, **kwargs)
        return None

    return wrapped
