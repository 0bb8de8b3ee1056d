"""Stand-in for ``polars`` (not installed here): lets ``import polars`` succeed; the pandas backend of the
reference never calls into it."""


class DataFrame:
    pass


class Series:
    pass


String = str


def _unavailable(*args, **kwargs):
    raise RuntimeError("polars is not installed on this machine; use --backend pandas")


read_csv = col = concat = lit = when = from_pandas = _unavailable
