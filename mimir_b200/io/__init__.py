"""File I/O: the ``.mim`` container, Parquet shards."""
from . import mim, metadata  # noqa: F401
