"""File I/O: the ``.mim`` container (``mim``, ``metadata``), its graph runtime (``graph``, ``graph_run``,
``export``), importers (``gguf``, ``safetensors``) and Parquet shards (``parquet``, imported on use
because it needs pyarrow)."""
from . import mim, metadata  # noqa: F401
from . import graph, graph_run, export  # noqa: F401,E402
from . import gguf, safetensors  # noqa: F401,E402
