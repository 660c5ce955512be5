"""Language models: tensor-parallel quantized decoding, model loading, sampling."""
from .tp_decode import LlamaConfig, TPDecoder  # noqa: F401
