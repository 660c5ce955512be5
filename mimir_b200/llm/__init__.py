"""Language models: loading from ``.mim`` files, tokenizers, sampling, LoRA adapters, and the
tensor-parallel quantized decoder."""
from .tp_decode import LlamaConfig, TPDecoder  # noqa: F401
from .model import Config, Model  # noqa: F401
from .tokenizer import BytePairs, SentencePiece, from_metadata as tokenizer_from_metadata  # noqa: F401
from .generate import Sampler, generate  # noqa: F401
