"""Language models: loading from ``.mim`` files, tokenizers, sampling, LoRA adapters, the
tensor-parallel quantized decoder for GPUs and the quantized decoder for the host."""
from .tp_decode import LlamaConfig, TPDecoder  # noqa: F401
from .model import Config, Model  # noqa: F401
from .tokenizer import BytePairs, SentencePiece, from_metadata as tokenizer_from_metadata  # noqa: F401
from .generate import Sampler, generate  # noqa: F401
from .cpu_decode import CPUDecoder  # noqa: F401
