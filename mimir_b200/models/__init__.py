from .gpt2 import GPT2Config, GPT2Engine  # noqa: F401
from .llama import LlamaEngine, LlamaTrainConfig  # noqa: F401
from .cnn import MnistCNN  # noqa: F401
