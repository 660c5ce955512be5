from .gpt2 import GPT2Config, GPT2Engine  # noqa: F401
