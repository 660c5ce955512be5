"""mimir_b200: a Blackwell-native (sm_100a) machine-learning framework with the
capabilities of gsoultan/mimir: lazy tensors with sticky errors, autograd, layers,
optimizers, a training loop, data-parallel / tensor-parallel / fully sharded
training over NVLink peer memory, quantized LLM inference and the ``.mim`` format.

Device picker facade (reference: mimir.go:36-49): ``auto()``, ``devices()``,
``cpu()``, ``gpu(i)``.
"""
from .tensor.core import CPU as cpu, GPU as gpu, auto, devices  # noqa: F401

__version__ = "0.1.0"
