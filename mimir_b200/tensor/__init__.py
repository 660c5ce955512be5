"""The lazy tensor layer: tensors, autograd, transforms, devices, groups, meshes."""
from .errors import *  # noqa: F401,F403
from .core import *  # noqa: F401,F403
from .core import Tensor, Device, CPU, GPU, devices, auto, default_device, set_default_device, tensor, from_torch, realize  # noqa: F401
from .autograd import Param, Buffer, backward, gradients, grad, vjp, jvp, jacobian, hessian, vmap, func, checkpoint  # noqa: F401
from .loop import scan, record, record_into, Recording, trace, TracedGraph  # noqa: F401
from .memory import set_memory_budget, memory_budget, memory_of  # noqa: F401
from .random import philox_uniform, philox_normal, splitmix64  # noqa: F401
from .pattern import Pattern, segment  # noqa: F401
from .linalg import (exp2, log2, greater, fmod, fft, ifft, rfft, irfft, cholesky, triangular_solve, solve, inv, det,  # noqa: F401
                     slogdet, qr, svd, eigh, rand_gamma, rand_poisson, from_slice, scalar, flatten)
from . import group  # noqa: F401,E402
from .group import Group, cpus  # noqa: F401,E402
from .core import from_bytes, from_bytes_func, realize_into  # noqa: F401,E402


def gpus():
    """One device handle per visible GPU (tensor.GPUs); empty without CUDA."""
    import torch
    return [GPU(i) for i in range(torch.cuda.device_count())] if torch.cuda.is_available() else []
