"""The lazy tensor layer: tensors, autograd, transforms, devices, groups, meshes."""
from .errors import *  # noqa: F401,F403
from .core import *  # noqa: F401,F403
from .core import Tensor, Device, CPU, GPU, devices, auto, default_device, set_default_device, tensor, from_torch, realize  # noqa: F401
from .autograd import Param, Buffer, backward, gradients, grad, vjp, jvp, jacobian, hessian, vmap, func, checkpoint  # noqa: F401
from .loop import scan, record, Recording, trace, TracedGraph  # noqa: F401
from .memory import set_memory_budget, memory_budget, memory_of  # noqa: F401
from .random import philox_uniform, philox_normal, splitmix64  # noqa: F401
from . import group  # noqa: F401,E402
from .group import Group, cpus  # noqa: F401,E402
