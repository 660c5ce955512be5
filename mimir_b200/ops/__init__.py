"""Python wrappers over the hand-written sm_100a kernels (``csrc/``)."""
from .gemm import gemm, GEMM_FLAGS  # noqa: F401
