from .fused import FusedTrainer  # noqa: F401
