"""Training: the generic ``fit`` loop and the fused kernel-sequence trainer."""
from .fused import FusedTrainer  # noqa: F401
from .fit import fit, evaluate, save_checkpoint, load_checkpoint, EpochReport, BatchReport  # noqa: F401
