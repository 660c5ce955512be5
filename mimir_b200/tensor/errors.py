"""Error values of the tensor layer (reference: backend/backend.go:31-54,
tensor/tensor.go:126-146).  Operations never raise: a failed operation returns a
tensor that carries one of these as a sticky error, and every tensor derived
from it carries the same error; ``Tensor.err`` exposes it and ``realize`` /
``item`` / ``data`` raise it.
"""
from __future__ import annotations


class MimirError(Exception):
    pass


class ErrShape(MimirError): pass
class ErrDType(MimirError): pass
class ErrIndex(MimirError): pass
class ErrDivideByZero(MimirError): pass
class ErrDevice(MimirError): pass
class ErrOutOfMemory(MimirError): pass
class ErrMemoryBudget(MimirError): pass
class ErrInternal(MimirError): pass
class ErrSingular(MimirError): pass
class ErrOverwritten(MimirError): pass
class ErrDonated(MimirError): pass
class ErrNoGrad(MimirError): pass
class ErrNotDifferentiable(MimirError): pass
class ErrNotBatchable(MimirError): pass
class ErrCheckpoint(MimirError): pass
class ErrFrozen(MimirError): pass
class ErrNilTensor(MimirError): pass
class ErrUnsupported(MimirError): pass


def classify(exc: BaseException) -> MimirError:
    """Maps an exception raised by the executor to the matching error value."""
    if isinstance(exc, MimirError):
        return exc
    msg = str(exc)
    low = msg.lower()
    if isinstance(exc, IndexError) or "index out of range" in low or "out of bounds" in low:
        return ErrIndex(msg)
    if isinstance(exc, ZeroDivisionError) or "division by zero" in low:
        return ErrDivideByZero(msg)
    if "out of memory" in low:
        return ErrOutOfMemory(msg)
    if "singular" in low or "not positive-definite" in low or "not positive definite" in low:
        return ErrSingular(msg)
    if isinstance(exc, TypeError) or "dtype" in low or "expected scalar type" in low or "must have the same dtype" in low:
        return ErrDType(msg)
    if "device" in low and "expected" in low:
        return ErrDevice(msg)
    if any(k in low for k in ("shape", "size", "dimension", "broadcast", "must match", "mat1 and mat2", "reduction dim", " dim ")):
        return ErrShape(msg)
    return ErrInternal(msg)
