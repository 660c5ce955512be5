"""What the classical models share (reference: tabular/tabular.go, and the conventions every model
package there follows): the task, feature standardisation with missing values, JSON round trips and
the ``nn.Module`` form of a fitted model.

* Every fit standardises each feature first (mean 0, deviation 1 over the rows that have it), so
  penalties, distances and kernel scales mean the same whatever the features' units.  A constant
  feature keeps scale 1.  A missing value (NaN) counts as the feature's mean, i.e. 0 after scaling.
* A fitted model keeps plain fields (tensors, numbers, strings, lists): ``to_json`` / ``from_json``
  save and load it without pickling code.
* ``module()`` serves the model as an ``nn.Module`` whose tables are buffers, not trained parameters:
  ``forward`` maps ``[batch, features]`` to ``[batch, classes]`` logits whose softmax is the model's
  probabilities (``[batch, 1]`` values for regression), in lazy tensor ops, so a fitted model runs,
  saves and loads wherever a network does.
"""
from __future__ import annotations

import enum
import json

import torch


class Task(enum.Enum):
    REGRESSION = "regression"
    CLASSIFICATION = "classification"

    def __str__(self):
        return self.value


REGRESSION, CLASSIFICATION = Task.REGRESSION, Task.CLASSIFICATION


def as_task(task) -> Task:
    return task if isinstance(task, Task) else Task(str(task))


def as_rows(X, features: int | None = None) -> torch.Tensor:
    """``X`` as float32 ``[rows, features]``; a flat list holds rows one after another."""
    X = torch.as_tensor(X)
    if not X.dtype.is_floating_point:
        X = X.float()
    X = X.float()
    if X.dim() == 1:
        if features is None or features <= 0 or X.numel() % features:
            raise ValueError(f"{X.numel()} numbers are not a whole number of rows of {features} features")
        X = X.reshape(-1, features)
    if X.dim() != 2 or (features is not None and X.shape[1] != features):
        raise ValueError(f"rows of shape {tuple(X.shape)}, want [rows, {features if features is not None else 'features'}]")
    return X


class Standard:
    """Per-feature mean and scale over the rows that have the feature."""

    def __init__(self, mean: torch.Tensor, scale: torch.Tensor):
        self.mean, self.scale = mean.float(), scale.float()

    @classmethod
    def fit(cls, X: torch.Tensor, raw: bool = False) -> "Standard":
        if not torch.isnan(X).any():
            # no missing values: one pass, sums kept in double without a double copy of the table
            var, mean = torch.var_mean(X.float(), 0, unbiased=False)
            mean, var = mean.double(), var.double()
            if raw:
                return cls(mean, torch.ones_like(mean))
            scale = var.sqrt()
            return cls(mean, torch.where(scale > 1e-12 * (1 + mean.abs()), scale, torch.ones_like(scale)))
        X = X.double()
        have = ~torch.isnan(X)
        n = have.sum(0).clamp_min(1)
        filled = torch.where(have, X, torch.zeros_like(X))
        mean = filled.sum(0) / n
        if raw:
            # features in their own units: only the fill value for a missing entry is kept
            return cls(mean, torch.ones_like(mean))
        var = (torch.where(have, X - mean, torch.zeros_like(X)) ** 2).sum(0) / n
        scale = var.sqrt()
        scale = torch.where(scale > 1e-12 * (1 + mean.abs()), scale, torch.ones_like(scale))
        return cls(mean, scale)

    def apply(self, X: torch.Tensor) -> torch.Tensor:
        Z = (X.float() - self.mean.to(X.device)) / self.scale.to(X.device)
        return torch.nan_to_num(Z, nan=0.0) if torch.isnan(Z).any() else Z


def count_classes(y: torch.Tensor, classes: int = 0) -> int:
    y = torch.as_tensor(y)
    if y.numel() == 0:
        return max(classes, 0)
    if (y < 0).any() or (y.float() != y.float().round()).any():
        raise ValueError("class targets must be whole numbers 0, 1, ...")
    return max(int(y.max()) + 1, classes)


# ------------------------------------------------------------------ JSON
def _enc(v):
    if isinstance(v, torch.Tensor):
        return {"__tensor__": v.tolist(), "dtype": str(v.dtype).replace("torch.", ""), "shape": list(v.shape)}
    if isinstance(v, Task):
        return {"__task__": v.value}
    if isinstance(v, Standard):
        return {"__standard__": [_enc(v.mean), _enc(v.scale)]}
    if isinstance(v, Model):
        return {"__model__": type(v).__module__ + ":" + type(v).__name__, "fields": v._state()}
    if isinstance(v, (list, tuple)):
        return [_enc(x) for x in v]
    if isinstance(v, dict):
        return {str(k): _enc(x) for k, x in v.items()}
    if isinstance(v, float) and v != v:
        return {"__nan__": True}
    return v


def _dec(v):
    if isinstance(v, dict):
        if "__tensor__" in v:
            return torch.tensor(v["__tensor__"], dtype=getattr(torch, v["dtype"])).reshape(v["shape"])
        if "__task__" in v:
            return Task(v["__task__"])
        if "__standard__" in v:
            m, s = v["__standard__"]
            return Standard(_dec(m), _dec(s))
        if "__model__" in v:
            import importlib
            mod, name = v["__model__"].split(":")
            if not mod.startswith(__package__):
                raise ValueError(f"model class {v['__model__']} is outside this package")
            cls = getattr(importlib.import_module(mod), name)
            return cls._from_state(v["fields"])
        if "__nan__" in v:
            return float("nan")
        return {k: _dec(x) for k, x in v.items()}
    if isinstance(v, list):
        return [_dec(x) for x in v]
    return v


class Model:
    """A fitted model of plain fields.  Subclasses list the fields in ``FIELDS``."""

    FIELDS: tuple = ()

    def _state(self):
        return {k: _enc(getattr(self, k)) for k in self.FIELDS}

    @classmethod
    def _from_state(cls, state):
        m = cls.__new__(cls)
        for k in cls.FIELDS:
            setattr(m, k, _dec(state[k]))
        return m

    def to_json(self) -> str:
        return json.dumps({"model": type(self).__name__, "fields": self._state()})

    @classmethod
    def from_json(cls, s: str):
        d = json.loads(s)
        if d.get("model") != cls.__name__:
            raise ValueError(f"JSON holds a {d.get('model')}, not a {cls.__name__}")
        return cls._from_state(d["fields"])

    # classification helpers shared by the models whose predict returns probabilities
    def classify(self, X):
        p = self.predict(X)
        return p.argmax(-1) if p.dim() == 2 else p


def softmax_rows(logits: torch.Tensor) -> torch.Tensor:
    return torch.softmax(logits.float(), -1)
