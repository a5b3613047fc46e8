"""Weights by tensor name: checking a checkpoint against what the parts declare,
and converting what passes for the engine.

The reference copies module by module out of a library model and raises on the
first mismatch (worker/src/inference/qwen2/model.py:383-452).  Here every part
declares its tensors (:class:`~distie_b200.parts.base.TensorSpec`), the checkpoint
is compared with the whole list, and ONE error names everything that is missing,
unexpected or of the wrong shape.

Conversion on the way to the device:

* ``matrix`` / ``table``: the engine's dtype, as the reference loads with the dtype
  it serves in (worker/src/inference/torch_engine.py:135-141).  float32 engine:
  everything becomes float32.  bfloat16 engine: bfloat16 and float16 tensors become
  bfloat16; what happens to a tensor stored in 32-bit is the ``float32_weights``
  policy.  ``"auto"`` (the default): a checkpoint that stores EVERY matrix in 32-bit
  is a float32 checkpoint and is cast; in a checkpoint that stores matrices in
  16-bit, one stored in 32-bit was kept wide on purpose and stays so (its products
  then run in float32).  ``"keep"``: 32-bit tensors always stay; ``"cast"``: never.
* ``bias`` / ``norm``: float32 (exact for bfloat16 inputs): stored in 32-bit they stay so.
* integer tensors: int32.
"""

from __future__ import annotations

import logging
from typing import Iterable, Mapping

import torch

from ..parts.base import TensorSpec
from .safetensors_io import ModelTensors


_log = logging.getLogger(__name__)
FLOAT32_POLICIES = ("auto", "keep", "cast")
_WIDE = (torch.float32, torch.float64)


class WeightsError(ValueError):
    """The checkpoint does not match the model: lists every problem at once."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_kind=()) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(
                f"  wrong shapes ({len(self.wrong_shape)}): "
                + ", ".join(f"{n}: checkpoint {tuple(have)}, model {tuple(want)}" for n, have, want in self.wrong_shape)
            )
        if self.wrong_kind:
            lines.append(
                f"  wrong element types ({len(self.wrong_kind)}): "
                + ", ".join(f"{n}: {dtype}" for n, dtype in self.wrong_kind)
            )
        super().__init__("\n".join(lines))


def check_checkpoint(
    shapes: Mapping[str, tuple[int, ...]],
    specs: Iterable[TensorSpec],
    tolerated: Iterable[str] = (),
    dtypes: Mapping[str, torch.dtype] | None = None,
) -> None:
    specs = list(specs)
    wanted = {s.name: s for s in specs}
    missing = [name for name in wanted if name not in shapes]
    allowed = set(tolerated)
    unexpected = sorted(name for name in shapes if name not in wanted and name not in allowed)
    wrong = [
        (name, shapes[name], spec.shape)
        for name, spec in wanted.items()
        if name in shapes and tuple(shapes[name]) != tuple(spec.shape)
    ]
    wrong_kind = []
    if dtypes is not None:
        for name in wanted:
            if name in dtypes and not dtypes[name].is_floating_point:
                wrong_kind.append((name, dtypes[name]))
    if missing or unexpected or wrong or wrong_kind:
        raise WeightsError(missing, unexpected, wrong, wrong_kind)


class WeightStore:
    """Hands converted device tensors to the parts, each name once (tied uses share the tensor)."""

    def __init__(self, source, specs: Iterable[TensorSpec], dtype: torch.dtype, device, float32_weights: str = "auto") -> None:
        if float32_weights not in FLOAT32_POLICIES:
            raise ValueError(f"float32_weights must be one of {FLOAT32_POLICIES}, got {float32_weights!r}")
        self._source = source  # anything with .tensor(name) -> CPU tensor
        self._roles = {s.name: s.role for s in specs}
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self._cache: dict[str, torch.Tensor] = {}
        self.keep_wide = False  # whether a matrix stored in 32-bit stays 32-bit in a 16-bit engine
        if dtype != torch.float32 and float32_weights != "cast":
            stored = [source.dtype(n) for n, role in self._roles.items() if role in ("matrix", "table") and n in set(source.keys())]
            wide = [d for d in stored if d in _WIDE]
            self.keep_wide = bool(wide) and (float32_weights == "keep" or len(wide) < len(stored))
            if self.keep_wide:
                _log.warning(
                    "%s of %s matrices are stored in 32-bit and stay so: their products run in float32, "
                    "not on the %s kernels (float32_weights='cast' converts them)", len(wide), len(stored), dtype,
                )

    def _convert(self, name: str, role: str) -> torch.Tensor:
        key = f"{role}:{name}"
        if key in self._cache:
            return self._cache[key]
        raw = self._source.tensor(name)
        if not raw.dtype.is_floating_point:
            target = torch.int32
        elif role in ("bias", "norm"):
            target = torch.float32
        elif self.dtype == torch.float32 or (self.keep_wide and raw.dtype in _WIDE):
            target = torch.float32
        else:
            target = self.dtype
        out = raw.to(dtype=target)
        if self.device is not None:
            out = out.to(self.device)
        out = out.contiguous()
        self._cache[key] = out
        return out

    def matrix(self, name: str) -> torch.Tensor:
        return self._convert(name, "matrix")

    table = matrix

    def vector(self, name: str) -> torch.Tensor:
        return self._convert(name, "bias")

    def has(self, name: str) -> bool:
        return name in self._roles

    def release(self) -> None:
        """Forget the per-name tensors once the parts hold (possibly fused) copies."""
        self._cache.clear()


class DictSource:
    """Adapter so that a plain dict of CPU tensors can stand in for a model folder."""

    def __init__(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self._tensors = tensors

    def keys(self):
        return self._tensors.keys()

    def shape(self, name):
        return tuple(self._tensors[name].shape)

    def dtype(self, name):
        return self._tensors[name].dtype

    def tensor(self, name):
        return self._tensors[name]


def open_weights(folder_or_dict, specs, tolerated, dtype: torch.dtype, device, float32_weights: str = "auto") -> WeightStore:
    """Open a model folder (or a dict of tensors), check it against ``specs``, return the store."""
    if isinstance(folder_or_dict, Mapping):
        source = DictSource(folder_or_dict)
    elif isinstance(folder_or_dict, (str, bytes)) or hasattr(folder_or_dict, "__fspath__"):
        source = ModelTensors(folder_or_dict)
    else:
        source = folder_or_dict  # anything with keys / shape / dtype / tensor
    specs = list(specs)
    names = list(source.keys())
    check_checkpoint(
        {name: source.shape(name) for name in names},
        specs,
        tolerated,
        {name: source.dtype(name) for name in names},
    )
    return WeightStore(source, specs, dtype, device, float32_weights)
