"""Random-weights mode: write a model folder from a configuration and a seed.

``config.json`` plus ``model.safetensors`` with the tensors the architecture's
parts declare, under their checkpoint names, so that the ordinary loader reads the
folder like any other.  Values come from one ``torch.Generator(seed)`` on the CPU,
drawn in float32 in the declared order of the tensors and then cast: products'
weights, tables and biases ``N(0, std)``, norm scales ``1 + N(0, norm_noise)``.
``std`` defaults to the configuration's ``initializer_range`` when it has one.
"""

from __future__ import annotations

import json
import os

import torch

from ..config.registry import architecture_of
from .safetensors_io import save_file

_DEFAULT_STD = 0.02


def random_tensors(specs, seed: int, std: float, norm_noise: float, dtype: torch.dtype) -> dict[str, torch.Tensor]:
    generator = torch.Generator().manual_seed(int(seed))
    out: dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.name in out:
            continue
        if spec.role == "norm":
            value = torch.ones(spec.shape)
            if norm_noise:
                value = value + torch.randn(spec.shape, generator=generator) * norm_noise
        else:
            value = torch.randn(spec.shape, generator=generator) * std
        out[spec.name] = value.to(dtype)
    return out


class RandomSource:
    """Random tensors made on demand on a device: a weight source without a folder.

    Same distributions as :func:`random_tensors` (not the same numbers: every tensor has
    its own generator, seeded by ``seed`` and its place in the declared order), for models
    too large to be worth a trip through the file system.
    """

    def __init__(self, specs, seed: int = 0, std: float = _DEFAULT_STD, norm_noise: float = 0.0,
                 dtype: torch.dtype = torch.bfloat16, device="cpu") -> None:
        self._specs = {}
        for index, spec in enumerate(specs):
            self._specs.setdefault(spec.name, (spec, index))
        self.seed, self.std, self.norm_noise, self._dtype, self.device = int(seed), std, norm_noise, dtype, torch.device(device)

    def keys(self):
        return self._specs.keys()

    def shape(self, name):
        return tuple(self._specs[name][0].shape)

    def dtype(self, name):
        return self._dtype

    def tensor(self, name):
        spec, index = self._specs[name]
        generator = torch.Generator(device=self.device).manual_seed(self.seed * 1_000_003 + index)
        if spec.role == "norm":
            value = torch.ones(spec.shape, device=self.device)
            if self.norm_noise:
                value += torch.randn(spec.shape, generator=generator, device=self.device) * self.norm_noise
        else:
            value = torch.randn(spec.shape, generator=generator, device=self.device) * self.std
        return value.to(self._dtype)


def write_random_model(
    folder: str,
    config: dict,
    seed: int = 0,
    std: float | None = None,
    norm_noise: float = 0.0,
    dtype: str | torch.dtype | None = None,
) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors``; returns ``folder``.

    ``config`` holds the architecture's own ``config.json`` keys, ``architectures`` included.
    """
    from ..models.decoder import model_tensor_specs

    arch = architecture_of(config)
    typed = arch.config_cls.from_dict(config)
    spec = arch.recipe(typed)
    if dtype is None:
        dtype = config.get("torch_dtype") or "bfloat16"
    if isinstance(dtype, str):
        dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}[dtype]
    if std is None:
        std = float(config.get("initializer_range", _DEFAULT_STD))
    tensors = random_tensors(model_tensor_specs(spec), seed, std, norm_noise, dtype)
    os.makedirs(folder, exist_ok=True)
    written = dict(config)
    written["torch_dtype"] = "bfloat16" if dtype == torch.bfloat16 else "float32"
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(written, handle, indent=2, sort_keys=True)
    save_file(tensors, os.path.join(folder, "model.safetensors"), {"format": "pt", "seed": str(seed)})
    return folder
