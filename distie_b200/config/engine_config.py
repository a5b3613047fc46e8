"""Engine knobs, typed, with the reference's environment names as defaults.

The reference reads ``WORKER_NUM_BLOCKS`` (1024), ``WORKER_MAX_SEQS`` (32),
``WORKER_TOKEN_BUDGET`` (2048), ``WORKER_DECODE_GRAPHS`` (1) and
``WORKER_STEP_STATS`` (0) from the environment (README.md:105-119,
worker/src/worker/config.py:22-57, worker/src/inference/torch_engine.py:212-225,
462-493).  The same names give this engine's defaults; explicit arguments win.

The cache is sized by a page count (``num_blocks``, the reference's only way,
torch_engine.py:416-446) or, with ``gpu_mem_fraction``, from the device memory that
is free once the weights are loaded: that fraction of it becomes pages
(``WORKER_GPU_MEM_FRACTION``; an explicit ``num_blocks`` argument wins over it).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, replace

DEFAULT_NUM_BLOCKS = 1024
DEFAULT_MAX_SEQS = 32
DEFAULT_TOKEN_BUDGET = 2048
DEFAULT_PAGE_SIZE = 16

_DTYPE_NAMES = {
    "bf16": "bfloat16",
    "bfloat16": "bfloat16",
    "fp32": "float32",
    "float32": "float32",
}


def resolve_dtype_name(name: str) -> str:
    """``bf16``/``bfloat16`` or ``fp32``/``float32`` (the reference's spelling and torch's)."""
    key = name.strip().lower()
    if key == "auto":
        return "bfloat16"
    if key not in _DTYPE_NAMES:
        raise ValueError(f"dtype must be one of auto, bf16, bfloat16, fp32, float32; got {name!r}")
    return _DTYPE_NAMES[key]


@dataclass(frozen=True)
class EngineConfig:
    num_blocks: int = DEFAULT_NUM_BLOCKS
    page_size: int = DEFAULT_PAGE_SIZE
    max_seqs: int = DEFAULT_MAX_SEQS
    token_budget: int = DEFAULT_TOKEN_BUDGET
    prefill_chunk: int | None = None
    max_model_len: int | None = None
    dtype: str = "bfloat16"
    decode_graphs: bool = True
    decode_ahead: bool = True  # launch a decode step before the tokens of the one ahead of it reached the host
    step_stats: int = 0
    device: str = "cuda:0"
    float32_weights: str = "auto"  # matrices stored in 32-bit under a 16-bit engine: "auto" | "keep" | "cast"
    gpu_mem_fraction: float | None = None  # size the cache from free device memory instead of num_blocks

    def __post_init__(self) -> None:
        for key in ("num_blocks", "page_size", "max_seqs", "token_budget"):
            if int(getattr(self, key)) < 1:
                raise ValueError(f"{key} must be >= 1")
        if self.prefill_chunk is not None and self.prefill_chunk < 1:
            raise ValueError("prefill_chunk must be >= 1")
        if self.step_stats < 0:
            raise ValueError("step_stats must be >= 0")
        if self.gpu_mem_fraction is not None and not 0.0 < float(self.gpu_mem_fraction) <= 1.0:
            raise ValueError("gpu_mem_fraction must lie in (0, 1]")
        if self.float32_weights not in ("auto", "keep", "cast"):
            raise ValueError("float32_weights must be one of 'auto', 'keep', 'cast'")
        object.__setattr__(self, "dtype", resolve_dtype_name(self.dtype))

    @classmethod
    def from_env(cls, **overrides) -> "EngineConfig":
        base = cls(
            num_blocks=_env_int("WORKER_NUM_BLOCKS", DEFAULT_NUM_BLOCKS),
            max_seqs=_env_int("WORKER_MAX_SEQS", DEFAULT_MAX_SEQS),
            token_budget=_env_int("WORKER_TOKEN_BUDGET", DEFAULT_TOKEN_BUDGET),
            decode_graphs=_env_bool("WORKER_DECODE_GRAPHS", True),
            decode_ahead=_env_bool("WORKER_DECODE_AHEAD", True),
            step_stats=_env_int("WORKER_STEP_STATS", 0, minimum=0),
            gpu_mem_fraction=_env_float("WORKER_GPU_MEM_FRACTION"),
        )
        given = {k: v for k, v in overrides.items() if v is not None}
        if "num_blocks" in given and "gpu_mem_fraction" not in given:
            given["gpu_mem_fraction"] = None  # an explicit page count wins over a fraction from the environment
        return replace(base, **given)

    def sized(self, num_blocks: int) -> "EngineConfig":
        """This configuration with the page count that ``gpu_mem_fraction`` came to."""
        return replace(self, num_blocks=int(num_blocks), gpu_mem_fraction=None)


def _env_int(key: str, default: int, minimum: int = 1) -> int:
    raw = os.getenv(key)
    if raw is None or raw.strip() == "":
        return default
    try:
        value = int(raw)
    except ValueError as exc:
        raise ValueError(f"{key} must be an integer") from exc
    if value < minimum:
        raise ValueError(f"{key} must be >= {minimum}")
    return value


def _env_float(key: str) -> float | None:
    raw = os.getenv(key)
    if raw is None or raw.strip() == "":
        return None
    try:
        return float(raw)
    except ValueError as exc:
        raise ValueError(f"{key} must be a number") from exc


def _env_bool(key: str, default: bool) -> bool:
    raw = os.getenv(key)
    if raw is None or raw.strip() == "":
        return default
    return raw.strip().lower() not in {"0", "false", "no", "off"}
