"""Architecture recipes (registered on import) and the decoder they build."""

from . import qwen2  # noqa: F401
from .decoder import DecoderModel, model_tensor_specs, slot_needs

__all__ = ["DecoderModel", "model_tensor_specs", "slot_needs"]
