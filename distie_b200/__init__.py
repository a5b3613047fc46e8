"""distie_b200: a single-GPU inference engine for the Qwen2 dense decoder on B200 (sm_100a).

From a model folder (``config.json`` + safetensors) to generated tokens: typed
configuration and architecture registry, weights by tensor name, layers composed
from parts, a paged cache manager, one step function over mixed batches, a
continuous-batching scheduler, sampling, and hand-written CUDA kernels in
bfloat16 and true float32.
"""

__version__ = "0.1.0"
