"""mimirmind_b200: a small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

From a model folder (``config.json`` + safetensors, or seeded random weights) to generated
tokens: typed configuration and architecture registry, weights by tensor name, layers
composed from parts, a paged cache manager, one step function for mixed batches, a
continuous-batching scheduler, device-side sampling, hand-written CUDA kernels.
"""
__version__ = "0.1.0"
