"""mimirmind_b200: a small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

From a model folder (``config.json`` + safetensors, or seeded random weights) to generated
tokens: typed configuration and architecture registry, weights by tensor name, layers
composed from parts, a paged cache manager, one step function for mixed batches, a
continuous-batching scheduler, device-side sampling, hand-written CUDA kernels.

    from mimirmind_b200 import Engine, SamplingParams
    engine = Engine.from_folder("/path/to/model", dtype="bfloat16")
    results = engine.generate([[1, 2, 3]], max_new_tokens=16)
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    if name == "write_random_model":
        from .weights.store import write_random_model
        return write_random_model
    raise AttributeError(name)
