"""tuff_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a), built
from parts, for the LFM2 / LFM2.5 dense decoder.

    from tuff_b200 import Engine, SamplingParams
    engine = Engine(model_dir, dtype="bfloat16")
    new_tokens = engine.generate([[1, 5, 9]], SamplingParams(max_new_tokens=16))
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    if name == "ModelRunner":
        from .engine.runner import ModelRunner
        return ModelRunner
    raise AttributeError(name)
