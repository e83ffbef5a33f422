"""A B200-native inference engine for the Qwen3 dense decoder: config.json and safetensors in, tokens out.

    from inferrs_b200 import Engine, SamplingParams
    engine = Engine("path/to/model", dtype="bf16")
    outputs = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=16))
"""
from .sampling.params import SamplingParams

__all__ = ["Engine", "SamplingParams"]


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
