"""mrun_b200: a one-GPU inference engine for B200 (sm_100a), from a model folder to tokens.

    from mrun_b200 import Engine
    engine = Engine.from_folder("model-dir", dtype="bfloat16")
    results = engine.generate([[1, 2, 3]], max_tokens=16)
"""
__version__ = "0.1.0"

from .sampling.mask import TokenMask  # noqa: E402
from .sampling.params import SamplingParams  # noqa: E402


def __getattr__(name):
    if name in ("Engine", "Generation"):
        from .engine import engine as _engine
        return getattr(_engine, name)
    raise AttributeError(name)


__all__ = ["Engine", "Generation", "SamplingParams", "TokenMask", "__version__"]
