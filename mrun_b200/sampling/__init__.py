from .mask import TokenMask
from .params import GREEDY, REPETITION_CONTEXT, SamplingParams, draw_key, fresh_seed, mix64

__all__ = ["GREEDY", "REPETITION_CONTEXT", "SamplingParams", "TokenMask", "draw_key", "fresh_seed", "mix64"]
