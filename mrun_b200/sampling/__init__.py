from .params import GREEDY, REPETITION_CONTEXT, SamplingParams, draw_key, fresh_seed, mix64

__all__ = ["GREEDY", "REPETITION_CONTEXT", "SamplingParams", "draw_key", "fresh_seed", "mix64"]
