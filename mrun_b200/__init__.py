"""mrun_b200: a one-GPU inference engine for B200 (sm_100a), from a model folder to tokens."""
__version__ = "0.1.0"
