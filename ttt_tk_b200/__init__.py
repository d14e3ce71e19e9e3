"""B200-native TTT-MLP forward / backward operator (sm_100a only, no fallback).

    from ttt_tk_b200 import ttt_forward, ttt_backward      # reference-compatible signatures
"""
from .ops import ttt_forward, ttt_backward, ttt_linear_forward, ttt_linear_backward, take_status  # noqa: F401

__all__ = ["ttt_forward", "ttt_backward", "ttt_linear_forward", "ttt_linear_backward", "take_status"]
