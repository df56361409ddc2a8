from .params import SamplingParams, xorshift64

__all__ = ["SamplingParams", "xorshift64"]
