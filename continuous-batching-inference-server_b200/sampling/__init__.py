from .params import SamplingParams, request_key

__all__ = ["SamplingParams", "request_key"]
