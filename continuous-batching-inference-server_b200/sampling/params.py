"""Sampling options and the key of a draw."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

_M64 = (1 << 64) - 1


@dataclass
class SamplingParams:
    """``temperature`` 0 is greedy (the reference's only rule: first maximum wins,
    src/server_demo.cpp:70-74); above 0 the token is drawn from softmax(logits / temperature)
    with a generator keyed by (``seed``, request, output index).  A request ends after
    ``max_new_tokens`` outputs (the reference's decode_len, src/server_demo.cpp:181), at
    ``eos_token_id`` unless ``ignore_eos``, or when the model's positions run out."""
    max_new_tokens: int = 16
    temperature: float = 0.0
    seed: int = 0
    eos_token_id: Optional[int] = None
    ignore_eos: bool = False


def _splitmix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def request_key(seed: int, request: int, output_index: int) -> int:
    """64-bit key of one draw, as a signed integer (for an int64 tensor).  The sampling kernel
    derives the uniform number of vocabulary entry i from key + (i+1) * 0x9E3779B97F4A7C15."""
    k = _splitmix64((seed & _M64) ^ _splitmix64(((request & 0xFFFFFFFF) << 32) | (output_index & 0xFFFFFFFF)))
    return k - (1 << 64) if k >= (1 << 63) else k
