"""Synthetic workload helpers (benchmarks, smoke tests): rewards computed from token ids only."""

from __future__ import annotations


async def mod7_reward(args, sample, **kwargs) -> float:
    """Fraction of response tokens whose id is divisible by 7."""
    n = sample.response_length
    if n == 0:
        return 0.0
    resp = sample.tokens[-n:]
    return sum(1 for t in resp if t % 7 == 0) / n


def random_prompts(num: int, length: int, vocab: int, seed: int = 0) -> list[list[int]]:
    import random

    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(length)] for _ in range(num)]
