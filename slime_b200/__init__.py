"""slime_b200: a Blackwell-native RL post-training framework.

Training backend (TP/SP/EP/DP/PP), rollout engine (continuous batching, paged
KV), weight sync and orchestration are implemented here from scratch for
sm_100a; CUDA kernels live in ``csrc/`` and are exposed through
``slime_b200.ops``.
"""

__version__ = "0.1.0"
