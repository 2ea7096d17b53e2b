"""Task generators for the rollout buffer; ``base_generator`` serves ``task_type = "math"`` and is the template."""

from .base_generator import BaseGenerator, ChatClient, query_single_turn

__all__ = ["BaseGenerator", "ChatClient", "query_single_turn"]
