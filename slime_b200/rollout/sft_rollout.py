"""SFT as a degenerate rollout: no generation, samples are tokenised conversations with an assistant-only loss mask.

``--rollout-function-path slime.rollout.sft_rollout.generate_rollout --loss-type sft_loss``; prompts are message
lists (``sample.prompt``), optional tool schemas come from ``sample.metadata["tools"]``.
Parity: slime/rollout/sft_rollout.py:17-68.
"""

from __future__ import annotations

import logging

from slime_b200.utils.mask_utils import MultiTurnLossMaskGenerator
from slime_b200.utils.processing_utils import load_processor, load_tokenizer

__all__ = ["generate_rollout"]
logger = logging.getLogger(__name__)
_state: dict = {}


def _lazy(args):
    if not _state:
        _state["tokenizer"] = load_tokenizer(args.hf_checkpoint, trust_remote_code=True)
        _state["processor"] = load_processor(args.hf_checkpoint, trust_remote_code=True)
        _state["masker"] = MultiTurnLossMaskGenerator(_state["tokenizer"], tokenizer_type=args.loss_mask_type)
        _state["shown"] = False
    return _state


def generate_rollout(args, rollout_id, data_buffer, evaluation=False):
    assert not evaluation, "the SFT rollout has no evaluation mode"
    assert args.rollout_global_dataset
    st = _lazy(args)
    groups = data_buffer.get_samples(args.rollout_batch_size)
    for group in groups:
        (sample,) = group  # n_samples_per_prompt must be 1
        tools = (sample.metadata or {}).get("tools")
        ids, mask = st["masker"].get_loss_mask(sample.prompt, tools=tools)
        if len(ids) != len(mask):
            raise ValueError(f"token ids ({len(ids)}) and loss mask ({len(mask)}) differ in length")
        n_resp = st["masker"].get_response_lengths([mask])[0]
        sample.tokens, sample.response_length, sample.reward = ids, n_resp, 0
        sample.loss_mask = mask[-n_resp:] if n_resp else []
        if not st["shown"]:
            st["shown"] = True
            logger.info("sft rollout example: %d tokens, %d trained, messages=%s", len(ids), sum(mask), sample.prompt)
    return groups
