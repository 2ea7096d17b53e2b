"""Prompt dataset loading.

``read_file`` streams ``.jsonl`` / ``.parquet`` rows and supports the
``path@[a:b]`` row-slice suffix. ``Dataset`` turns rows into ``Sample``s
(optional chat template, tools, multimodal placeholders, prompt-length filter)
and reshuffles per epoch with ``seed + epoch``.
Parity: slime/utils/data.py:24-84 (read_file), :214-301 (Dataset), :304-318.
"""

from __future__ import annotations

import itertools
import json
import logging
import os
import random
import re

from slime_b200.utils.types import MultimodalTypes, Sample

logger = logging.getLogger(__name__)
__all__ = ["Dataset", "get_source", "read_file", "process_rollout_data"]

_SLICE_RE = re.compile(r"^(?P<path>.*)@\[(?P<a>-?\d*):(?P<b>-?\d*)\]$")


def parse_sliced_path(spec: str):
    m = _SLICE_RE.match(spec)
    if m is None:
        return spec, None
    a = int(m["a"]) if m["a"] else None
    b = int(m["b"]) if m["b"] else None
    return m["path"], slice(a, b)


def _iter_jsonl(path):
    with open(path, encoding="utf-8") as f:
        for n, line in enumerate(f):
            line = line.strip()
            if not line:
                continue
            try:
                yield json.loads(line)
            except json.JSONDecodeError as e:
                logger.warning("%s line %d is not valid JSON (%s); skipped", path, n, e)


def _iter_parquet(path):
    import pyarrow.parquet as pq

    for batch in pq.ParquetFile(path).iter_batches():
        yield from batch.to_pylist()


def read_file(path):
    path, rows = parse_sliced_path(path)
    if not os.path.exists(path):
        raise FileNotFoundError(f"Prompt dataset path '{path}' does not exist.")
    if path.endswith(".jsonl"):
        it = _iter_jsonl(path)
    elif path.endswith(".parquet"):
        it = _iter_parquet(path)
    else:
        raise ValueError(f"Unsupported file format: {path}. Supported formats are .jsonl and .parquet.")
    if rows is not None:
        negative = (rows.start or 0) < 0 or (rows.stop or 0) < 0
        it = iter(list(it)[rows]) if negative else itertools.islice(it, rows.start, rows.stop)
    yield from it


def _expand_multimodal(messages, row, multimodal_keys):
    """Replace ``<image>``-style placeholders in string contents by typed content parts."""
    pools = {}
    for type_name, key in multimodal_keys.items():
        mt = MultimodalTypes.get(type_name)
        if mt is not None and row.get(key) is not None:
            pools[mt.placeholder] = (mt, list(row[key]))
    if not pools:
        return messages
    splitter = re.compile("(" + "|".join(re.escape(p) for p in pools) + ")")
    for msg in messages:
        content = msg["content"]
        if isinstance(content, list):
            continue
        if not isinstance(content, str):
            raise ValueError(f"Unsupported content type: {type(content)}, expected str or list of dicts")
        parts = []
        for seg in splitter.split(content):
            if not seg:
                continue
            if seg in pools:
                mt, pool = pools[seg]
                assert pool, f"more '{mt.placeholder}' placeholders in prompt than {mt.name}s provided in data"
                item = pool.pop(0)
                parts.append(item if isinstance(item, dict) else {"type": mt.name, mt.name: item})
            else:
                parts.append({"type": "text", "text": seg})
        msg["content"] = parts
    for ph, (mt, pool) in pools.items():
        assert not pool, f"{len(pool)} more {mt.name}(s) than '{ph}' placeholders in prompt"
    return messages


def build_prompt(row: dict, prompt_key: str, as_conversation: bool, multimodal_keys=None):
    prompt = row.get(prompt_key)
    if isinstance(prompt, str):
        if not as_conversation:
            return prompt
        prompt = [{"role": "user", "content": prompt}]
    if multimodal_keys:
        prompt = _expand_multimodal(prompt, row, multimodal_keys)
    return prompt


def filter_long_prompt(samples: list[Sample], tokenizer, processor, max_length: int | None) -> list[Sample]:
    if max_length is None or not samples:
        return samples
    if not isinstance(samples[0].prompt, str):
        logger.warning("prompt is a message list; set apply_chat_template=True to enable length filtering")
        return samples
    keep = []
    text_idx = []
    for i, s in enumerate(samples):
        mm = s.multimodal_inputs and any(v is not None for v in s.multimodal_inputs.values())
        if processor is not None and mm:
            from slime_b200.utils.processing_utils import process_vision_info

            ids = processor(text=s.prompt, **process_vision_info(s.prompt, processor))["input_ids"][0]
            if len(ids) <= max_length:
                keep.append(i)
        else:
            text_idx.append(i)
    if text_idx:
        enc = tokenizer([samples[i].prompt for i in text_idx], add_special_tokens=False)["input_ids"]
        keep += [i for i, ids in zip(text_idx, enc) if len(ids) <= max_length]
    keep.sort()
    logger.info("Filtered %d samples longer than max_length=%s.", len(samples) - len(keep), max_length)
    return [samples[i] for i in keep]


class Dataset:
    def __init__(
        self,
        path,
        tokenizer,
        processor,
        max_length,
        *,
        prompt_key="text",
        multimodal_keys=None,
        label_key=None,
        tool_key=None,
        metadata_key="metadata",
        seed=42,
        apply_chat_template=False,
        apply_chat_template_kwargs=None,
    ):
        rows = []
        conv = apply_chat_template or multimodal_keys is not None
        for row in read_file(path):
            prompt = build_prompt(row, prompt_key, conv, multimodal_keys)
            metadata = row.get(metadata_key) or {}
            tools = None
            if tool_key is not None and tool_key in row:
                tools = row[tool_key]
                if isinstance(tools, str):
                    tools = json.loads(tools)
                elif hasattr(tools, "tolist"):
                    tools = tools.tolist()
                assert isinstance(tools, list), f"tools must be a list, got {type(tools)} instead"
                metadata["tools"] = tools
            text = prompt
            if apply_chat_template:
                text = tokenizer.apply_chat_template(
                    prompt, tools=tools, tokenize=False, add_generation_prompt=True, **(apply_chat_template_kwargs or {})
                )
            mm = None
            if processor:
                from slime_b200.utils.processing_utils import process_vision_info

                assert isinstance(prompt, list), "prompt must be a message list when a processor is used"
                mm = process_vision_info(prompt, processor)
            rows.append(
                Sample(
                    prompt=text,
                    label=row[label_key] if label_key is not None else None,
                    metadata=metadata,
                    multimodal_inputs=mm,
                )
            )
        self.origin_samples = filter_long_prompt(rows, tokenizer, processor, max_length)
        self.samples = self.origin_samples
        self.epoch_id = -1
        self.seed = seed

    def shuffle(self, new_epoch_id):
        if self.epoch_id == new_epoch_id:
            return
        rng = random.Random(self.seed + new_epoch_id)
        perm = list(range(len(self.origin_samples)))
        rng.shuffle(perm)
        self.samples = [self.origin_samples[i] for i in perm]
        self.epoch_id = new_epoch_id

    def __getitem__(self, idx):
        return self.samples[idx]

    def __len__(self):
        return len(self.samples)


def process_rollout_data(args, rollout_data_ref, dp_rank, dp_size):
    """Fetch this DP rank's payload from the object store and localise whole-batch fields."""
    from slime_b200.observability.timer import Timer
    from slime_b200.runtime import object_store

    assert len(rollout_data_ref) == dp_size
    data = object_store.get(rollout_data_ref[dp_rank].inner)
    part = data["partition"]
    totals = data["total_lengths"]
    Timer().seq_lens = totals
    data["total_lengths"] = [totals[i] for i in part]
    if "raw_reward" in data:
        data["local_raw_reward"] = [data["raw_reward"][i] for i in part]
    return data


def get_source(sample: Sample) -> str:
    if getattr(sample, "source", None):
        return sample.source
    md = getattr(sample, "metadata", None) or {}
    return md.get("source_name") or "unknown"
