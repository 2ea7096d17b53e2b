"""Prompt sources feeding the rollout loop.

``RolloutDataSource`` reads the global prompt dataset and yields groups of
``n_samples_per_prompt`` deep-copied ``Sample``s; its cursor (epoch, offset,
sample index) is checkpointed under ``{save}/rollout/``.
``RolloutDataSourceWithBuffer`` puts a FIFO of returned (partial / aborted /
over-sampled) groups in front of it.
Parity: slime/rollout/data_source.py:17-48, :50-165, :168-229.
"""

from __future__ import annotations

import abc
import copy
import logging
import os

import torch

from slime_b200.utils.data import Dataset
from slime_b200.utils.misc import load_function
from slime_b200.utils.types import Sample

logger = logging.getLogger(__name__)


class DataSource(abc.ABC):
    @abc.abstractmethod
    def get_samples(self, num_samples: int) -> list[list[Sample]]:
        """Return ``num_samples`` groups (one group per prompt)."""

    @abc.abstractmethod
    def add_samples(self, samples: list[list[Sample]]):
        """Give groups back to the source (buffering)."""

    @abc.abstractmethod
    def save(self, rollout_id):
        ...

    @abc.abstractmethod
    def load(self, rollout_id=None):
        ...

    @abc.abstractmethod
    def __len__(self) -> int:
        ...


class RolloutDataSource(DataSource):
    def __init__(self, args):
        self.args = args
        self.epoch_id = 0
        self.sample_group_index = 0
        self.sample_index = 0
        self.sample_offset = 0
        self.metadata = {}
        self.dataset = None
        if getattr(args, "rollout_global_dataset", True) and getattr(args, "prompt_data", None):
            from slime_b200.utils.processing_utils import load_processor, load_tokenizer

            tok = load_tokenizer(args.hf_checkpoint, trust_remote_code=True)
            proc = load_processor(args.hf_checkpoint, trust_remote_code=True)
            self.dataset = Dataset(
                args.prompt_data,
                tokenizer=tok,
                processor=proc,
                max_length=args.rollout_max_prompt_len,
                prompt_key=args.input_key,
                multimodal_keys=args.multimodal_keys,
                label_key=args.label_key,
                metadata_key=args.metadata_key,
                tool_key=args.tool_key,
                apply_chat_template=args.apply_chat_template,
                apply_chat_template_kwargs=args.apply_chat_template_kwargs,
                seed=args.rollout_seed,
            )
            if args.rollout_shuffle:
                self.dataset.shuffle(self.epoch_id)

    def _next_prompts(self, n: int) -> list[Sample]:
        if self.dataset is None:
            return [Sample() for _ in range(n)]
        out = []
        while len(out) < n:
            take = min(n - len(out), len(self.dataset) - self.sample_offset)
            out += self.dataset.samples[self.sample_offset : self.sample_offset + take]
            self.sample_offset += take
            if self.sample_offset >= len(self.dataset):
                self.epoch_id += 1
                self.sample_offset = 0
                if self.args.rollout_shuffle:
                    self.dataset.shuffle(self.epoch_id)
        return out

    def get_samples(self, num_samples):
        groups = []
        for prompt in self._next_prompts(num_samples):
            group = []
            for _ in range(self.args.n_samples_per_prompt):
                s = copy.deepcopy(prompt)
                s.group_index = self.sample_group_index
                s.index = self.sample_index
                self.sample_index += 1
                group.append(s)
            self.sample_group_index += 1
            groups.append(group)
        return groups

    def add_samples(self, samples):
        raise RuntimeError(f"Cannot add samples to {self.__class__.__name__}. This is a read-only data source.")

    def _state_path(self, base, rollout_id):
        return os.path.join(base, "rollout", f"global_dataset_state_dict_{rollout_id}.pt")

    def save(self, rollout_id):
        if not getattr(self.args, "rollout_global_dataset", True) or self.args.save is None:
            return
        path = self._state_path(self.args.save, rollout_id)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save(
            {
                "sample_offset": self.sample_offset,
                "epoch_id": self.epoch_id,
                "sample_group_index": self.sample_group_index,
                "sample_index": self.sample_index,
                "metadata": self.metadata,
            },
            path,
        )

    def load(self, rollout_id=None):
        if not getattr(self.args, "rollout_global_dataset", True) or self.args.load is None:
            return
        path = self._state_path(self.args.load, rollout_id)
        if not os.path.exists(path):
            logger.info("Checkpoint %s does not exist.", path)
            return
        state = torch.load(path, weights_only=False)
        self.sample_offset = state.get("sample_offset", 0)
        self.epoch_id = state.get("epoch_id", 0)
        self.sample_group_index = state.get("sample_group_index", 0)
        self.sample_index = state.get("sample_index", 0)
        self.metadata = state.get("metadata", {})
        if self.dataset is not None and self.args.rollout_shuffle:
            self.dataset.shuffle(self.epoch_id)

    def __len__(self) -> int:
        return len(self.dataset) if self.dataset is not None else 0


def pop_first(args, rollout_id, buffer: list[list[Sample]], num_samples: int) -> list[list[Sample]]:
    n = min(len(buffer), num_samples)
    taken = buffer[:n]
    del buffer[:n]
    return taken


class RolloutDataSourceWithBuffer(RolloutDataSource):
    def __init__(self, args):
        super().__init__(args)
        self.buffer: list[list[Sample]] = []
        path = getattr(args, "buffer_filter_path", None)
        self.buffer_filter = load_function(path) if path else pop_first

    def get_samples(self, num_samples: int):
        groups = self._get_samples_from_buffer(num_samples)
        missing = num_samples - len(groups)
        if missing > 0:
            groups += super().get_samples(missing)
        return groups

    def _get_samples_from_buffer(self, num_samples: int):
        if not self.buffer or num_samples == 0:
            return []
        return self.buffer_filter(self.args, None, self.buffer, num_samples)

    def add_samples(self, samples: list[list[Sample]]):
        if not samples:
            return
        assert isinstance(samples, list) and isinstance(samples[0], list), "add_samples expects list[list[Sample]]"
        for g in samples:
            assert len(g) == self.args.n_samples_per_prompt, (
                f"group of {len(g)} samples, expected n_samples_per_prompt={self.args.n_samples_per_prompt}"
            )
            self.buffer.append(g)

    def update_metadata(self, metadata: dict):
        self.metadata.update(metadata)

    def get_metadata(self):
        return self.metadata

    def get_buffer_length(self):
        return len(self.buffer)
