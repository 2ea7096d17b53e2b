"""Public in-process API: one colocated trainer + rollout engine per GPU.

``ColocatedGRPO`` is the shortest path through the framework's own components: prompts ->
rollout engine (continuous batching, paged KV, fused sampling) -> ``Sample`` objects -> reward hook
-> GRPO group normalisation -> DP schedule -> packed forward/backward with the fused loss ->
sharded Adam -> device-side weight sync back into the engine. ``train.py`` composes the same
objects through the actor runtime; this class keeps them in one process per GPU, which is what a
single 8xB200 box with colocated placement wants (no IPC between trainer and engine).
"""

from __future__ import annotations

import asyncio
import time
from argparse import Namespace

import torch
import torch.distributed as dist

from slime_b200.backends.train.actor import TrainActor
from slime_b200.engine.engine import Engine
from slime_b200.engine.request import SamplingParams
from slime_b200.engine.server_args import ServerArgs
from slime_b200.models.config import ModelConfig
from slime_b200.parallel import state as mpu
from slime_b200.rollout import train_data as td
from slime_b200.rollout.rm_hub import async_rm
from slime_b200.utils.types import Sample


class ColocatedGRPO:
    def __init__(self, args: Namespace, device=None, engine_pages: int | None = None, server_args: ServerArgs | None = None):
        self.args = args
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        )
        self.actor = TrainActor(args, role="actor")
        self.actor.init(device=self.device)
        cfg = self.actor.model.cfg
        sa = server_args or ServerArgs(
            context_length=getattr(args, "rollout_max_context_len", None) or 4096,
            max_running_requests=getattr(args, "sglang_max_running_requests", None) or 512,
            mem_fraction_static=getattr(args, "sglang_mem_fraction_static", None) or 0.5,
            page_size=getattr(args, "sglang_page_size", None) or 16,
            random_seed=args.rollout_seed + mpu.get_data_parallel_rank(),
            disable_cuda_graph=bool(getattr(args, "sglang_disable_cuda_graph", False)),
            quantization=getattr(args, "sglang_quantization", None),
            ep_size=getattr(args, "sglang_ep_size", None) or 1,
            enable_return_routed_experts=bool(getattr(args, "use_rollout_routing_replay", False)),
        )
        # One engine per tensor-parallel group of the trainer, sharded the same way: rank r of the group holds shard r
        # of both the trainer's and the engine's weights, so weight sync is a device-local copy and the ranks of a
        # group step the engine in lockstep (same requests, same seeds, same tokens).
        tps = mpu.get_tensor_model_parallel_world_size()
        self.engine = Engine(cfg, sa, device=self.device, num_pages=engine_pages,
                             tp_group=mpu.get_tensor_model_parallel_group() if tps > 1 else None, tp_size=tps,
                             tp_rank=mpu.get_tensor_model_parallel_rank())  # fmt: skip
        self.actor.connect_rollout_engines([self.engine])
        self.actor.update_weights()
        self.rollout_id = 0
        self.sample_index = 0
        self.timings: dict[str, float] = {}

    # ------------------------------------------------------------------ rollout
    def generate(self, prompts: list[list[int]], max_new_tokens: list[int] | int, n_samples: int | None = None) -> list[Sample]:
        """Generate ``n_samples`` per prompt; returns flat list of Samples in group order."""
        a = self.args
        n = n_samples or a.n_samples_per_prompt
        reqs, samples = [], []
        for g, p in enumerate(prompts):
            for j in range(n):
                mnt = max_new_tokens[g * n + j] if isinstance(max_new_tokens, (list, tuple)) else max_new_tokens
                sp = SamplingParams(temperature=a.rollout_temperature, top_p=a.rollout_top_p, top_k=a.rollout_top_k,
                                    max_new_tokens=mnt, ignore_eos=getattr(a, "rollout_ignore_eos", False),
                                    stop_token_ids=a.rollout_stop_token_ids,
                                    sampling_seed=a.rollout_seed * 1_000_003 + self.sample_index)  # fmt: skip
                if a.rollout_top_p != 1.0:
                    sp.custom_params = {"return_top_p_token_ids": True}
                reqs.append(self.engine.add_request(p, sp, return_routed_experts=self.engine.runner.record_routed))
                s = Sample(group_index=self.rollout_id * len(prompts) + g, index=self.sample_index, prompt="", tokens=list(p))
                self.sample_index += 1
                samples.append(s)
        while self.engine.has_work():
            self.engine.step()
        for s, r in zip(samples, reqs):
            s.append_response_tokens(a, tokens=r.output_ids, log_probs=r.output_logprobs, meta_info=self.engine.meta_info(r))
        return samples

    def reward(self, samples: list[Sample]):
        async def run():
            return await asyncio.gather(*[async_rm(self.args, s) for s in samples])

        for s, r in zip(samples, asyncio.run(run())):
            s.reward = r
        return samples

    # -------------------------------------------------------------------- train
    def train_on(self, samples: list[Sample]):
        a = self.args
        data = td.convert_samples_to_train_data(a, samples)
        cfg = {"dp_size": 1, "cp_size": mpu.get_context_parallel_world_size(),
               "vpp_size": mpu.get_virtual_pipeline_model_parallel_world_size() or 1,
               "microbatch_group_size_per_vp_stage": a.microbatch_group_size_per_vp_stage or 1}  # fmt: skip
        # every DP rank generated its own slice of the global batch: schedule locally, reduce globally
        local_args = Namespace(**{**vars(a), "global_batch_size": max(1, a.global_batch_size // mpu.get_data_parallel_world_size())})
        payload = td.split_train_data_by_dp(local_args, data, cfg, pin=self.device.type == "cuda")[0]
        payload["global_batch_sizes"] = [a.global_batch_size] * len(payload["global_batch_sizes"])
        return self.actor.train(self.rollout_id, payload)

    def step(self, prompts: list[list[int]], max_new_tokens) -> dict:
        """One full GRPO step: generate -> reward -> train -> weight sync. Returns timing + metrics."""
        t0 = time.perf_counter()
        samples = self.generate(prompts, max_new_tokens)
        t1 = time.perf_counter()
        self.reward(samples)
        metrics = self.train_on(samples)
        t2 = time.perf_counter()
        self.actor.update_weights()
        t3 = time.perf_counter()
        self.rollout_id += 1
        tokens = sum(len(s.tokens) for s in samples)
        return {"tokens": tokens, "response_tokens": sum(s.response_length for s in samples), "rollout_s": t1 - t0,
                "train_s": t2 - t1, "sync_s": t3 - t2, "metrics": metrics[-1] if metrics else {}}  # fmt: skip
