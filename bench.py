"""Headline benchmark: colocated GRPO step throughput (rollout + train + weight sync).

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...            # the unmodified reference (if runnable)

Workloads (random init, bf16, synthetic data; weak scaling: per-GPU work is fixed as N grows):

``--config qwen2.5-0.5b`` (default): Qwen2.5-0.5B architecture, data parallel only. Per GPU and per step 32 prompts of
256 random token ids, 8 samples each at temperature 1.0 with ``ignore_eos`` and a response length drawn uniformly
from [128, 1024].

``--config qwen3-4b``: Qwen3-4B architecture (36 layers, hidden 2560, 32 Q / 8 KV heads of 128, QK-norm, FFN 9728),
trainer TP2 + sequence parallel x DP N/2, one TP2 rollout engine per GPU pair (TP1 on a single GPU), 8 prompts of
512 ids per GPU x 8 samples, response length uniform in [1024, 8192]: 64 prompts x 8 samples on 8 GPUs. A step of
this config takes about a minute per GPU (the decode phase alone streams ~140 TB of KV cache per GPU), so it is
not the default: give it a small ``--steps``.

Both: reward = fraction of response tokens whose id is divisible by 7; GRPO group-normalised advantages, clipped
policy loss (eps 0.2 / 0.28), one optimizer step per rollout, then the trainer's weights are synced into the
rollout engine (``perf/update_weights_time`` in the output).

``value`` = tokens (prompt + response of every sample) per second over the whole job, from CUDA-event
time around exactly K steps (max over ranks). ``e2e`` = the same metric from a separate wall-clock
measurement of K steps through the public API (``slime_b200.api.ColocatedGRPO.step``) where every
step stages its prompts in pinned host memory, copies them to the device, and reads the loss back.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "grpo_step_tokens_per_s"
_SMI_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
               "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
               "clocks_event_reasons.sw_power_cap")  # fmt: skip


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference", "library"])
    p.add_argument("--config", type=str, default="qwen2.5-0.5b", choices=sorted(CONFIGS))
    p.add_argument("--model", type=str, default=None)
    p.add_argument("--prompts-per-gpu", type=int, default=None)
    p.add_argument("--n-samples", type=int, default=8)
    p.add_argument("--prompt-len", type=int, default=None)
    p.add_argument("--min-response", type=int, default=None)
    p.add_argument("--max-response", type=int, default=None)
    p.add_argument("--max-tokens-per-gpu", type=int, default=None)
    p.add_argument("--tp", type=int, default=None, help="tensor-parallel size of trainer and engines (config default)")
    p.add_argument("--recompute", type=str, default=None, choices=["full", "none", "auto"])
    p.add_argument("--e2e-steps", type=int, default=None, help="steps of the end-to-end arm (default: --steps)")
    p.add_argument("--no-e2e", action="store_true")
    a = p.parse_args()
    for k, v in CONFIGS[a.config].items():
        if getattr(a, k, None) is None:
            setattr(a, k, v)
    return a


CONFIGS = {
    "qwen2.5-0.5b": dict(model="qwen2.5-0.5b", prompts_per_gpu=32, prompt_len=256, min_response=128, max_response=1024,
                         max_tokens_per_gpu=16384, tp=1, recompute="none", mem_fraction=0.45),
    # recompute: "auto" = none under TP2 (a 9216-token micro-batch keeps ~22 GB of activations per rank, which 180 GB
    # holds next to the trainer state and the KV pool), full on a single GPU where the whole optimizer state is local
    "qwen3-4b": dict(model="qwen3-4b", prompts_per_gpu=8, prompt_len=512, min_response=1024, max_response=8192,
                     max_tokens_per_gpu=9216, tp=2, recompute="auto", mem_fraction=0.72),
    # MoE config: trainer TP4 (+ sequence parallel) with the experts spread over all ranks (EP = world, at most 8), one
    # rollout engine per tensor-parallel group with its experts sharded over the group and block-fp8 resident weights
    "qwen3-30b-a3b": dict(model="qwen3-30b-a3b", prompts_per_gpu=4, prompt_len=512, min_response=1024, max_response=8192,
                          max_tokens_per_gpu=20480, tp=4, ep=8, recompute="full", mem_fraction=0.6, quantization="fp8"),
}  # fmt: skip


def reference_arm(a):
    """The reference's GRPO step runs through ``train.py`` -> Ray -> Megatron-LM + SGLang. The package
    itself installs offline (``baseline/_ref``, --no-deps) but its engines are external pinned
    dependencies that are not in this image and cannot be built offline."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    missing = []
    for mod in ("ray", "megatron.core", "sglang"):
        try:
            __import__(mod)
        except Exception:  # noqa: BLE001
            missing.append(mod)
    if missing:
        print(json.dumps({"impl": "reference", "unavailable": "reference train.py needs " + ", ".join(missing)
                          + " (external engines, not installable offline); only its CPU math imports"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "reference engines import but no runnable offline recipe is wired"}))
    return 0


class ClockSampler:
    def __init__(self, gpu_index: int):
        import tempfile

        self.proc, self.path = None, os.path.join(tempfile.gettempdir(), f"slime_b200_bench_clocks_{os.getpid()}.csv")
        self.gpu = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={_SMI_FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)  # fmt: skip
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}  # fmt: skip


def build_args(a, world, tp):
    from slime_b200.models.config import apply_to_args, get_preset
    from slime_b200.utils.arguments import namespace_from_dict

    ns = namespace_from_dict(dict(
        rollout_batch_size=a.prompts_per_gpu * world, n_samples_per_prompt=a.n_samples, num_rollout=10**6,
        global_batch_size=a.prompts_per_gpu * a.n_samples * world, num_steps_per_rollout=1, colocate=True,
        use_dynamic_batch_size=True, max_tokens_per_gpu=a.max_tokens_per_gpu, lr=1e-6, weight_decay=0.1, adam_beta2=0.98,
        eps_clip=0.2, eps_clip_high=0.28, advantage_estimator="grpo", rollout_temperature=1.0, rollout_ignore_eos=True,
        rollout_max_context_len=a.prompt_len + a.max_response + 16, custom_rm_path="slime_b200.rollout.synthetic.mod7_reward",
        actor_num_nodes=1, actor_num_gpus_per_node=world, rollout_num_gpus=world, rollout_num_gpus_per_engine=tp,
        sglang_mem_fraction_static=a.mem_fraction, sglang_max_running_requests=a.prompts_per_gpu * a.n_samples * tp,
        rollout_seed=42, seed=1234, tensor_model_parallel_size=tp, sequence_parallel=tp > 1,
        recompute_granularity="full" if a.recompute == "full" else None,
        expert_model_parallel_size=getattr(a, "ep_used", 1), expert_tensor_parallel_size=1,
        sglang_quantization=getattr(a, "quantization", None), sglang_ep_size=tp if getattr(a, "ep_used", 1) > 1 else 1,
    ))  # fmt: skip
    apply_to_args(get_preset(a.model), ns)
    ns.kv_channels = ns.kv_channels or ns.hidden_size // ns.num_attention_heads
    if tp > 1:  # vocab-parallel embedding / LM head
        mult = 128 * tp
        ns.padded_vocab_size = -(-ns.vocab_size // mult) * mult
    return ns


def main():
    a = parse()
    if a.impl == "reference":
        return reference_arm(a)
    if a.impl == "library":
        os.environ["SLIME_B200_LIBRARY_OPS"] = "1"  # read by slime_b200.ops at import: see ops.library_mode()

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N>1"
    assert torch.cuda.is_available(), "bench.py needs a GPU"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from slime_b200.api import ColocatedGRPO
    from slime_b200.ops import _lib
    from slime_b200.parallel import state as mpu

    tp = min(a.tp, world)
    if a.recompute == "auto":
        a.recompute = "none" if tp > 1 else "full"
    assert world % tp == 0, f"{world} GPUs do not split into tensor-parallel groups of {tp}"
    a.ep_used = min(getattr(a, "ep", None) or 1, world)
    mpu.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=a.ep_used,
                                  expert_tensor_parallel_size=1 if a.ep_used > 1 else None)
    args = build_args(a, world, tp)
    runner = ColocatedGRPO(args)
    # one data stream per data-parallel rank: the ranks of a tensor-parallel group see the same prompts
    gen = torch.Generator().manual_seed(1000 + mpu.get_data_parallel_rank())
    G, n = a.prompts_per_gpu * tp, a.n_samples
    # inputs staged in pinned host memory, one fresh batch per step (> L2: the step touches ~GBs of weights/KV)
    e2e_steps = 0 if a.no_e2e else (a.e2e_steps or a.steps)
    total_steps = a.warmup + a.steps + e2e_steps
    prompts_host = torch.randint(0, args.vocab_size, (total_steps, G, a.prompt_len), generator=gen, dtype=torch.int32).pin_memory()
    resp_lens = torch.randint(a.min_response, a.max_response + 1, (total_steps, G * n), generator=gen)
    dev_prompts = torch.empty(G, a.prompt_len, dtype=torch.int32, device="cuda")
    h2d = {"bytes": 0}

    def one_step(i):
        dev_prompts.copy_(prompts_host[i], non_blocking=True)  # H2D of the step's inputs from pinned memory
        h2d["bytes"] = prompts_host[i].numel() * 4
        out = runner.step(prompts_host[i].tolist(), resp_lens[i].tolist())
        loss = out["metrics"].get("train/loss", 0.0)  # python float: already read back D2H
        if rank == 0:  # progress on stderr: a long step of the large config is otherwise silent for minutes
            kind = "warmup" if i < a.warmup else "step"
            print(f"[bench] {kind} {i}: rollout {out['rollout_s']:.2f} s, train {out['train_s']:.2f} s, sync {out['sync_s']:.3f} s, "
                  f"{out['tokens'] // tp} tokens on this data-parallel rank", file=sys.stderr, flush=True)
        return out, loss

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(a.warmup):
        one_step(i)
    sync()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = _lib.launch_count() + runner.engine.runner.replayed_launches
    e0 = dict(runner.engine.stats)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    tokens, parts = 0, {"rollout_s": 0.0, "train_s": 0.0, "sync_s": 0.0}
    for i in range(a.warmup, a.warmup + a.steps):
        out, _ = one_step(i)
        tokens += out["tokens"] / tp  # every rank of a tensor-parallel group reports the group's tokens
        for k in parts:
            parts[k] += out[k]
    end.record()
    sync()
    ms = start.elapsed_time(end)
    launches = _lib.launch_count() + runner.engine.runner.replayed_launches - l0
    clocks = sampler.stop() if rank == 0 else None

    e2e = None
    if not a.no_e2e:
        sync()
        t0 = time.perf_counter()
        e2e_tokens = 0
        for i in range(a.warmup + a.steps, a.warmup + a.steps + e2e_steps):
            out, loss = one_step(i)
            e2e_tokens += out["tokens"] / tp
        sync()
        e2e_s = time.perf_counter() - t0
        stats = runner.engine.stats
        e2e = {"tokens": e2e_tokens, "seconds": e2e_s,
               "h2d": (h2d["bytes"] + stats.get("h2d_bytes", 0) / max(stats["steps"], 1)),
               "d2h": stats.get("d2h_bytes", 0) / max(stats["steps"], 1)}  # fmt: skip

    t = torch.tensor([ms, float(tokens), e2e["seconds"] if e2e else 0.0, float(e2e["tokens"]) if e2e else 0.0,
                      float(launches), parts["rollout_s"], parts["train_s"], parts["sync_s"]], dtype=torch.float64, device="cuda")  # fmt: skip
    phase_max = {k: v / a.steps for k, v in parts.items()}
    if world > 1:
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, tokens, launches = float(mx[0]), float(sm[1]), float(sm[4])
        phase_max = {"rollout_s": float(mx[5]) / a.steps, "train_s": float(mx[6]) / a.steps, "sync_s": float(mx[7]) / a.steps}
        if e2e:
            e2e["seconds"], e2e["tokens"] = float(mx[2]), float(sm[3])
    if rank == 0:
        value = tokens / (ms / 1e3)
        steps_engine = max(runner.engine.stats["steps"] - e0["steps"], 1)
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random prompt ids, random-init weights)", "impl": a.impl,
            "config": {"model": a.model, "layers": args.num_layers, "hidden": args.hidden_size,
                       "global_batch": a.prompts_per_gpu * n * world, "seq_len": f"{a.prompt_len}+U[{a.min_response},{a.max_response}]",
                       "parallelism": (f"tp{tp}xdp{world // tp}" if tp > 1 else f"dp{world}") + (f"+ep{a.ep_used}" if a.ep_used > 1 else ""),
                       "rollout": f"{world // tp} engine(s) x tp{tp}", "prompts_per_gpu": a.prompts_per_gpu,
                       "n_samples_per_prompt": n, "colocated": True, "recompute": a.recompute,
                       "l2": "inputs larger than L2 (fresh prompts each step; weights+KV+activations >> 126 MB)",
                       "phase_seconds_rank0": {k: v / a.steps for k, v in parts.items()},
                       "phase_seconds_max_over_ranks": phase_max,
                       "perf/update_weights_time": phase_max["sync_s"]},
            "clocks": clocks, "gpu_launches": int(launches),
        }  # fmt: skip
        if a.impl == "library":
            line["library_replaces"] = ("explanatory arm, not the reference framework: GEMMs -> cuBLAS (torch.mm), training / prefill "
                                        "attention -> flash-attn, RMSNorm / RoPE / SwiGLU / embedding -> eager PyTorch, fused loss -> "
                                        "logits + PyTorch ops, peer-memory collectives -> NCCL; the engine's decode attention, KV write "
                                        "and sampling kernels stay")
        if e2e:
            line["e2e"] = {"value": e2e["tokens"] / e2e["seconds"], "unit": "tokens/s", "steps": e2e_steps,
                           "h2d_bytes_per_step": int(runner_h2d_bytes(runner, a, G, n)),
                           "d2h_bytes_per_step": int(runner_d2h_bytes(runner, a, G, n))}  # fmt: skip
        print(json.dumps(line), flush=True)
    if world > 1:
        _finish(runner.engine)
    return 0


def _finish(engine, grace_s: float = 60.0):
    """The result line is out. Tear the process groups down in order (graphs that captured NCCL collectives first);
    should the teardown itself stall, leave after ``grace_s`` instead of holding the GPUs."""
    import threading

    from slime_b200.utils.distributed_utils import shutdown_distributed

    t = threading.Thread(target=shutdown_distributed, args=([engine],), daemon=True)
    t.start()
    t.join(grace_s)
    sys.stdout.flush()
    sys.stderr.flush()
    if t.is_alive():
        os._exit(0)


def runner_h2d_bytes(runner, a, G, n):
    """Bytes copied host->device per step, counted from the tensors: the staged prompt batch, the engine's
    prefill/decode input uploads and the trainer's token / mask / log-prob tensors."""
    st = runner.engine.stats
    steps = max(runner.rollout_id, 1)
    return G * a.prompt_len * 4 + (st.get("h2d_bytes", 0) + runner.actor.__dict__.get("h2d_bytes", 0)) / steps


def runner_d2h_bytes(runner, a, G, n):
    st = runner.engine.stats
    steps = max(runner.rollout_id, 1)
    return (st.get("d2h_bytes", 0) + runner.actor.__dict__.get("d2h_bytes", 0)) / steps


if __name__ == "__main__":
    sys.exit(main())
