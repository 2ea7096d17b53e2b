"""Model/optimizer construction and the forward-only / train-step loops.

Replaces what the reference gets from Megatron (``setup_model_and_optimizer``,
``get_forward_backward_func`` with 1F1B, DDP grad buffers, DistributedOptimizer)
and the slime glue around it: slime/backends/megatron_utils/model.py:269-321
(setup), :347-509 (forward_only), :512-702 (train_one_step), :710-943 (train).
"""

from __future__ import annotations

import logging
import math
import os
from argparse import Namespace

import torch
import torch.distributed as dist

from slime_b200.backends.train import fused_loss
from slime_b200.backends.train.buffers import FlatBuffer
from slime_b200.backends.train.data import DataIterator, get_batch
from slime_b200.backends.train.loss import get_log_probs_and_entropy, get_values, loss_function
from slime_b200.backends.train.optimizer import DistributedOptimizer, get_optimizer_param_scheduler
from slime_b200.models.config import ModelConfig
from slime_b200.models.gpt import GPTModel, named_parameters_with_layer_offset, pipeline_layer_range
from slime_b200.parallel import pipeline, state as mpu
from slime_b200.utils.misc import load_function

logger = logging.getLogger(__name__)

BATCH_KEYS = [
    "tokens", "total_lengths", "response_lengths", "loss_masks", "log_probs", "ref_log_probs", "rollout_log_probs",
    "advantages", "returns", "values", "rollout_mask_sums", "teacher_log_probs", "opd_reverse_kl", "sample_indices",
    "rollout_top_p_token_ids", "rollout_top_p_token_offsets", "rollout_routed_experts", "multimodal_train_inputs",
]  # fmt: skip


class TrainModel:
    """One role's (actor / critic) model chunk(s), flat buffers and sharded optimizer on this rank."""

    def __init__(self, args: Namespace, role: str = "actor", device=None, with_optimizer: bool = True):
        self.args, self.role = args, role
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.cfg = ModelConfig.from_args(args)
        if getattr(args, "allgather_cp", False):
            from slime_b200.models import mixers

            mixers.set_allgather_cp(True)
        if getattr(args, "max_tokens_per_gpu", None):
            from slime_b200.parallel import fused_tp

            fused_tp.set_max_tokens(args.max_tokens_per_gpu)
        pp, ppr = mpu.get_pipeline_model_parallel_world_size(), mpu.get_pipeline_model_parallel_rank()
        vpp = mpu.get_virtual_pipeline_model_parallel_world_size() or 1
        dtype = torch.bfloat16 if getattr(args, "bf16", True) else torch.float32
        provider = load_function(args.custom_model_provider_path) if getattr(args, "custom_model_provider_path", None) else None
        self.chunks: list[GPTModel] = []
        spec = getattr(args, "spec", None)
        if spec and len(spec) == 2 and not spec[0].startswith("slime_plugins."):
            # --spec <module> <function>: a per-layer mixer factory (the reference passes Megatron layer specs this way,
            # e.g. scripts/models/qwen3-next-80B-A3B.sh; its own plug-in names select the built-in mixers instead)
            from slime_b200.models import mixers

            mixers.set_custom_builder(load_function(f"{spec[0]}.{spec[1]}"))
        for v in range(vpp):
            rng = pipeline_layer_range(self.cfg, pp, ppr, getattr(args, "decoder_first_pipeline_num_layers", None),
                                       getattr(args, "decoder_last_pipeline_num_layers", None), vpp, v)  # fmt: skip
            pre = ppr == 0 and v == 0
            post = ppr == pp - 1 and v == vpp - 1
            if provider is not None:
                m = provider(pre_process=pre, post_process=post, vp_stage=v)
            else:
                m = GPTModel(self.cfg, dtype=dtype, device=self.device, sequence_parallel=getattr(args, "sequence_parallel", False),
                             pre_process=pre, post_process=post, layer_range=rng, value_head=(role == "critic"),
                             recompute_granularity=getattr(args, "recompute_granularity", None), seed=args.seed)  # fmt: skip
            if getattr(args, "enable_mtp_training", False) and hasattr(m, "mtp_training"):
                m.mtp_training = True
            self.chunks.append(m)
        from slime_b200.observability import layerwise_dump

        self.layer_dump = layerwise_dump.enable_from_env(self, prefix=f"{role}_")
        self._freeze_params()
        self._build_buffers()
        self.optimizer = self.scheduler = None
        if with_optimizer:
            self.optimizer = DistributedOptimizer(
                self.buffers, lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
                weight_decay=args.weight_decay, clip_grad=args.clip_grad, stateless=getattr(args, "use_stateless_adam", False),
                cpu_offload=getattr(args, "optimizer_cpu_offload", False),
            )  # fmt: skip
            self.scheduler = get_optimizer_param_scheduler(args)

    # ------------------------------------------------------------------ construction
    def _freeze_params(self):
        import re

        only = getattr(self.args, "only_train_params_name_list", None)
        freeze = getattr(self.args, "freeze_params_name_list", None)
        for name, p in self.named_parameters():
            if only:
                p.requires_grad_(any(re.search(pat, name) for pat in only))
            elif freeze and any(re.search(pat, name) for pat in freeze):
                p.requires_grad_(False)

    def _build_buffers(self):
        dense, dense_names, expert, expert_names = [], [], [], []
        for name, p in self.named_parameters():
            if getattr(p, "is_expert", False):
                expert.append(p)
                expert_names.append(name)
            else:
                dense.append(p)
                dense_names.append(name)
        self.buffers: list[FlatBuffer] = []
        alloc = getattr(self, "_allocator", None)
        from slime_b200.parallel.fused_dp import symmetric_memory_usable

        dp = mpu.get_data_parallel_world_size(with_context_parallel=True)
        # Peer-memory optimizer step: needs buffers that stay mapped, so not with a trainer that releases its memory
        # between phases, and not with optimizer state on the host.
        symmetric = (symmetric_memory_usable(dp, self.device) and mpu.get_pipeline_model_parallel_world_size() == 1
                     and not getattr(self.args, "offload_train", False) and not getattr(self.args, "optimizer_cpu_offload", False)
                     and getattr(self.args, "fused_dp_step", True))  # fmt: skip
        self.dense_buffer = FlatBuffer(dense, dense_names, lambda: mpu.get_data_parallel_group(with_context_parallel=True), dp,
                                       mpu.get_data_parallel_rank(with_context_parallel=True), self.device, allocator=alloc,
                                       symmetric=symmetric)  # fmt: skip
        self.buffers.append(self.dense_buffer)
        self.expert_buffer = None
        if expert:
            self.expert_buffer = FlatBuffer(expert, expert_names, mpu.get_expert_data_parallel_group,
                                            mpu.get_expert_data_parallel_world_size(), mpu.get_expert_data_parallel_rank(),
                                            self.device, allocator=alloc)  # fmt: skip
            self.buffers.append(self.expert_buffer)

    def named_parameters(self):
        for chunk in self.chunks:
            yield from named_parameters_with_layer_offset(chunk)

    def parameters(self):
        for _n, p in self.named_parameters():
            yield p

    def named_buffers(self):
        for chunk in self.chunks:
            for name, b in chunk.named_buffers():
                parts = name.split(".")
                if len(parts) > 2 and parts[1] == "layers":
                    parts[2] = str(int(parts[2]) + chunk.layer_offset)
                yield ".".join(parts), b

    def train(self, mode=True):
        for c in self.chunks:
            c.train(mode)

    def eval(self):
        self.train(False)

    # ------------------------------------------------------------------ grad sync
    def zero_grad_buffer(self):
        for b in self.buffers:
            b.zero_grad()

    def finalize_grads(self):
        """Fold stray ``.grad``s, all-reduce grads of TP-replicated params fed by sharded activations
        (SP layer norms, qk-norms), tie embeddings across pipeline ends, then reduce over DP."""
        for b in self.buffers:
            b.fold_autograd_grads()
        tps = mpu.get_tensor_model_parallel_world_size()
        if tps > 1:
            flat = [p.main_grad for _n, p in self.named_parameters()
                    if getattr(p, "sequence_parallel", False) or getattr(p, "needs_tp_grad_reduce", False)]  # fmt: skip
            # coalesced, at most ~1 GiB per collective (the staging copy of a very large model's norm grads stays bounded)
            limit, batch, size = int(os.environ.get("SLIME_GRAD_COALESCE_CHUNK_BYTES", 1 << 30)), [], 0
            for g in flat + [None]:
                if g is not None:
                    batch.append(g)
                    size += g.numel() * g.element_size()
                if batch and (g is None or size >= limit):
                    coalesced = torch.cat([x.reshape(-1) for x in batch])
                    dist.all_reduce(coalesced, group=mpu.get_tensor_model_parallel_group())
                    off = 0
                    for x in batch:
                        x.copy_(coalesced[off : off + x.numel()].view_as(x))
                        off += x.numel()
                    batch, size = [], 0
        if mpu.get_pipeline_model_parallel_world_size() > 1 and self.cfg.tie_word_embeddings:
            w = None
            if self.chunks[0].pre_process:
                w = self.chunks[0].embedding.word_embeddings.weight
            elif self.chunks[-1].post_process and self.chunks[-1].output_layer is not None:
                w = self.chunks[-1].output_layer.weight
            if w is not None:
                dist.all_reduce(w.main_grad, group=mpu.get_embedding_group())
        for b in self.buffers:
            b.reduce_scatter_grads()


# ---------------------------------------------------------------------------- forward only
@torch.no_grad()
def forward_only(f, args, model: TrainModel, data_iterator: list[DataIterator], num_microbatches: list[int],
                 store_prefix: str = "") -> dict:
    """Eval-mode pass over all micro-batches collecting ``f``'s per-sample outputs
    (``f`` is get_log_probs_and_entropy or get_values) re-ordered to local sample order."""
    model.eval()
    for it in data_iterator:
        it.reset()
    hook = getattr(args, "custom_megatron_before_log_prob_hook_path", None)
    if hook:
        load_function(hook)(args, model.chunks, store_prefix)
    total_mb = sum(num_microbatches)
    use_fused = _can_use_fused_logprob(args, f, model)

    def forward_step(batch, chunk, input_tensor):
        chunk.set_input_tensor(input_tensor)
        out = chunk(batch["tokens"], batch["position_ids"], packed_seq_params=batch["packed_seq_params"], **batch.get("multimodal", {}),
                    return_hidden=use_fused)  # fmt: skip
        if not chunk.post_process:
            return out, None
        if use_fused:
            res = _fused_logprob_from_hidden(args, chunk, out, batch)
        else:
            _, res = f(out, args=args, unconcat_tokens=batch["unconcat_tokens"], total_lengths=batch["total_lengths"],
                       response_lengths=batch["response_lengths"], with_entropy=getattr(args, "use_rollout_entropy", False))  # fmt: skip
        return out, res

    results = pipeline.run_forward_only(model, data_iterator[0], total_mb, forward_step, args)
    out: dict[str, list] = {}
    if mpu.is_pipeline_last_stage():
        order = [i for mb in data_iterator[0].micro_batch_indices for i in mb]
        for key in results[0].keys() if results else []:
            flat = [t for r in results for t in r[key]]
            ordered = [None] * len(flat)
            for pos, t in zip(order, flat):
                ordered[pos] = t
            out[f"{store_prefix}{key}"] = ordered
    model.train()
    return out


def _can_use_fused_logprob(args, f, model) -> bool:
    return (
        f is get_log_probs_and_entropy
        and model.device.type == "cuda"
        and mpu.get_context_parallel_world_size() == 1
        and getattr(args, "rollout_top_p", 1.0) == 1.0
        and getattr(args, "fused_loss", True)
        and os.environ.get("SLIME_B200_LIBRARY_OPS") != "1"
    )


def _response_rows(batch, device):
    """Row indices (into the packed stream) that predict response tokens, and the target token ids."""
    rows, tgts, lens = [], [], []
    end = 0
    for tok, tl, rl in zip(batch["unconcat_tokens"], batch["total_lengths"], batch["response_lengths"]):
        end += tl
        rows.append(torch.arange(end - rl - 1, end - 1, device=device))
        tgts.append(tok[-rl:])
        lens.append(rl)
    return torch.cat(rows), torch.cat(tgts).to(torch.int32), lens


def _fused_logprob_from_hidden(args, chunk, hidden, batch):
    rows, tgts, lens = _response_rows(batch, hidden.device)
    h = hidden.index_select(0, rows)
    lp, ent = fused_loss.logprob_entropy_rows(
        h, chunk.output_weight(), tgts, inv_temperature=1.0 / getattr(args, "rollout_temperature", 1.0),
        vocab_lo=chunk.vocab_start, tp_group=mpu.get_tensor_model_parallel_group(),
        with_entropy=getattr(args, "use_rollout_entropy", False),
    )  # fmt: skip
    res = {"log_probs": list(lp.split(lens))}
    if ent is not None:
        res["entropy"] = list(ent.split(lens))
    return res


# ------------------------------------------------------------------------------ train step
def _fused_policy_eligible(args, model) -> bool:
    return (
        args.loss_type == "policy_loss" and args.advantage_estimator in ("grpo", "cispo", "ppo", "reinforce_plus_plus",
                                                                         "reinforce_plus_plus_baseline")
        and model.device.type == "cuda" and mpu.get_context_parallel_world_size() == 1
        and not args.use_opsm and not args.use_kl_loss and not args.get_mismatch_metrics
        and args.custom_tis_function_path is None and getattr(args, "custom_pg_loss_reducer_function_path", None) is None
        and getattr(args, "rollout_top_p", 1.0) == 1.0 and getattr(args, "fused_loss", True)
        and not getattr(args, "recompute_loss_function", False) and os.environ.get("SLIME_B200_LIBRARY_OPS") != "1"
    )  # fmt: skip


def _fused_policy_step(args, chunk, hidden, batch, step_gbs, step_total_tokens):
    """Fast path: per-token weights carry mask, per-rollout denominators and the step normalisation."""
    dev = hidden.device
    rows, tgts, lens = _response_rows(batch, dev)
    h = hidden.index_select(0, rows)
    masks = torch.cat(batch["loss_masks"]).to(torch.float32)
    if args.calculate_per_token_loss:
        w = masks / step_total_tokens
    else:
        denoms = batch.get("rollout_mask_sums") or [m.sum() for m in batch["loss_masks"]]
        d = torch.cat([torch.clamp_min(torch.as_tensor(dn, dtype=torch.float32, device=dev), 1).expand(n) for dn, n in zip(denoms, lens)])
        w = masks / d / step_gbs
    adv = torch.cat(batch["advantages"]).to(torch.float32)
    old = batch["rollout_log_probs"] if args.use_rollout_logprobs else batch.get("log_probs")
    old = torch.cat(old).to(torch.float32).contiguous() if old else None
    tis = None
    if args.use_tis:
        train_old = torch.cat(batch["log_probs"]) if batch.get("log_probs") else None
        ro = torch.cat(batch["rollout_log_probs"]).to(torch.float32)
        base = train_old if train_old is not None else ro  # without a stored train log-prob the ratio is 1
        tis = torch.exp(base - ro).clamp(min=args.tis_clip_low, max=args.tis_clip).contiguous()
    loss, logp, ent, metrics = fused_loss.fused_policy_loss(
        h, chunk.output_weight(), tgts, old, adv, w.contiguous(), eps_clip=args.eps_clip, eps_clip_high=args.eps_clip_high,
        eps_clip_c=args.eps_clip_c, cispo=args.advantage_estimator == "cispo", entropy_coef=args.entropy_coef,
        temperature=getattr(args, "rollout_temperature", 1.0), tis=tis,
    )  # fmt: skip
    # metrics are already normalised sums: report in the same units as the general path (x gbs)
    scale = 1.0 if args.calculate_per_token_loss else float(step_gbs)
    log = {"loss": loss.detach() * scale, "pg_loss": metrics[0] * scale, "entropy_loss": metrics[3] * scale,
           "pg_clipfrac": metrics[1] * scale, "ppo_kl": metrics[2] * scale}  # fmt: skip
    if batch.get("rollout_log_probs"):
        ro = torch.cat(batch["rollout_log_probs"]).to(torch.float32)
        cmp = logp if (args.use_rollout_logprobs or old is None) else old
        log["train_rollout_logprob_abs_diff"] = ((cmp - ro).abs() * w).sum() * scale
    ntok = masks.sum().clamp_min(1)
    vals = torch.stack([ntok if args.calculate_per_token_loss else torch.zeros((), device=dev)] + [v.reshape(()).float() for v in log.values()])
    return loss, {"keys": list(log.keys()), "values": vals}


def train_one_step(args, rollout_id, step_id, data_iterator, model: TrainModel, num_microbatches: int, step_gbs: int):
    """zero grads -> 1F1B forward/backward over the step's micro-batches -> grad sync -> optimizer -> metrics."""
    model.zero_grad_buffer()
    hook = getattr(args, "custom_megatron_before_train_step_hook_path", None)
    if hook:
        load_function(hook)(args, rollout_id, step_id, model.chunks, model.optimizer, model.scheduler)
    fused = _fused_policy_eligible(args, model)

    step_total_tokens = None
    if args.calculate_per_token_loss:
        it = data_iterator[0]
        tok = sum(float(torch.clamp_min(m.sum(), 1)) for mb in it.micro_batch_indices[it.offset : it.offset + num_microbatches]
                  for m in (it.rollout_data["loss_masks"][i] for i in mb))  # fmt: skip
        t = torch.tensor([tok], dtype=torch.float64, device=model.device)
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(t, group=mpu.get_data_parallel_group(with_context_parallel=False))
        step_total_tokens = float(t.item())

    def forward_step(batch, chunk, input_tensor):
        chunk.set_input_tensor(input_tensor)
        out = chunk(batch["tokens"], batch["position_ids"], packed_seq_params=batch["packed_seq_params"], **batch.get("multimodal", {}), return_hidden=fused)
        if not chunk.post_process:
            return out, None
        if fused:
            loss, log = _fused_policy_step(args, chunk, out, batch, step_gbs, step_total_tokens)
        else:
            loss, _norm, log = loss_function(args, batch, num_microbatches, step_gbs, out, step_total_tokens)
        aux = [l.mlp.aux_loss for l in chunk.decoder.layers if getattr(l.mlp, "aux_loss", None) is not None]
        if aux:
            loss = loss + sum(aux) / max(num_microbatches, 1)
        if getattr(args, "enable_mtp_training", False) and getattr(chunk, "mtp", None) is not None:
            # the draft head learns the tokens actually sampled (cross entropy), scaled like Megatron's MTP loss
            mtp = chunk.mtp_loss(batch["full_loss_masks"])
            loss = loss + args.mtp_loss_scaling_factor * mtp / max(num_microbatches, 1)
            log = dict(log, mtp_loss=mtp.detach()) if isinstance(log, dict) and "keys" not in log else log
        return loss, log

    logs = pipeline.run_forward_backward(model, data_iterator[0], num_microbatches, forward_step, args)
    model.finalize_grads()
    if getattr(args, "ci_test", False) and getattr(args, "enable_mtp_training", False) and getattr(args, "ci_check_mtp_only_grad", False):
        from slime_b200.backends.train.ci_utils import check_mtp_only_grad

        check_mtp_only_grad(model, step_id)

    # non-finite guard on the device: the flag makes the Adam kernel a no-op (no host sync)
    opt = model.optimizer
    lr = model.scheduler.get_lr()
    grad_norm = opt.step(grad_scale=1.0, lr=lr, skip_on_nonfinite=getattr(args, "check_for_nan_in_loss_and_grad", True))
    model.scheduler.step(increment=step_gbs)
    if any(getattr(b, "fused", None) is not None for b in model.buffers):
        # the peer-memory optimizer step has bounded waits: an expired one made every rank skip the update (the skip
        # flag is all-reduced with the norm) and left a status word, which is surfaced here instead of training on
        from slime_b200.ops import _lib

        _lib.check_status(model.device)
    return reduce_train_step_metrics(args, logs, step_gbs), grad_norm


def reduce_train_step_metrics(args, logs: list[dict], step_gbs: int) -> dict:
    """Sum micro-batch metric vectors, all-reduce over DP x CP, divide by the step denominator."""
    if not mpu.is_pipeline_last_stage() or not logs:
        return {}
    keys = logs[0]["keys"]
    vals = torch.stack([l["values"] for l in logs]).sum(0)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(vals, group=mpu.get_data_parallel_group(with_context_parallel=True))
    denom = vals[0] if args.calculate_per_token_loss else float(step_gbs)
    cp = mpu.get_context_parallel_world_size()
    return {k: (vals[i + 1] / denom) for i, k in enumerate(keys)}


def train(rollout_id, model: TrainModel, data_iterator, num_microbatches: list[int], global_batch_sizes: list[int]):
    """All optimizer steps of one rollout; returns the per-step reduced metrics."""
    args = model.args
    model.train()
    for it in data_iterator:
        it.reset()
    history = []
    steps = enumerate(zip(num_microbatches, global_batch_sizes))
    if getattr(args, "use_pytorch_profiler", False):  # --profile-target train_actor: one profiler step per optimizer step
        from slime_b200.observability.profile_utils import _profile_simple_loop

        steps = _profile_simple_loop(steps, args, "train_actor")
    for step_id, (nmb, gbs) in steps:
        metrics, grad_norm = train_one_step(args, rollout_id, step_id, data_iterator, model, nmb, gbs)
        history.append((metrics, grad_norm))
    return history
