"""Sharded (ZeRO-1) Adam on flat buffers, LR schedule and stateless Adam.

Each data-parallel rank keeps fp32 master weights and Adam moments for its slice
of every ``FlatBuffer``. ``step()``:
  1. reduce-scatter grads (already done by the DDP wrapper, possibly overlapped),
  2. global grad-norm (device-side, no host sync) over all shards and model-parallel ranks,
  3. fused unscale + clip + Adam + bf16 write-back on the shard (one sm_100a kernel),
  4. all-gather the updated bf16 parameters.
Replaces Megatron's DistributedOptimizer + apex FusedAdam used by the reference
(slime/backends/megatron_utils/model.py:300-320,661-686). ``StatelessAdam``
(moments restart from zero every step) mirrors slime/backends/megatron_utils/stateless_adam.py.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist

from slime_b200.backends.train.buffers import FlatBuffer
from slime_b200.ops import _lib

P = _lib.ptr


class OptimizerParamScheduler:
    """Warm-up + {constant, linear, cosine} decay keyed by *samples consumed* (increment = global batch)."""

    def __init__(self, max_lr, min_lr, warmup_steps, decay_steps, decay_style="constant", init_lr=0.0):
        self.max_lr, self.min_lr, self.init_lr = max_lr, min_lr, init_lr
        self.warmup_steps, self.decay_steps, self.decay_style = warmup_steps, max(decay_steps, 1), decay_style
        self.num_steps = 0

    def get_lr(self) -> float:
        n = self.num_steps
        if self.warmup_steps > 0 and n <= self.warmup_steps:
            return self.init_lr + (self.max_lr - self.init_lr) * n / self.warmup_steps
        if self.decay_style == "constant":
            return self.max_lr
        if n > self.decay_steps:
            return self.min_lr
        frac = (n - self.warmup_steps) / max(self.decay_steps - self.warmup_steps, 1)
        if self.decay_style == "linear":
            coeff = 1.0 - frac
        elif self.decay_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * frac) + 1.0)
        else:
            raise ValueError(f"unknown lr decay style {self.decay_style}")
        return self.min_lr + coeff * (self.max_lr - self.min_lr)

    def step(self, increment: int = 1):
        self.num_steps += increment

    def state_dict(self):
        return {"num_steps": self.num_steps, "max_lr": self.max_lr, "min_lr": self.min_lr}

    def load_state_dict(self, sd):
        self.num_steps = sd.get("num_steps", 0)


def get_optimizer_param_scheduler(args) -> OptimizerParamScheduler:
    """LR schedule length derived from the rollout plan (parity: model.py:181-234)."""
    gbs = args.global_batch_size
    total_samples = (args.num_rollout or 1) * args.rollout_batch_size * args.n_samples_per_prompt
    decay = total_samples if args.lr_decay_iters is None else args.lr_decay_iters * gbs
    warm = int(args.lr_warmup_fraction * decay) if args.lr_warmup_fraction else args.lr_warmup_iters * gbs
    return OptimizerParamScheduler(args.lr, args.min_lr, warm, decay, args.lr_decay_style, args.lr_warmup_init)


class DistributedOptimizer:
    def __init__(self, buffers: list[FlatBuffer], *, lr=1e-6, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 clip_grad=1.0, stateless=False, norm_groups=(), cpu_offload=False):  # fmt: skip
        self.buffers = buffers
        self.lr, self.betas, self.eps, self.weight_decay, self.clip_grad = lr, betas, eps, weight_decay, clip_grad
        self.stateless, self.cpu_offload = stateless, cpu_offload
        self.norm_groups = [g for g in norm_groups if g is not None]
        self.step_count = 0
        self.state = []
        for b in buffers:
            dev = "cpu" if cpu_offload else b.param_data.device
            master = b.param_shard().to(dev, torch.float32).clone()
            if cpu_offload and torch.cuda.is_available():
                master = master.pin_memory()
            st = {"master": master}
            if not stateless:
                st["exp_avg"] = torch.zeros_like(master)
                st["exp_avg_sq"] = torch.zeros_like(master)
            self.state.append(st)
        dev = buffers[0].param_data.device if buffers else "cpu"
        self.ctl = torch.zeros(2, dtype=torch.float32, device=dev)  # [grad sq-norm, skip flag]
        self._partials = torch.zeros(1024, dtype=torch.float32, device=dev)
        self.last_grad_norm = None

    # ---- gradient norm ----------------------------------------------------------------------
    def _no_dup_mask_needed(self) -> bool:
        return False

    def compute_grad_sqnorm(self, grad_scale: float = 1.0) -> torch.Tensor:
        """Sum of squares of this rank's grad shards into ``ctl[0]`` and all-reduced over the
        groups that partition the model (DP shards; TP/PP/EP ranks hold different parameters).
        Parameters replicated over TP are counted once per TP rank by this simple sum; the
        replicated tensors are norms/biases and contribute negligibly, and every rank applies
        the same coefficient, so training stays consistent."""
        self.ctl.zero_()  # [squared norm, skip flag]; a fused reduce raises the flag itself when one of its waits gave up
        for b in self.buffers:
            g = b.grad_shard()
            if getattr(b, "fused", None) is not None:
                b.fused.reduce_shard(self.ctl)  # reduce-scatter over peer memory and the shard's squared norm in one pass
            elif g.is_cuda:
                n = min(1024, max(1, g.numel() // 4096))
                rc = _lib.lib().sb_sqnorm(P(g), g.numel(), int(g.dtype == torch.bfloat16), P(self._partials), n,
                                          P(self.ctl), 1, _lib.stream())
                _lib.check(rc, "sb_sqnorm")
            else:
                self.ctl[0] += g.float().pow(2).sum()
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            # shards are disjoint across DP ranks and model-parallel ranks hold different parameters,
            # so one sum over the whole trainer world gives the global norm
            dist.all_reduce(self.ctl)  # the skip flag travels with the norm: every rank takes the same decision
        return self.ctl[0:1]

    # ---- update -----------------------------------------------------------------------------------
    def step(self, grad_scale: float = 1.0, lr: float | None = None, gather_params: bool = True,
             skip_on_nonfinite: bool = True):
        """``grad_scale`` multiplies the accumulated grads (loss normalisation) before clipping."""
        lr = self.lr if lr is None else lr
        self.step_count += 1
        b1, b2 = self.betas
        bc1 = 1.0 - b1**self.step_count
        bc2 = 1.0 - b2**self.step_count
        if self.stateless:
            bc1, bc2 = 1.0 - b1, 1.0 - b2
        self.compute_grad_sqnorm(grad_scale)
        # non-finite guard stays on the device: the flag turns the Adam kernel into a no-op
        if skip_on_nonfinite:
            self.ctl[1] += (~torch.isfinite(self.ctl[0])).float()
        self.last_grad_norm = self.ctl[0:1].sqrt() * grad_scale  # device tensor; .item() only when logged
        for b, st in zip(self.buffers, self.state):
            g = b.grad_shard()
            if getattr(b, "fused", None) is not None:
                b.fused.adam_bcast(st, lr=lr, b1=b1, b2=b2, eps=self.eps, wd=self.weight_decay, bc1=bc1, bc2=bc2,
                                   grad_scale=grad_scale, clip=self.clip_grad, ctl=self.ctl, stateless=self.stateless)
            elif g.is_cuda and not self.cpu_offload:
                rc = _lib.lib().sb_adam(
                    P(st["master"]), P(st.get("exp_avg")), P(st.get("exp_avg_sq")), P(g), int(g.dtype == torch.bfloat16),
                    P(b.param_shard()), g.numel(), lr, b1, b2, self.eps, self.weight_decay, bc1, bc2, grad_scale,
                    float(self.clip_grad or 0.0), P(self.ctl), int(self.stateless), _lib.stream(),
                )  # fmt: skip
                _lib.check(rc, "sb_adam")
            else:
                self._adam_host(b, st, g, lr, b1, b2, bc1, bc2, grad_scale)
        if gather_params:
            for b in self.buffers:
                b.all_gather_params()
        return self.last_grad_norm

    def _adam_host(self, b, st, g, lr, b1, b2, bc1, bc2, grad_scale):
        """CPU path (tests, and --optimizer-cpu-offload: grads D2H, update on host, params H2D)."""
        master = st["master"]
        gf = g.to(master.device, torch.float32) * grad_scale
        norm = float(self.ctl[0].sqrt()) * grad_scale
        if self.clip_grad and self.clip_grad > 0:
            gf = gf * min(1.0, self.clip_grad / (norm + 1e-6))
        if self.stateless:
            m, v = (1 - b1) * gf, (1 - b2) * gf * gf
        else:
            m = st["exp_avg"].mul_(b1).add_(gf, alpha=1 - b1)
            v = st["exp_avg_sq"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
        master.mul_(1 - lr * self.weight_decay)
        master.addcdiv_(m / bc1, (v / bc2).sqrt() + self.eps, value=-lr)
        b.param_shard().copy_(master.to(b.param_data.dtype), non_blocking=True)

    def reload_model_params(self):
        """Refresh the fp32 masters from the (externally modified) bf16 parameters."""
        for b, st in zip(self.buffers, self.state):
            st["master"].copy_(b.param_shard().to(st["master"].device, torch.float32))

    def reset_states(self):
        self.step_count = 0
        for st in self.state:
            for k in ("exp_avg", "exp_avg_sq"):
                if k in st:
                    st[k].zero_()

    def zero_grad(self):
        for b in self.buffers:
            b.zero_grad()

    # ---- checkpoint ---------------------------------------------------------------------------------
    def state_dict(self):
        """Placement-independent: step lives at top level, tensors keyed per buffer/shard."""
        return {
            "step": self.step_count,
            "shards": [{k: v.detach().cpu() for k, v in st.items()} for st in self.state],
            "shard_ranges": [b.shard_range() for b in self.buffers],
        }

    def load_state_dict(self, sd):
        self.step_count = sd.get("step", 0)
        for st, saved in zip(self.state, sd["shards"]):
            for k, v in saved.items():
                if k in st:
                    st[k].copy_(v)


class StatelessAdam(torch.optim.Optimizer):
    """Adam whose moments start from zero every step: ``p -= lr * g / (|g| + eps')`` up to bias terms.
    Keeps no state tensors, so it costs no optimizer memory. Every step equals the first step of a freshly created
    ``torch.optim.AdamW`` (``adam_w_mode``, decoupled decay) or ``torch.optim.Adam`` (decay added to the gradient)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adam_w_mode: bool = True):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adam_w_mode=adam_w_mode))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad if p.grad.dtype == torch.float64 else p.grad.float()
                if group["weight_decay"] and group["adam_w_mode"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                elif group["weight_decay"]:
                    g = g + group["weight_decay"] * p.to(g.dtype)
                m = (1 - b1) * g
                v = (1 - b2) * g * g
                upd = (m / (1 - b1)) / ((v / (1 - b2)).sqrt() + group["eps"])
                p.add_(upd.to(p.dtype), alpha=-group["lr"])
        return loss
