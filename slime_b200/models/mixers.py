"""Token mixers beyond the fused GQA attention path: attention variants, gated delta-net, latent attention, sparse
latent attention with a lightning indexer.

``ModelConfig.mixer(layer)`` names the mixer of a layer and ``build_mixer`` constructs it; every mixer has the calling
convention of ``gpt.SelfAttention``: ``forward(x, residual, rope_table, packed) -> (out, residual)`` on packed
(``thd``) rows, doing its own pre-norm with the fused add + RMSNorm.

* ``GeneralSelfAttention``: tensor-parallel GQA attention composed from separate ops, for the variants the fused
  RoPE + attention kernel does not cover: partial rotary embeddings (GLM-4 family, Qwen3-Next), interleaved rotary
  pairs, a sigmoid output gate carried by the query projection (Qwen3-Next), RMSNorm over all heads at once
  (MiniMax-M2; slime_plugins/models/minimax_m2.py:12 in the reference) and learnable softmax sinks
  (slime_plugins/models/learnable_softmax_attention.py:23). The attention core is the flash kernel pair.
* ``GatedDeltaNet``: the linear-attention layer of Qwen3-Next / Qwen3.5 (slime_plugins/models/qwen3_next.py:27,
  qwen3_5.py:31): short causal depthwise convolution, gated delta rule evaluated chunk by chunk (a triangular solve and
  matmuls per chunk, so autograd provides the backward), gated RMSNorm. ``gated_delta_rule_recurrent`` is the
  token-by-token definition the chunked form is tested against.
* ``MLASelfAttention``: multi-head latent attention (DeepSeek-V3, Kimi-K2, Moonlight): low-rank query and key/value
  projections with a shared rotary key.
* ``DSASelfAttention``: the same with a lightning indexer that picks ``index_topk`` keys per query; layers can reuse the
  choice of an earlier layer (slime_plugins/models/glm5/glm5.py:264-281,302-550 in the reference).

The last three keep their parameters replicated over the tensor-parallel group and compute on the full sequence on
every rank (sequence-parallel rows are gathered before and split after), the way the reference wraps Hugging Face
modules (slime_plugins/models/hf_attention.py:63-173); their math is plain PyTorch ops.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from slime_b200 import ops
from slime_b200.models.config import ModelConfig
from slime_b200.parallel import state as mpu
from slime_b200.parallel import tensor_parallel as tp


def _param(shape, dtype, device, std=None, ones=False, generator=None):
    t = torch.empty(*shape, dtype=torch.float32, device=device)
    if ones:
        t.fill_(1.0)
    elif std == 0.0:
        t.zero_()
    else:
        t.normal_(0.0, std, generator=generator)
    return nn.Parameter(t.to(dtype))


def _replicated(shape, dtype, device, std=None, ones=False):
    gen = tp.get_rng_tracker().states.get("default")
    return tp.set_tp_attrs(_param(shape, dtype, device, std, ones, gen), False)


# ------------------------------------------------------------------------------------------------- rotary helpers
def rotary_cos_sin(table: torch.Tensor, positions: torch.Tensor, band_axes: torch.Tensor | None = None):
    """``table`` [max_pos, rot] = [cos(rot/2) | sin(rot/2)] -> (cos, sin) [T, 1, rot/2] for ``positions`` [T], or for the
    three position streams ``positions`` [3, T] of vision inputs with ``band_axes`` [rot/2] naming each band's stream."""
    if positions.dim() == 2:
        from slime_b200.models.vision import mrope_cos_sin

        return mrope_cos_sin(table, positions, band_axes)
    cs = table[positions.long()]
    half = cs.shape[-1] // 2
    return cs[:, None, :half], cs[:, None, half:]


def apply_rotary(x: torch.Tensor, cos, sin, interleaved: bool = False) -> torch.Tensor:
    """Rotate the first ``2 * cos.shape[-1]`` channels of ``x`` [T, H, D]; the rest passes through (partial rotary)."""
    rot = 2 * cos.shape[-1]
    xr, rest = x[..., :rot].float(), x[..., rot:]
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    else:
        a, b = xr[..., : rot // 2], xr[..., rot // 2 :]
        out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    return torch.cat([out.to(x.dtype), rest], dim=-1)


def _rms(x, w, eps):
    y = x.float()
    y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


def dense_causal_attention(q, k, v, cu_seqlens, scale, allowed=None, q_offset: int = 0):
    """Per-sequence causal attention with explicit matrices: q [Tq, H, Dqk], k [T, H, Dqk], v [T, H, Dv] (query / key and
    value widths may differ), ``allowed`` [Tq, Lmax] bool optional extra mask per query row over the keys of ITS sequence
    (column j = j-th token of the sequence). The query rows are rows ``q_offset .. q_offset + Tq`` of the packed stream
    that ``k`` / ``v`` / ``cu_seqlens`` describe (all of it by default; a contiguous window under all-gather context
    parallelism). fp32 math; meant for correctness, not for long sequences."""
    Tq = q.shape[0]
    out = torch.zeros(Tq, q.shape[1], v.shape[-1], dtype=torch.float32, device=q.device)
    pieces = []
    cu = cu_seqlens.tolist()
    for a, b in zip(cu[:-1], cu[1:]):
        lo, hi = max(a, q_offset), min(b, q_offset + Tq)  # this sequence's rows inside the window
        if hi <= lo:
            continue
        qs = q[lo - q_offset : hi - q_offset].float().transpose(0, 1)
        ks, vs = (t[a:hi].float().transpose(0, 1) for t in (k, v))  # keys up to the window's last row of the sequence
        att = (qs @ ks.transpose(-1, -2)) * scale
        mask = torch.arange(a, hi, device=q.device)[None, :] <= torch.arange(lo, hi, device=q.device)[:, None]
        if allowed is not None:
            mask = mask & allowed[lo - q_offset : hi - q_offset, : hi - a]
        att = att.masked_fill(~mask, float("-inf"))
        pieces.append((lo - q_offset, hi - q_offset, (att.softmax(-1) @ vs).transpose(0, 1)))
    for a, b, o in pieces:
        out = out + F.pad(o, (0, 0, 0, 0, a, Tq - b))
    return out.to(q.dtype)


# ------------------------------------------------------------------------------------- all-gather context parallelism
ALLGATHER_CP = False


def set_allgather_cp(on: bool):
    """``--allgather-cp``: the packed stream of a micro-batch is cut into contiguous pieces, one per context-parallel rank;
    latent-attention layers compute their own rows against keys / values gathered from all ranks (every other layer is
    token-local). Same role as the all-gather mode of slime_plugins/models/glm5/glm5.py:850-852,921-928 in the reference."""
    global ALLGATHER_CP
    ALLGATHER_CP = bool(on)


def allgather_cp_active() -> bool:
    return ALLGATHER_CP and mpu.get_context_parallel_world_size() > 1


class _GatherFromContextParallel(torch.autograd.Function):
    """Rank-major concatenation of equally sized pieces along dim 0; the gradient of a rank's piece is the sum over ranks
    of the gradients of that slice."""

    @staticmethod
    def forward(ctx, x):
        group = mpu.get_context_parallel_group()
        n = mpu.get_context_parallel_world_size()
        out = torch.empty(n * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        torch.distributed.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        group = mpu.get_context_parallel_group()
        n, r = mpu.get_context_parallel_world_size(), mpu.get_context_parallel_rank()
        g = g.contiguous()
        rows = g.shape[0] // n
        if torch.distributed.get_backend(group) == "nccl":
            out = torch.empty(rows, *g.shape[1:], dtype=g.dtype, device=g.device)
            torch.distributed.reduce_scatter_tensor(out, g, group=group)
            return out
        torch.distributed.all_reduce(g, group=group)
        return g[r * rows : (r + 1) * rows].clone()


def gather_from_context_parallel(x):
    return _GatherFromContextParallel.apply(x)


# -------------------------------------------------------------------------------------------- attention variants
class GeneralSelfAttention(nn.Module):
    """Tensor-parallel GQA attention for the variants listed in the module docstring. Parameter names and shard layouts
    are those of ``gpt.SelfAttention`` (rows of the fused projection: [q heads | gate heads if gated | k heads | v heads]
    of the local shard), plus ``softmax_offset`` [local heads] when the model has sinks."""

    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
        super().__init__()
        self.cfg, self.sp = cfg, sequence_parallel
        tps = mpu.get_tensor_model_parallel_world_size()
        assert cfg.num_attention_heads % tps == 0 and cfg.num_query_groups % tps == 0, "heads must divide by tp"
        assert mpu.get_context_parallel_world_size() == 1, "the composed attention path has no context-parallel form"
        self.hq, self.hkv, self.d = cfg.num_attention_heads // tps, cfg.num_query_groups // tps, cfg.head_dim
        self.gated = cfg.attention_output_gate
        self.rot = int(self.d * cfg.rotary_percent) // 2 * 2
        h = cfg.hidden_size
        gen = tp.get_rng_tracker().states.get("tp")
        out_std = cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers)
        rows = ((2 if self.gated else 1) * self.hq + 2 * self.hkv) * self.d
        self.linear_qkv = nn.Module()
        self.linear_qkv.weight = tp.set_tp_attrs(_param((rows, h), dtype, device, cfg.init_method_std, generator=gen), True, 0, 1, "column")
        self.linear_qkv.layer_norm_weight = tp.set_tp_attrs(_param((h,), dtype, device, ones=True), False)
        self.linear_qkv.layer_norm_weight.sequence_parallel = sequence_parallel
        self.linear_qkv.bias = tp.set_tp_attrs(_param((rows,), dtype, device, 0.0), True, 0, 1, "column") if cfg.add_qkv_bias else None
        self.q_layernorm = self.k_layernorm = None
        if cfg.qk_layernorm or cfg.qk_layernorm_full:
            # per head: one [d] vector shared by the heads; over all heads: one vector per projection, sharded like it
            self.q_layernorm, self.k_layernorm = nn.Module(), nn.Module()
            full = cfg.qk_layernorm_full
            qn, kn = (self.hq * self.d, self.hkv * self.d) if full else (self.d, self.d)
            self.q_layernorm.weight = tp.set_tp_attrs(_param((qn,), dtype, device, ones=True), full, 0, 1)
            self.k_layernorm.weight = tp.set_tp_attrs(_param((kn,), dtype, device, ones=True), full, 0, 1)
            if not full:
                self.q_layernorm.weight.needs_tp_grad_reduce = True
                self.k_layernorm.weight.needs_tp_grad_reduce = True
        if cfg.softmax_sinks:
            self.softmax_offset = tp.set_tp_attrs(_param((self.hq,), torch.float32, device, 0.0), True, 0, 1)
        else:
            self.softmax_offset = None
        self.linear_proj = nn.Module()
        self.linear_proj.weight = tp.set_tp_attrs(_param((h, self.hq * self.d), dtype, device, out_std, generator=gen), True, 1, 1, "row")
        self._rope = None

    def _table(self, device, need: int):
        if self._rope is None or self._rope.shape[0] < need or self._rope.device != torch.device(device):
            self._rope = ops.rope_table(self.cfg, max(need, 4096), self.rot, device)
        return self._rope

    def _full_norm(self, t, w, eps):
        """RMSNorm over all heads of the model: the sum of squares crosses tensor-parallel ranks."""
        T = t.shape[0]
        flat = t.reshape(T, -1).float()
        ss = flat.pow(2).sum(-1, keepdim=True)
        n = flat.shape[-1]
        if mpu.get_tensor_model_parallel_world_size() > 1:
            # summed over ranks in the forward pass AND in the backward pass: every rank's output depends on the total
            ss = tp.reduce_from_tensor_model_parallel_region(tp.copy_to_tensor_model_parallel_region(ss))
            n = n * mpu.get_tensor_model_parallel_world_size()
        return (flat * torch.rsqrt(ss / n + eps) * w.float()).to(t.dtype).view_as(t)

    def forward(self, x, residual, rope_table, packed):
        cfg, d, hq, hkv = self.cfg, self.d, self.hq, self.hkv
        normed, residual = ops.rmsnorm(x, self.linear_qkv.layer_norm_weight, cfg.norm_epsilon, residual)
        inp = tp.gather_from_sequence_parallel_region(normed) if self.sp else tp.copy_to_tensor_model_parallel_region(normed)
        qkv = ops.linear(inp, self.linear_qkv.weight, self.linear_qkv.bias)
        T = qkv.shape[0]
        sizes = [hq * d] + ([hq * d] if self.gated else []) + [hkv * d, hkv * d]
        parts = qkv.split(sizes, dim=-1)
        q, gate = parts[0].view(T, hq, d), (parts[1] if self.gated else None)
        k, v = parts[-2].view(T, hkv, d), parts[-1].view(T, hkv, d)
        if self.q_layernorm is not None:
            if cfg.qk_layernorm_full:
                q = self._full_norm(q, self.q_layernorm.weight, cfg.norm_epsilon)
                k = self._full_norm(k, self.k_layernorm.weight, cfg.norm_epsilon)
            else:
                q, k = _rms(q, self.q_layernorm.weight, cfg.norm_epsilon), _rms(k, self.k_layernorm.weight, cfg.norm_epsilon)
        if self.rot > 0:
            streams = getattr(packed, "mrope_positions", None) if cfg.mrope_section else None
            if streams is not None:  # vision inputs: three position streams, one per group of frequency bands
                from slime_b200.models.vision import mrope_band_axes

                axes = mrope_band_axes(cfg.mrope_section, self.rot // 2, cfg.mrope_interleaved, q.device)
                cos, sin = rotary_cos_sin(self._table(q.device, int(packed.max_seqlen) + 1), streams, axes)
            else:
                cos, sin = rotary_cos_sin(self._table(q.device, int(packed.max_seqlen) + 1), packed.position_ids.reshape(-1))
            q, k = apply_rotary(q, cos, sin, cfg.rotary_interleaved), apply_rotary(k, cos, sin, cfg.rotary_interleaved)
        ctx = ops.varlen_attention(q.contiguous(), k.contiguous(), v.contiguous(), packed.cu_seqlens, packed.max_seqlen,
                                   sinks=self.softmax_offset).reshape(T, hq * d)  # fmt: skip
        if gate is not None:
            ctx = ctx * torch.sigmoid(gate.float()).to(ctx.dtype)
        out = ops.linear(ctx, self.linear_proj.weight)
        out = tp.reduce_scatter_to_sequence_parallel_region(out) if self.sp else tp.reduce_from_tensor_model_parallel_region(out)
        return out, residual


# ------------------------------------------------------------------------------------------------ gated delta net
def _l2norm(x, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def gated_delta_rule_recurrent(q, k, v, g, beta, cu_seqlens):
    """Definition, one token at a time. q / k [T, H, Dk], v [T, H, Dv], g [T, H] (log decay, <= 0), beta [T, H];
    the state ``S`` [H, Dk, Dv] starts at zero for every sequence:

        S <- exp(g_t) S;  delta = beta_t (v_t - S^T k_t);  S <- S + k_t delta^T;  o_t = S^T q_t

    with q and k L2-normalised and q scaled by ``Dk ** -0.5``."""
    q, k = _l2norm(q.float()) * q.shape[-1] ** -0.5, _l2norm(k.float())
    v, g, beta = v.float(), g.float(), beta.float()
    out = torch.zeros_like(v)
    cu = cu_seqlens.tolist()
    for a, b in zip(cu[:-1], cu[1:]):
        S = torch.zeros(q.shape[1], q.shape[2], v.shape[2], dtype=torch.float32, device=q.device)
        for t in range(a, b):
            S = S * g[t].exp()[:, None, None]
            delta = (v[t] - torch.einsum("hkv,hk->hv", S, k[t])) * beta[t][:, None]
            S = S + k[t][:, :, None] * delta[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def gated_delta_rule_chunked(q, k, v, g, beta, cu_seqlens, chunk: int = 64, initial_states=None, return_final_states: bool = False):
    """The same function, ``chunk`` tokens at a time. Inside a chunk with cumulative log decay ``G`` and incoming state
    ``S0`` the updates ``delta`` solve the unit lower-triangular system

        (I + A) delta = beta * (V - exp(G) K S0),   A[i, j] = beta_i exp(G_i - G_j) <k_i, k_j>  (j < i),

    then ``O = exp(G) Q S0 + (tril(exp(G_i - G_j)) * Q K^T) delta`` and ``S <- exp(G_C) S0 + (exp(G_C - G) K)^T delta``.
    Everything is matmuls and one triangular solve per chunk, all differentiable. ``initial_states``: one ``[H, Dk, Dv]``
    tensor (or None) per sequence to start from; ``return_final_states`` also returns the state after each sequence's last
    token (what a decode step continues from)."""
    Dk = q.shape[-1]
    qf, kf = _l2norm(q.float()) * Dk**-0.5, _l2norm(k.float())
    vf, gf, bf = v.float(), g.float(), beta.float()
    outs, finals = [], []
    cu = cu_seqlens.tolist()
    for si, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        n = b - a
        if n <= 0:
            finals.append(None if initial_states is None else initial_states[si])
            continue
        pad = (-n) % chunk
        # [H, n_chunks, C, *]
        shape = lambda t: F.pad(t[a:b], (0, 0) * (t.dim() - 1) + (0, pad)).transpose(0, 1).reshape(t.shape[1], -1, chunk, *t.shape[2:])  # noqa: E731
        Q, K, V, Gc, B = shape(qf), shape(kf), shape(vf), shape(gf), shape(bf)
        G = Gc.cumsum(-1)  # padded tokens have g = 0, beta = 0: they change nothing
        diff = G[..., :, None] - G[..., None, :]
        tri = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
        decay = torch.where(tri, diff, torch.full_like(diff, float("-inf"))).exp()  # [H, N, C, C], zero above the diagonal
        KK = K @ K.transpose(-1, -2)
        A = (B[..., :, None] * decay * KK).tril(-1)
        eye = torch.eye(chunk, device=q.device)
        QK = (Q @ K.transpose(-1, -2)) * decay
        eG = G.exp()[..., None]
        S = torch.zeros(q.shape[1], Dk, v.shape[-1], dtype=torch.float32, device=q.device)
        if initial_states is not None and initial_states[si] is not None:
            S = initial_states[si].float()
        seq_out = []
        for c in range(Q.shape[1]):
            rhs = B[:, c, :, None] * (V[:, c] - eG[:, c] * (K[:, c] @ S))
            delta = torch.linalg.solve_triangular(eye + A[:, c], rhs, upper=False, unitriangular=True)
            seq_out.append(eG[:, c] * (Q[:, c] @ S) + QK[:, c] @ delta)
            last = G[:, c, -1]
            S = last.exp()[:, None, None] * S + ((last[:, None] - G[:, c]).exp()[..., None] * K[:, c]).transpose(-1, -2) @ delta
        o = torch.stack(seq_out, 1).reshape(q.shape[1], -1, v.shape[-1])[:, :n].transpose(0, 1)
        outs.append(o)
        finals.append(S)  # padded tokens (g = 0, beta = 0) left it untouched
    out = torch.cat(outs) if outs else vf[:0]
    return (out, finals) if return_final_states else out


def gated_delta_rule_step(q, k, v, g, beta, S):
    """One token per row: q / k [B, H, Dk], v [B, H, Dv], g / beta [B, H], state ``S`` [B, H, Dk, Dv] (updated in place).
    Returns the outputs [B, H, Dv]."""
    q, k = _l2norm(q.float()) * q.shape[-1] ** -0.5, _l2norm(k.float())
    S.mul_(g.float().exp()[:, :, None, None])
    delta = (v.float() - torch.einsum("bhkv,bhk->bhv", S, k)) * beta.float()[:, :, None]
    S.add_(k[:, :, :, None] * delta[:, :, None, :])
    return torch.einsum("bhkv,bhk->bhv", S, q)


def causal_short_conv(x, weight, positions, activation=True, history=None, cu_seqlens=None):
    """Depthwise causal convolution over time with zero history at every sequence start. x [T, C], weight [C, K]
    (tap K-1 multiplies the current token), ``positions`` [T] the index of each token inside its sequence (of THIS call:
    a continued sequence starts at 0 again and brings ``history``). ``history``: per sequence of ``cu_seqlens`` a
    ``[K-1, C]`` tensor of the inputs that preceded this call (or None), oldest first."""
    K = weight.shape[1]
    acc = x.float() * weight[:, K - 1].float()
    pos = positions.reshape(-1)
    for s in range(1, K):
        shifted = F.pad(x.float(), (0, 0, s, 0))[: x.shape[0]]
        acc = acc + torch.where((pos >= s)[:, None], shifted, torch.zeros_like(shifted)) * weight[:, K - 1 - s].float()
    if history is not None:
        add = torch.zeros_like(acc)
        for si, (a, b) in enumerate(zip(cu_seqlens.tolist()[:-1], cu_seqlens.tolist()[1:])):
            h = history[si]
            if h is None or b <= a:
                continue
            hf = h.float()
            for t in range(min(K - 1, b - a)):  # token t of the call still sees K-1-t history rows
                for s in range(t + 1, K):
                    add[a + t] += hf[K - 1 - (s - t)] * weight[:, K - 1 - s].float()
        acc = acc + add
    return (F.silu(acc) if activation else acc).to(x.dtype)


def short_conv_step(x, weight, state):
    """One token per row: x [B, C], ``state`` [B, K-1, C] the previous inputs (oldest first, updated in place)."""
    window = torch.cat([state.float(), x.float()[:, None, :]], dim=1)  # [B, K, C]
    y = (window * weight.float().t()[None]).sum(1)
    state.copy_(window[:, 1:].to(state.dtype))
    return F.silu(y).to(x.dtype)


class GatedDeltaNet(nn.Module):
    """Qwen3-Next / Qwen3.5 linear-attention layer. Parameters (replicated over tensor-parallel ranks):
    ``in_proj_qkvz`` [2 Kdim + 2 Vdim, H] (rows grouped per key head: q, k, then that head's value and gate heads) and
    ``in_proj_ba`` [2 Hv, H] for Qwen3-Next, or ``in_proj_qkv`` [2 Kdim + Vdim, H], ``in_proj_z`` [Vdim, H],
    ``in_proj_b`` / ``in_proj_a`` [Hv, H] for Qwen3.5; ``conv1d.weight`` [2 Kdim + Vdim, K], ``A_log`` / ``dt_bias`` [Hv], ``norm.weight`` [Dv],
    ``out_proj`` [H, Vdim], ``input_layernorm.weight`` [H]."""

    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
        super().__init__()
        self.cfg, self.sp = cfg, sequence_parallel
        self.hk, self.hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        assert self.hv % self.hk == 0
        self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
        h, std = cfg.hidden_size, cfg.init_method_std
        self.input_layernorm = nn.Module()
        self.input_layernorm.weight = _replicated((h,), dtype, device, ones=True)
        self.input_layernorm.weight.sequence_parallel = sequence_parallel
        self.conv1d, self.norm, self.out_proj = (nn.Module() for _ in range(3))
        # Qwen3-Next fuses the input projections (rows grouped per key head); Qwen3.5 keeps four plain ones
        self.fused_in_proj = "qwen3next" in (cfg.model_arch or "").lower().replace("_", "")
        if self.fused_in_proj:
            self.in_proj_qkvz, self.in_proj_ba = nn.Module(), nn.Module()
            self.in_proj_qkvz.weight = _replicated((2 * self.key_dim + 2 * self.value_dim, h), dtype, device, std)
            self.in_proj_ba.weight = _replicated((2 * self.hv, h), dtype, device, std)
        else:
            self.in_proj_qkv, self.in_proj_z, self.in_proj_b, self.in_proj_a = (nn.Module() for _ in range(4))
            self.in_proj_qkv.weight = _replicated((2 * self.key_dim + self.value_dim, h), dtype, device, std)
            self.in_proj_z.weight = _replicated((self.value_dim, h), dtype, device, std)
            self.in_proj_b.weight = _replicated((self.hv, h), dtype, device, std)
            self.in_proj_a.weight = _replicated((self.hv, h), dtype, device, std)
        self.conv1d.weight = _replicated((2 * self.key_dim + self.value_dim, cfg.linear_conv_kernel_dim), dtype, device, 0.2)
        self.dt_bias = _replicated((self.hv,), torch.float32, device, ones=True)
        gen = tp.get_rng_tracker().states.get("default")
        a = torch.empty(self.hv, dtype=torch.float32, device=device).uniform_(1e-3, 16.0, generator=gen)
        self.A_log = tp.set_tp_attrs(nn.Parameter(a.log()), False)
        self.norm.weight = _replicated((self.dv,), dtype, device, ones=True)
        self.out_proj.weight = _replicated((h, self.value_dim), dtype, device, std / math.sqrt(2.0 * cfg.num_layers))

    def _split(self, qkvz, ba):
        """Undo the per-key-head grouping of the fused projections."""
        T, r = qkvz.shape[0], self.hv // self.hk
        qkvz = qkvz.view(T, self.hk, 2 * self.dk + 2 * r * self.dv)
        q, k, v, z = qkvz.split([self.dk, self.dk, r * self.dv, r * self.dv], dim=-1)
        b, a = ba.view(T, self.hk, 2 * r).split([r, r], dim=-1)
        return (q, k, v.reshape(T, self.hv, self.dv), z.reshape(T, self.hv, self.dv), b.reshape(T, self.hv), a.reshape(T, self.hv))

    def forward(self, x, residual, rope_table, packed):
        cfg = self.cfg
        normed, residual = ops.rmsnorm(x, self.input_layernorm.weight, cfg.norm_epsilon, residual)
        inp = tp.gather_from_sequence_parallel_region_no_reduce(normed) if self.sp else normed
        T = inp.shape[0]
        if self.fused_in_proj:
            q, k, v, z, b, a = self._split(F.linear(inp, self.in_proj_qkvz.weight), F.linear(inp, self.in_proj_ba.weight))
            mixed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=-1)
        else:
            mixed = F.linear(inp, self.in_proj_qkv.weight)
            z = F.linear(inp, self.in_proj_z.weight).view(T, self.hv, self.dv)
            b, a = F.linear(inp, self.in_proj_b.weight), F.linear(inp, self.in_proj_a.weight)
        mixed = causal_short_conv(mixed, self.conv1d.weight, packed.position_ids)
        q, k, v = mixed.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q, k, v = q.view(T, self.hk, self.dk), k.view(T, self.hk, self.dk), v.view(T, self.hv, self.dv)
        beta = torch.sigmoid(b.float())
        g = -self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias.float())
        r = self.hv // self.hk
        if r > 1:
            q, k = q.repeat_interleave(r, dim=1), k.repeat_interleave(r, dim=1)
        o = gated_delta_rule_chunked(q, k, v, g, beta, packed.cu_seqlens)  # the alignment padding is a sequence of its own
        if o.shape[0] < T:  # rows past the last sequence (alignment padding of the packed stream)
            o = F.pad(o, (0, 0, 0, 0, 0, T - o.shape[0]))
        o = _rms(o, self.norm.weight, cfg.norm_epsilon).float() * F.silu(z.float())
        out = F.linear(o.to(inp.dtype).reshape(T, self.value_dim), self.out_proj.weight)
        return (tp.scatter_to_sequence_parallel_region(out) if self.sp else out), residual


# ---------------------------------------------------------------------------------------------- latent attention
def mla_rope_table(cfg: ModelConfig, need: int, device) -> torch.Tensor:
    """Rotary table of the latent-attention rotary part (YaRN frequencies when the model asks for them)."""
    if cfg.rotary_scaling_type == "yarn" and cfg.rotary_scaling_factor > 1:
        from slime_b200.ops import reference

        return reference.rope_cos_sin_yarn(need, cfg.qk_pos_emb_head_dim, cfg.rotary_base, cfg.rotary_scaling_factor,
                                           cfg.rotary_original_max_position, cfg.yarn_beta_fast, cfg.yarn_beta_slow, cfg.mscale,
                                           cfg.mscale_all_dim, device=device)  # fmt: skip
    return ops.rope_cos_sin(need, cfg.qk_pos_emb_head_dim, cfg.rotary_base, device=device, scaling_factor=cfg.rotary_scaling_factor)


def mla_softmax_scale(cfg: ModelConfig) -> float:
    scale = (cfg.qk_head_dim + cfg.qk_pos_emb_head_dim) ** -0.5
    if cfg.rotary_scaling_type == "yarn" and cfg.rotary_scaling_factor > 1 and cfg.mscale_all_dim:
        from slime_b200.ops.reference import yarn_mscale

        scale *= yarn_mscale(cfg.rotary_scaling_factor, cfg.mscale_all_dim) ** 2  # YaRN's attention temperature
    return scale


class MLASelfAttention(nn.Module):
    """Multi-head latent attention. Parameters (replicated over tensor-parallel ranks), Megatron names:
    ``linear_q_down_proj`` [q_lora, H] + ``q_layernorm`` + ``linear_q_up_proj`` [Hq (Dn + Dr), q_lora] (or ``linear_q_proj``
    when the model has no query compression), ``linear_kv_down_proj`` [kv_lora + Dr, H], ``kv_layernorm``,
    ``linear_kv_up_proj`` [Hq (Dn + Dv), kv_lora], ``linear_proj`` [H, Hq Dv], ``input_layernorm``."""

    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
        super().__init__()
        self.cfg, self.sp, self.layer_number = cfg, sequence_parallel, layer_number
        self.hq, self.dn, self.dr, self.dv = cfg.num_attention_heads, cfg.qk_head_dim, cfg.qk_pos_emb_head_dim, cfg.v_head_dim
        h, std = cfg.hidden_size, cfg.init_method_std
        mk = lambda *shape, **kw: _replicated(shape, dtype, device, **kw)  # noqa: E731
        self.input_layernorm = nn.Module()
        self.input_layernorm.weight = mk(h, ones=True)
        self.input_layernorm.weight.sequence_parallel = sequence_parallel
        names = ["linear_q_down_proj", "q_layernorm", "linear_q_up_proj", "linear_q_proj", "linear_kv_down_proj", "kv_layernorm",
                 "linear_kv_up_proj", "linear_proj"]  # fmt: skip
        for n in names:
            setattr(self, n, nn.Module())
        if cfg.q_lora_rank:
            self.linear_q_down_proj.weight = mk(cfg.q_lora_rank, h, std=std)
            self.q_layernorm.weight = mk(cfg.q_lora_rank, ones=True)
            self.linear_q_up_proj.weight = mk(self.hq * (self.dn + self.dr), cfg.q_lora_rank, std=std)
            del self.linear_q_proj
        else:
            self.linear_q_proj.weight = mk(self.hq * (self.dn + self.dr), h, std=std)
            del self.linear_q_down_proj, self.q_layernorm, self.linear_q_up_proj
        self.linear_kv_down_proj.weight = mk(cfg.kv_lora_rank + self.dr, h, std=std)
        self.kv_layernorm.weight = mk(cfg.kv_lora_rank, ones=True)
        self.linear_kv_up_proj.weight = mk(self.hq * (self.dn + self.dv), cfg.kv_lora_rank, std=std)
        self.linear_proj.weight = mk(h, self.hq * self.dv, std=std / math.sqrt(2.0 * cfg.num_layers))
        self.scale = mla_softmax_scale(cfg)
        self._rope = None

    def _table(self, device, need):
        if self._rope is None or self._rope.shape[0] < need or self._rope.device != torch.device(device):
            self._rope = mla_rope_table(self.cfg, max(need, 4096), device)
        return self._rope

    def _qkv(self, inp, packed):
        cfg, T = self.cfg, inp.shape[0]
        if cfg.q_lora_rank:
            q_latent = _rms(F.linear(inp, self.linear_q_down_proj.weight), self.q_layernorm.weight, cfg.norm_epsilon)
            q = F.linear(q_latent, self.linear_q_up_proj.weight)
        else:
            q_latent, q = inp, F.linear(inp, self.linear_q_proj.weight)
        q = q.view(T, self.hq, self.dn + self.dr)
        kv_down = F.linear(inp, self.linear_kv_down_proj.weight)
        c_kv, k_pe = kv_down.split([cfg.kv_lora_rank, self.dr], dim=-1)
        kv = F.linear(_rms(c_kv, self.kv_layernorm.weight, cfg.norm_epsilon), self.linear_kv_up_proj.weight)
        k_nope, v = kv.view(T, self.hq, self.dn + self.dv).split([self.dn, self.dv], dim=-1)
        cos, sin = rotary_cos_sin(self._table(inp.device, int(packed.max_seqlen) + 1), packed.position_ids.reshape(-1))
        q_pe = apply_rotary(q[..., self.dn :], cos, sin, cfg.rotary_interleaved)
        k_pe = apply_rotary(k_pe.view(T, 1, self.dr), cos, sin, cfg.rotary_interleaved)
        q = torch.cat([q[..., : self.dn], q_pe], dim=-1)
        k = torch.cat([k_nope, k_pe.expand(T, self.hq, self.dr)], dim=-1)
        return q, k, v, q_latent, (cos, sin)

    def _allowed(self, inp, q_latent, rope, packed, q_offset=0):
        return None

    def forward(self, x, residual, rope_table, packed):
        cfg = self.cfg
        normed, residual = ops.rmsnorm(x, self.input_layernorm.weight, cfg.norm_epsilon, residual)
        inp = tp.gather_from_sequence_parallel_region_no_reduce(normed) if self.sp else normed
        q, k, v, q_latent, rope = self._qkv(inp, packed)
        q_offset = 0
        if allgather_cp_active():  # this rank's rows against every rank's keys and values
            q_offset = mpu.get_context_parallel_rank() * inp.shape[0]
            k, v = gather_from_context_parallel(k), gather_from_context_parallel(v)
        elif mpu.get_context_parallel_world_size() > 1:
            raise NotImplementedError("latent attention under context parallelism needs --allgather-cp")
        ctx = dense_causal_attention(q, k, v, packed.cu_seqlens, self.scale, self._allowed(inp, q_latent, rope, packed, q_offset), q_offset)
        out = F.linear(ctx.reshape(inp.shape[0], -1), self.linear_proj.weight)
        return (tp.scatter_to_sequence_parallel_region(out) if self.sp else out), residual


def indexer_logits(q_idx, k_idx, weights):
    """Lightning indexer: ``logits[t, s] = sum_h weights[t, h] * relu(<q_idx[t, h], k_idx[s]>)``; q_idx [T, Hi, Di],
    k_idx [S, Di], weights [T, Hi] -> [T, S] fp32."""
    return torch.einsum("thd,sd->ths", q_idx.float(), k_idx.float()).relu_().mul_(weights.float()[:, :, None]).sum(1)


def select_topk_keys(logits_fn, cu_seqlens, T: int, topk: int, device, q_offset: int = 0) -> torch.Tensor:
    """Per query row the ``topk`` best-scoring keys among the causally visible ones of its own sequence, as a boolean
    matrix [T, Lmax] over in-sequence key positions (rows with fewer visible keys keep all of them). The ``T`` query rows
    are rows ``q_offset .. q_offset + T`` of the packed stream. ``logits_fn(q0, q1, k0, k1)`` returns the score block of
    query rows ``q0 .. q1`` (counted inside the window) against keys ``k0 .. k1`` (counted in the whole stream)."""
    cu = cu_seqlens.tolist()
    lmax = max((b - a for a, b in zip(cu[:-1], cu[1:])), default=0)
    allowed = torch.zeros(T, lmax, dtype=torch.bool, device=device)
    for a, b in zip(cu[:-1], cu[1:]):
        lo, hi = max(a, q_offset), min(b, q_offset + T)
        if hi <= lo:
            continue
        n = hi - a  # keys the window's last row of this sequence can see
        causal = torch.arange(a, hi, device=device)[None, :] <= torch.arange(lo, hi, device=device)[:, None]
        if n <= topk:
            allowed[lo - q_offset : hi - q_offset, :n] = causal
            continue
        scores = logits_fn(lo - q_offset, hi - q_offset, a, hi).masked_fill(~causal, float("-inf"))
        idx = scores.topk(topk, dim=-1).indices
        pick = torch.zeros(hi - lo, n, dtype=torch.bool, device=device).scatter_(1, idx, True)
        allowed[lo - q_offset : hi - q_offset, :n] = pick & causal
    return allowed


class DSASelfAttention(MLASelfAttention):
    """Latent attention restricted to the keys a lightning indexer picks. Extra parameters: ``wq_b`` [Hi Di, q_lora],
    ``wk`` [Di, H], ``k_norm`` (LayerNorm weight and bias [Di]), ``weights_proj`` [Hi, H]. The first ``Dr`` channels of
    the indexer's queries and key are rotated like the attention's rotary part. A layer for which
    ``max(layer - index_skip_topk_offset, 0) % index_topk_freq != 0`` (1-based layer numbers) reuses the choice of the
    nearest earlier layer that computed one; the choice travels on the micro-batch's ``packed`` object, so it is
    per micro-batch and survives activation recomputation."""

    _HOLDER = "_dsa_topk"

    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
        super().__init__(cfg, layer_number, dtype, device, sequence_parallel)
        assert cfg.q_lora_rank, "the indexer reads the compressed query"
        self.hi, self.di = cfg.index_n_heads, cfg.index_head_dim
        mk = lambda *shape, **kw: _replicated(shape, dtype, device, **kw)  # noqa: E731
        one_based = layer_number + 1
        self.skip = (max(one_based - cfg.index_skip_topk_offset, 0) % cfg.index_topk_freq) != 0
        src = one_based
        while (max(src - cfg.index_skip_topk_offset, 0) % cfg.index_topk_freq) != 0:
            src -= 1
        self.source_layer = src - 1
        if not self.skip:
            self.wq_b, self.wk, self.k_norm, self.weights_proj = (nn.Module() for _ in range(4))
            self.wq_b.weight = mk(self.hi * self.di, cfg.q_lora_rank, std=cfg.init_method_std)
            self.wk.weight = mk(self.di, cfg.hidden_size, std=cfg.init_method_std)
            self.k_norm.weight, self.k_norm.bias = mk(self.di, ones=True), mk(self.di, std=0.0)
            self.weights_proj.weight = mk(self.hi, cfg.hidden_size, std=cfg.init_method_std)

    def _allowed(self, inp, q_latent, rope, packed, q_offset=0):
        holder = getattr(packed, self._HOLDER, None)
        if holder is None:
            holder = {}
            setattr(packed, self._HOLDER, holder)
        if self.skip:
            if self.source_layer not in holder:
                raise AssertionError(f"layer {self.layer_number} reuses the key choice of layer {self.source_layer}, which did not "
                                     "run before it in this pipeline stage: every stage must start on a computing layer")  # fmt: skip
            return holder[self.source_layer]
        cfg, T = self.cfg, inp.shape[0]
        cos, sin = rope
        with torch.no_grad():  # the choice is discrete: no gradient reaches the indexer through it
            il = cfg.rotary_interleaved if cfg.index_rotary_interleaved is None else cfg.index_rotary_interleaved
            q_idx = apply_rotary(F.linear(q_latent, self.wq_b.weight).view(T, self.hi, self.di), cos, sin, il)
            k_idx = F.layer_norm(F.linear(inp, self.wk.weight).float(), (self.di,), self.k_norm.weight.float(), self.k_norm.bias.float())
            k_idx = apply_rotary(k_idx.view(T, 1, self.di), cos, sin, il).view(T, self.di)
            w = F.linear(inp, self.weights_proj.weight).float() * (self.hi**-0.5) * (self.di**-0.5)
            if allgather_cp_active():  # the indexer's keys of every rank (no gradient flows through the choice)
                k_idx = gather_from_context_parallel(k_idx)
            allowed = select_topk_keys(lambda q0, q1, k0, k1: indexer_logits(q_idx[q0:q1], k_idx[k0:k1], w[q0:q1]),
                                       packed.cu_seqlens, T, cfg.index_topk, inp.device, q_offset)  # fmt: skip
        holder[self.layer_number] = allowed
        return allowed


class HuggingfaceAttention(nn.Module):
    """Run a Hugging Face style token-mixing module as a layer of this model: the pre-norm, the sequence-parallel gather
    before and the split after are done here, ``hf_forward`` sees ``[1, T, H]`` hidden states of the whole packed stream
    plus the packing metadata. Its parameters are replicated over tensor-parallel ranks. Subclass and override
    ``hf_forward``, or pass ``module`` whose ``forward(hidden_states, position_ids=..., cu_seqlens=...)`` returns the
    mixed hidden states (a tuple's first element is taken). Same role as slime_plugins/models/hf_attention.py:63-173 in
    the reference."""

    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool, module: nn.Module | None = None):
        super().__init__()
        self.cfg, self.sp, self.layer_number = cfg, sequence_parallel, layer_number
        self.input_layernorm = nn.Module()
        self.input_layernorm.weight = _replicated((cfg.hidden_size,), dtype, device, ones=True)
        self.input_layernorm.weight.sequence_parallel = sequence_parallel
        self.hf_module = module
        if module is not None:
            module.to(device=device, dtype=dtype)
            for p in module.parameters():
                tp.set_tp_attrs(p, False)

    def hf_forward(self, hidden_states, packed):
        out = self.hf_module(hidden_states, position_ids=packed.position_ids.reshape(1, -1).long(), cu_seqlens=packed.cu_seqlens)
        return out[0] if isinstance(out, tuple) else out

    def forward(self, x, residual, rope_table, packed):
        normed, residual = ops.rmsnorm(x, self.input_layernorm.weight, self.cfg.norm_epsilon, residual)
        inp = tp.gather_from_sequence_parallel_region_no_reduce(normed) if self.sp else normed
        out = self.hf_forward(inp.unsqueeze(0), packed).squeeze(0)
        return (tp.scatter_to_sequence_parallel_region(out) if self.sp else out), residual


_CUSTOM_BUILDER = None


def set_custom_builder(fn) -> None:
    """``fn(cfg, layer_number, dtype, device, sequence_parallel) -> module | None`` is asked first for every layer's
    mixer (``--spec <module> <function>`` installs it); None falls through to the built-in choice."""
    global _CUSTOM_BUILDER
    _CUSTOM_BUILDER = fn


def build_mixer(cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
    if _CUSTOM_BUILDER is not None:
        custom = _CUSTOM_BUILDER(cfg, layer_number, dtype, device, sequence_parallel)
        if custom is not None:
            return custom
    kind = cfg.mixer(layer_number)
    if kind == "attention":
        from slime_b200.models.gpt import SelfAttention

        return SelfAttention(cfg, layer_number, dtype, device, sequence_parallel)
    cls = {"general_attention": GeneralSelfAttention, "gated_delta_net": GatedDeltaNet, "mla": MLASelfAttention,
           "dsa": DSASelfAttention}[kind]  # fmt: skip
    return cls(cfg, layer_number, dtype, device, sequence_parallel)
