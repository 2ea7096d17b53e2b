"""Kernel micro-benchmarks: ``python -m slime_b200.ops.microbench {gemm,decode,norm} [options]``.

Every number is a CUDA-event time on the launching stream after warm-up, median over ``--iters`` timed
repetitions with an L2 flush (a 256 MiB memset) between them. One JSON object per line on stdout.

    gemm    tcgen05 GEMM vs cuBLAS (torch.matmul) for forward / dgrad / wgrad layouts
    decode  each kernel of one rollout decode step at a given batch and context length
    norm    RMSNorm forward/backward bandwidth
    attn    flash attention forward / backward (own kernels; the flash-attn library on the same tensors for comparison)
    fused_emul  the peer-memory kernels (DP reduce / Adam, TP all-reduce + norm) with all ranks emulated on one GPU

``--small`` shrinks the working set to a case suitable for a profiler capture (a few launches, < 1 GB).
"""

from __future__ import annotations

import argparse
import json
import math
import os

import torch

from slime_b200 import ops
from slime_b200.ops import _lib

_FLUSH = None


def _flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_ms(fn, iters: int = 20, warmup: int = 3, reps: int = 1, flush: bool = True) -> float:
    """Median device time of ``reps`` back-to-back calls of ``fn`` (divided by ``reps``)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            _flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) / reps)
    times.sort()
    return times[len(times) // 2]


def _emit(**kw):
    print(json.dumps(kw), flush=True)


# ------------------------------------------------------------------------------------ gemm
GEMM_SHAPES = [(16384, 1152, 896), (16384, 896, 896), (16384, 9728, 896), (16384, 896, 4864), (8192, 8192, 8192),
               (4096, 151936, 896), (256, 1152, 896), (256, 9728, 896), (256, 151936, 896)]  # fmt: skip
GRAD_SHAPES = [(16384, 9728, 896), (16384, 896, 4864), (16384, 1152, 896)]  # (tokens, out features, in features)


def bench_gemm(a):
    shapes, grads = (GEMM_SHAPES, GRAD_SHAPES) if not a.small else ([(4096, 4096, 4096)], [])
    if a.shape:
        shapes, grads = [tuple(a.shape)], []
    bf = torch.bfloat16
    for M, N, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=bf)
        w = torch.randn(N, K, device="cuda", dtype=bf)
        fl = 2.0 * M * N * K
        for bn in (128, 256):
            t = time_ms(lambda: ops.gemm(x, w, bn=bn), a.iters)
            _emit(kind="nt", M=M, N=N, K=K, bn=bn, ms=t, tflops=fl / t / 1e9)
        if not a.no_cublas:
            t = time_ms(lambda: x @ w.t(), a.iters)
            _emit(kind="cublas_nt", M=M, N=N, K=K, ms=t, tflops=fl / t / 1e9)
    for T, O, I in grads:
        dy = torch.randn(T, O, device="cuda", dtype=bf)
        w = torch.randn(O, I, device="cuda", dtype=bf)
        x = torch.randn(T, I, device="cuda", dtype=bf)
        acc = torch.zeros(O, I, device="cuda", dtype=torch.float32)
        fl = 2.0 * T * O * I
        for name, fn, ref in (
            ("dgrad", lambda: ops.gemm(dy, w, b_mn=True), lambda: dy @ w),
            ("wgrad", lambda: ops.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32), lambda: dy.t() @ x),
            ("wgrad_accumulate", lambda: ops.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True), None),
        ):
            t = time_ms(fn, a.iters)
            _emit(kind=name, T=T, O=O, I=I, ms=t, tflops=fl / t / 1e9)
            if ref is not None and not a.no_cublas:
                t = time_ms(ref, a.iters)
                _emit(kind="cublas_" + name, T=T, O=O, I=I, ms=t, tflops=fl / t / 1e9)
    _lib.check_status("cuda")


# ---------------------------------------------------------------------------------- decode
def bench_decode(a):
    """Times each kernel of a decode step in isolation (back-to-back launches, no L2 flush: in a real step the
    weights of a 0.5B model stay L2-resident), then one full layer loop, so shares and launch gaps are visible."""
    from slime_b200.models.config import get_preset

    cfg = get_preset(a.model)
    B, ctx, ps = a.batch, a.context, 16
    d, hq, hkv, H, F, V = cfg.head_dim, cfg.num_attention_heads, cfg.num_query_groups, cfg.hidden_size, cfg.ffn_hidden_size, cfg.vocab_size
    bf, dev = torch.bfloat16, "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: (0.02 * torch.randn(*s, device=dev, generator=g)).to(bf)  # noqa: E731
    x, res = rnd(B, H), rnd(B, H)
    x32 = x.float()
    ln = torch.ones(H, device=dev, dtype=bf)
    wqkv, bqkv = rnd((hq + 2 * hkv) * d, H), (rnd((hq + 2 * hkv) * d) if cfg.add_qkv_bias else None)
    wo, wgu, wdn, wlm = rnd(H, hq * d), rnd(2 * F, H), rnd(H, F), rnd(V, H)
    pages = B * math.ceil((ctx + 1) / ps) + 1
    kc, vc = rnd(pages * ps, hkv, d), rnd(pages * ps, hkv, d)
    per = math.ceil((ctx + 1) / ps)
    bt = (1 + torch.arange(B * per, device=dev, dtype=torch.int32)).view(B, per).contiguous()
    seq = torch.full((B,), ctx, device=dev, dtype=torch.int32)
    pos = seq - 1
    slots = (bt[:, -1] * ps).to(torch.int32)
    rope = ops.rope_cos_sin(ctx + 8, d, cfg.rotary_base, device=dev)
    qn = torch.ones(d, device=dev, dtype=bf) if cfg.qk_layernorm else None
    temp = torch.ones(B, device=dev)
    seeds = torch.arange(B, device=dev, dtype=torch.int64)
    outp = torch.zeros(B, device=dev, dtype=torch.int32)

    qkv = ops.gemm(x, wqkv, bias=bqkv)
    q3 = qkv.view(B, hq + 2 * hkv, d)
    attn = ops.paged_decode_attention(q3[:, :hq], kc, vc, bt, seq, ps)
    gu = ops.gemm(x, wgu)
    act = ops.swiglu(gu)
    logits = ops.gemm(x, wlm, out_dtype=torch.float32)
    steps = {
        "rmsnorm_add": lambda: ops.rmsnorm(x32, ln, 1e-6, res),  # reads the fp32 projection output
        "gemm_qkv": lambda: ops.gemm(x, wqkv, bias=bqkv),
        "rope_qk": lambda: ops.rope_qk(qkv, pos, rope, hq, hkv, d, qn, qn, 1e-6),
        "kv_write": lambda: ops.kv_write(q3[:, hq : hq + hkv].reshape(B, -1), q3[:, hq + hkv :].reshape(B, -1), slots, kc, vc),
        "rope_kv_write": lambda: ops.rope_kv_write(qkv, pos, rope, slots, kc, vc, hq, hkv, d, qn, qn, 1e-6),
        "paged_attention": lambda: ops.paged_decode_attention(q3[:, :hq], kc, vc, bt, seq, ps),
        "gemm_o": lambda: ops.gemm(attn.reshape(B, -1), wo, out_dtype=torch.float32),
        "gemm_gate_up": lambda: ops.gemm(x, wgu),
        "swiglu": lambda: ops.swiglu(gu),
        "gemm_down": lambda: ops.gemm(act, wdn, out_dtype=torch.float32),  # split-K, summed in fp32
        "gemm_lm_head": lambda: ops.gemm(x, wlm, out_dtype=torch.float32),
        "sample": lambda: ops.sample(logits, temp, None, None, None, seeds, outp, 0),
    }
    # rope_qk and kv_write (training-style ops, four launches) are timed for comparison; the engine uses the fused one
    per_layer = ["rmsnorm_add", "gemm_qkv", "rope_kv_write", "paged_attention", "gemm_o", "rmsnorm_add", "gemm_gate_up",
                 "swiglu", "gemm_down"]  # fmt: skip
    def attn_forced(flag, **kw):  # SLIME_B200_DECODE_ATTN_WS = "1": warp-specialised kernel, "0": the two-chain kernel
        os.environ["SLIME_B200_DECODE_ATTN_WS"] = flag
        try:
            return ops.paged_decode_attention(q3[:, :hq], kc, vc, bt, seq, ps, **kw)
        finally:
            os.environ.pop("SLIME_B200_DECODE_ATTN_WS", None)

    def attn_ws():
        return attn_forced("1", splits=a.splits)

    def attn_ws_loads():  # the same kernel with every landed tile handed straight back: the cost of its copy path alone
        _lib.lib().sb_paged_decode_ws_load_path_only(1)
        try:
            return attn_ws()
        finally:
            _lib.lib().sb_paged_decode_ws_load_path_only(0)

    if d == 64:
        steps["paged_attention_warp_specialised"] = attn_ws
        steps["paged_attention_two_chain"] = lambda: attn_forced("0")
        steps["paged_attention_warp_specialised_load_path"] = attn_ws_loads
    steps["paged_attention_cuda_cores"] = lambda: ops.paged_decode_attention(q3[:, :hq], kc, vc, bt, seq, ps,
                                                                             use_tensor_cores=False)
    t_of = {}
    for name, fn in steps.items():
        # `reps` launches inside one CUDA graph: device time per launch without the host's launch cost
        fn()
        gk = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gk):
            for _ in range(a.reps):
                fn()
        t_of[name] = time_ms(gk.replay, a.iters, flush=False) / a.reps
        _emit(kind="decode_kernel", name=name, batch=B, context=ctx, us=1e3 * t_of[name])
    try:  # a measurement build (-DSB_WS_CHAIN_TIMING) also reports where a softmax group's time per tile goes
        import ctypes

        ticks_fn = _lib.bind("sb_paged_decode_ws_chain_ticks", [ctypes.c_void_p, ctypes.c_int])
    except AttributeError:
        ticks_fn = None
    if ticks_fn is not None and d == 64:
        buf = (ctypes.c_ulonglong * 16)()
        torch.cuda.synchronize()
        ticks_fn(ctypes.addressof(buf), 1)
        attn_ws()
        torch.cuda.synchronize()
        ticks_fn(ctypes.addressof(buf), 0)
        tiles = max(1, buf[6])
        names = ["wait_s", "tmem_ld_max", "group_exchange", "merge_prev", "exp_p_fence", "end_of_item"]
        _emit(kind="decode_attn_ws_chain", batch=B, context=ctx, tiles=int(buf[6]),
              cycles_per_tile={k: buf[i] / tiles for i, k in enumerate(names)})
        inames = ["s_queue", "s_wait_k", "s_wait_group", "s_issue", "o_wait_p", "o_wait_v", "o_wait_group", "o_issue"]
        # the issuers handle the tiles of all four groups: per tile of the CTA (4 x the tiles the clocked group saw)
        _emit(kind="decode_attn_ws_issuers", batch=B, context=ctx,
              cycles_per_cta_tile={k: buf[8 + i] / (4 * tiles) for i, k in enumerate(inames)})
    est = cfg.num_layers * sum(t_of[k] for k in per_layer) + t_of["gemm_lm_head"] + t_of["sample"] + t_of["rmsnorm_add"]

    def layer_loop():
        for _ in range(cfg.num_layers):
            for k in per_layer:
                steps[k]()

    eager = time_ms(layer_loop, max(3, a.iters // 4), flush=False)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        layer_loop()
    graphed = time_ms(gr.replay, max(3, a.iters // 4), flush=False)
    kv_bytes = 2.0 * B * ctx * hkv * d * 2 * cfg.num_layers
    w_bytes = 2.0 * (cfg.num_params() - (0 if cfg.tie_word_embeddings else V * H))
    _emit(kind="decode_step", batch=B, context=ctx, model=a.model, sum_of_kernels_ms=est, layers_eager_ms=eager,
          layers_graph_ms=graphed, kv_bytes=kv_bytes, weight_bytes=w_bytes)
    _lib.check_status("cuda")


# ------------------------------------------------------------------------------------ norm
def bench_norm(a):
    for T, H in ((131072, 896), (1048576, 128), (16384, 4096), (65536, 2560)) if not a.small else ((4096, 4096),):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        t = time_ms(lambda: ops.rmsnorm(x.detach(), w.detach(), 1e-6, r), a.iters)
        _emit(kind="rmsnorm_fwd", T=T, H=H, ms=t, gbs=4 * T * H * 2 / t / 1e6)  # read x, r; write y, h
        y, h = ops.rmsnorm(x, w, 1e-6, r)
        gy, gh = torch.randn_like(y), torch.randn_like(h)
        t = time_ms(lambda: torch.autograd.grad([y, h], [x], [gy, gh], retain_graph=True), a.iters)
        _emit(kind="rmsnorm_bwd", T=T, H=H, ms=t, gbs=4 * T * H * 2 / t / 1e6)  # read dy, dres, h; write dh


def bench_fp8(a):
    """Block-scaled fp8 GEMM against this library's bf16 GEMM and torch._scaled_mm (per-tensor scales: a different,
    cheaper scaling scheme, shown only as the library fp8 ceiling)."""
    shapes = [(4096, 4096, 7168), (16384, 2048, 7168), (8192, 1536, 2048), (256, 4096, 7168)] if not a.small else [(1024, 1024, 1024)]
    for M, N, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.1
        xq, xs = ops.block_fp8_quant(x, (1, 128))
        wq, ws = ops.block_fp8_quant(w, (128, 128))
        fl = 2.0 * M * N * K
        t = time_ms(lambda: ops.fp8_block_gemm(xq, xs, wq, ws), a.iters)
        _emit(kind="fp8_block", M=M, N=N, K=K, ms=t, tflops=fl / t / 1e9)
        t = time_ms(lambda: ops.gemm(x, w), a.iters)
        _emit(kind="bf16_ours", M=M, N=N, K=K, ms=t, tflops=fl / t / 1e9)
        t = time_ms(lambda: ops.fp8_act_quant(x), a.iters)
        _emit(kind="act_quant_1x128", M=M, K=K, ms=t, gbs=3.0 * M * K / t / 1e6)
        if not a.no_cublas:
            one = torch.ones((), device="cuda")
            try:
                t = time_ms(lambda: torch._scaled_mm(xq, wq.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16), a.iters)
                _emit(kind="scaled_mm_per_tensor", M=M, N=N, K=K, ms=t, tflops=fl / t / 1e9)
            except Exception as e:  # noqa: BLE001
                _emit(kind="scaled_mm_per_tensor", error=repr(e)[:200])
    _lib.check_status("cuda")


def bench_moe(a):
    """Expert MLP of Qwen3-30B-A3B (hidden 2048, expert FFN 768, 16 local experts of 128 under EP8): grouped GEMMs
    against the per-expert loop over the same GEMM kernel, for a training-sized and a decode-sized token count."""
    from slime_b200.ops import grouped

    E, H, F = 16, 2048, 768
    w13 = torch.randn(E, 2 * F, H, device="cuda", dtype=torch.bfloat16) * 0.02
    w2 = torch.randn(E, H, F, device="cuda", dtype=torch.bfloat16) * 0.02
    for rows in ((16384, 2048) if not a.small else (2048,)):
        g = torch.Generator(device="cuda").manual_seed(rows)
        cuts = torch.sort(torch.randint(0, rows, (E - 1,), device="cuda", generator=g)).values.tolist()
        counts = [b - c for c, b in zip([0] + cuts, cuts + [rows])]
        x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
        lay = grouped.PaddedLayout(counts, "cuda")
        xp = lay.pad(x)

        def fused():
            return grouped.grouped_gemm(ops.swiglu(grouped.grouped_gemm(xp, w13, lay)), w2, lay)

        def loop():
            outs, s = [], 0
            for e, n in enumerate(counts):
                if n:
                    outs.append(ops.gemm(ops.swiglu(ops.gemm(x[s : s + n], w13[e])), w2[e]))
                    s += n
            return outs

        fl = 2.0 * rows * (2 * F * H + H * F)
        t = time_ms(fused, a.iters)
        _emit(kind="moe_grouped", rows=rows, experts=E, ms=t, tflops=fl / t / 1e9)
        t = time_ms(loop, a.iters)
        _emit(kind="moe_expert_loop", rows=rows, experts=E, ms=t, tflops=fl / t / 1e9)
    _lib.check_status("cuda")


def bench_attn(a):
    """Flash attention forward / backward (own tcgen05 kernels) on packed equal-length sequences, and the flash-attn
    library (an mma.sync-class kernel) on the same tensors when it is importable. FLOPs: causal, 4 * S^2 * H * D / 2 per
    sequence forward, 2.5 x that backward."""
    from slime_b200.ops import attention

    try:
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward, _flash_attn_varlen_forward
    except Exception:  # noqa: BLE001
        _flash_attn_varlen_forward = None
    cases = [(14, 2, 64, 1024, 16), (14, 2, 64, 4096, 4), (32, 8, 128, 2048, 4), (32, 8, 128, 8192, 1), (16, 4, 128, 8192, 1)]
    if a.small:
        cases = [(32, 8, 128, 2048, 2)]
    for Hq, Hkv, D, S_, nseq in cases:
        T = S_ * nseq
        qkv = (torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda") * 0.5).to(torch.bfloat16)
        x3 = qkv.view(T, Hq + 2 * Hkv, D)
        q, k, v = x3[:, :Hq], x3[:, Hq : Hq + Hkv], x3[:, Hq + Hkv :]
        cu = torch.arange(0, T + 1, S_, dtype=torch.int32, device="cuda")
        seg = attention.segments_from_cu_seqlens(cu)
        scale = 1.0 / math.sqrt(D)
        fwd_flops = 4.0 * S_ * S_ * Hq * D / 2 * nseq
        out, lse = attention.flash_fwd(q, k, v, seg, scale)
        d_o = torch.randn_like(out)
        dqkv = torch.zeros_like(qkv)
        d3 = dqkv.view(T, Hq + 2 * Hkv, D)
        tf = time_ms(lambda: attention.flash_fwd(q, k, v, seg, scale, out=out), a.iters)
        tb = time_ms(lambda: attention.flash_bwd(q, k, v, out, d_o, lse, seg, scale, dq=d3[:, :Hq], dk=d3[:, Hq : Hq + Hkv],
                                                 dv=d3[:, Hq + Hkv :]), a.iters)  # fmt: skip
        rec = dict(kind="flash_attn", Hq=Hq, Hkv=Hkv, D=D, seqlen=S_, nseq=nseq, fwd_ms=tf, fwd_tflops=fwd_flops / tf / 1e9,
                   bwd_ms=tb, bwd_tflops=2.5 * fwd_flops / tb / 1e9)  # fmt: skip
        if _flash_attn_varlen_forward is not None and not a.no_cublas:
            res = _flash_attn_varlen_forward(q, k, v, cu, cu, S_, S_, 0.0, scale, causal=True)
            lo, llse, rng = res[0], res[1], res[3]
            lf = time_ms(lambda: _flash_attn_varlen_forward(q, k, v, cu, cu, S_, S_, 0.0, scale, causal=True), a.iters)
            lb = time_ms(lambda: _flash_attn_varlen_backward(d_o, q, k, v, lo, llse, d3[:, :Hq], d3[:, Hq : Hq + Hkv],
                                                             d3[:, Hq + Hkv :], cu, cu, S_, S_, 0.0, scale, True, -1, -1, 0.0,
                                                             None, False, rng), a.iters)  # fmt: skip
            rec.update(lib_fwd_ms=lf, lib_bwd_ms=lb, lib_fwd_tflops=fwd_flops / lf / 1e9, lib_bwd_tflops=2.5 * fwd_flops / lb / 1e9)
        _emit(**rec)
    _lib.check_status("cuda")


def bench_fused_emul(a):
    """The peer-memory kernels with every "rank" a buffer of THIS GPU (profilers attach to one process on one GPU, and
    kernels that wait on one another must not run as separate launches on one device): the data path, instruction mix
    and DRAM behaviour are those of the multi-GPU run, the NVLink hop is not. Flags are preset so no wait occurs."""
    import ctypes

    lib, P = _lib.lib(), _lib.ptr
    dev = torch.device("cuda")
    status = _lib.status_word(dev)
    # ---- data-parallel reduce-scatter shard + squared norm, then Adam + all-gather stores (world = 4)
    world, n = 4, (8 if a.small else 64) * 1024 * 1024
    grads = [torch.randn(n, device=dev) for _ in range(world)]
    params = [torch.zeros(n, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    gp = (ctypes.c_void_p * world)(*[g.data_ptr() for g in grads])
    pp = (ctypes.c_void_p * world)(*[p.data_ptr() for p in params])
    shard = n // world
    partials, ctl = torch.zeros(148 * 8, device=dev), torch.zeros(2, device=dev)
    master, m, v = (torch.zeros(shard, device=dev) for _ in range(3))

    def reduce():
        _lib.check(lib.sb_dp_reduce_shard(gp, world, 0, 0, 0, shard, P(grads[0][:shard]), P(partials), P(ctl), P(status),
                                          _lib.stream()), "sb_dp_reduce_shard")  # fmt: skip

    def adam():
        _lib.check(lib.sb_dp_adam_bcast(P(master), P(m), P(v), P(grads[0][:shard]), pp, world, 0, 0, 0, shard, 1e-6, 0.9, 0.98,
                                        1e-8, 0.1, 0.1, 0.02, 1.0, 1.0, P(ctl), 0, _lib.stream()), "sb_dp_adam_bcast")  # fmt: skip

    t = time_ms(reduce, a.iters)
    _emit(kind="dp_reduce_shard_emulated", world=world, shard_elems=shard, ms=t, read_gbs=world * shard * 4 / t / 1e6)
    t = time_ms(adam, a.iters)
    _emit(kind="dp_adam_bcast_emulated", world=world, shard_elems=shard, ms=t,
          bytes_gbs=(shard * (4 * 4 + 3 * 4) + world * shard * 2) / t / 1e6)  # fmt: skip
    # ---- tensor-parallel all-reduce + residual + RMSNorm (world = 2)
    T, H, world = 256, 2560, 2
    parts = [torch.randn(T, H, device=dev).to(torch.bfloat16) for _ in range(world)]
    flags = torch.full((148 * 8,), 1 << 30, dtype=torch.int32, device=dev)  # every peer "has arrived" already
    epochs = torch.zeros(148, dtype=torch.int32, device=dev)
    res, w = torch.randn(T, H, device=dev).to(torch.bfloat16), torch.ones(H, device=dev, dtype=torch.bfloat16)
    y, r = torch.empty_like(res), torch.empty_like(res)
    ptrs = (ctypes.c_void_p * world)(*[x.data_ptr() for x in parts])
    fl = (ctypes.c_void_p * world)(*[flags.data_ptr()] * world)

    def ar():
        _lib.check(lib.sb_tp_ar_add_rmsnorm(ptrs, fl, P(epochs), P(res), P(w), P(y), P(r), T, H, 1e-6, 0, world, 0, P(status),
                                            _lib.stream()), "sb_tp_ar_add_rmsnorm")  # fmt: skip

    t = time_ms(ar, a.iters)
    _emit(kind="tp_ar_add_rmsnorm_emulated", T=T, H=H, world=world, us=t * 1e3, gbs=(world + 3) * T * H * 2 / t / 1e6)
    want = (parts[0].float() + parts[1].float() + res.float())
    want = want * torch.rsqrt(want.pow(2).mean(-1, keepdim=True) + 1e-6)
    assert (y.float() - want).abs().max() < 0.05
    _lib.check_status(dev)


def main(argv=None):
    p = argparse.ArgumentParser(prog="python -m slime_b200.ops.microbench")
    p.add_argument("what", choices=["gemm", "decode", "norm", "fp8", "moe", "attn", "fused_emul"])
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--reps", type=int, default=20, help="back-to-back launches per timed repetition (decode)")
    p.add_argument("--small", action="store_true")
    p.add_argument("--no-cublas", action="store_true")
    p.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"))
    p.add_argument("--model", default="qwen2.5-0.5b")
    p.add_argument("--batch", type=int, default=256)
    p.add_argument("--context", type=int, default=768)
    p.add_argument("--splits", type=int, default=None, help="sequence splits of the warp-specialised decode attention")
    a = p.parse_args(argv)
    from slime_b200.ops import build

    build.build()
    {"gemm": bench_gemm, "decode": bench_decode, "norm": bench_norm, "fp8": bench_fp8, "moe": bench_moe, "attn": bench_attn, "fused_emul": bench_fused_emul}[a.what](a)


if __name__ == "__main__":
    main()
