"""Block-scaled fp8 GEMM (tcgen05 kind::f8f6f4 with per-K-block promotion) against the dequantised fp32 product."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,dtype", [(128, 128, 128, torch.float32), (300, 200, 256, torch.bfloat16),
                                          (1024, 1536, 2048, torch.bfloat16), (4096, 768, 7168, torch.float32)])
def test_fp8_block_gemm_matches_dequantised_product(kernels, M, N, K, dtype):
    from slime_b200 import ops
    from slime_b200.ops import _lib

    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda") * 1.5
    w = torch.randn(N, K, device="cuda") * 0.1
    # make the scales differ strongly between blocks so a wrong scale index cannot hide
    x[:, : K // 2] *= 7.0
    w[: N // 2] *= 3.0
    xq, xs = ops.block_fp8_quant(x.to(torch.bfloat16), (1, 128))
    wq, ws = ops.block_fp8_quant(w.to(torch.bfloat16), (128, 128))
    out = ops.fp8_block_gemm(xq, xs, wq, ws, out_dtype=dtype)
    torch.cuda.synchronize()
    _lib.check_status(out.device)
    a = xq.float() * xs.repeat_interleave(128, dim=1)
    b = wq.float() * ws.repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1)
    ref = a @ b.t()
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-3
    assert (out.float() - ref).abs().max() <= tol * ref.abs().max(), float((out.float() - ref).abs().max() / ref.abs().max())
    # and the quantised product is close to the bf16 one (sanity of the whole W8A8 path)
    full = x.to(torch.bfloat16).float() @ w.to(torch.bfloat16).float().t()
    assert (out.float() - full).abs().max() <= 0.08 * full.abs().max()


def test_activation_quant_kernel_matches_block_quant(kernels):
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(3)
    x = (torch.randn(777, 1024, device="cuda") * torch.rand(777, 1, device="cuda") * 20).to(torch.bfloat16)
    q, s, st = ops.fp8_act_quant(x)
    qr, sr = reference.block_fp8_quant(x.cpu(), (1, 128), False)
    torch.testing.assert_close(s.cpu(), sr, rtol=1e-6, atol=0)
    assert torch.equal(st, s.t())
    # the kernel multiplies by 1/scale where the reference divides: a value on a rounding boundary may land one code off
    same = (q.cpu().view(torch.uint8) == qr.view(torch.uint8)).float().mean().item()
    assert same > 0.999, same
    deq, deq_ref = q.cpu().float() * s.cpu().repeat_interleave(128, 1), qr.float() * sr.repeat_interleave(128, 1)
    assert (deq - deq_ref).abs().max() <= 0.13 * deq_ref.abs().max()
    q2, s2 = ops.block_fp8_quant(x, (1, 128))  # the generic entry point takes the same fast path
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s)


@pytest.mark.parametrize("counts,N,K", [([300, 0, 77, 129], 256, 256), ([1000, 40, 513, 2, 128, 700], 768, 2048)])
def test_grouped_fp8_gemm_matches_dequantised_product_per_expert(kernels, counts, N, K):
    """Expert stack [E, N, K] in block fp8: every 128-row tile multiplies its own expert's bytes and scales."""
    from slime_b200 import ops
    from slime_b200.ops import _lib, grouped

    torch.manual_seed(len(counts) + N)
    E = len(counts)
    lay = grouped.PaddedLayout(counts, "cuda")
    x = torch.randn(sum(counts), K, device="cuda").to(torch.bfloat16)
    w = torch.randn(E, N, K, device="cuda") * 0.1
    w *= torch.arange(1, E + 1, device="cuda").view(E, 1, 1)  # scales differ by expert: a wrong table cannot hide
    wq = torch.empty(E, N, K, dtype=torch.float8_e4m3fn, device="cuda")
    ws = torch.empty(E, -(-N // 128), K // 128, dtype=torch.float32, device="cuda")
    for e in range(E):
        ops.block_fp8_quant(w[e].to(torch.bfloat16), (128, 128), out=(wq[e], ws[e]))
    xp = lay.pad(x)
    out = grouped.grouped_gemm_fp8(xp, wq, ws, lay, out_dtype=torch.float32)
    torch.cuda.synchronize()
    _lib.check_status(out.device)
    aq, a_s, _ = ops.fp8_act_quant(xp)
    a = aq.float() * a_s.repeat_interleave(128, 1)
    for e, (s, n) in enumerate(zip(lay.padded_starts, counts)):
        if n == 0:
            continue
        b = wq[e].float() * ws[e].repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)
        ref = a[s : s + n] @ b.t()
        err = (out[s : s + n] - ref).abs().max() / ref.abs().max()
        assert err <= 2e-3, (e, float(err))


def test_fp8_engine_on_gpu_tracks_the_bf16_engine(kernels):
    """quantization='fp8': resident e4m3 matrices, fp8 tensor-core GEMMs (dense and grouped) in prefill and in captured
    decode steps; its log-probs for the bf16 engine's tokens stay within W8A8 error of the bf16 engine's own."""
    import numpy as np

    from slime_b200.engine.engine import Engine
    from slime_b200.engine.quant import Fp8Weight
    from slime_b200.engine.server_args import ServerArgs
    from slime_b200.models.config import ModelConfig

    cfg = ModelConfig(num_layers=3, hidden_size=256, num_attention_heads=4, num_query_groups=2, kv_channels=64, ffn_hidden_size=512,
                      vocab_size=1024, rotary_base=1e4, tie_word_embeddings=False, num_experts=4, moe_ffn_hidden_size=128,
                      moe_router_topk=2, moe_layer_freq=[0, 1, 1])  # fmt: skip
    g = torch.Generator(device="cuda").manual_seed(0)
    mat = lambda *s, std=0.05: (torch.randn(*s, device="cuda", generator=g) * std).to(torch.bfloat16)  # noqa: E731
    h, d, f, fe = cfg.hidden_size, 64, cfg.ffn_hidden_size, cfg.moe_ffn_hidden_size
    weights = [("model.embed_tokens.weight", mat(cfg.vocab_size, h, std=0.5)), ("model.norm.weight", 1 + mat(h)),
               ("lm_head.weight", mat(cfg.vocab_size, h, std=0.5))]  # fmt: skip
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        weights += [(p + "input_layernorm.weight", 1 + mat(h)), (p + "post_attention_layernorm.weight", 1 + mat(h)),
                    (p + "self_attn.q_proj.weight", mat(4 * d, h)), (p + "self_attn.k_proj.weight", mat(2 * d, h)),
                    (p + "self_attn.v_proj.weight", mat(2 * d, h)), (p + "self_attn.o_proj.weight", mat(h, 4 * d))]  # fmt: skip
        if cfg.is_moe_layer(i):
            weights.append((p + "mlp.gate.weight", mat(cfg.num_experts, h, std=0.5)))
            for e in range(cfg.num_experts):
                weights += [(p + f"mlp.experts.{e}.gate_proj.weight", mat(fe, h)), (p + f"mlp.experts.{e}.up_proj.weight", mat(fe, h)),
                            (p + f"mlp.experts.{e}.down_proj.weight", mat(h, fe))]  # fmt: skip
        else:
            weights += [(p + "mlp.gate_proj.weight", mat(f, h)), (p + "mlp.up_proj.weight", mat(f, h)), (p + "mlp.down_proj.weight", mat(h, f))]
    prompts = [[(7 * i + 3 * j) % 1000 for j in range(5 + i)] for i in range(4)]
    engines = {}
    for q in (None, "fp8"):
        e = Engine(cfg, ServerArgs(page_size=16, max_running_requests=4, context_length=128, quantization=q), device="cuda", num_pages=64)
        assert not e.weights.load_weights(weights)
        engines[q] = e
    L = engines["fp8"].weights.layers
    assert isinstance(L[0]["gate_up"], Fp8Weight) and isinstance(L[1]["w13"], Fp8Weight) and isinstance(L[1]["qkv"], Fp8Weight)
    base = engines[None].generate(prompts, dict(max_new_tokens=8, temperature=0, ignore_eos=True))
    own = engines["fp8"].generate(prompts, dict(max_new_tokens=8, temperature=0, ignore_eos=True))  # decode through graphs
    assert all(len(r.output_ids) == 8 for r in own) and engines["fp8"].runner.graphs
    diffs = []
    for r in base:
        ids = r.input_ids + r.output_ids
        a = engines[None].generate([ids], [dict(max_new_tokens=0)], logprob_start_len=0)[0].input_logprobs[len(r.input_ids):]
        b = engines["fp8"].generate([ids], [dict(max_new_tokens=0)], logprob_start_len=0)[0].input_logprobs[len(r.input_ids):]
        diffs += [abs(x - y) for x, y in zip(a, b)]
    # random weights put many router logits near ties: a route that flips under W8A8 moves single tokens by a nat or
    # so, which bounds the mean and the median but not the maximum
    assert float(np.median(diffs)) < 0.15 and float(np.mean(diffs)) < 0.35, (float(np.median(diffs)), float(np.mean(diffs)))
    for e in engines.values():
        e.shutdown()
