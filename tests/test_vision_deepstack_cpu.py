"""Qwen3-VL: an image encoder whose intermediate blocks also feed the language model's first layers ("deepstack"),
checked against the Transformers implementation with random weights (the library is the oracle, nothing else uses it)."""

import inspect

import pytest
import torch

from slime_b200.models.config import ModelConfig
from slime_b200.models.gpt import GPTModel, PackedSeqParams
from slime_b200.weight_sync import convert

IMG, VID, VSTART, VEND = 190, 191, 192, 193


def _per_expert(sd: dict) -> dict:
    """The library keeps a layer's experts in two fused tensors; checkpoint names (used everywhere here) name each expert."""
    out = {}
    for k, v in sd.items():
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(v.shape[0]):
                g, u = v[e].chunk(2, 0)
                out[k.replace("gate_up_proj", f"{e}.gate_proj.weight")], out[k.replace("gate_up_proj", f"{e}.up_proj.weight")] = g, u
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(v.shape[0]):
                out[k.replace("down_proj", f"{e}.down_proj.weight")] = v[e]
        else:
            out[k] = v
    return out


@pytest.fixture(scope="module", params=["dense", "moe"])
def pair(request):
    vis = dict(depth=3, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=64, num_position_embeddings=64, in_channels=3, deepstack_visual_indexes=[0, 1])  # fmt: skip
    text = dict(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, rms_norm_eps=1e-6, max_position_embeddings=512,
                rope_parameters=dict(rope_type="default", rope_theta=10000.0, mrope_section=[4, 2, 2], mrope_interleaved=True))  # fmt: skip
    if request.param == "dense":
        from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLConfig as C
        from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLForConditionalGeneration as M
    else:
        from transformers.models.qwen3_vl_moe.configuration_qwen3_vl_moe import Qwen3VLMoeConfig as C
        from transformers.models.qwen3_vl_moe.modeling_qwen3_vl_moe import Qwen3VLMoeForConditionalGeneration as M

        text.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=1, mlp_only_layers=[])
    hf_cfg = C(text_config=text, vision_config=vis, image_token_id=IMG, video_token_id=VID, vision_start_token_id=VSTART,
               vision_end_token_id=VEND)  # fmt: skip
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = M(hf_cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    d = hf_cfg.to_dict()
    d["architectures"] = [M.__name__]
    cfg = ModelConfig.from_hf(d)
    assert cfg.vision["deepstack_visual_indexes"] == [0, 1] and cfg.mrope_section == [4, 2, 2] and cfg.mrope_interleaved
    ours = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=1)
    sd = _per_expert(hf.state_dict())
    with torch.no_grad():
        for name, p in list(ours.named_parameters()) + list(ours.named_buffers()):
            names, rule = convert.hf_sources_for(cfg, name)
            p.copy_(convert.merge_hf_sources(rule, [sd[n] for n in names], cfg))
    return hf, cfg, ours, sd


def _inputs(seed=3):
    ids = torch.tensor([[5, 6, VSTART] + [IMG] * 6 + [VEND, 7, 8, VSTART] + [IMG] * 8 + [VEND, 9, 10, 11]])
    grids = [[1, 4, 6], [1, 8, 4]]
    g = torch.Generator().manual_seed(seed)
    px = torch.randn(sum(t * h * w for t, h, w in grids), 3 * 2 * 4 * 4, generator=g)
    return ids, px, torch.tensor(grids)


def test_encoder_and_its_side_outputs_match_the_library(pair):
    hf, _, ours, _ = pair
    _, px, grid = _inputs()
    with torch.no_grad():
        want = hf.model.visual(px, grid_thw=grid)
        got, extras = ours.vision(px, grid, with_deepstack=True)
    want_main = want.pooler_output if hasattr(want, "pooler_output") else want[0]
    want_deep = want.deepstack_features if hasattr(want, "deepstack_features") else want[1]
    assert (got - torch.as_tensor(want_main)).abs().max() < 2e-5
    assert len(extras) == len(want_deep) == 2
    for a, b in zip(extras, want_deep):
        assert (a - b).abs().max() < 2e-5


def test_whole_model_matches_the_library_and_names_round_trip(pair):
    hf, cfg, ours, sd = pair
    ids, px, grid = _inputs()
    with torch.no_grad():
        kw = dict(mm_token_type_ids=(ids == IMG).int()) if "mm_token_type_ids" in inspect.signature(hf.forward).parameters else {}
        want = hf(input_ids=ids, pixel_values=px, image_grid_thw=grid, **kw).logits[0]
        got = ours(ids, pixel_values=px, image_grid_thw=grid)[0]
    assert (got - want).abs().max() < 3e-4, float((got - want).abs().max())
    packed = PackedSeqParams(torch.tensor([0, ids.numel(), 2 * ids.numel()], dtype=torch.int32), ids.numel())
    with torch.no_grad():
        both = ours(torch.cat([ids[0], ids[0]]), packed_seq_params=packed, pixel_values=torch.cat([px, px]), image_grid_thw=torch.cat([grid, grid]))[0]
    assert (both[: ids.numel()] - got).abs().max() < 1e-4 and (both[ids.numel() :] - got).abs().max() < 1e-4
    out = dict(x for n, p in list(ours.named_parameters()) + list(ours.named_buffers()) for x in convert.convert_to_hf(cfg, n, p.detach()))
    assert set(out) == set(sd), (sorted(set(out) - set(sd))[:5], sorted(set(sd) - set(out))[:5])
    for k in sd:
        assert torch.allclose(out[k], sd[k], atol=1e-6), k


@pytest.mark.parametrize("chunk", [8192, 5])
def test_engine_adds_the_side_outputs_after_the_first_layers(pair, chunk):
    """Prompt and greedy-decode log-probs of a request with two images equal the trainer's teacher-forced ones, also when
    an image spans several prefill chunks."""
    import numpy as np

    from slime_b200.engine.engine import Engine
    from slime_b200.engine.server_args import ServerArgs

    hf, cfg, ours, sd = pair
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=4, context_length=128, disable_cuda_graph=True, chunked_prefill_size=chunk),
               device="cpu", num_pages=96)  # fmt: skip
    assert not e.weights.load_weights(list(sd.items()))
    ids, px, grid = _inputs()
    ids = ids[0].tolist()
    mm = dict(pixel_values=px, image_grid_thw=grid)

    def trainer_logprobs(tokens):
        with torch.no_grad():
            lg = ours(torch.tensor(tokens), pixel_values=px, image_grid_thw=grid)[0]
        return lg.log_softmax(-1)[:-1].gather(-1, torch.tensor(tokens[1:])[:, None]).squeeze(-1).numpy()

    r = e.generate([ids], [dict(max_new_tokens=0)], logprob_start_len=0, mm=mm)[0]
    assert np.abs(np.array(r.input_logprobs[1:]) - trainer_logprobs(ids)).max() < 3e-4
    a = e.generate([ids], [dict(max_new_tokens=6, temperature=0, ignore_eos=True)], mm=mm)[0]
    ref = trainer_logprobs(ids + a.output_ids)[len(ids) - 1 :]
    assert np.abs(np.array(a.output_logprobs) - ref).max() < 3e-4, np.abs(np.array(a.output_logprobs) - ref).max()


def test_files_with_stacked_experts_load_into_trainer_and_engine(pair, tmp_path):
    """Qwen3-VL-MoE files hold a layer's experts as [experts, hidden, 2 x width] and [experts, width, hidden] stacks."""
    from safetensors.torch import save_file

    from slime_b200.checkpoint.hf_loader import SafetensorReader, load_hf_weights
    from slime_b200.engine.engine import Engine
    from slime_b200.engine.server_args import ServerArgs

    hf, cfg, ours, sd = pair
    if not cfg.num_experts:
        pytest.skip("dense model: nothing is stacked")
    files = {k: (v.transpose(1, 2) if k.endswith(("experts.gate_up_proj", "experts.down_proj")) else v).contiguous().clone()
             for k, v in hf.state_dict().items()}  # fmt: skip
    assert files["model.language_model.layers.0.mlp.experts.down_proj"].shape == (4, 32, 64)
    parts = dict(x for k, v in files.items() for x in (convert.split_stacked_experts(cfg, k, v) or [(k, v)]))
    assert set(parts) == set(sd) and all(torch.equal(parts[k], sd[k]) for k in sd)
    save_file(files, str(tmp_path / "model.safetensors"))
    reader = SafetensorReader(str(tmp_path))
    name = "model.language_model.layers.1.mlp.experts.2.up_proj.weight"
    assert name in reader and torch.equal(reader.get(name, cfg), sd[name])
    fresh = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=7)
    assert not load_hf_weights(str(tmp_path), fresh)
    for (n, a), (_, b) in zip(fresh.named_parameters(), ours.named_parameters()):
        assert torch.equal(a, b), n
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=2, context_length=64, disable_cuda_graph=True), device="cpu", num_pages=32)
    assert not e.weights.load_weights(list(files.items()))
    f = Engine(cfg, ServerArgs(page_size=4, max_running_requests=2, context_length=64, disable_cuda_graph=True), device="cpu", num_pages=32)
    assert not f.weights.load_weights(list(sd.items()))
    for a, b in zip(e.weights.tensors(), f.weights.tensors()):
        assert torch.equal(a, b)


def test_engine_takes_encoder_outputs_computed_elsewhere(pair):
    """``image_embeds`` + ``image_deepstack_embeds`` in place of pixel values skip the engine's encoder and give the same
    tokens and log-probs; a request that leaves the deepstack vectors out is refused."""
    from slime_b200.engine.engine import Engine
    from slime_b200.engine.server_args import ServerArgs

    hf, cfg, ours, sd = pair
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=4, context_length=128, disable_cuda_graph=True), device="cpu", num_pages=96)
    assert not e.weights.load_weights(list(sd.items()))
    ids, px, grid = _inputs()
    ids = ids[0].tolist()
    sp = dict(max_new_tokens=5, temperature=0, ignore_eos=True)
    want = e.generate([ids], [sp], mm=dict(pixel_values=px, image_grid_thw=grid))[0]
    with torch.no_grad():
        out, extras = ours.vision(px, grid, with_deepstack=True)
    e.weights.vision = None  # the language-model side of a split deployment holds no encoder
    got = e.generate([ids], [sp], mm=dict(image_embeds=out, image_deepstack_embeds=extras, image_grid_thw=grid))[0]
    assert got.output_ids == want.output_ids
    assert max(abs(a - b) for a, b in zip(got.output_logprobs, want.output_logprobs)) < 1e-5
    with pytest.raises(Exception, match="deepstack_embeds"):
        e.generate([ids], [sp], mm=dict(image_embeds=out, image_grid_thw=grid))
