"""Vision inputs: the image encoder, the multi-axis rotary positions and the whole model against the Transformers
implementation of Qwen3.5 with random weights (the library serves as the oracle here, nothing else uses it)."""

import pytest
import torch

from slime_b200.models import vision
from slime_b200.models.config import ModelConfig
from slime_b200.models.gpt import GPTModel, PackedSeqParams
from slime_b200.weight_sync import convert

IMG, VID, VSTART, VEND = 190, 191, 192, 193


def _hf_model():
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5Config
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForConditionalGeneration

    text = dict(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2,
                linear_num_value_heads=4, full_attention_interval=2, rms_norm_eps=1e-6, max_position_embeddings=512,
                layer_types=["linear_attention", "full_attention"] * 2,
                rope_parameters=dict(rope_type="default", rope_theta=10000.0, partial_rotary_factor=0.5, mrope_section=[4, 2, 2],
                                     mrope_interleaved=True))  # fmt: skip
    vis = dict(depth=2, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=64, num_position_embeddings=64, in_channels=3)  # fmt: skip
    cfg = Qwen3_5Config(text_config=text, vision_config=vis, image_token_id=IMG, video_token_id=VID, vision_start_token_id=VSTART,
                        vision_end_token_id=VEND)  # fmt: skip
    torch.manual_seed(0)
    model = Qwen3_5ForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():  # the library's init leaves norms at 1 / biases at 0: make every tensor matter
            p.add_(torch.randn_like(p) * 0.05)
    return cfg, model


@pytest.fixture(scope="module")
def pair():
    hf_cfg, hf = _hf_model()
    d = hf_cfg.to_dict()
    d["architectures"] = ["Qwen3_5ForConditionalGeneration"]
    cfg = ModelConfig.from_hf(d)
    assert cfg.vision["depth"] == 2 and cfg.image_token_id == IMG and cfg.mrope_section == [4, 2, 2] and cfg.mrope_interleaved
    assert cfg.rotary_percent == 0.5 and cfg.full_attention_interval == 2
    ours = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=1)
    sd = hf.state_dict()
    with torch.no_grad():
        for name, p in list(ours.named_parameters()) + list(ours.named_buffers()):
            names, rule = convert.hf_sources_for(cfg, name)
            p.copy_(convert.merge_hf_sources(rule, [sd[n] for n in names], cfg))
    return hf_cfg, hf, cfg, ours


def _image_inputs(grids, seed=0):
    g = torch.Generator().manual_seed(seed)
    n = sum(t * h * w for t, h, w in grids)
    return torch.randn(n, 3 * 2 * 4 * 4, generator=g), torch.tensor(grids)


def test_vision_tower_matches_the_library_encoder(pair):
    _, hf, _, ours = pair
    px, grid = _image_inputs([[1, 4, 6], [1, 8, 4], [2, 4, 4]])
    with torch.no_grad():
        want = hf.model.visual(px, grid_thw=grid).pooler_output
        got = ours.vision(px, grid)
    assert got.shape == want.shape == (6 + 8 + 8, 64)
    assert (got - want).abs().max() < 2e-5, float((got - want).abs().max())


def test_position_streams_match_the_library(pair):
    _, hf, cfg, _ = pair
    ids = torch.tensor([[5, 6, VSTART] + [IMG] * 6 + [VEND, 7, 8, VSTART] + [IMG] * 8 + [VEND, 9, 10, 11]])
    grid = torch.tensor([[1, 4, 6], [1, 8, 4]])
    import inspect

    kw = dict(mm_token_type_ids=(ids == IMG).int()) if "mm_token_type_ids" in inspect.signature(hf.model.get_rope_index).parameters else {}
    want, want_delta = hf.model.get_rope_index(ids, image_grid_thw=grid, **kw)
    got, delta = vision.mrope_position_ids(ids, [0, ids.numel()], grid, None, image_token_id=IMG, video_token_id=VID, spatial_merge_size=2)
    assert torch.equal(got, want[:, 0]) and delta[0] == int(want_delta.reshape(-1)[0])
    # packed: every sequence restarts at zero and consumes its own grids
    two, d2 = vision.mrope_position_ids(torch.cat([ids[0], ids[0]]), [0, ids.numel(), 2 * ids.numel()], torch.cat([grid, grid]), None,
                                        image_token_id=IMG, video_token_id=VID)  # fmt: skip
    assert torch.equal(two[:, : ids.numel()], got) and torch.equal(two[:, ids.numel() :], got) and d2 == [delta[0]] * 2
    with pytest.raises(ValueError, match="more grids"):
        vision.mrope_position_ids(ids, [0, ids.numel()], torch.cat([grid, grid]), None, image_token_id=IMG)
    with pytest.raises(ValueError, match="shorter than its grid"):
        vision.mrope_position_ids(ids[:, :8], [0, 8], grid[:1], None, image_token_id=IMG)
    axes = vision.mrope_band_axes([4, 2, 2], 8, True)
    assert axes.tolist() == [0, 1, 2, 0, 1, 2, 0, 0]
    assert vision.mrope_band_axes([4, 2, 2], 8, False).tolist() == [0, 0, 0, 0, 1, 1, 2, 2]


def test_whole_model_with_an_image_matches_the_library(pair):
    _, hf, cfg, ours = pair
    ids = torch.tensor([[5, 6, VSTART] + [IMG] * 6 + [VEND, 7, 8, VSTART] + [IMG] * 8 + [VEND, 9, 10, 11]])
    px, grid = _image_inputs([[1, 4, 6], [1, 8, 4]], seed=3)
    with torch.no_grad():
        import inspect

        kw = dict(mm_token_type_ids=(ids == IMG).int()) if "mm_token_type_ids" in inspect.signature(hf.forward).parameters else {}
        want = hf(input_ids=ids, pixel_values=px, image_grid_thw=grid, **kw).logits[0]
        got = ours(ids, pixel_values=px, image_grid_thw=grid)[0]
        text_only = ours(ids)[0]
    assert (got - want).abs().max() < 2e-4, float((got - want).abs().max())
    assert (text_only - want).abs().max() > 1e-2  # the image matters
    # two samples packed into one stream give each sample's own logits
    packed = PackedSeqParams(torch.tensor([0, ids.numel(), 2 * ids.numel()], dtype=torch.int32), ids.numel())
    with torch.no_grad():
        both = ours(torch.cat([ids[0], ids[0]]), packed_seq_params=packed, pixel_values=torch.cat([px, px]), image_grid_thw=torch.cat([grid, grid]))[0]
    assert (both[: ids.numel()] - got).abs().max() < 1e-4 and (both[ids.numel() :] - got).abs().max() < 1e-4


def test_image_encoder_receives_gradients_and_names_round_trip(pair):
    _, hf, cfg, ours = pair
    ids = torch.tensor([[5, VSTART] + [IMG] * 4 + [VEND, 7, 8]])
    px, grid = _image_inputs([[1, 4, 4]], seed=5)
    ours.zero_grad()
    ours(ids, pixel_values=px, image_grid_thw=grid).float().logsumexp(-1).sum().backward()
    assert float(ours.vision.merger.linear_fc2.weight.grad.abs().sum()) > 0 and float(ours.vision.patch_embed.proj.weight.grad.abs().sum()) > 0
    sd = hf.state_dict()
    out = dict(x for n, p in list(ours.named_parameters()) + list(ours.named_buffers()) for x in convert.convert_to_hf(cfg, n, p.detach()))
    assert set(out) == set(sd), (sorted(set(out) - set(sd))[:5], sorted(set(sd) - set(out))[:5])
    for k in sd:
        assert torch.allclose(out[k], sd[k], atol=1e-6), k


def _engine(pair, **kw):
    from slime_b200.engine.engine import Engine
    from slime_b200.engine.server_args import ServerArgs

    _, hf, cfg, _ = pair
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=4, context_length=128, disable_cuda_graph=True, **kw), device="cpu", num_pages=96)
    missing = e.weights.load_weights(list(hf.state_dict().items()))  # the checkpoint's own names, language model nested
    assert not missing, missing
    return e


@pytest.mark.parametrize("chunk", [8192, 5])
def test_engine_with_images_reproduces_the_trainer(pair, chunk):
    """Prompt log-probs (prefill, also when an image spans several chunks) and greedy decode log-probs of a request with
    two images equal the trainer's teacher-forced ones; a text-only request next to it is unaffected."""
    import numpy as np

    _, _, cfg, ours = pair
    e = _engine(pair, chunked_prefill_size=chunk)
    ids = [5, 6, VSTART] + [IMG] * 6 + [VEND, 7, 8, VSTART] + [IMG] * 8 + [VEND, 9, 10, 11]
    px, grid = _image_inputs([[1, 4, 6], [1, 8, 4]], seed=3)
    mm = dict(pixel_values=px, image_grid_thw=grid)

    def trainer_logprobs(tokens):
        with torch.no_grad():
            lg = ours(torch.tensor(tokens), pixel_values=px, image_grid_thw=grid)[0]
        return lg.log_softmax(-1)[:-1].gather(-1, torch.tensor(tokens[1:])[:, None]).squeeze(-1).numpy()

    r = e.generate([ids], [dict(max_new_tokens=0)], logprob_start_len=0, mm=mm)[0]
    assert np.abs(np.array(r.input_logprobs[1:]) - trainer_logprobs(ids)).max() < 2e-4
    text = [5, 6, 7, 8, 9, 10, 11, 12]
    a = e.add_request(ids, dict(max_new_tokens=7, temperature=0, ignore_eos=True), mm=mm)
    b = e.add_request(text, dict(max_new_tokens=7, temperature=0, ignore_eos=True))
    while e.has_work():
        e.step()
    assert a.rope_delta == (3 - 6) + (4 - 8)  # an image of 2 x 3 (4 x 2) merged patches advances the position by 3 (4), not by 6 (8)
    ref = trainer_logprobs(ids + a.output_ids)[len(ids) - 1 :]
    assert np.abs(np.array(a.output_logprobs) - ref).max() < 2e-4, np.abs(np.array(a.output_logprobs) - ref).max()
    with torch.no_grad():
        lg = ours(torch.tensor(text + b.output_ids))[0].log_softmax(-1)
    ref_b = lg[len(text) - 1 : -1].gather(-1, torch.tensor(b.output_ids)[:, None]).squeeze(-1).numpy()
    assert np.abs(np.array(b.output_logprobs) - ref_b).max() < 2e-4
    # prompts with images neither offer nor reuse cached prefixes (placeholder ids do not identify the image)
    again = e.generate([ids], [dict(max_new_tokens=2, temperature=0, ignore_eos=True)], mm=dict(pixel_values=px * 0.5, image_grid_thw=grid))[0]
    assert again.num_cached_tokens == 0 and again.output_logprobs != a.output_logprobs[:2]


def test_generate_endpoint_takes_images(pair):
    import base64
    import io

    import numpy as np
    import requests
    from PIL import Image

    from slime_b200.engine.http_server import EngineServer
    from slime_b200.utils.image_processing import ImageProcessor, expand_image_placeholders

    _, _, cfg, _ = pair
    e = _engine(pair)
    srv = EngineServer(e, port=0).start(block=False)
    try:
        url = f"http://127.0.0.1:{srv.port}"
        rng = np.random.default_rng(0)
        imgs = [Image.fromarray(rng.integers(0, 255, (16, 24, 3), dtype=np.uint8)), Image.fromarray(rng.integers(0, 255, (32, 16, 3), dtype=np.uint8))]

        def b64(im):
            buf = io.BytesIO()
            im.save(buf, format="PNG")
            return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()

        short = [5, VSTART, IMG, VEND, 7, VSTART, IMG, VEND, 9]  # one placeholder per image, as a chat template writes them
        body = {"input_ids": short, "image_data": [b64(i) for i in imgs], "return_logprob": True,
                "sampling_params": {"max_new_tokens": 5, "temperature": 0, "ignore_eos": True}}  # fmt: skip
        out = requests.post(url + "/generate", json=body, timeout=60).json()
        ip = ImageProcessor.from_vision_config(cfg.vision)
        mm = ip(imgs)
        counts = [ip.tokens_for(g) for g in mm["image_grid_thw"].tolist()]  # small images are scaled up to the minimum area
        full = expand_image_placeholders(short, IMG, counts)
        assert out["meta_info"]["prompt_tokens"] == len(full) == len(short) + sum(counts) - 2
        want = e.generate([full], [dict(max_new_tokens=5, temperature=0, ignore_eos=True)], mm=mm)[0]
        assert out["output_ids"] == want.output_ids
        # an already expanded prompt is taken as it is; a prompt whose runs do not fit its images is refused
        out2 = requests.post(url + "/generate", json=dict(body, input_ids=full), timeout=60).json()
        assert out2["output_ids"] == want.output_ids
        bad = requests.post(url + "/generate", json=dict(body, input_ids=short[:4]), timeout=60)
        assert bad.status_code == 400 and "image" in bad.json()["error"]
    finally:
        srv.shutdown()


def test_image_processor_matches_the_library_patch_layout():
    import numpy as np
    from PIL import Image
    from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor

    from slime_b200.utils.image_processing import ImageProcessor, smart_resize

    rng = np.random.default_rng(0)
    exact = [Image.fromarray(rng.integers(0, 255, (32, 48, 3), dtype=np.uint8))]  # already a multiple of patch * merge: no resize
    odd = [Image.fromarray(rng.integers(0, 255, (37, 61, 3), dtype=np.uint8)), Image.fromarray(rng.integers(0, 255, (64, 32, 3), dtype=np.uint8))]
    kw = dict(patch_size=4, temporal_patch_size=2, merge_size=2, min_pixels=16 * 16, max_pixels=64 * 64)
    hf, mine = Qwen2VLImageProcessor(**kw), ImageProcessor(**kw)
    a, b = hf(images=exact, return_tensors="pt"), mine(exact)
    assert a["image_grid_thw"].tolist() == b["image_grid_thw"].tolist() == [[1, 8, 12]]
    assert (a["pixel_values"] - b["pixel_values"]).abs().max() < 1e-5
    a, b = hf(images=odd, return_tensors="pt"), mine(odd)
    assert a["image_grid_thw"].tolist() == b["image_grid_thw"].tolist()
    assert (a["pixel_values"] - b["pixel_values"]).abs().max() < 0.05  # resampling filters differ by a grey level
    assert smart_resize(1000, 3000, 32, 56 * 56, 64 * 64 * 4)[0] * smart_resize(1000, 3000, 32, 56 * 56, 64 * 64 * 4)[1] <= 64 * 64 * 4
    assert mine.tokens_for([1, 8, 12]) == 24


def test_micro_batch_concatenates_processor_outputs_in_stream_order(pair):
    """Samples with and without images in one micro-batch: the model kwargs are the per-sample tensors joined in order."""
    from slime_b200.backends.train.data import DataIterator, get_batch

    _, _, cfg, ours = pair
    a = [5, VSTART] + [IMG] * 4 + [VEND, 7, 8]
    b = [9, 10, 11]
    c = [6, VSTART] + [IMG] * 6 + [VEND, 12]
    pa, ga = _image_inputs([[1, 4, 4]], seed=1)
    pc, gc = _image_inputs([[1, 4, 6]], seed=2)
    data = {"tokens": [torch.tensor(a), torch.tensor(b), torch.tensor(c)],
            "multimodal_train_inputs": [dict(pixel_values=pa, image_grid_thw=ga), None, dict(pixel_values=pc, image_grid_thw=gc)]}  # fmt: skip
    batch = get_batch(DataIterator(data, [[0, 1, 2]]), ["tokens", "multimodal_train_inputs"], pad_multiplier=1)
    mm = batch["multimodal"]
    assert torch.equal(mm["pixel_values"], torch.cat([pa, pc])) and mm["image_grid_thw"].tolist() == [[1, 4, 4], [1, 4, 6]]
    with torch.no_grad():
        packed = ours(batch["tokens"], batch["position_ids"], packed_seq_params=batch["packed_seq_params"], **mm)[0]
        alone = ours(torch.tensor(c), pixel_values=pc, image_grid_thw=gc)[0]
    assert (packed[len(a) + len(b) :] - alone).abs().max() < 1e-4


def test_position_streams_golden_vector_and_packed_reset():
    """Two identical samples [start, 4 image tokens of a 4 x 4 grid merged 2 x 2, end, text]: temporal stays, height and
    width spread over the 2 x 2 grid, text continues after the larger side; every packed sample restarts at zero."""
    ids = torch.tensor([99, 10, 10, 10, 10, 98, 7, 99, 10, 10, 10, 10, 98, 8])
    got, delta = vision.mrope_position_ids(ids, [0, 7, 14], torch.tensor([[1, 4, 4], [1, 4, 4]]), None, image_token_id=10, video_token_id=20)
    want = torch.tensor([[0, 1, 1, 1, 1, 3, 4], [0, 1, 1, 2, 2, 3, 4], [0, 1, 2, 1, 2, 3, 4]])
    assert torch.equal(got[:, :7], want) and torch.equal(got[:, 7:], want) and delta == [-2, -2]
    with pytest.raises(ValueError, match="more grids"):
        vision.mrope_position_ids(torch.tensor([1, 2, 3]), [0, 3], torch.tensor([[1, 4, 4]]), None, image_token_id=10, video_token_id=20)
    # a two-frame video is two one-frame runs, each between its own markers
    vid = torch.tensor([99, 20, 20, 20, 20, 98, 99, 20, 20, 20, 20, 98, 5])
    got, _ = vision.mrope_position_ids(vid, [0, 13], None, torch.tensor([[2, 4, 4]]), image_token_id=10, video_token_id=20)
    assert got[0].tolist() == [0, 1, 1, 1, 1, 3, 4, 5, 5, 5, 5, 7, 8] and got[2].tolist() == [0, 1, 2, 1, 2, 3, 4, 5, 6, 5, 6, 7, 8]


def test_generate_endpoint_takes_video_frames(pair):
    """A clip arrives as a list of frames; frame pairs form one temporal patch each, every pair has its own placeholder
    run, and the engine's answer equals the direct call's and the trainer's."""
    import base64
    import io

    import numpy as np
    import requests
    from PIL import Image

    from slime_b200.engine.http_server import EngineServer
    from slime_b200.utils.image_processing import ImageProcessor

    _, _, cfg, ours = pair
    ip = ImageProcessor.from_vision_config(cfg.vision, min_pixels=16 * 16, max_pixels=64 * 64)
    rng = np.random.default_rng(1)
    frames = [Image.fromarray(rng.integers(0, 255, (16, 24, 3), dtype=np.uint8)) for _ in range(3)]
    rows, grid = ip.video(frames)
    assert grid == [2, 4, 6] and rows.shape == (48, 3 * 2 * 4 * 4)
    still, g1 = ip.one(frames[2])
    assert g1 == [1, 4, 6] and torch.equal(rows[24:], still)  # the odd last frame repeats, like a still image
    pair01 = rows[:24].reshape(24, 3, 2, 16)
    assert torch.equal(pair01[:, :, 0], ip.one(frames[0])[0].reshape(24, 3, 2, 16)[:, :, 0])
    assert torch.equal(pair01[:, :, 1], ip.one(frames[1])[0].reshape(24, 3, 2, 16)[:, :, 0])

    e = _engine(pair)
    srv = EngineServer(e, port=0).start(block=False)
    try:
        def b64(im):
            buf = io.BytesIO()
            im.save(buf, format="PNG")
            return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()

        short = [5, VSTART, VID, VEND, 6, VSTART, VID, VEND, 9]  # one placeholder per frame pair, each between its own markers
        body = {"input_ids": short, "video_data": [[b64(f) for f in frames]], "return_logprob": True,
                "sampling_params": {"max_new_tokens": 4, "temperature": 0, "ignore_eos": True}}  # fmt: skip
        out = requests.post(f"http://127.0.0.1:{srv.port}/generate", json=body, timeout=60).json()
        own = ImageProcessor.from_vision_config(cfg.vision)(videos=[frames])
        n = int(own["video_grid_thw"][0, 1] * own["video_grid_thw"][0, 2]) // 4
        full = [5, VSTART] + [VID] * n + [VEND, 6, VSTART] + [VID] * n + [VEND, 9]
        assert out["meta_info"]["prompt_tokens"] == len(full)
        want = e.generate([full], [dict(max_new_tokens=4, temperature=0, ignore_eos=True)], mm=own)[0]
        assert out["output_ids"] == want.output_ids
        with torch.no_grad():
            toks = full + want.output_ids
            lg = ours(torch.tensor(toks), pixel_values_videos=own["pixel_values_videos"], video_grid_thw=own["video_grid_thw"])[0]
        ref = lg.log_softmax(-1)[len(full) - 1 : -1].gather(-1, torch.tensor(want.output_ids)[:, None]).squeeze(-1)
        assert (torch.tensor(want.output_logprobs) - ref).abs().max() < 2e-4
        bad = requests.post(f"http://127.0.0.1:{srv.port}/generate", json=dict(body, input_ids=short[:4]), timeout=60)
        assert bad.status_code == 400 and "vision inputs" in bad.json()["error"]
    finally:
        srv.shutdown()


def test_video_patch_layout_matches_the_library_processor():
    import numpy as np

    from slime_b200.utils.image_processing import ImageProcessor

    vp_mod = pytest.importorskip("transformers.models.qwen3_vl.video_processing_qwen3_vl")
    try:
        vp = vp_mod.Qwen3VLVideoProcessor(patch_size=4, temporal_patch_size=2, merge_size=2, do_sample_frames=False,
                                          size={"shortest_edge": 16 * 16, "longest_edge": 64 * 64 * 8})  # fmt: skip
    except ImportError as e:  # the library's processor wants torchvision
        pytest.skip(str(e))
    clip = np.random.default_rng(0).integers(0, 255, (4, 32, 48, 3), dtype=np.uint8)
    want = vp(videos=[torch.from_numpy(clip).permute(0, 3, 1, 2)], return_tensors="pt")
    ip = ImageProcessor(patch_size=4, temporal_patch_size=2, merge_size=2, min_pixels=16 * 16, max_pixels=64 * 64,
                        mean=tuple(vp.image_mean), std=tuple(vp.image_std))  # fmt: skip
    rows, grid = ip.video(list(clip))
    assert grid == want["video_grid_thw"][0].tolist() == [2, 8, 12]
    assert (rows - want["pixel_values_videos"]).abs().max() < 1e-6
