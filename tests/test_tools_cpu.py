"""Converter tools on CPU: HF -> torch_dist -> HF is the identity on a tiny model."""

import json
import os

import torch


def _tiny_hf_dir(path):
    from safetensors.torch import save_file

    from slime_b200.backends.train.model import TrainModel
    from slime_b200.checkpoint.hf_saver import iter_hf_tensors
    from slime_b200.models.config import get_preset
    from slime_b200.utils.arguments import namespace_from_dict

    os.makedirs(path, exist_ok=True)
    cfg = get_preset("tiny")
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_hf_dict(), f)
    args = namespace_from_dict(dict(hf_checkpoint=path, num_rollout=0, rollout_batch_size=1, seed=7))
    model = TrainModel(args, device=torch.device("cpu"), with_optimizer=False)
    tensors = {n: t.detach().clone().contiguous() for n, t in iter_hf_tensors(model)}
    save_file(tensors, os.path.join(path, "model.safetensors"))
    return tensors


def test_hf_torch_dist_roundtrip(tmp_path):
    from safetensors import safe_open

    from slime_b200.tools import convert_hf_to_torch_dist, convert_torch_dist_to_hf

    hf = str(tmp_path / "hf")
    original = _tiny_hf_dir(hf)
    native = str(tmp_path / "native")
    convert_hf_to_torch_dist.main(["--hf-checkpoint", hf, "--save", native, "--device", "cpu"])
    assert open(os.path.join(native, "latest_checkpointed_iteration.txt")).read().strip() == "release"
    back = str(tmp_path / "back")
    convert_torch_dist_to_hf.main(["--input-dir", os.path.join(native, "release"), "--output-dir", back, "--origin-hf-dir", hf,
                                   "--chunk-size", "200000"])  # fmt: skip
    index = json.load(open(os.path.join(back, "model.safetensors.index.json")))["weight_map"]
    assert set(index) == set(original) and len(set(index.values())) > 1  # several shards were written
    for name, fname in index.items():
        with safe_open(os.path.join(back, fname), framework="pt") as f:
            assert torch.equal(f.get_tensor(name), original[name]), name
    assert os.path.exists(os.path.join(back, "config.json"))


def test_fp8_convert_and_cast_back(tmp_path):
    from safetensors import safe_open

    from slime_b200.tools import convert_hf_to_fp8, fp8_cast_bf16

    hf = str(tmp_path / "hf")
    original = _tiny_hf_dir(hf)
    fp8 = str(tmp_path / "fp8")
    wm = convert_hf_to_fp8.convert(hf, fp8, "block", (128, 128), device="cpu")
    cfg = json.load(open(os.path.join(fp8, "config.json")))
    assert cfg["quantization_config"]["weight_block_size"] == [128, 128]
    q_name = "model.layers.0.mlp.down_proj.weight"
    assert q_name + "_scale_inv" in wm and "model.embed_tokens.weight_scale_inv" not in wm
    with safe_open(os.path.join(fp8, wm[q_name]), framework="pt") as f:
        q, s = f.get_tensor(q_name), f.get_tensor(q_name + "_scale_inv")
        assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32
        assert s.shape == (-(-q.shape[0] // 128), -(-q.shape[1] // 128))
        assert f.get_tensor("model.norm.weight").dtype == torch.bfloat16
    back = str(tmp_path / "bf16")
    assert fp8_cast_bf16.convert(fp8, back, device="cpu") > 0
    assert "quantization_config" not in json.load(open(os.path.join(back, "config.json")))
    with safe_open(os.path.join(back, "model.safetensors"), framework="pt") as f:
        w = f.get_tensor(q_name).float()
    ref = original[q_name].float()
    assert (w - ref).abs().max() <= 0.07 * ref.abs().max()  # e4m3 has 3 mantissa bits
    for strategy in ("channel", "tensor"):
        wm2 = convert_hf_to_fp8.convert(hf, str(tmp_path / strategy), strategy, device="cpu")
        assert q_name + "_scale" in wm2


def test_int4_direct_conversion(tmp_path):
    from safetensors import safe_open

    from slime_b200.tools import convert_hf_to_int4_direct as tool

    hf = str(tmp_path / "hf")
    original = _tiny_hf_dir(hf)
    out = str(tmp_path / "int4")
    assert tool.convert(hf, out, 32, device="cpu")["quantised"] == 0  # dense model: the default list keeps everything bf16
    stats = tool.convert(hf, out, 32, ignore=[r".*embed.*", r".*norm.*", r".*lm_head.*"], device="cpu")
    assert stats["quantised"] > 0
    name = "model.layers.1.mlp.down_proj"
    with safe_open(os.path.join(out, "model.safetensors"), framework="pt") as f:
        packed, scale, shape = (f.get_tensor(f"{name}.weight_{k}") for k in ("packed", "scale", "shape"))
        assert f"{name}.weight" not in f.keys()
    w = original[name + ".weight"].float()
    assert shape.tolist() == list(w.shape) and packed.shape == (w.shape[0], w.shape[1] // 8)
    codes = torch.stack([((packed >> (4 * i)) & 0xF) - 8 for i in range(8)], -1).reshape(w.shape).float()
    deq = (codes.view(w.shape[0], -1, 32) * scale.float()[..., None]).view(w.shape)
    assert (deq - w).abs().max() <= w.abs().max() / 7 * 0.51 + 1e-3  # half a quantisation step of the largest group
    cfg = json.load(open(os.path.join(out, "config.json")))["quantization_config"]
    assert cfg["format"] == "pack-quantized" and cfg["config_groups"]["group_0"]["weights"]["group_size"] == 32
    # and back: the packed triples become bf16 weights again, within half a quantisation step of the originals
    from slime_b200.tools import convert_int4_to_bf16 as back

    restored_dir = str(tmp_path / "bf16")
    stats2 = back.convert(out, restored_dir, device="cpu")
    assert stats2["restored"] == stats["quantised"] and "quantization_config" not in json.load(open(os.path.join(restored_dir, "config.json")))
    with safe_open(os.path.join(restored_dir, "model.safetensors"), framework="pt") as f:
        names = set(f.keys())
        assert not any(n.endswith(("weight_packed", "weight_scale", "weight_shape")) for n in names) and names == set(original)
        got = f.get_tensor(name + ".weight")
    assert got.dtype == torch.bfloat16 and (got.float() - deq).abs().max() <= deq.abs().max() * 2**-8


def test_model_presets_round_trip_through_flags():
    """Every supported preset, printed as flags and parsed back, gives the same architecture."""
    import dataclasses

    from slime_b200.models import presets
    from slime_b200.models.config import PRESETS, ModelConfig, _register_more_presets, get_preset
    from slime_b200.utils.arguments import parse_args

    _register_more_presets()
    assert {"qwen2.5-7b", "qwen3-14b", "qwen3-235b-a22b", "llama3.1-8b-instruct", "mimo-7b-rl"} <= set(PRESETS)
    for name in sorted(PRESETS):
        cfg = get_preset(name)
        args = parse_args(presets.to_flags(cfg) + ["--rollout-batch-size", "1", "--num-rollout", "1", "--debug-train-only"])
        if cfg.vision:
            args.hf_checkpoint = f"preset:{name}"  # the image encoder has no flags: it is read from the checkpoint's config
        back = ModelConfig.from_args(args)
        for f in dataclasses.fields(ModelConfig):
            if f.name in ("model_arch", "padded_vocab_size", "init_method_std"):
                continue
            a, b = getattr(cfg, f.name), getattr(back, f.name)
            if f.name == "moe_layer_freq" and a is not None:
                a, b = list(a), list(b) if not isinstance(b, int) else b
            assert a == b, (name, f.name, a, b)
    vl = get_preset("qwen3.5-35b-a3b-vl")
    assert vl.vision["depth"] == 27 and vl.mixer(3) == "general_attention" and vl.num_params() - get_preset("qwen3.5-35b-a3b").num_params() > 4e8
    assert abs(get_preset("qwen3-vl-8b").num_params() / 1e9 - 8.77) < 0.01  # the published size, deepstack mergers included
    assert get_preset("qwen3-235b-a22b").num_params() > 2.3e11
    # the parameter counts of the latent-attention and hybrid families agree with the published sizes
    for name, billions in (("deepseek-v3", 671), ("kimi-k2", 1026), ("glm5-744b-a40b", 744), ("qwen3-next-80b-a3b", 80),
                           ("minimax-m2", 229), ("moonlight", 16)):  # fmt: skip
        assert abs(get_preset(name).num_params() / 1e9 - billions) < 1.0, name
    kinds = [get_preset("qwen3-next-80b-a3b").mixer(i) for i in range(8)]
    assert kinds == ["gated_delta_net"] * 3 + ["general_attention"] + ["gated_delta_net"] * 3 + ["general_attention"]
    assert get_preset("glm5-744b-a40b").mixer(0) == "dsa" and get_preset("kimi-k2").mixer(5) == "mla"


def test_run_recipes_produce_parseable_command_lines(tmp_path):
    """Every recipe, in DRY_RUN mode, prints a command line that the argument parser accepts."""
    import glob
    import os
    import subprocess

    ckpt, data = tmp_path / "ckpt", tmp_path / "data"
    models = ["Qwen2.5-0.5B-Instruct", "Qwen3-4B", "Qwen3-30B-A3B", "Qwen3-8B", "Qwen3-32B", "Qwen3-235B-A22B", "Qwen3-4B-Base",
              "Qwen3-4B-retool-sft", "GLM-Z1-9B-0414", "GLM-4.7-30B-A3B", "GLM-4.5-355B-A32B", "GLM-5", "GLM-5.2", "Kimi-K2-Instruct",
              "Kimi-K2-Thinking", "DeepSeek-R1", "MiMo-7B-RL", "MiniMax-M2", "Moonlight-16B-A3B", "Qwen3-Next-80B-A3B-Thinking",
              "Qwen3.5-27B", "Qwen3.5-35B-A3B"]  # fmt: skip
    for d in [m + suffix for m in models for suffix in ("", "_torch_dist")]:
        (ckpt / d).mkdir(parents=True)
    for f in ("gsm8k/train.jsonl", "gsm8k/test.jsonl", "dapo-math-17k/dapo-math-17k.jsonl", "aime-2024/aime-2024.jsonl",
              "openhermes2_5/openhermes2_5.parquet"):
        (data / f).parent.mkdir(parents=True, exist_ok=True)
        (data / f).write_text("")

    from slime_b200.utils.arguments import parse_args

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    scripts = sorted(glob.glob(os.path.join(root, "recipes", "run-*.sh")))
    assert len(scripts) >= 23  # one per launch recipe of the reference's scripts/ folder
    # launch lines of the script-based examples go through the same parser
    examples = [os.path.join(root, "examples", p) for p in (
        "delta_weight_sync/run-qwen3-30B-A3B-delta.sh", "on_policy_distillation/run-qwen3-8B-opd.sh",
        "fully_async/run-qwen2.5-0.5B-fully_async.sh", "eval_multi_task/multi_task.sh", "retool/retool_qwen3_4b_rl.sh")]  # fmt: skip
    for script in examples:
        r = subprocess.run(["bash", script], env=dict(os.environ, DRY_RUN="1", NUM_GPUS="8", CKPT_DIR=str(ckpt), DATA_DIR=str(data)), capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr[-2000:]
        argv = r.stdout.strip().split("\n")
        args = parse_args(argv[1:])
        if "delta" in script:
            assert args.update_weight_mode == "delta" and args.update_weight_delta_encoding == "xor"
        if "opd" in script:
            assert args.use_opd and args.opd_type == "megatron" and args.opd_kl_coef == 1.0
        if "multi_task" in script:
            assert args.eval_config.endswith("multi_task.yaml")
    for script in scripts:
        r = subprocess.run(["bash", script], env=dict(os.environ, DRY_RUN="1", NUM_GPUS="8", CKPT_DIR=str(ckpt), DATA_DIR=str(data)), capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr[-2000:]
        argv = r.stdout.strip().split("\n")
        assert argv[0] in ("train.py", "train_async.py")
        args = parse_args(argv[1:])
        assert args.num_layers > 0
        if "sft" in script:
            assert args.loss_type == "sft_loss" and args.debug_train_only and args.rollout_batch_size == 128
        else:
            assert args.rollout_batch_size in (8, 32, 64, 128) and args.n_samples_per_prompt in (4, 8)
        base = os.path.basename(script)
        if base == "run-deepseek-r1.sh":
            assert args.multi_latent_attention and args.q_lora_rank == 1536 and args.sglang_quantization == "fp8"
            assert args.moe_router_num_groups == 8 and args.expert_model_parallel_size == 32 and args.actor_num_nodes == 16
        if base == "run-glm5-744B-A40B.sh":
            assert args.index_topk == 2048 and args.v_head_dim == 256 and args.context_parallel_size == 2
        if base == "run-qwen3-next-80B-A3B.sh":
            assert args.full_attention_interval == 4 and args.attention_output_gate and args.advantage_estimator == "gspo"
        if base == "run-mimo-7B-rl-mtp.sh":
            assert args.enable_mtp_training and args.mtp_num_layers == 1
        if base == "run-glm4-9B.sh":
            assert args.rotary_percent == 0.5 and args.rotary_interleaved and args.post_mlp_layernorm
        if base == "run-minimax-m2.sh":
            assert args.qk_layernorm_full and args.moe_router_score_function == "sigmoid"
        if "qwen3-8B" in script:
            assert args.use_critic and args.advantage_estimator == "ppo"
        if base == "run-qwen3-32B.sh":
            assert args.tensor_model_parallel_size == 4 and args.rollout_num_gpus == 4 and not args.colocate
        if "reproducibility" in script:
            assert args.deterministic_mode
        if base == "run-qwen3-30B-A3B.sh":
            assert args.num_experts == 128 and args.expert_model_parallel_size == 8 and args.sglang_ep_size == 8
        if "async" in script:
            assert args.rollout_function_path.endswith("generate_rollout_fully_async") and not args.colocate
