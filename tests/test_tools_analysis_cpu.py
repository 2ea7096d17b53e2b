"""Profile analyser and rollout timeline viewer on small synthetic inputs."""

import gzip
import json

import pytest
import torch

from slime_b200.observability import trace_utils
from slime_b200.tools import analyze_profile as ap
from slime_b200.tools import trace_timeline_viewer as tv
from slime_b200.utils.types import Sample


def _trace():
    ev = []

    def k(name, ts, dur, tid=7, cat="kernel"):
        ev.append({"ph": "X", "cat": cat, "name": name, "ts": ts, "dur": dur, "tid": tid, "pid": 0})

    k("void sb::gemm_bf16_kernel<256, 4>(...)", 100, 50)
    k("void sb::decode_attn_kernel<64, 7>(...)", 150, 30)
    k("ncclDevKernel_AllReduce_Sum_bf16", 200, 20, tid=9)
    k("sb::rmsnorm_fwd_kernel", 1000, 10)
    k("Memcpy HtoD", 1010, 5, cat="gpu_memcpy")
    ev.append({"ph": "X", "cat": "cpu_op", "name": "aten::copy_", "ts": 300, "dur": 650, "tid": 1, "pid": 0})
    for i, ts in enumerate((90, 95, 98, 900, 905)):
        ev.append({"ph": "X", "cat": "cuda_runtime", "name": "cudaGraphLaunch", "ts": ts, "dur": 2, "tid": 1, "pid": 0})
    ev.append({"ph": "X", "cat": "cuda_runtime", "name": "cudaStreamSynchronize", "ts": 1020, "dur": 4, "tid": 1, "pid": 0})
    return {"traceEvents": ev, "deviceProperties": [{"name": "B200", "numSms": 148, "totalGlobalMem": 180 * 2**30}],
            "cuda_runtime_version": 12090, "distributedInfo": {"nccl_version": "2.28.9", "world_size": 2}}


def test_analyze_profile(tmp_path, capsys):
    assert ap.classify_kernel("void sb::gemm_bf16_kernel<128, 6>") == "gemm"
    assert ap.classify_kernel("flash::flash_fwd_kernel") == "attention"
    assert ap.classify_kernel("sb::dp_reduce_shard_kernel<true>") == "communication"
    assert ap.classify_kernel("sb::swiglu_fwd_kernel") == "norm+activation"
    assert ap.classify_kernel("mystery") == "other"
    r = ap.analyze_trace(_trace(), "rank0")
    assert r.gpu_name == "B200" and r.cuda_version == "12.9" and r.world_size == 2
    assert r.kernel_count == 4 and r.kernel_us == 110
    assert r.gpu_busy_us == 115 and r.gpu_span_us == 915  # 100..180, 200..220 and 1000..1015
    assert r.categories["gemm"].total_us == 50 and r.comm_us == 20
    assert r.top_gaps[0]["gap_us"] == 780 and r.top_gaps[0]["cause"] == "aten::copy_"
    assert r.graph_launches == 5 and len(r.decode_steps) == 2
    assert r.copy_count == 1 and r.sync_count == 1 and set(r.streams) == {"7", "9"}
    for i in range(2):
        with gzip.open(tmp_path / f"engine-rank{i}.trace.json.gz", "wt") as f:
            json.dump(_trace(), f)
    out_json = tmp_path / "out.json"
    assert ap.main(["--profile-dir", str(tmp_path), "--all-ranks", "--json", str(out_json)]) == 0
    text = capsys.readouterr().out
    assert "across ranks" in text and "GPU utilisation" in text and "gemm" in text
    assert len(json.loads(out_json.read_text())) == 2
    assert ap.main(["--profile-dir", str(tmp_path), "--rank", "1"]) == 0
    assert "rank1" in capsys.readouterr().out
    assert ap.main(["--profile-dir", str(tmp_path / "none")]) == 1


def test_timeline_viewer(tmp_path):
    samples = []
    for i in range(3):
        s = Sample(index=i, group_index=i // 2, prompt="p", reward=float(i), response_length=4)
        with trace_utils.trace_span(s, "generate", {"turn": 0}) as h:
            with trace_utils.trace_span(s, "engine_call"):
                trace_utils.trace_event(s, "first_token", {"n": 1})
            h.set("tokens", 4)
        samples.append(s.to_dict())
    samples.append(Sample(index=9, prompt="untraced").to_dict())
    # a span that never closed
    samples[0]["trace"]["events"].append({"type": "span_start", "name": "reward", "span_id": "zz", "parent_span_id": None,
                                          "ts": samples[0]["trace"]["events"][-1]["ts"], "attrs": {}})
    pt = tmp_path / "rollout_3.pt"
    torch.save({"rollout_id": 3, "samples": samples}, pt)
    data = tv.ensure_cache(pt)
    assert data["num_samples"] == 4 and data["num_lanes"] == 3 and data["rollout_id"] == 3
    lane = data["lanes"][0]
    by_name = {s["name"]: s for s in lane["spans"]}
    assert by_name["generate"]["depth"] == 0 and by_name["engine_call"]["depth"] == 1
    assert by_name["generate"]["attrs"] == {"turn": 0, "tokens": 4} and by_name["reward"].get("open") is True
    assert lane["events"][0]["name"] == "first_token" and lane["events"][0]["parent"] == by_name["engine_call"]["id"]
    assert data["span_summary"]["generate"]["count"] == 3 and data["lanes"][0]["spans"][0]["t0"] >= 0
    cache_path, html_path = tv.timeline_paths(pt)
    mtime = cache_path.stat().st_mtime_ns
    assert tv.ensure_cache(pt)["num_lanes"] == 3 and cache_path.stat().st_mtime_ns == mtime  # cache reused
    assert tv.main([str(pt)]) == 0
    page = html_path.read_text()
    assert "rollout_3.pt" in page and '"span_summary"' in page and "__DATA__" not in page
    assert tv.main([str(tmp_path / "missing.pt")]) == 1
    assert {"p50_s", "p95_s"} <= set(data["span_summary"]["generate"]) and 'id="srt"' in page


def test_timeline_analysis_of_concurrency_stragglers_and_idle_time():
    def lane(i, t0, t1, spans):
        return {"lane": i, "label": f"s{i}", "t0": t0, "t1": t1, "response_length": 10 * (i + 1),
                "spans": [{"name": n, "t0": a, "t1": b, "depth": d} for n, a, b, d in spans]}  # fmt: skip

    lanes = [lane(i, 0.0, 1.0, [("generate", 0.0, 1.0, 0)]) for i in range(19)]
    lanes.append(lane(19, 0.0, 5.0, [("generate", 0.0, 2.0, 0), ("tool", 0.5, 0.7, 1), ("generate", 3.0, 5.0, 0)]))
    a = tv.analyse_lanes(lanes)
    c = a["concurrency"]
    assert c["wall_s"] == 5.0 and c["thin_means_at_most"] == 2
    assert c["mean_in_flight"] == pytest.approx((20 * 1.0 + 1 * 4.0) / 5.0) and c["thin_tail_s"] == pytest.approx(4.0)
    assert a["stragglers"][0]["label"] == "s19" and a["stragglers"][0]["longest_span"] == {"name": "generate", "s": 2.0}
    assert a["idle"]["total_s"] == pytest.approx(1.0) and list(a["idle"]["worst"])[0] == "s19"  # the gap between its two turns
    assert tv.analyse_lanes([]) == {"concurrency": {}, "stragglers": [], "idle": {}}


def test_layerwise_dump_and_compare(tmp_path, monkeypatch):
    import torch

    from slime_b200.models.config import get_preset
    from slime_b200.models.gpt import GPTModel
    from slime_b200.observability import layerwise_dump as ld

    cfg = get_preset("tiny")
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(0))
    for tag, seed in (("a", 1), ("b", 1), ("c", 2)):
        model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=seed)
        dump = ld.LayerDump(str(tmp_path), None, prefix=f"{tag}_")
        assert dump.register(model) == cfg.num_layers
        model(ids)
        model(ids + 1 - 1)  # a second pass does not overwrite the first
        dump.remove()
    same = ld.compare(str(tmp_path / "a_rank0"), str(tmp_path / "b_rank0"))
    assert [r["layer"] for r in same] == [0, 1] and all(r["max_abs"] == 0 and not r["over"] for r in same)
    diff = ld.compare(str(tmp_path / "a_rank0"), str(tmp_path / "c_rank0"))
    assert all(r["over"] for r in diff)
    assert ld.main([str(tmp_path / "a_rank0"), str(tmp_path / "c_rank0"), "1e-3"]) == 0


def test_command_utils_build_commands(monkeypatch, capsys):
    from slime_b200.utils.external_utils import command_utils as U

    monkeypatch.setenv("DRY_RUN", "1")
    monkeypatch.setenv("SLIME_SCRIPT_EXTRA_ENV_VARS", "A=1 B=two")
    assert U._parse_extra_env_vars("A=1 B=two junk") == {"A": "1", "B": "two"}
    assert U.execute_train("--num-rollout 1", 2, model_preset="qwen2.5-0.5B") == 0
    out = capsys.readouterr().out
    assert "train.py --swiglu" in out and "--num-layers 24" in out and "--actor-num-gpus-per-node 2" in out
    assert U.get_bool_env_var("DRY_RUN") and not U.get_bool_env_var("NOT_SET_ANYWHERE")
    import pytest

    monkeypatch.setenv("X_BAD", "maybe")
    with pytest.raises(ValueError):
        U.get_bool_env_var("X_BAD")
    assert len(U.create_run_id().split("-")) == 3


def test_ci_check_that_the_draft_loss_does_not_leak(monkeypatch):
    import torch

    from slime_b200.backends.train.ci_utils import check_mtp_loss, check_mtp_only_grad

    class P:
        def __init__(self, g):
            self.main_grad = torch.tensor(g)

    class M:
        def __init__(self, d):
            self.d = d

        def named_parameters(self):
            return list(self.d.items())

    check_mtp_only_grad(M({"mtp.layers.0.eh_proj.weight": P([1.0]), "decoder.layers.0.mlp.linear_fc1.weight": P([0.0])}))
    import pytest

    with pytest.raises(AssertionError, match="policy parameters received"):
        check_mtp_only_grad(M({"mtp.layers.0.eh_proj.weight": P([1.0]), "decoder.layers.0.x": P([0.5])}))
    with pytest.raises(AssertionError, match="no draft-head"):
        check_mtp_only_grad(M({"mtp.layers.0.eh_proj.weight": P([0.0])}))
    check_mtp_loss(0.3)
    with pytest.raises(AssertionError):
        check_mtp_loss(2.0)
