"""Profile analyser and rollout timeline viewer on small synthetic inputs."""

import gzip
import json

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
