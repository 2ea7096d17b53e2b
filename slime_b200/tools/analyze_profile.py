"""Summarise torch-profiler traces of the rollout engine or the trainer.

    python -m slime_b200.tools.analyze_profile --profile-dir /tmp/engine_profile            # first trace found
    python -m slime_b200.tools.analyze_profile --profile-dir ... --rank 3
    python -m slime_b200.tools.analyze_profile --profile-dir ... --all-ranks --json out.json

Input: Chrome-trace files (``*.json`` / ``*.json.gz``) as written by ``torch.profiler`` (the engine's
``/start_profile`` endpoint and the trainer's ``--use-pytorch-profiler`` both produce them). Per trace the report gives
  * device and distributed facts recorded in the trace,
  * GPU busy time vs the span between first and last GPU event, and the largest idle gaps with the CPU-side event that
    covers most of each (what the GPU was waiting for),
  * kernel time by category (GEMM, attention, normalisation/activation, sampling+loss, optimizer, communication,
    memory copies, other) and the top kernels,
  * per-stream utilisation,
  * CUDA-graph launches grouped into decode steps (launches closer together than ``--step-gap-us``), with the spread of
    step durations,
  * host overhead indicators (``aten::copy_``, ``cudaStreamSynchronize``, gloo time).
With ``--all-ranks`` a cross-rank table follows, which is where stragglers show. Parity: tools/analyze_profile.py:67-730.
"""

from __future__ import annotations

import argparse
import bisect
import dataclasses
import glob
import gzip
import json
import os
import re
import statistics
import sys
from collections import defaultdict

CATEGORIES = (
    ("communication", re.compile(r"nccl|dp_reduce_shard|dp_adam_bcast|symm_barrier|all_?reduce|all_?gather|reduce_?scatter|deep_ep|multimem", re.I)),
    ("gemm", re.compile(r"gemm|cutlass|cublas|sm\d+_xmma|ampere_|hopper_|matmul|router_gemm", re.I)),
    ("attention", re.compile(r"attn|attention|flash|fmha|mla", re.I)),
    ("sampling+loss", re.compile(r"sample|softmax|dlogits|pg_loss|logprob|topk|top_p|argmax|multinomial", re.I)),
    ("optimizer", re.compile(r"adam|sqnorm|multi_tensor|clip", re.I)),
    ("norm+activation", re.compile(r"rmsnorm|layer_?norm|rope|rotary|swiglu|silu|gelu|embedding|kv_write|decode_prepare|decode_advance", re.I)),
    ("quantisation", re.compile(r"fp8|int4|quant", re.I)),
    ("memory", re.compile(r"memcpy|memset|copy_kernel|fill", re.I)),
    ("elementwise", re.compile(r"elementwise|vectorized|reduce_kernel|cat|index|gather|scatter", re.I)),
)


def classify_kernel(name: str) -> str:
    for cat, pat in CATEGORIES:
        if pat.search(name):
            return cat
    return "other"


@dataclasses.dataclass
class KernelStat:
    name: str
    category: str
    count: int = 0
    total_us: float = 0.0

    @property
    def avg_us(self) -> float:
        return self.total_us / max(self.count, 1)


@dataclasses.dataclass
class TraceAnalysis:
    rank_name: str = ""
    gpu_name: str = ""
    num_sms: int = 0
    vram_gb: float = 0.0
    cuda_version: str = ""
    nccl_version: str = ""
    world_size: int = 0
    total_events: int = 0
    wall_us: float = 0.0
    gpu_span_us: float = 0.0
    gpu_busy_us: float = 0.0
    kernel_count: int = 0
    kernel_us: float = 0.0
    categories: dict[str, KernelStat] = dataclasses.field(default_factory=dict)
    top_kernels: list[KernelStat] = dataclasses.field(default_factory=list)
    top_gaps: list[dict] = dataclasses.field(default_factory=list)
    streams: dict[str, dict] = dataclasses.field(default_factory=dict)
    graph_launches: int = 0
    graph_launch_cpu_us: float = 0.0
    decode_steps: list[float] = dataclasses.field(default_factory=list)
    comm_us: float = 0.0
    gloo_us: float = 0.0
    copy_count: int = 0
    copy_us: float = 0.0
    sync_count: int = 0
    sync_us: float = 0.0

    @property
    def gpu_util_pct(self) -> float:
        return 100.0 * self.gpu_busy_us / self.gpu_span_us if self.gpu_span_us > 0 else 0.0


def load_trace(path: str) -> dict:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt") as f:
        return json.load(f)


def merge_intervals(intervals: list[tuple[float, float]]) -> list[tuple[float, float]]:
    out: list[list[float]] = []
    for s, e in sorted(intervals):
        if out and s <= out[-1][1]:
            out[-1][1] = max(out[-1][1], e)
        else:
            out.append([s, e])
    return [(s, e) for s, e in out]


def analyze_trace(data: dict, rank_name: str = "", top_n: int = 20, step_gap_us: float = 200.0) -> TraceAnalysis:
    r = TraceAnalysis(rank_name=rank_name)
    events = [e for e in data.get("traceEvents", []) if e.get("ph") == "X" and "ts" in e]
    r.total_events = len(data.get("traceEvents", []))
    props = data.get("deviceProperties") or []
    if props:
        r.gpu_name, r.num_sms = props[0].get("name", ""), props[0].get("numSms", 0)
        r.vram_gb = props[0].get("totalGlobalMem", 0) / 2**30
    rt = data.get("cuda_runtime_version", 0) or 0
    r.cuda_version = f"{rt // 1000}.{rt % 1000 // 10}" if rt else ""
    dist = data.get("distributedInfo") or {}
    r.nccl_version, r.world_size = str(dist.get("nccl_version", "")), int(dist.get("world_size", 0) or 0)

    kernels = [e for e in events if e.get("cat") == "kernel"]
    per_name: dict[str, KernelStat] = {}
    for e in kernels:
        name, dur = e.get("name", "?"), float(e.get("dur", 0))
        st = per_name.get(name)
        if st is None:
            st = per_name[name] = KernelStat(name, classify_kernel(name))
        st.count += 1
        st.total_us += dur
        cat = r.categories.setdefault(st.category, KernelStat(st.category, st.category))
        cat.count += 1
        cat.total_us += dur
    r.kernel_count, r.kernel_us = len(kernels), sum(s.total_us for s in per_name.values())
    r.top_kernels = sorted(per_name.values(), key=lambda s: -s.total_us)[:top_n]
    r.comm_us = r.categories["communication"].total_us if "communication" in r.categories else 0.0

    gpu = [e for e in events if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset")]
    if events:
        r.wall_us = max(e["ts"] + e.get("dur", 0) for e in events) - min(e["ts"] for e in events)
    if gpu:
        merged = merge_intervals([(e["ts"], e["ts"] + e.get("dur", 0)) for e in gpu])
        r.gpu_busy_us = sum(e - s for s, e in merged)
        r.gpu_span_us = merged[-1][1] - merged[0][0]
        gaps = sorted(((merged[i][0] - merged[i - 1][1], merged[i - 1][1], merged[i][0]) for i in range(1, len(merged))),
                      reverse=True)[:15]  # fmt: skip
        cpu = sorted((e for e in events if e.get("cat") in ("cpu_op", "user_annotation", "cuda_runtime", "python_function")),
                     key=lambda e: e["ts"])  # fmt: skip
        starts = [e["ts"] for e in cpu]
        for gap, g0, g1 in gaps:
            # the host event that covers most of the gap: what the CPU was doing while the GPU had nothing to run
            i = bisect.bisect_right(starts, g1)
            cause, best = "unknown", 0.0
            for e in cpu[max(0, i - 256):i]:
                overlap = min(e["ts"] + e.get("dur", 0), g1) - max(e["ts"], g0)
                if overlap > best:
                    cause, best = e.get("name", "?"), overlap
            r.top_gaps.append({"gap_us": gap, "start": g0, "end": g1, "cause": cause})
        by_stream: dict[str, list] = defaultdict(list)
        for e in gpu:
            by_stream[str(e.get("tid"))].append(e)
        for tid, evs in by_stream.items():
            busy = sum(e.get("dur", 0) for e in evs)
            span = max(e["ts"] + e.get("dur", 0) for e in evs) - min(e["ts"] for e in evs)
            r.streams[tid] = {"count": len(evs), "busy_us": busy, "span_us": span, "util_pct": 100 * busy / span if span else 0.0}

    launches = sorted((e for e in events if e.get("name") == "cudaGraphLaunch"), key=lambda e: e["ts"])
    r.graph_launches, r.graph_launch_cpu_us = len(launches), sum(e.get("dur", 0) for e in launches)
    if launches:  # a decode step = a run of launches with less than step_gap_us between consecutive ones
        start = prev_end = None
        for e in launches:
            if start is None or e["ts"] - prev_end > step_gap_us:
                if start is not None:
                    r.decode_steps.append(prev_end - start)
                start = e["ts"]
            prev_end = e["ts"] + e.get("dur", 0)
        r.decode_steps.append(prev_end - start)
    for e in events:
        name = e.get("name", "")
        if name == "aten::copy_":
            r.copy_count, r.copy_us = r.copy_count + 1, r.copy_us + e.get("dur", 0)
        elif name in ("cudaStreamSynchronize", "cudaDeviceSynchronize", "cudaEventSynchronize"):
            r.sync_count, r.sync_us = r.sync_count + 1, r.sync_us + e.get("dur", 0)
        elif "gloo" in name.lower():
            r.gloo_us += e.get("dur", 0)
    return r


def _bar(pct: float, width: int = 30) -> str:
    n = max(0, min(width, int(round(pct / 100 * width))))
    return "#" * n + "." * (width - n)


def format_analysis(r: TraceAnalysis) -> str:
    out = [f"=== {r.rank_name or 'trace'} ==="]
    if r.gpu_name:
        out.append(f"device: {r.gpu_name}, {r.num_sms} SMs, {r.vram_gb:.0f} GiB; CUDA {r.cuda_version or '?'}; "
                   f"NCCL {r.nccl_version or '?'}; world {r.world_size or '?'}")  # fmt: skip
    out.append(f"events {r.total_events}, wall {r.wall_us / 1e3:.2f} ms, GPU span {r.gpu_span_us / 1e3:.2f} ms, "
               f"busy {r.gpu_busy_us / 1e3:.2f} ms")  # fmt: skip
    out.append(f"GPU utilisation [{_bar(r.gpu_util_pct)}] {r.gpu_util_pct:5.1f} %")
    out.append("-- kernel time by category")
    for c in sorted(r.categories.values(), key=lambda c: -c.total_us):
        pct = 100 * c.total_us / r.kernel_us if r.kernel_us else 0
        out.append(f"  {c.name:<16} [{_bar(pct, 20)}] {pct:5.1f} %  {c.total_us / 1e3:9.2f} ms  {c.count:7d} launches")
    out.append("-- top kernels")
    for k in r.top_kernels:
        out.append(f"  {k.total_us / 1e3:9.2f} ms {k.count:7d}x {k.avg_us:9.1f} us  [{k.category}] {k.name[:90]}")
    if r.top_gaps:
        out.append("-- largest GPU idle gaps (host event covering most of the gap)")
        for g in r.top_gaps[:10]:
            out.append(f"  {g['gap_us']:10.1f} us  {g['cause'][:80]}")
    if r.streams:
        out.append("-- streams")
        for tid, s in sorted(r.streams.items(), key=lambda kv: -kv[1]["busy_us"]):
            out.append(f"  stream {tid:>6}: {s['count']:7d} events, busy {s['busy_us'] / 1e3:9.2f} ms, {s['util_pct']:5.1f} % of its span")
    if r.graph_launches:
        d = r.decode_steps
        out.append(f"-- CUDA graphs: {r.graph_launches} launches, {r.graph_launch_cpu_us / 1e3:.2f} ms of host time, "
                   f"{len(d)} steps")  # fmt: skip
        if d:
            out.append(f"  step host span: median {statistics.median(d):.1f} us, min {min(d):.1f}, max {max(d):.1f}")
    out.append(f"-- host: aten::copy_ {r.copy_count}x {r.copy_us / 1e3:.2f} ms; synchronize {r.sync_count}x "
               f"{r.sync_us / 1e3:.2f} ms; gloo {r.gloo_us / 1e3:.2f} ms; communication kernels {r.comm_us / 1e3:.2f} ms")  # fmt: skip
    return "\n".join(out)


def format_cross_rank(rs: list[TraceAnalysis]) -> str:
    out = ["=== across ranks ===", f"  {'rank':<28}{'util %':>8}{'busy ms':>10}{'kernels ms':>12}{'comm ms':>10}{'steps':>7}"]
    for r in rs:
        out.append(f"  {r.rank_name[:27]:<28}{r.gpu_util_pct:8.1f}{r.gpu_busy_us / 1e3:10.2f}{r.kernel_us / 1e3:12.2f}"
                   f"{r.comm_us / 1e3:10.2f}{len(r.decode_steps):7d}")  # fmt: skip
    busy = [r.gpu_busy_us for r in rs]
    if len(busy) > 1 and min(busy) > 0:
        out.append(f"  busy-time spread: max/min = {max(busy) / min(busy):.3f}")
    return "\n".join(out)


def find_traces(profile_dir: str) -> list[str]:
    pats = ("*.trace.json.gz", "*.trace.json", "*.json.gz", "*.json")
    found: list[str] = []
    for p in pats:
        found += glob.glob(os.path.join(profile_dir, "**", p), recursive=True)
    return sorted(set(found))


def pick_rank(files: list[str], rank: int) -> list[str]:
    pat = re.compile(rf"(rank|TP|DP|tp|dp)[-_]?{rank}(\D|$)")
    hit = [f for f in files if pat.search(os.path.basename(f))]
    return hit or files[rank : rank + 1]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--profile-dir", required=True)
    ap.add_argument("--rank", type=int, default=None)
    ap.add_argument("--all-ranks", action="store_true")
    ap.add_argument("--top-n", type=int, default=20)
    ap.add_argument("--step-gap-us", type=float, default=200.0)
    ap.add_argument("--json", default=None, help="also write the analyses as JSON to this path")
    a = ap.parse_args(argv)
    files = find_traces(a.profile_dir)
    if not files:
        print(f"no trace files under {a.profile_dir}", file=sys.stderr)
        return 1
    if a.rank is not None:
        files = pick_rank(files, a.rank)
    elif not a.all_ranks:
        files = files[:1]
    results = [analyze_trace(load_trace(f), os.path.basename(f), a.top_n, a.step_gap_us) for f in files]
    for r in results:
        print(format_analysis(r))
    if len(results) > 1:
        print(format_cross_rank(results))
    if a.json:
        with open(a.json, "w") as f:
            json.dump([dataclasses.asdict(r) for r in results], f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
