"""Interactive timeline of a rollout: one lane per sample, nested spans, point events.

    python -m slime_b200.tools.trace_timeline_viewer /dumps/rollout_12.pt            # writes .timeline.json + .html
    python -m slime_b200.tools.trace_timeline_viewer /dumps/rollout_12.pt --serve --port 9999

Input: a debug rollout dump (``--save-debug-rollout-data``): ``{"rollout_id", "samples": [Sample.to_dict(), ...]}`` whose
samples carry ``trace = {"events": [span_start / span_end / event ...]}`` as recorded by
``slime_b200.observability.trace_utils``. The dump is read with a tolerant unpickler, so a dump that references classes
of user plug-ins which are not importable here still loads (those objects become attribute bags).

Output, written beside the dump: ``<stem>.timeline.json`` (the cache: lanes, spans with depth, events, summary; rebuilt
when the dump is newer or ``--rebuild``) and ``<stem>.timeline.html`` (self-contained viewer: wheel to zoom, drag to pan,
hover for attributes, click a lane label to fold it, filter box for span names).
Parity: tools/trace_timeline_viewer.py:30-2379 (same inputs, cache + HTML beside the dump, ``--serve``).
"""

from __future__ import annotations

import argparse
import functools
import http.server
import json
import pickle
import socketserver
import sys
import types
from pathlib import Path
from typing import Any

CACHE_VERSION = 2


class _Bag:
    """Stand-in for a pickled object whose class cannot be imported."""

    def __init__(self, *a, **k):
        pass

    def __setstate__(self, state):
        self.__dict__.update(state if isinstance(state, dict) else {"_state": state})


class _TolerantUnpickler(pickle.Unpickler):
    def find_class(self, module, name):
        try:
            return super().find_class(module, name)
        except Exception:  # noqa: BLE001
            return type(name, (_Bag,), {"__module__": module})


def load_dump(path: Path) -> dict:
    import torch

    tolerant = types.ModuleType("tolerant_pickle")
    tolerant.Unpickler, tolerant.load, tolerant.__name__ = _TolerantUnpickler, pickle.load, "pickle"
    for k in ("dumps", "loads", "dump", "HIGHEST_PROTOCOL", "DEFAULT_PROTOCOL", "UnpicklingError", "PickleError"):
        setattr(tolerant, k, getattr(pickle, k))
    return torch.load(str(path), map_location="cpu", weights_only=False, pickle_module=tolerant)


def _plain(v: Any, depth: int = 0) -> Any:
    """JSON-safe, size-bounded copy of an attribute value."""
    if v is None or isinstance(v, (bool, int)):
        return v
    if isinstance(v, float):
        return round(v, 6)
    if isinstance(v, str):
        return v if len(v) <= 256 else v[:253] + "..."
    if depth >= 3:
        return str(type(v).__name__)
    if isinstance(v, dict):
        return {str(k): _plain(x, depth + 1) for k, x in list(v.items())[:32]}
    if isinstance(v, (list, tuple)):
        return [_plain(x, depth + 1) for x in list(v)[:16]] + (["..."] if len(v) > 16 else [])
    if hasattr(v, "item") and getattr(v, "numel", lambda: 2)() == 1:
        return _plain(v.item(), depth)
    return str(v)[:128]


def _as_dict(sample: Any) -> dict:
    if isinstance(sample, dict):
        return sample
    if hasattr(sample, "to_dict"):
        return sample.to_dict()
    return dict(getattr(sample, "__dict__", {}))


def build_lane(sample: dict, idx: int) -> dict | None:
    """Pair span_start / span_end by span_id, give every span a depth from its parent chain, keep point events."""
    trace = sample.get("trace")
    trace = trace if isinstance(trace, dict) else getattr(trace, "__dict__", None)
    events = (trace or {}).get("events") or []
    if not events:
        return None
    open_spans: dict[str, dict] = {}
    spans: list[dict] = []
    points: list[dict] = []
    last_ts = max((e.get("ts") or 0.0) for e in events)
    for e in sorted(events, key=lambda e: e.get("ts") or 0.0):
        kind = e.get("type")
        if kind == "span_start":
            open_spans[e.get("span_id")] = {"id": e.get("span_id"), "parent": e.get("parent_span_id"), "name": e.get("name", "?"),
                                            "t0": e.get("ts"), "t1": None, "attrs": dict(e.get("attrs") or {})}  # fmt: skip
        elif kind == "span_end":
            s = open_spans.pop(e.get("span_id"), None)
            if s is None:
                continue
            s["t1"] = e.get("ts")
            s["attrs"].update(e.get("attrs") or {})
            if e.get("error"):
                s["error"] = str(e["error"])[:256]
            spans.append(s)
        else:
            points.append({"name": e.get("name", "?"), "t": e.get("ts"), "parent": e.get("parent_span_id"),
                           "attrs": _plain(e.get("attrs") or {})})  # fmt: skip
    for s in open_spans.values():  # never closed (aborted or still running when dumped): runs to the lane's last event
        s["t1"], s["open"] = last_ts, True
        spans.append(s)
    by_id = {s["id"]: s for s in spans}

    def depth(s, seen=()):
        p = by_id.get(s["parent"])
        return 0 if p is None or s["id"] in seen else 1 + depth(p, seen + (s["id"],))

    for s in spans:
        s["depth"] = depth(s)
        s["attrs"] = _plain(s["attrs"])
    spans.sort(key=lambda s: (s["t0"], s["depth"]))
    md = sample.get("metadata") or {}
    status = sample.get("status")
    return {"lane": idx, "sample_index": sample.get("index"), "group_index": sample.get("group_index"),
            "label": f"g{sample.get('group_index')}/s{sample.get('index')}", "status": getattr(status, "value", status),
            "reward": _plain(sample.get("reward")), "response_length": sample.get("response_length"),
            "source": md.get("source") or md.get("data_source") or md.get("rm_type"),
            "attempt": (trace or {}).get("attempt", 0), "spans": spans, "events": points,
            "t0": min([s["t0"] for s in spans] + [p["t"] for p in points]),
            "t1": max([s["t1"] for s in spans] + [p["t"] for p in points])}  # fmt: skip


def build_cache(pt_path: Path) -> dict:
    dump = load_dump(pt_path)
    samples = [_as_dict(s) for s in (dump.get("samples") if isinstance(dump, dict) else dump) or []]
    lanes = [lane for i, s in enumerate(samples) if (lane := build_lane(s, i)) is not None]
    t0 = min((ln["t0"] for ln in lanes), default=0.0)
    for ln in lanes:  # times relative to the first event, in seconds
        ln["t0"], ln["t1"] = ln["t0"] - t0, ln["t1"] - t0
        for s in ln["spans"]:
            s["t0"], s["t1"] = round(s["t0"] - t0, 6), round(s["t1"] - t0, 6)
        for p in ln["events"]:
            p["t"] = round(p["t"] - t0, 6)
    per_name: dict[str, list[float]] = {}
    for ln in lanes:
        for s in ln["spans"]:
            per_name.setdefault(s["name"], []).append(s["t1"] - s["t0"])
    def pct(d, q):
        d = sorted(d)
        return d[min(len(d) - 1, int(q * len(d)))]

    summary = {n: {"count": len(d), "total_s": round(sum(d), 6), "mean_s": round(sum(d) / len(d), 6), "p50_s": round(pct(d, 0.5), 6),
                   "p95_s": round(pct(d, 0.95), 6), "max_s": round(max(d), 6)}
               for n, d in sorted(per_name.items(), key=lambda kv: -sum(kv[1]))}  # fmt: skip
    return {"version": CACHE_VERSION, "analysis": analyse_lanes(lanes), "source": pt_path.name, "rollout_id": dump.get("rollout_id") if isinstance(dump, dict) else None,
            "num_samples": len(samples), "num_lanes": len(lanes), "origin_ts": t0,
            "duration_s": round(max((ln["t1"] for ln in lanes), default=0.0), 6), "span_summary": summary, "lanes": lanes}  # fmt: skip


def analyse_lanes(lanes: list[dict]) -> dict:
    """What a rollout's wall time went to. ``concurrency``: time-weighted mean number of samples in flight and the share
    of the wall time during which fewer than a tenth of the lanes were active (the long tail a partial-rollout or
    over-sampling setting would cut). ``stragglers``: the five lanes that finished last with their longest top-level
    span. ``idle``: per lane, the time inside its extent that no top-level span covers (waiting between turns)."""
    if not lanes:
        return {"concurrency": {}, "stragglers": [], "idle": {}}
    edges = sorted([(ln["t0"], 1) for ln in lanes] + [(ln["t1"], -1) for ln in lanes])
    end = max(ln["t1"] for ln in lanes)
    active, last, area, tail = 0, edges[0][0], 0.0, 0.0
    thin = max(1, len(lanes) // 10)
    for t, d in edges:
        area += active * (t - last)
        if 0 < active <= thin:
            tail += t - last
        active, last = active + d, t
    wall = max(end - edges[0][0], 1e-9)
    stragglers = []
    for ln in sorted(lanes, key=lambda x: -x["t1"])[:5]:
        top = max((s for s in ln["spans"] if s["depth"] == 0), key=lambda s: s["t1"] - s["t0"], default=None)
        stragglers.append({"label": ln["label"], "end_s": round(ln["t1"], 4), "duration_s": round(ln["t1"] - ln["t0"], 4),
                           "response_length": ln.get("response_length"),
                           "longest_span": None if top is None else {"name": top["name"], "s": round(top["t1"] - top["t0"], 4)}})  # fmt: skip
    idle = {}
    for ln in lanes:
        tops = sorted((s["t0"], s["t1"]) for s in ln["spans"] if s["depth"] == 0)
        covered, cur = 0.0, None
        for a, b in tops:
            if cur is None or a > cur[1]:
                covered += 0.0 if cur is None else cur[1] - cur[0]
                cur = [a, b]
            else:
                cur[1] = max(cur[1], b)
        covered += 0.0 if cur is None else cur[1] - cur[0]
        idle[ln["label"]] = round(max(ln["t1"] - ln["t0"] - covered, 0.0), 6)
    worst_idle = dict(sorted(idle.items(), key=lambda kv: -kv[1])[:5])
    return {"concurrency": {"mean_in_flight": round(area / wall, 3), "wall_s": round(wall, 4), "thin_tail_s": round(tail, 4),
                            "thin_tail_share": round(tail / wall, 4), "thin_means_at_most": thin},
            "stragglers": stragglers, "idle": {"total_s": round(sum(idle.values()), 4), "worst": worst_idle}}  # fmt: skip


def timeline_paths(pt_path: Path) -> tuple[Path, Path]:
    return pt_path.with_suffix(".timeline.json"), pt_path.with_suffix(".timeline.html")


def ensure_cache(pt_path: Path, rebuild: bool = False) -> dict:
    cache_path, _ = timeline_paths(pt_path)
    if not rebuild and cache_path.exists() and cache_path.stat().st_mtime >= pt_path.stat().st_mtime:
        try:
            data = json.loads(cache_path.read_text())
            if data.get("version") == CACHE_VERSION:
                return data
        except (OSError, ValueError):
            pass
    data = build_cache(pt_path)
    cache_path.write_text(json.dumps(data, separators=(",", ":")))
    return data


_HTML = r"""<!doctype html><html><head><meta charset="utf-8"><title>__TITLE__</title><style>
body{margin:0;font:12px system-ui,sans-serif;background:#111;color:#ddd}#bar{padding:6px 10px;background:#1b1b1b;display:flex;gap:12px;align-items:center}
#wrap{display:flex;height:calc(100vh - 34px)}#labels{width:150px;overflow:hidden;background:#161616}#labels div{height:__LANE__px;line-height:__LANE__px;padding-left:8px;border-bottom:1px solid #222;cursor:pointer;white-space:nowrap}
canvas{flex:1;display:block}#tip{position:fixed;pointer-events:none;background:#000d;border:1px solid #555;padding:6px 8px;max-width:460px;white-space:pre-wrap;display:none;z-index:9}
input{background:#222;color:#ddd;border:1px solid #444;padding:2px 6px}</style></head><body>
<div id="bar"><b>__TITLE__</b><span id="info"></span><input id="flt" placeholder="filter span names"><select id="srt"><option value="lane">order: dump</option><option value="t0">start</option><option value="dur">duration</option><option value="t1">end</option><option value="reward">reward</option></select><span id="sum"></span></div>
<div id="wrap"><div id="labels"></div><canvas id="cv"></canvas></div><div id="tip"></div><script>
const D=__DATA__,LH=__LANE__,cv=document.getElementById('cv'),cx=cv.getContext('2d'),tip=document.getElementById('tip');
let x0=0,x1=Math.max(D.duration_s,1e-3),scroll=0,flt='',hidden=new Set(),hit=[];
const colors={};function col(n){if(!colors[n]){let h=0;for(const c of n)h=(h*31+c.charCodeAt(0))%360;colors[n]=`hsl(${h},55%,45%)`}return colors[n]}
let srt='lane';const key={lane:l=>l.lane,t0:l=>l.t0,dur:l=>-(l.t1-l.t0),t1:l=>-l.t1,reward:l=>-(+l.reward||0)};
function lanes(){return D.lanes.filter(l=>!hidden.has(l.lane)).sort((a,b)=>key[srt](a)-key[srt](b))}
function draw(){const W=cv.width=cv.clientWidth,H=cv.height=cv.clientHeight;cx.clearRect(0,0,W,H);hit=[];const L=lanes(),sx=t=>(t-x0)/(x1-x0)*W;
 const lab=document.getElementById('labels');lab.innerHTML='';L.forEach((l,i)=>{const y=i*LH-scroll;if(y<-LH||y>H)return;const d=document.createElement('div');d.textContent=`${l.label} r=${l.reward} ${l.status||''}`;d.style.position='absolute';d.style.top=(y+34)+'px';d.style.width='142px';d.onclick=()=>{hidden.add(l.lane);draw()};lab.appendChild(d);
  cx.fillStyle=i%2?'#151515':'#191919';cx.fillRect(0,y,W,LH);
  for(const s of l.spans){if(flt&&!s.name.includes(flt))continue;const a=sx(s.t0),b=Math.max(sx(s.t1),a+1);if(b<0||a>W)continue;const h=Math.max(3,(LH-4)/(1+s.depth*0.6)),yy=y+2+s.depth*3;cx.fillStyle=s.error?'#c33':col(s.name);cx.globalAlpha=s.open?0.5:1;cx.fillRect(a,yy,b-a,Math.min(h,LH-4-s.depth*3));cx.globalAlpha=1;if(b-a>50){cx.fillStyle='#fff';cx.fillText(s.name,a+3,yy+10)}hit.push([a,yy,b,yy+h,s,l])}
  for(const p of l.events){const a=sx(p.t);if(a<0||a>W)continue;cx.fillStyle='#fd4';cx.beginPath();cx.arc(a,y+LH-5,3,0,7);cx.fill();hit.push([a-4,y+LH-9,a+4,y+LH-1,p,l])}});
 cx.fillStyle='#888';for(let k=0;k<=10;k++){const t=x0+(x1-x0)*k/10;cx.fillText(t.toFixed(3)+'s',k*W/10+2,H-4)}
 document.getElementById('info').textContent=`${D.num_lanes}/${D.num_samples} samples with traces, ${D.duration_s.toFixed(2)} s, rollout ${D.rollout_id}`}
cv.onwheel=e=>{e.preventDefault();if(e.shiftKey){scroll=Math.max(0,scroll+e.deltaY);draw();return}const f=e.deltaY>0?1.25:0.8,t=x0+(x1-x0)*e.offsetX/cv.clientWidth;x0=t-(t-x0)*f;x1=t+(x1-t)*f;draw()};
let drag=null;cv.onmousedown=e=>drag=[e.clientX,e.clientY,x0,x1,scroll];window.onmouseup=()=>drag=null;
window.onmousemove=e=>{if(drag){const dt=(e.clientX-drag[0])/cv.clientWidth*(drag[3]-drag[2]);x0=drag[2]-dt;x1=drag[3]-dt;scroll=Math.max(0,drag[4]-(e.clientY-drag[1]));draw();return}
 const r=cv.getBoundingClientRect(),x=e.clientX-r.left,y=e.clientY-r.top;let f=null;for(const h of hit)if(x>=h[0]&&x<=h[2]&&y>=h[1]&&y<=h[3])f=h;
 if(f){const o=f[4];tip.style.display='block';tip.style.left=(e.clientX+12)+'px';tip.style.top=(e.clientY+12)+'px';tip.textContent=`${o.name}  [${f[5].label}]\n`+(o.t0!==undefined?`${o.t0.toFixed(4)} -> ${o.t1.toFixed(4)} s  (${((o.t1-o.t0)*1e3).toFixed(2)} ms)${o.open?'  (never closed)':''}\n`:`at ${o.t.toFixed(4)} s\n`)+(o.error?`error: ${o.error}\n`:'')+JSON.stringify(o.attrs,null,1)}else tip.style.display='none'};
document.getElementById('flt').oninput=e=>{flt=e.target.value;draw()};document.getElementById('srt').onchange=e=>{srt=e.target.value;draw()};window.onresize=draw;
document.getElementById('sum').textContent=Object.entries(D.span_summary).slice(0,4).map(([n,s])=>`${n}: ${s.count}x mean ${(s.mean_s*1e3).toFixed(1)} ms`).join(' | ');draw();
</script></body></html>"""


def ensure_html(pt_path: Path, data: dict, lane_px: int = 26) -> Path:
    _, html_path = timeline_paths(pt_path)
    page = (_HTML.replace("__TITLE__", f"rollout timeline: {pt_path.name}").replace("__LANE__", str(lane_px))
            .replace("__DATA__", json.dumps(data, separators=(",", ":")).replace("</", "<\\/")))  # fmt: skip
    html_path.write_text(page)
    return html_path


def serve_directory(directory: Path, port: int) -> None:
    class Quiet(http.server.SimpleHTTPRequestHandler):
        def log_message(self, *a):
            pass

    handler = functools.partial(Quiet, directory=str(directory))
    with socketserver.TCPServer(("0.0.0.0", port), handler) as srv:
        srv.serve_forever()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("pt_path", help="rollout debug dump (.pt)")
    ap.add_argument("--rebuild", action="store_true", help="rebuild the JSON cache even if it is current")
    ap.add_argument("--serve", action="store_true", help="serve the dump's directory over HTTP after building")
    ap.add_argument("--port", type=int, default=9999)
    a = ap.parse_args(argv)
    pt = Path(a.pt_path)
    if not pt.exists():
        print(f"no such file: {pt}", file=sys.stderr)
        return 1
    data = ensure_cache(pt, a.rebuild)
    html = ensure_html(pt, data)
    print(f"{data['num_lanes']} lanes, {data['duration_s']:.2f} s -> {html}")
    for name, s in list(data["span_summary"].items())[:10]:
        print(f"  {name:<32} {s['count']:6d}x  mean {s['mean_s'] * 1e3:9.2f} ms  p50 {s['p50_s'] * 1e3:9.2f}  p95 {s['p95_s'] * 1e3:9.2f}"
              f"  max {s['max_s'] * 1e3:9.2f} ms")
    an = data.get("analysis") or {}
    c = an.get("concurrency") or {}
    if c:
        print(f"  in flight: {c['mean_in_flight']:.1f} samples on average over {c['wall_s']:.2f} s; at most {c['thin_means_at_most']} "
              f"active for {c['thin_tail_s']:.2f} s ({100 * c['thin_tail_share']:.1f} % of the wall time)")
        for st in an.get("stragglers", [])[:3]:
            ls = st["longest_span"]
            print(f"  straggler {st['label']}: ended at {st['end_s']:.2f} s after {st['duration_s']:.2f} s, {st['response_length']} response "
                  f"tokens" + (f", longest span {ls['name']} {ls['s']:.2f} s" if ls else ""))
        print(f"  idle inside lanes (no top-level span): {an['idle']['total_s']:.2f} s in total")
    if a.serve:
        print(f"http://0.0.0.0:{a.port}/{html.name}")
        serve_directory(pt.parent, a.port)
    return 0


if __name__ == "__main__":
    sys.exit(main())
