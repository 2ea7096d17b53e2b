"""Start or stop the engines' profiler on every worker behind a router.

    python -m slime_b200.tools.profile_rollout --router-url http://127.0.0.1:3000 --action start --num-steps 3
    python -m slime_b200.tools.profile_rollout --router-url http://127.0.0.1:3000 --action stop

Workers are read from ``GET <router>/workers``; each gets ``POST /start_profile`` (output dir, number of scheduler steps,
activities, per-stage split, stacks, shapes) or ``POST /stop_profile``. Parity: tools/profile_rollout.py:1-77.
"""

from __future__ import annotations

import argparse
import sys

import requests


def list_workers(router_url: str) -> list[str]:
    r = requests.get(f"{router_url.rstrip('/')}/workers", timeout=30)
    r.raise_for_status()
    return [w["url"] for w in r.json().get("workers", []) if w.get("url")]


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--router-url", required=True)
    p.add_argument("--action", choices=["start", "stop"], default="start")
    p.add_argument("--output-dir", default="/tmp/engine_profile")
    p.add_argument("--num-steps", type=int, default=3)
    p.add_argument("--activities", nargs="+", default=["GPU"])
    p.add_argument("--profile-by-stage", action="store_true")
    p.add_argument("--with-stack", action="store_true")
    p.add_argument("--record-shapes", action="store_true")
    a = p.parse_args(argv)
    try:
        workers = list_workers(a.router_url)
    except requests.RequestException as e:
        print(f"cannot list workers at {a.router_url}: {e}")
        return 1
    if not workers:
        print("the router has no workers registered")
        return 1
    body = {} if a.action == "stop" else {"output_dir": a.output_dir, "num_steps": a.num_steps, "activities": a.activities,
                                          "profile_by_stage": a.profile_by_stage, "with_stack": a.with_stack,
                                          "record_shapes": a.record_shapes}  # fmt: skip
    failed = 0
    for url in workers:
        try:
            requests.post(f"{url}/{a.action}_profile", json=body, timeout=60).raise_for_status()
            print(f"{a.action} profile: {url} ok")
        except requests.RequestException as e:
            failed += 1
            print(f"{a.action} profile: {url} failed: {e}")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
