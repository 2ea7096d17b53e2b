"""Multi-process orchestration on CPU: driver -> rollout manager -> engine actors (HTTP) -> trainer actors.

Failures are injected on the host only (an engine that stops answering); no GPU is involved.
"""

import json
import os
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture()
def prompt_file(tmp_path):
    path = tmp_path / "prompts.jsonl"
    with open(path, "w") as f:
        for i in range(64):
            f.write(json.dumps({"prompt": [1 + i % 50, 2, 3 + i % 7, 4], "label": str(i % 7)}) + "\n")
    return str(path)


COMMON = ["--hf-checkpoint", "preset:tiny", "--input-key", "prompt", "--label-key", "label", "--rollout-batch-size", "4",
          "--n-samples-per-prompt", "4", "--global-batch-size", "16", "--rollout-max-response-len", "8",
          "--actor-num-nodes", "1", "--actor-num-gpus-per-node", "1", "--rollout-num-gpus", "1",
          "--custom-rm-path", "slime_b200.rollout.synthetic.mod7_reward"]  # fmt: skip


def _run(script, extra, prompt_file, timeout=240):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, script), *COMMON, "--prompt-data", prompt_file, *extra]
    return subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=timeout)


@pytest.mark.timeout(300)
def test_train_py_runs_two_rollouts(prompt_file):
    r = _run("train.py", ["--num-rollout", "2", "--colocate"], prompt_file)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    log = r.stdout + r.stderr
    assert "step 0:" in log and "step 1:" in log
    assert "train_rollout_logprob_abs_diff" in log


@pytest.mark.timeout(300)
def test_train_async_py_overlaps_rollout_and_training(prompt_file):
    r = _run("train_async.py", ["--num-rollout", "3", "--update-weights-interval", "2"], prompt_file)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    log = r.stdout + r.stderr
    assert "step 2:" in log


@pytest.mark.timeout(300)
def test_external_engine_is_discovered_and_used(prompt_file):
    """An engine somebody else started: probe it, front it with an actor, route generation through it."""
    from slime_b200.engine import external
    from slime_b200.engine.http_server import launch_server
    from slime_b200.engine.server_args import ServerArgs
    from slime_b200.runtime import actors
    from slime_b200.runtime.rollout_manager import RolloutManager
    from slime_b200.utils.arguments import parse_args
    from slime_b200.utils.http_utils import find_available_port

    port = find_available_port(17000)
    server = launch_server(ServerArgs(model_path="preset:tiny", host="127.0.0.1", port=port, load_format="dummy"), block=False)
    try:
        infos = external.discover_external_engines([f"127.0.0.1:{port}"])
        assert infos[0].worker_type == "regular" and infos[0].num_gpus == 1 and infos[0].parallel_config["tp_size"] == 1
        with pytest.raises(ValueError):
            external.normalize_external_engine_addr("ftp://x")
        args = parse_args([*COMMON, "--prompt-data", prompt_file, "--num-rollout", "2", "--debug-rollout-only",
                           "--rollout-external-engine-addrs", f"127.0.0.1:{port}"])  # fmt: skip
        mgr = RolloutManager(args, None)
        try:
            assert args.rollout_num_engines == 1 and len(mgr.rollout_engines) == 1
            engines, _lock, num_new, counts, offsets, cfgs = mgr.get_updatable_engines_and_lock()
            assert num_new == 1 and counts == [1] and offsets == [0] and cfgs[0]["tp_size"] == 1
            assert actors.get(engines[0].get_url.remote()) == f"http://127.0.0.1:{port}"
            mgr.generate(0)
            assert server.engine.stats["steps"] > 0  # the tokens came from the pre-launched engine
        finally:
            mgr.dispose()
            actors.shutdown()
    finally:
        server.shutdown()


@pytest.mark.timeout(300)
def test_engine_crash_is_detected_and_recovered(prompt_file):
    from slime_b200.runtime import actors
    from slime_b200.runtime.rollout_manager import RolloutManager
    from slime_b200.utils.arguments import parse_args

    args = parse_args([*COMMON, "--prompt-data", prompt_file, "--num-rollout", "4", "--debug-rollout-only", "--use-fault-tolerance",
                       "--rollout-health-check-interval", "0.2", "--rollout-health-check-timeout", "2",
                       "--rollout-num-gpus", "2"])  # fmt: skip
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    mgr = RolloutManager(args, None)
    try:
        assert len(mgr.rollout_engines) == 2 and mgr.num_dead_engines() == 0
        assert mgr.generate(0) is None  # debug-rollout-only: samples are produced and logged, nothing is returned
        victim = mgr.server.server_groups[0].all_engines[0]
        actors.get(victim.simulate_crash.remote())
        deadline = time.time() + 30
        while mgr.num_dead_engines() == 0 and time.time() < deadline:
            time.sleep(0.1)
        assert mgr.num_dead_engines() == 1, "the health monitor did not notice the crashed engine"
        assert not victim.is_alive()
        mgr.generate(1)  # the surviving engine serves the whole batch
        assert mgr.recover_updatable_engines() == 1
        assert mgr.num_dead_engines() == 0
        engines, _lock, num_new, counts, offsets, _cfgs = mgr.get_updatable_engines_and_lock()
        assert num_new == 1 and len(engines) == 2 and counts == [1, 1] and offsets == [0, 1]
        mgr.generate(2)
    finally:
        mgr.dispose()
        actors.shutdown()
