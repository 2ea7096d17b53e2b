"""Shell-level helpers for end-to-end launchers and CI scripts: convert a checkpoint, run a training job, small utilities.

    from slime_b200.utils.external_utils import command_utils as U
    U.convert_checkpoint("Qwen3-4B", "qwen3-4B", num_gpus_per_node=4)
    U.execute_train(train_args="--num-rollout 3 ...", num_gpus_per_node=4, model_preset="qwen3-4B")

Every command goes through ``run`` (printed, then executed with ``check=True``); ``DRY_RUN=1`` prints only. Same role as
slime/utils/external_utils/command_utils.py:21-263 in the reference (there the jobs are submitted to a Ray cluster; here
``train.py`` starts its own actor runtime, so a job is one process tree).
"""

from __future__ import annotations

import datetime
import os
import random
import shlex
import subprocess
import sys
import tempfile

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def run(cmd: str, env: dict | None = None) -> int:
    print(f"+ {cmd}", flush=True)
    if get_bool_env_var("DRY_RUN"):
        return 0
    return subprocess.run(cmd, shell=True, check=True, env={**os.environ, **(env or {})}, cwd=REPO_ROOT).returncode


def model_flags(preset: str) -> str:
    return subprocess.check_output([sys.executable, "-m", "slime_b200.models.presets", preset], cwd=REPO_ROOT, text=True).strip()


def convert_checkpoint(model_name: str, preset: str, num_gpus_per_node: int = 1, dir_src: str = "~/models", dir_dst: str = "~/models",
                       extra_args: str = "") -> str:  # fmt: skip
    """Hugging Face directory -> ``<name>_torch_dist`` (skipped when it already exists). Returns the destination."""
    dir_src, dir_dst = os.path.expanduser(dir_src), os.path.expanduser(dir_dst)
    dst = os.path.join(dir_dst, f"{model_name}_torch_dist")
    if os.path.exists(os.path.join(dst, "latest_checkpointed_iteration.txt")):
        print(f"convert_checkpoint: {dst} exists, skipping")
        return dst
    launcher = (f"{sys.executable} -m torch.distributed.run --nnodes=1 --nproc-per-node {num_gpus_per_node} --master-addr 127.0.0.1"
                if num_gpus_per_node > 1 else sys.executable)  # fmt: skip
    run(f"{launcher} -m slime_b200.tools.convert_hf_to_torch_dist {model_flags(preset)} --hf-checkpoint {shlex.quote(os.path.join(dir_src, model_name))} "
        f"--save {shlex.quote(dst)} {extra_args}")  # fmt: skip
    return dst


def fp8_cast_bf16(path_src: str, path_dst: str) -> None:
    if os.path.exists(path_dst):
        print(f"fp8_cast_bf16: {path_dst} exists, skipping")
        return
    run(f"{sys.executable} -m slime_b200.tools.fp8_cast_bf16 --input-fp8-hf-path {shlex.quote(path_src)} --output-bf16-hf-path {shlex.quote(path_dst)}")


def rsync_simple(path_src: str, path_dst: str) -> None:
    run(f"mkdir -p {shlex.quote(path_dst)} && rsync -a --info=progress2 {shlex.quote(path_src.rstrip('/'))}/ {shlex.quote(path_dst)}")


def hf_download_dataset(full_name: str, dst_root: str = "~/datasets") -> None:
    _, name = full_name.split("/")
    dst_root = os.path.expanduser(dst_root)
    run(f"hf download --repo-type dataset {full_name} --local-dir {os.path.join(dst_root, name)}")


def execute_train(train_args: str, num_gpus_per_node: int, model_preset: str | None = None, train_script: str = "train.py",
                  before_hook=None, extra_env_vars: dict | None = None) -> int:  # fmt: skip
    """Run one training job to completion. ``model_preset`` adds the architecture flags; ``extra_env_vars`` and
    ``SLIME_SCRIPT_EXTRA_ENV_VARS`` (``K=V K2=V2``) are exported to it."""
    if before_hook is not None:
        before_hook()
    env = {"PYTHONPATH": f"{REPO_ROOT}:{os.environ.get('PYTHONPATH', '')}", "MASTER_ADDR": os.environ.get("MASTER_ADDR", "127.0.0.1"),
           "CUDA_DEVICE_MAX_CONNECTIONS": "1", **_parse_extra_env_vars(os.environ.get("SLIME_SCRIPT_EXTRA_ENV_VARS", "")),
           **(extra_env_vars or {})}  # fmt: skip
    flags = model_flags(model_preset) + " " if model_preset else ""
    gpus = "" if "--actor-num-gpus-per-node" in train_args else f" --actor-num-nodes 1 --actor-num-gpus-per-node {num_gpus_per_node}"
    return run(f"{sys.executable} {os.path.join(REPO_ROOT, train_script)} {flags}{train_args}{gpus}", env=env)


def _parse_extra_env_vars(text: str) -> dict:
    return dict(item.split("=", 1) for item in text.split() if "=" in item)


def check_has_nvlink() -> bool:
    try:
        out = subprocess.check_output(["nvidia-smi", "topo", "-m"], text=True, stderr=subprocess.DEVNULL)
    except (OSError, subprocess.CalledProcessError):
        return False
    return "NV" in out


def get_default_wandb_args(test_file: str, run_name_prefix: str | None = None, run_id: str | None = None) -> str:
    if not os.environ.get("WANDB_API_KEY"):
        return ""
    name = os.path.basename(test_file).removesuffix(".py")
    run = f"{run_name_prefix + '-' if run_name_prefix else ''}{name}-{run_id or create_run_id()}"
    return f"--use-wandb --wandb-project slime-b200-ci --wandb-group {run} --wandb-key {os.environ['WANDB_API_KEY']} --disable-wandb-random-suffix"


def create_run_id() -> str:
    return datetime.datetime.now(datetime.timezone.utc).strftime("%y%m%d-%H%M%S") + f"-{random.Random().randint(0, 999):03d}"


def get_bool_env_var(name: str, default: str = "false") -> bool:
    value = os.environ.get(name, default).strip().lower()
    if value in ("1", "true", "yes", "y", "on"):
        return True
    if value in ("0", "false", "no", "n", "off", ""):
        return False
    raise ValueError(f"{name}={value!r} is not a boolean")


def get_env_enable_infinite_run() -> bool:
    return get_bool_env_var("SLIME_TEST_ENABLE_INFINITE_RUN")


def save_to_temp_file(text: str, ext: str) -> str:
    with tempfile.NamedTemporaryFile("w", suffix=f".{ext}", delete=False) as f:
        f.write(text)
        return f.name
