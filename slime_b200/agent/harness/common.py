"""Life cycle of a coding agent (a CLI such as Claude Code or Codex) inside a sandbox.

A harness knows three things about its CLI: how to install it, which config files it wants, and how to run it on a
prompt so that its model calls go to an adapter URL with the session id as the credential. Everything else is shared
here: creating the unprivileged user, the run skeleton, launching detached and polling for the exit code, installing an
npm-packaged CLI on top of a Node runtime tarball. The harness knows nothing about the task; preparing the workspace
and scoring the result belong to the caller. Parity: slime/agent/harness/common.py:43-178.
"""

from __future__ import annotations

import abc
import asyncio
import dataclasses
import lzma
import os
import shutil
import tempfile
from pathlib import Path

from slime_b200.agent import sandbox as sbx
from slime_b200.utils.misc import SingletonMeta

NPM_INSTALL_RETRIES = 3
NPM_INSTALL_BACKOFF_SEC = 2.0


class _SingletonABC(abc.ABCMeta, SingletonMeta):
    pass


@dataclasses.dataclass(frozen=True)
class HarnessContext:
    workdir: str
    session_id: str
    adapter_url: str
    model_label: str = "slime-actor"  # what the CLI is told the model is called; the adapter serves whatever is loaded


class BaseHarness(abc.ABC, metaclass=_SingletonABC):
    name = ""

    @abc.abstractmethod
    async def install_cli(self, sb: sbx.Sandbox) -> None: ...

    @abc.abstractmethod
    async def write_config(self, sb: sbx.Sandbox, ctx: HarnessContext) -> None: ...

    @abc.abstractmethod
    async def launch_and_wait(self, sb: sbx.Sandbox, ctx: HarnessContext, prompt: str, time_budget_sec: int) -> int: ...

    async def run(self, sb: sbx.Sandbox, *, workdir: str, session_id: str, adapter_url: str, time_budget_sec: int,
                  prompt: str) -> int:  # fmt: skip
        """agent user -> config -> launch; returns the CLI's exit code (``EXIT_TIME_BUDGET_EXCEEDED`` on overrun)."""
        await sbx.ensure_agent_user(sb, workdir)
        ctx = HarnessContext(workdir, session_id, adapter_url)
        await self.write_config(sb, ctx)
        return await self.launch_and_wait(sb, ctx, prompt, time_budget_sec)

    # ---- shared by the CLI harnesses: `<base command> <extra args from the environment>` and env overrides as JSON
    extra_args_env = ""
    extra_envs_env = ""

    def _finish_command(self, cmd: str, env: dict[str, str]) -> tuple[str, dict[str, str]]:
        import json

        extra = os.environ.get(self.extra_args_env, "").strip() if self.extra_args_env else ""
        if extra:
            cmd = f"{cmd} {extra}"
        more = os.environ.get(self.extra_envs_env, "").strip() if self.extra_envs_env else ""
        if more:
            env = {**env, **json.loads(more)}
        return cmd, env


async def run_agent(sb: sbx.Sandbox, *, workdir: str, start_cmd: str, env: dict[str, str], time_budget_sec: int) -> int:
    """Run ``start_cmd`` as ``agent`` in ``workdir`` to completion; its output goes to ``.harness/trajectory.jsonl``."""
    meta = f"{workdir}/.harness"
    await sb.exec(f"mkdir -p {meta} && chown agent:agent {meta}", user="root", check=True, timeout=30)
    code, _ = await sbx.exec_and_wait(sb, cmd=start_cmd, user="agent", env=env, workdir=workdir,
                                      out_file=f"{meta}/trajectory.jsonl", time_budget_sec=time_budget_sec, tag="run")  # fmt: skip
    return code


def _plain_tar(tarball: Path) -> Path:
    """``.tar.xz`` -> cached ``.tar`` on the host, so a sandbox image without xz can still unpack it."""
    if tarball.suffix != ".xz":
        return tarball
    plain = Path(tempfile.gettempdir()) / f"sb200_agent.{tarball.stem}"
    if not plain.exists():
        part = plain.with_suffix(plain.suffix + ".partial")
        with lzma.open(tarball, "rb") as src, open(part, "wb") as dst:
            shutil.copyfileobj(src, dst)
        os.replace(part, plain)
    return plain


async def install_node22(sb: sbx.Sandbox, host_tarball: Path) -> None:
    await sb.write_file("/tmp/node22.tar", _plain_tar(Path(host_tarball)))
    links = " && ".join(f"ln -sf /opt/node22/bin/{b} /usr/local/bin/{b}" for b in ("node", "npm", "npx"))
    await sb.exec(f"set -e && mkdir -p /opt/node22 && tar xf /tmp/node22.tar -C /opt/node22 --strip-components=1 && "
                  f"{links} && node --version && npm --version", user="root", timeout=180, check=True)  # fmt: skip


async def install_npm_cli(sb: sbx.Sandbox, *, node_runtime: Path, npm_package: Path, check_cmd: str) -> None:
    """Node runtime, then a global install of the CLI's package tarball, then ``check_cmd``; the install runs detached
    and is retried in place a few times, which is much cheaper than the caller recreating the sandbox."""
    await install_node22(sb, node_runtime)
    await sb.write_file("/tmp/harness-cli.tgz", Path(npm_package))
    cmd = f"npm install -g --prefix=/usr/local --no-audit --no-fund /tmp/harness-cli.tgz && {check_cmd}"
    code, log = 1, ""
    for attempt in range(NPM_INSTALL_RETRIES):
        code, log = await sbx.exec_and_wait(sb, cmd=cmd, user="root", time_budget_sec=300, tag="harness-npm-install")
        if code == 0:
            return
        if attempt + 1 < NPM_INSTALL_RETRIES:
            await asyncio.sleep(NPM_INSTALL_BACKOFF_SEC * (attempt + 1))
    raise RuntimeError(f"npm install failed after {NPM_INSTALL_RETRIES} attempts (exit={code}):\n{log[-1000:]}")
