"""Codex CLI as a sandbox-resident agent, speaking the OpenAI chat protocol to the adapter.

Codex honours ``OPENAI_BASE_URL`` only for its built-in provider, so a custom provider with the URL inline is written
to ``~/.codex/config.toml``; the file is shipped base64-encoded so no shell quoting can mangle it. The session id goes
in ``OPENAI_API_KEY`` and reaches the adapter as the bearer token. Host-side inputs: ``SLIME_AGENT_NODE_TARBALL``,
``SLIME_AGENT_CODEX_TARBALL``; optional ``SLIME_AGENT_CODEX_EXTRA_ARGS`` / ``SLIME_AGENT_CODEX_EXTRA_ENVS``.
Parity: slime/agent/harness/codex.py:21-86.
"""

from __future__ import annotations

import base64
import os
import shlex
from pathlib import Path

from .common import BaseHarness, HarnessContext, install_npm_cli, run_agent


class CodexHarness(BaseHarness):
    name = "codex"
    node_tarball_env = "SLIME_AGENT_NODE_TARBALL"
    cli_tarball_env = "SLIME_AGENT_CODEX_TARBALL"
    extra_args_env = "SLIME_AGENT_CODEX_EXTRA_ARGS"
    extra_envs_env = "SLIME_AGENT_CODEX_EXTRA_ENVS"
    exec_flags = "--skip-git-repo-check"  # shallow or odd clones fail the CLI's own git check
    provider = "slime"

    def config_toml(self, ctx: HarnessContext) -> str:
        return (f'model = "{ctx.model_label}"\nmodel_provider = "{self.provider}"\n\n'
                f'[model_providers.{self.provider}]\nname = "{self.provider}"\nbase_url = "{ctx.adapter_url}/v1"\n'
                f'env_key = "OPENAI_API_KEY"\nwire_api = "chat"\n')  # fmt: skip

    async def install_cli(self, sb) -> None:
        await install_npm_cli(sb, node_runtime=Path(os.environ[self.node_tarball_env]),
                              npm_package=Path(os.environ[self.cli_tarball_env]), check_cmd="codex --version")  # fmt: skip

    async def write_config(self, sb, ctx: HarnessContext) -> None:
        blob = shlex.quote(base64.b64encode(self.config_toml(ctx).encode()).decode())
        await sb.exec(f"mkdir -p /home/agent/.codex && echo {blob} | base64 -d > /home/agent/.codex/config.toml && "
                      f"chown -R agent:agent /home/agent/.codex", user="root", check=True, timeout=60)  # fmt: skip

    async def launch_and_wait(self, sb, ctx: HarnessContext, prompt: str, time_budget_sec: int) -> int:
        cmd, env = self._finish_command(f"codex exec {self.exec_flags} {shlex.quote(prompt)}",
                                        {"OPENAI_API_KEY": ctx.session_id, "OPENAI_BASE_URL": f"{ctx.adapter_url}/v1"})
        return await run_agent(sb, workdir=ctx.workdir, start_cmd=cmd, env=env, time_budget_sec=time_budget_sec)
