"""Claude Code CLI as a sandbox-resident agent. Its Anthropic-protocol calls go to the adapter URL; the session id
travels as the auth token. Host-side inputs: ``SLIME_AGENT_NODE_TARBALL``, ``SLIME_AGENT_CC_TARBALL``; optional
``SLIME_AGENT_CC_EXTRA_ARGS`` (appended to the command) and ``SLIME_AGENT_CC_EXTRA_ENVS`` (JSON object).
Parity: slime/agent/harness/claude_code.py:15-71.
"""

from __future__ import annotations

import json
import os
import shlex
from pathlib import Path

from .common import BaseHarness, HarnessContext, install_npm_cli, run_agent


class ClaudeCodeHarness(BaseHarness):
    name = "claude_code"
    node_tarball_env = "SLIME_AGENT_NODE_TARBALL"
    cli_tarball_env = "SLIME_AGENT_CC_TARBALL"
    extra_args_env = "SLIME_AGENT_CC_EXTRA_ARGS"
    extra_envs_env = "SLIME_AGENT_CC_EXTRA_ENVS"
    binary = "/usr/local/bin/claude"
    launch_flags = ("--permission-mode bypassPermissions --output-format stream-json --include-partial-messages "
                    "--include-hook-events --verbose")  # fmt: skip
    static_env = {"CLAUDE_CODE_DISABLE_NONESSENTIAL_TRAFFIC": "1", "CLAUDE_CODE_DISABLE_EXPERIMENTAL_BETAS": "1",
                  "CLAUDE_CODE_ATTRIBUTION_HEADER": "0"}  # fmt: skip

    async def install_cli(self, sb) -> None:
        await install_npm_cli(sb, node_runtime=Path(os.environ[self.node_tarball_env]),
                              npm_package=Path(os.environ[self.cli_tarball_env]),
                              check_cmd=f"ls -la {self.binary} && {self.binary} --version")  # fmt: skip

    async def write_config(self, sb, ctx: HarnessContext) -> None:
        # both onboarding and the bypass-permissions prompt are acknowledged up front, so the CLI starts headless
        settings = shlex.quote(json.dumps({"hasCompletedOnboarding": True, "bypassPermissionsModeAccepted": True}))
        await sb.exec(f"mkdir -p /home/agent/.claude && echo {settings} | "
                      f"tee /home/agent/.claude.json /home/agent/.claude/settings.json > /dev/null && "
                      f"chown -R agent:agent /home/agent/.claude /home/agent/.claude.json",
                      user="root", check=True, timeout=60)  # fmt: skip

    async def launch_and_wait(self, sb, ctx: HarnessContext, prompt: str, time_budget_sec: int) -> int:
        cmd, env = self._finish_command(
            f"{self.binary} -p {shlex.quote(prompt)} {self.launch_flags}",
            {"ANTHROPIC_BASE_URL": ctx.adapter_url, "ANTHROPIC_AUTH_TOKEN": ctx.session_id,
             "ANTHROPIC_MODEL": ctx.model_label, **self.static_env})  # fmt: skip
        return await run_agent(sb, workdir=ctx.workdir, start_cmd=cmd, env=env, time_budget_sec=time_budget_sec)
