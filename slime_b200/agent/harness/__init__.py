"""Coding-agent harnesses: ``HARNESSES[name]()`` gives the (singleton) harness for ``claude_code`` or ``codex``."""

from .claude_code import ClaudeCodeHarness
from .codex import CodexHarness
from .common import BaseHarness, HarnessContext, install_npm_cli, run_agent

HARNESSES = {h.name: h for h in (ClaudeCodeHarness, CodexHarness)}
__all__ = ["HARNESSES", "BaseHarness", "ClaudeCodeHarness", "CodexHarness", "HarnessContext", "install_npm_cli", "run_agent"]
