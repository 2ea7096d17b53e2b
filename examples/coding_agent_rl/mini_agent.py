"""A small coding agent that needs nothing but Python in the sandbox, and its harness.

The agent is one file (``AGENT_SOURCE``) written into the sandbox: it talks the OpenAI chat-completions protocol to the
adapter with three tools (``read_file``, ``write_file``, ``run``), executes the calls inside the workspace and stops
when the model answers without a tool call or after ``MAX_STEPS`` steps. It stands in for the CLI agents of
``slime_b200.agent.harness`` (Claude Code, Codex) where those cannot be installed, and is what the example's tests
drive; the RL side cannot tell the difference, since it only sees the turns the adapter recorded.
"""

from __future__ import annotations

import shlex
import sys

from slime_b200.agent import sandbox as sbx
from slime_b200.agent.harness.common import BaseHarness, HarnessContext

AGENT_SOURCE = r'''
import json, os, subprocess, sys, urllib.request

URL, SID, MODEL = os.environ["ADAPTER_URL"], os.environ["SESSION_ID"], os.environ.get("MODEL_LABEL", "model")
MAX_STEPS = int(os.environ.get("MAX_STEPS", "24"))
TOOLS = [
    {"type": "function", "function": {"name": "read_file", "description": "Return a file of the workspace.",
        "parameters": {"type": "object", "properties": {"path": {"type": "string"}}, "required": ["path"]}}},
    {"type": "function", "function": {"name": "write_file", "description": "Create or replace a file of the workspace.",
        "parameters": {"type": "object", "properties": {"path": {"type": "string"}, "content": {"type": "string"}},
                       "required": ["path", "content"]}}},
    {"type": "function", "function": {"name": "run", "description": "Run a shell command in the workspace (60 s).",
        "parameters": {"type": "object", "properties": {"cmd": {"type": "string"}}, "required": ["cmd"]}}},
]

def inside(path):
    full = os.path.realpath(os.path.join(os.getcwd(), path))
    if not full.startswith(os.path.realpath(os.getcwd()) + os.sep):
        raise ValueError("path leaves the workspace")
    return full

def call(name, a):
    try:
        if name == "read_file":
            return open(inside(a["path"]), errors="replace").read()[:20000]
        if name == "write_file":
            full = inside(a["path"])
            os.makedirs(os.path.dirname(full), exist_ok=True)
            open(full, "w").write(a["content"])
            return "written"
        if name == "run":
            r = subprocess.run(a["cmd"], shell=True, capture_output=True, text=True, timeout=60)
            return ("exit %d\n" % r.returncode + r.stdout + r.stderr)[-8000:]
        return "unknown tool " + name
    except Exception as e:
        return "error: %r" % (e,)

def chat(messages):
    req = urllib.request.Request(URL.rstrip("/") + "/v1/chat/completions", method="POST",
        data=json.dumps({"model": MODEL, "messages": messages, "tools": TOOLS}).encode(),
        headers={"Content-Type": "application/json", "Authorization": "Bearer " + SID})
    with urllib.request.urlopen(req, timeout=3600) as r:
        return json.loads(r.read())["choices"][0]

messages = [{"role": "system", "content": "You are a software engineer working in a git repository. Use the tools to "
             "inspect and change files and to run commands. When the task is done, reply without a tool call."},
            {"role": "user", "content": sys.stdin.read()}]
for step in range(MAX_STEPS):
    choice = chat(messages)
    msg = choice["message"]
    messages.append(msg)
    print(json.dumps({"step": step, "finish_reason": choice.get("finish_reason"), "tool_calls": len(msg.get("tool_calls") or [])}), flush=True)
    if not msg.get("tool_calls"):
        break
    for tc in msg["tool_calls"]:
        try:
            args = json.loads(tc["function"]["arguments"] or "{}")
        except ValueError:
            args = {}
        messages.append({"role": "tool", "tool_call_id": tc["id"], "content": call(tc["function"]["name"], args)})
'''


class MiniAgentHarness(BaseHarness):
    name = "mini"

    async def install_cli(self, sb) -> None:  # nothing to install: the interpreter is the only dependency
        return None

    async def write_config(self, sb, ctx: HarnessContext) -> None:
        await sb.write_file(f"{ctx.workdir}/.harness/agent.py", AGENT_SOURCE)

    async def launch_and_wait(self, sb, ctx: HarnessContext, prompt: str, time_budget_sec: int) -> int:
        await sb.write_file(f"{ctx.workdir}/.harness/prompt.txt", prompt)
        env = {"ADAPTER_URL": ctx.adapter_url, "SESSION_ID": ctx.session_id, "MODEL_LABEL": ctx.model_label}
        cmd = (f"cd {shlex.quote(ctx.workdir)} && {shlex.quote(sys.executable)} .harness/agent.py < .harness/prompt.txt "
               f"> .harness/trajectory.jsonl 2> .harness/stderr.log")  # fmt: skip
        code, _, _ = await sb.exec(cmd, env=env, timeout=time_budget_sec)
        return sbx.EXIT_TIME_BUDGET_EXCEEDED if code == 124 else code

    async def run(self, sb, *, workdir: str, session_id: str, adapter_url: str, time_budget_sec: int, prompt: str) -> int:
        ctx = HarnessContext(workdir, session_id, adapter_url)  # no separate account: this agent runs as the sandbox's user
        await self.write_config(sb, ctx)
        return await self.launch_and_wait(sb, ctx, prompt, time_budget_sec)
