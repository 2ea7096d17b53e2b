"""Sandbox contract, detached execution and harness plumbing, on the local backend (no containers, no network)."""

import asyncio
import base64
import json

import pytest

from slime_b200.agent import sandbox as sbx
from slime_b200.agent.harness import HARNESSES, ClaudeCodeHarness, CodexHarness, HarnessContext


@pytest.fixture(autouse=True)
def fast_poll(monkeypatch):
    monkeypatch.setattr(sbx, "POLL_INTERVAL_SEC", 0.05)


def run(coro):
    return asyncio.run(coro)


def test_local_sandbox_contract():
    async def body():
        async with sbx.LocalSandbox() as sb:
            assert isinstance(sb, sbx.Sandbox) and sb.sandbox_id.startswith("local-")
            await sb.write_file("/work/a.txt", "hello")
            await sb.write_file("/work/b.bin", b"\x00\x01")
            assert await sb.read_file("/work/a.txt") == "hello"
            assert await sb.read_file("/work/missing") == ""
            code, out, _ = await sb.exec("cat work/a.txt; echo $FOO", env={"FOO": "bar"})
            assert code == 0 and out == "hellobar\n"
            code, _, _ = await sb.exec("exit 3")
            assert code == 3
            with pytest.raises(RuntimeError):
                await sb.exec("exit 3", check=True)
            code, _, err = await sb.exec("sleep 5", timeout=0.2)
            assert code == 124 and err == "timeout"

    run(body())


def test_exec_and_wait_detached_and_retagged():
    async def body():
        async with sbx.LocalSandbox() as sb:
            scratch = sb.root + "/tmp"
            await sb.exec(f"mkdir -p {scratch}")
            code, out = await sbx.exec_and_wait(sb, cmd="echo one; sleep 0.1; echo two", time_budget_sec=5, tag="t",
                                                want_output=True, scratch=scratch)
            assert code == 0 and out == "one\ntwo\n"
            # same tag again: the earlier marker must not leak into this run
            code, tail = await sbx.exec_and_wait(sb, cmd="echo boom >&2; exit 7", time_budget_sec=5, tag="t", scratch=scratch)
            assert code == 7 and "boom" in tail
            code, _ = await sbx.exec_and_wait(sb, cmd="sleep 3", time_budget_sec=0.2, tag="slow", scratch=scratch)
            assert code == sbx.EXIT_TIME_BUDGET_EXCEEDED

    run(body())


class _Recorder:
    """A sandbox that records calls and answers success, with a scripted marker for detached commands."""

    sandbox_id = "rec"

    def __init__(self):
        self.calls, self.files = [], {}

    async def exec(self, cmd, *, user="root", env=None, timeout=120, check=False, idempotent=True):
        self.calls.append((cmd, user, env))
        if cmd.startswith("test -f"):
            return 0, "0\n", ""
        return 0, "", ""

    async def write_file(self, path, content, *, user="root"):
        self.files[path] = content

    async def read_file(self, path, *, user="root"):
        return ""


def test_harness_commands_and_env(monkeypatch):
    monkeypatch.setenv("SLIME_AGENT_CC_EXTRA_ARGS", "--max-turns 5")
    monkeypatch.setenv("SLIME_AGENT_CODEX_EXTRA_ENVS", json.dumps({"RUST_LOG": "info"}))
    assert set(HARNESSES) == {"claude_code", "codex"} and ClaudeCodeHarness() is ClaudeCodeHarness()

    async def body():
        rec = _Recorder()
        code = await ClaudeCodeHarness().run(rec, workdir="/w", session_id="sid-1", adapter_url="http://a:1",
                                             time_budget_sec=5, prompt="fix the 'bug'")
        assert code == 0
        launcher = rec.files["/tmp/.run.sh"]
        assert "/usr/local/bin/claude -p" in launcher and "--max-turns 5" in launcher and "cd /w" in launcher
        spawn = next(c for c in rec.calls if "setsid" in c[0])
        assert spawn[1] == "agent" and spawn[2]["ANTHROPIC_BASE_URL"] == "http://a:1"
        assert spawn[2]["ANTHROPIC_AUTH_TOKEN"] == "sid-1"
        assert any("useradd" in c[0] for c in rec.calls) and any(".claude/settings.json" in c[0] for c in rec.calls)

        rec = _Recorder()
        await CodexHarness().run(rec, workdir="/w", session_id="sid-2", adapter_url="http://a:1", time_budget_sec=5,
                                 prompt="p")
        spawn = next(c for c in rec.calls if "setsid" in c[0])
        assert spawn[2] == {"OPENAI_API_KEY": "sid-2", "OPENAI_BASE_URL": "http://a:1/v1", "RUST_LOG": "info"}
        cfg = next(c[0] for c in rec.calls if "config.toml" in c[0])
        blob = cfg.split("echo ")[1].split(" |")[0].strip("'")
        toml = base64.b64decode(blob).decode()
        assert 'base_url = "http://a:1/v1"' in toml and 'wire_api = "chat"' in toml
        assert "codex exec --skip-git-repo-check p" in rec.files["/tmp/.run.sh"]

    run(body())


def test_e2b_retry_policy():
    class ReadError(Exception):
        pass

    class SandboxException(Exception):
        pass

    sb = sbx.E2BSandbox("img", image_metadata_key="ns/image", rpc_retries=3, size="lg")
    sb.BACKOFF_BASE_SEC = 0.0
    assert sb.metadata() == {"ns/image": "img", "ns/size": "lg"}
    assert sb.is_transient(ReadError()) and sb.is_transient(SandboxException("reset"))
    assert not sb.is_transient(SandboxException("sandbox does not exist")) and not sb.is_transient(ValueError())
    n = {"calls": 0}

    async def flaky():
        n["calls"] += 1
        if n["calls"] < 3:
            raise ReadError()
        return "ok"

    assert run(sb._retry("x", flaky)) == "ok" and n["calls"] == 3
    n["calls"] = 0
    with pytest.raises(ReadError):  # a non-idempotent call is never replayed
        run(sb._retry("x", flaky, idempotent=False))
    assert n["calls"] == 1


def test_serve_in_thread():
    import urllib.request

    from aiohttp import web

    from slime_b200.agent.aiohttp_threaded import serve_in_thread

    async def hi(_):
        return web.json_response({"ok": True})

    app = web.Application()
    app.router.add_get("/hi", hi)
    h = serve_in_thread(app, host="127.0.0.1")
    try:
        assert h.port > 0 and json.loads(urllib.request.urlopen(h.url + "/hi", timeout=5).read()) == {"ok": True}
    finally:
        h.stop()
    assert not h.thread.is_alive()
