"""Where an agent's commands run: a small async sandbox contract and two backends.

Contract (``Sandbox``): ``async with`` life cycle, ``exec(cmd) -> (exit_code, stdout, stderr)``, ``write_file`` (text,
bytes or a host ``Path`` streamed in) and ``read_file``. Task set-up, agent launch and scoring are written against
this contract only, so the provider can be swapped.

Backends:
  ``LocalSandbox``  a scratch directory on this host, commands run with ``bash -c`` as the current user. No isolation:
                    for tests, debugging and trusted tools.
  ``E2BSandbox``    a remote micro-VM through the ``e2b`` client (imported lazily). Transport failures of idempotent
                    calls are retried with jittered exponential back-off; a call marked non-idempotent is never
                    replayed, because a severed response does not say whether the command ran.

``exec_and_wait`` runs a long command *detached*: it writes a launcher script (the command in a subshell, so even an ``exit`` inside it still leaves the marker), starts it under ``setsid`` with output
redirected to a file, and polls for an exit-code marker. Every remote call it makes is short and idempotent, so no
single response stream has to outlive the command, and the polling keeps an idle-collected sandbox alive.
Parity: slime/agent/sandbox.py:28-399.
"""

from __future__ import annotations

import asyncio
import logging
import os
import random
import shlex
import shutil
import tempfile
import time
import uuid
from pathlib import Path
from typing import Protocol, runtime_checkable

logger = logging.getLogger(__name__)

ExecResult = tuple[int, str, str]
FileContent = str | bytes | Path
EXIT_TIME_BUDGET_EXCEEDED = -1
POLL_INTERVAL_SEC = 5.0  # tests lower this


@runtime_checkable
class Sandbox(Protocol):
    sandbox_id: str

    async def __aenter__(self) -> "Sandbox": ...

    async def __aexit__(self, exc_type, exc, tb) -> None: ...

    async def exec(self, cmd: str, *, user: str = "root", env: dict[str, str] | None = None, timeout: int = 120,
                   check: bool = False, idempotent: bool = True) -> ExecResult: ...  # fmt: skip

    async def write_file(self, sandbox_path: str, content: FileContent, *, user: str = "root") -> None: ...

    async def read_file(self, sandbox_path: str, *, user: str = "root") -> str: ...


async def _poll_done_marker(sb: Sandbox, done_file: str, *, user: str, time_budget_sec: float) -> int:
    end = time.monotonic() + time_budget_sec
    q = shlex.quote(done_file)
    while time.monotonic() < end:
        await asyncio.sleep(POLL_INTERVAL_SEC)
        code, out, _ = await sb.exec(f"test -f {q} && cat {q}", user=user, timeout=15)
        if code == 0 and out.strip():
            return int(out.strip())
    return EXIT_TIME_BUDGET_EXCEEDED


async def exec_and_wait(sb: Sandbox, *, cmd: str, time_budget_sec: float, tag: str, user: str = "root",
                        env: dict[str, str] | None = None, workdir: str | None = None, out_file: str | None = None,
                        want_output: bool = False, scratch: str = "/tmp") -> tuple[int, str]:  # fmt: skip
    """Run ``cmd`` detached to completion -> ``(exit_code, output)``.

    ``output`` is the whole log if ``want_output``, the last 512 bytes if the command failed, else empty. The exit
    code is ``EXIT_TIME_BUDGET_EXCEEDED`` when the marker did not appear in time. Two calls with the same ``tag`` must
    not overlap; state left by an earlier call with the tag is cleared first, in its own call, so that a replay of the
    guarded spawn (the ``mkdir`` lock de-duplicates transport retries) can never see a stale marker.
    """
    out_file = out_file or f"{scratch}/.{tag}.out"
    done, launcher, lock = f"{scratch}/.{tag}.done", f"{scratch}/.{tag}.sh", f"{scratch}/.{tag}.spawned"
    head = f"cd {shlex.quote(workdir)}\n" if workdir else ""
    if workdir and user != "root":
        head += f"export HOME=/home/{user}\n"
    await sb.write_file(launcher, f"#!/bin/bash\n{head}(\n{cmd}\n)\necho $? > {done}\n", user=user)
    await sb.exec(f"rm -rf {lock}; rm -f {out_file} {done}", user=user, timeout=30, check=True)
    await sb.exec(f"chmod +x {launcher}; mkdir {lock} 2>/dev/null || exit 0; "
                  f"setsid bash {launcher} < /dev/null > {out_file} 2>&1 &",
                  user=user, env=env, timeout=30, check=True)  # fmt: skip
    code = await _poll_done_marker(sb, done, user=user, time_budget_sec=time_budget_sec)
    if want_output:
        return code, await sb.read_file(out_file, user=user)
    if code == 0:
        return code, ""
    _, tail, _ = await sb.exec(f"tail -c 512 {out_file} 2>/dev/null", user=user, timeout=15)
    return code, tail or ""


async def ensure_agent_user(sb: Sandbox, workdir: str) -> None:
    """An unprivileged ``agent`` account that owns ``workdir`` (agents refuse to run as root; git needs safe.directory)."""
    await sb.exec(f"id agent >/dev/null 2>&1 || useradd -m -s /bin/bash agent && "
                  f"chown -R agent:agent /home/agent {shlex.quote(workdir)} && "
                  f"git config --system --add safe.directory '*' && id agent",
                  user="root", check=True, timeout=60)  # fmt: skip


class LocalSandbox:
    """Commands run on this host inside a private scratch directory (removed on exit). ``user`` is ignored."""

    def __init__(self, root: str | None = None, keep: bool = False):
        self._given_root, self.keep = root, keep
        self.root = ""
        self.sandbox_id = ""

    async def __aenter__(self) -> "LocalSandbox":
        self.root = self._given_root or tempfile.mkdtemp(prefix="sb200-sandbox-")
        os.makedirs(self.root, exist_ok=True)
        self.sandbox_id = f"local-{uuid.uuid4().hex[:12]}"
        return self

    async def __aexit__(self, exc_type, exc, tb) -> None:
        if not self.keep and not self._given_root:
            shutil.rmtree(self.root, ignore_errors=True)

    def _host_path(self, sandbox_path: str) -> str:
        return sandbox_path if sandbox_path.startswith(self.root) else os.path.join(self.root, sandbox_path.lstrip("/"))

    async def exec(self, cmd, *, user="root", env=None, timeout=120, check=False, idempotent=True) -> ExecResult:
        proc = await asyncio.create_subprocess_exec("bash", "-c", cmd, cwd=self.root, env={**os.environ, **(env or {})},
                                                    stdout=asyncio.subprocess.PIPE, stderr=asyncio.subprocess.PIPE,
                                                    stdin=asyncio.subprocess.DEVNULL)  # fmt: skip
        try:
            out, err = await asyncio.wait_for(proc.communicate(), timeout)
        except asyncio.TimeoutError:
            proc.kill()
            await proc.wait()
            if check:
                raise RuntimeError(f"command timed out after {timeout}s: {cmd[:120]}") from None
            return 124, "", "timeout"
        code = proc.returncode
        if check and code != 0:
            raise RuntimeError(f"command failed (exit={code}): {cmd[:120]}\n{err.decode(errors='replace')[:400]}")
        return code, out.decode(errors="replace"), err.decode(errors="replace")

    async def write_file(self, sandbox_path, content, *, user="root") -> None:
        dst = self._host_path(sandbox_path)
        os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
        if isinstance(content, Path):
            shutil.copyfile(content, dst)
        else:
            with open(dst, "wb") as f:
                f.write(content.encode() if isinstance(content, str) else content)

    async def read_file(self, sandbox_path, *, user="root") -> str:
        try:
            with open(self._host_path(sandbox_path), errors="replace") as f:
                return f.read()
        except OSError:
            return ""


def _env_first(names: tuple[str, ...], default: str = "") -> str:
    """First non-blank value among ``names`` (canonical name first, legacy aliases after)."""
    for n in names:
        v = os.environ.get(n)
        if v is not None and v.strip():
            return v
    return default


class E2BSandbox:
    """``e2b.AsyncSandbox`` behind the ``Sandbox`` contract.

    Settings (environment; the ``SWE_*`` names are accepted as aliases): ``SLIME_AGENT_SANDBOX_IMAGE_METADATA_KEY``
    (required: the metadata key the gateway routes images by), ``SLIME_AGENT_SANDBOX_LIFETIME_SEC`` (3600),
    ``SLIME_AGENT_SANDBOX_RPC_RETRIES`` (6), ``SLIME_AGENT_E2B_SANDBOX_SIZE`` ("md").
    """

    ENV_IMAGE_KEY = ("SLIME_AGENT_SANDBOX_IMAGE_METADATA_KEY", "SWE_SANDBOX_IMAGE_METADATA_KEY")
    ENV_LIFETIME = ("SLIME_AGENT_SANDBOX_LIFETIME_SEC", "SWE_SANDBOX_LIFETIME_SEC")
    ENV_RETRIES = ("SLIME_AGENT_SANDBOX_RPC_RETRIES", "SWE_RPC_RETRIES")
    ENV_SIZE = ("SLIME_AGENT_E2B_SANDBOX_SIZE", "SWE_E2B_SANDBOX_SIZE")
    BACKOFF_BASE_SEC, BACKOFF_CAP_SEC = 1.0, 32.0
    # exception class names of the http stack underneath that mean "the transport broke", not "the call was wrong"
    TRANSIENT = frozenset({"ProtocolError", "LocalProtocolError", "RemoteProtocolError", "WriteError", "ReadError",
                           "ConnectError", "ConnectTimeout", "ReadTimeout", "WriteTimeout", "PoolTimeout", "SSLError"})  # fmt: skip

    def __init__(self, image: str, *, timeout: int | None = None, image_metadata_key: str | None = None,
                 rpc_retries: int | None = None, size: str | None = None):  # fmt: skip
        self.image = image
        self.timeout = int(_env_first(self.ENV_LIFETIME, "3600")) if timeout is None else timeout
        self.image_metadata_key = image_metadata_key or _env_first(self.ENV_IMAGE_KEY) or None
        self.rpc_retries = int(_env_first(self.ENV_RETRIES, "6")) if rpc_retries is None else rpc_retries
        self.size = _env_first(self.ENV_SIZE, "md") if size is None else size
        self._sb = None
        self.sandbox_id = ""

    @classmethod
    def is_transient(cls, e: BaseException) -> bool:
        name = type(e).__name__
        if name in cls.TRANSIENT:
            return True
        if name == "SandboxException":  # the client's catch-all; a sandbox that is gone stays gone
            return not ("does not exist" in str(e) or "STOPPED state" in str(e))
        return False

    async def _retry(self, what: str, make_call, *, idempotent: bool = True):
        last = None
        for attempt in range(max(self.rpc_retries, 1)):
            try:
                return await make_call()
            except Exception as e:  # noqa: BLE001
                if not self.is_transient(e) or not idempotent:
                    raise
                last = e
                if attempt + 1 < self.rpc_retries:
                    await self._drop_connections()
                    pause = random.uniform(0.0, min(self.BACKOFF_CAP_SEC, self.BACKOFF_BASE_SEC * 2**attempt))
                    logger.debug("sandbox %s: transient %s, retry %d/%d in %.1fs", what, type(e).__name__,
                                 attempt + 1, self.rpc_retries, pause)  # fmt: skip
                    await asyncio.sleep(pause)
        raise last

    async def _drop_connections(self) -> None:
        try:
            await self._sb._transport.pool.aclose()  # next call reconnects
        except Exception:  # noqa: BLE001
            pass

    def metadata(self) -> dict[str, str]:
        md = {self.image_metadata_key: self.image}
        if self.size:
            ns = self.image_metadata_key.rsplit("/", 1)[0] if "/" in self.image_metadata_key else ""
            md[f"{ns}/size" if ns else "size"] = self.size
        return md

    async def __aenter__(self) -> "E2BSandbox":
        if self.image_metadata_key is None:
            raise RuntimeError(f"{self.ENV_IMAGE_KEY[0]} is not set: export the metadata key your E2B gateway uses "
                               f"for image routing ({self.ENV_IMAGE_KEY[1]} is accepted too)")  # fmt: skip
        from e2b import AsyncSandbox

        self._sb = await self._retry("create", lambda: AsyncSandbox.create(timeout=self.timeout, metadata=self.metadata()))
        self.sandbox_id = self._sb.sandbox_id
        return self

    async def __aexit__(self, exc_type, exc, tb) -> None:
        try:
            if self._sb is not None:
                await self._sb.kill()
        except Exception as e:  # noqa: BLE001
            logger.warning("sandbox %s: kill failed: %s", self.sandbox_id[:8], e)

    async def exec(self, cmd, *, user="root", env=None, timeout=120, check=False, idempotent=True) -> ExecResult:
        try:
            r = await self._retry(f"exec({cmd[:60]!r})",
                                  lambda: self._sb.commands.run(cmd, user=user, envs=env, timeout=timeout,
                                                                on_stdout=lambda s: None, on_stderr=lambda s: None),
                                  idempotent=idempotent)  # fmt: skip
            return r.exit_code, r.stdout or "", r.stderr or ""
        except Exception as e:  # noqa: BLE001
            if type(e).__name__ != "CommandExitException":
                raise
            if check:
                raise RuntimeError(f"sandbox exec failed (exit={e.exit_code}): {cmd[:120]}\n{(e.stderr or '')[:400]}") from None
            return e.exit_code, e.stdout or "", e.stderr or ""

    async def write_file(self, sandbox_path, content, *, user="root") -> None:
        if isinstance(content, Path):
            async def send():  # reopen per attempt: a retried upload must start from byte 0
                with open(content, "rb") as f:
                    return await self._sb.files.write(sandbox_path, f, user=user)
        else:
            data = content.encode() if isinstance(content, str) else content

            async def send():
                return await self._sb.files.write(sandbox_path, data, user=user)
        await self._retry(f"write_file({sandbox_path})", send)

    async def read_file(self, sandbox_path, *, user="root") -> str:
        try:
            return await self._retry(f"read_file({sandbox_path})", lambda: self._sb.files.read(sandbox_path, user=user))
        except Exception:  # noqa: BLE001
            return ""
