"""Task layer of the coding-agent example: what a dataset row means, how its workspace is built, how a patch is graded.

Row schema (``sample.metadata``, or ``sample.label`` as a JSON string / dict):

    instance_id   str
    problem       str   what the agent is asked to do (falls back to the sample's prompt)
    files         {path: content}   the repository at the base commit, inline      -- or --
    repo_url, base_commit           a git remote and the commit to check out
    setup_cmd     str   optional, run once in the workspace (install dependencies, build)
    test_cmd      str   command whose exit code 0 means "solved" (run in a FRESH copy of the workspace + the patch)
    test_files    {path: content}   optional hidden tests written only into the grading copy
    image         str   optional sandbox image (providers that have images)

Grading never trusts the agent's workspace: the patch (``git diff`` against the base commit) is applied to a clean
workspace in a second sandbox, hidden tests are added there and ``test_cmd`` decides. A patch that does not apply,
an empty patch or a timeout scores 0. Same role as examples/coding_agent_rl/swe.py in the reference (its SWE-bench /
Scale-SWE protocols need their graders' packages; this schema needs git and the task's own test command only).
"""

from __future__ import annotations

import dataclasses
import json
import shlex

WORKDIR = "workspace"
_GIT_ID = "-c user.email=agent@example.invalid -c user.name=agent"


@dataclasses.dataclass
class Task:
    instance_id: str
    problem: str
    test_cmd: str
    files: dict | None = None
    repo_url: str | None = None
    base_commit: str | None = None
    setup_cmd: str | None = None
    test_files: dict | None = None
    image: str | None = None


def get_task(sample) -> Task:
    md = sample.metadata if isinstance(getattr(sample, "metadata", None), dict) and sample.metadata.get("test_cmd") else sample.label
    if isinstance(md, str):
        md = json.loads(md)
    if not isinstance(md, dict) or not md.get("test_cmd"):
        raise ValueError("a coding task needs 'test_cmd' (and 'files' or 'repo_url') in the sample's metadata or label")
    if not md.get("files") and not md.get("repo_url"):
        raise ValueError("a coding task needs 'files' or 'repo_url'")
    prompt = md.get("problem") or sample.prompt
    if isinstance(prompt, list):  # chat-format prompt: the user turns, joined
        prompt = "\n\n".join(m.get("content", "") for m in prompt if m.get("role") == "user")
    names = {f.name for f in dataclasses.fields(Task)}
    return Task(**{**{k: v for k, v in md.items() if k in names}, "problem": str(prompt),
                   "instance_id": str(md.get("instance_id", getattr(sample, "index", "task")))})  # fmt: skip


async def prepare_workspace(sb, task: Task, workdir: str = WORKDIR, hidden_tests: bool = False) -> None:
    """A git repository at the task's base state, committed, so that ``git diff`` later is exactly the agent's work."""
    q = shlex.quote(workdir)
    if task.repo_url:
        await sb.exec(f"git clone -q {shlex.quote(task.repo_url)} {q} && cd {q} && git checkout -q {shlex.quote(task.base_commit or 'HEAD')}",
                      check=True, timeout=600)  # fmt: skip
    else:
        await sb.exec(f"mkdir -p {q} && cd {q} && git init -q", check=True, timeout=60)
        for path, content in task.files.items():
            await sb.write_file(f"{workdir}/{path}", content)
        await sb.exec(f"cd {q} && git add -A && git {_GIT_ID} commit -q -m base", check=True, timeout=60)
    if task.setup_cmd:
        await sb.exec(f"cd {q} && {task.setup_cmd}", check=True, timeout=1800)
    if hidden_tests and task.test_files:
        for path, content in task.test_files.items():
            await sb.write_file(f"{workdir}/{path}", content)


async def git_diff(sb, workdir: str = WORKDIR) -> str:
    """Everything the agent changed, new files included, as one patch against the base commit."""
    code, out, _ = await sb.exec(f"cd {shlex.quote(workdir)} && git add -A -N . && git diff HEAD --no-color -- . ':!.harness'", timeout=120)
    return out if code == 0 else ""


async def grade(task: Task, diff_text: str, sandbox_factory, timeout_sec: int = 600) -> tuple[float, dict]:
    """(reward, details). ``sandbox_factory()`` returns a fresh sandbox (async context manager)."""
    if not diff_text.strip():
        return 0.0, {"verdict": "empty_patch"}
    async with sandbox_factory() as ev:
        await prepare_workspace(ev, task, hidden_tests=True)
        await ev.write_file(f"{WORKDIR}/.model.patch", diff_text)
        code, _, err = await ev.exec(f"cd {WORKDIR} && git apply --whitespace=nowarn .model.patch", timeout=120)
        if code != 0:
            return 0.0, {"verdict": "patch_does_not_apply", "stderr": err[-400:]}
        code, out, err = await ev.exec(f"cd {WORKDIR} && {task.test_cmd}", timeout=timeout_sec)
        verdict = "solved" if code == 0 else ("timeout" if code == 124 else "tests_fail")
        return (1.0 if code == 0 else 0.0), {"verdict": verdict, "exit_code": code, "tail": (out + err)[-600:]}
