"""Minimal actor runtime: the ``remote()`` / ``get()`` programming model without a cluster manager.

The reference orchestrates its processes with Ray (slime/ray/*.py). On a single 8-GPU box the same
structure needs far less: every actor is a child process (``spawn``) that serves method calls over
a ``multiprocessing.connection`` listener on a Unix socket. Handles are plain picklable addresses,
so any process (driver or another actor) can call any actor; calls return futures.

    h = ActorClass.options(name="rollout", env={"CUDA_VISIBLE_DEVICES": "0"}).remote(args)
    ref = h.generate.remote(3)        # -> ObjectRef (future)
    out = get(ref)                    # blocks; raises ActorDiedError if the process is gone
    kill(h)

Large results can be parked in the node-local object store (``runtime.object_store``) and passed
around as references.
"""

from __future__ import annotations

import atexit
import itertools
import multiprocessing as mp
import os
import pickle
import tempfile
import threading
import time
import traceback
import uuid
from concurrent.futures import Future
from multiprocessing.connection import Client, Listener

_AUTH = b"slime-b200-actors"
_SOCK_DIR = os.environ.get("SLIME_B200_SOCK_DIR") or tempfile.gettempdir()


class ActorDiedError(RuntimeError):
    pass


class RemoteError(RuntimeError):
    """An exception raised inside the actor; carries the remote traceback text."""


class ObjectRef:
    """Future of a remote call (or a value wrapped by ``put``)."""

    __slots__ = ("_future", "_value", "_has_value")

    def __init__(self, future: Future | None = None, value=None, has_value=False):
        self._future, self._value, self._has_value = future, value, has_value

    def result(self, timeout=None):
        if self._has_value:
            return self._value
        return self._future.result(timeout)

    def done(self) -> bool:
        return self._has_value or self._future.done()

    def __reduce__(self):  # a ref crossing a process boundary travels by value
        return (ObjectRef, (None, self.result(), True))


def put(value) -> ObjectRef:
    return ObjectRef(value=value, has_value=True)


def get(refs, timeout: float | None = None):
    if isinstance(refs, (list, tuple)):
        return [get(r, timeout) for r in refs]
    return refs.result(timeout) if isinstance(refs, ObjectRef) else refs


def wait(refs: list[ObjectRef], num_returns: int = 1, timeout: float | None = None):
    deadline = None if timeout is None else time.time() + timeout
    while True:
        done = [r for r in refs if r.done()]
        if len(done) >= num_returns or (deadline is not None and time.time() >= deadline):
            return done, [r for r in refs if not r.done()]
        time.sleep(0.001)


# ----------------------------------------------------------------------------- server side
def _serve(cls, args, kwargs, address, env, ready_path, max_concurrency):
    os.environ.update({k: str(v) for k, v in (env or {}).items()})
    try:  # die with the parent (actors are not daemonic because they may start actors of their own)
        import ctypes
        import signal

        ctypes.CDLL("libc.so.6", use_errno=True).prctl(1, signal.SIGKILL)  # PR_SET_PDEATHSIG
    except Exception:  # noqa: BLE001
        pass
    try:
        instance = cls(*args, **kwargs)
        init_error = None
    except BaseException as e:  # noqa: BLE001
        instance, init_error = None, "".join(traceback.format_exception(e))
    listener = Listener(address, family="AF_UNIX", authkey=_AUTH)
    with open(ready_path, "w") as f:
        f.write(init_error or "ok")
    gate = threading.Semaphore(max_concurrency)
    stop = threading.Event()

    def handle(conn):
        send_lock = threading.Lock()

        def run(call_id, method, a, k):
            with gate:
                try:
                    if init_error is not None:
                        raise RuntimeError("actor constructor failed:\n" + init_error)
                    if method == "__ping__":
                        res = "pong"
                    else:
                        res = getattr(instance, method)(*a, **k)
                    payload = (call_id, True, res)
                except BaseException as e:  # noqa: BLE001
                    payload = (call_id, False, "".join(traceback.format_exception(e)))
            try:
                with send_lock:
                    conn.send(payload)
            except (OSError, pickle.PicklingError, TypeError) as e:
                with send_lock:
                    conn.send((call_id, False, f"result of {method} could not be sent: {e!r}"))

        try:
            while not stop.is_set():
                msg = conn.recv()
                if msg[0] == "__exit__":
                    stop.set()
                    os._exit(0)
                call_id, method, a, k = msg
                if max_concurrency > 1:
                    threading.Thread(target=run, args=(call_id, method, a, k), daemon=True).start()
                else:
                    run(call_id, method, a, k)
        except (EOFError, OSError):
            pass

    while not stop.is_set():
        try:
            conn = listener.accept()
        except OSError:
            break
        threading.Thread(target=handle, args=(conn,), daemon=True).start()


# ----------------------------------------------------------------------------- client side
class _Channel:
    """One connection per (process, actor); a reader thread resolves futures."""

    def __init__(self, address, pid):
        self.address, self.pid = address, pid
        self.conn = Client(address, family="AF_UNIX", authkey=_AUTH)
        self.lock = threading.Lock()
        self.pending: dict[int, Future] = {}
        self.ids = itertools.count()
        self.dead = False
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        try:
            while True:
                call_id, ok, res = self.conn.recv()
                fut = self.pending.pop(call_id, None)
                if fut is None:
                    continue
                if ok:
                    fut.set_result(res)
                else:
                    fut.set_exception(RemoteError(res))
        except (EOFError, OSError):
            self.dead = True
            for fut in list(self.pending.values()):
                if not fut.done():
                    fut.set_exception(ActorDiedError(f"actor at {self.address} died"))
            self.pending.clear()

    def call(self, method, args, kwargs) -> ObjectRef:
        fut: Future = Future()
        if self.dead:
            fut.set_exception(ActorDiedError(f"actor at {self.address} died"))
            return ObjectRef(fut)
        call_id = next(self.ids)
        self.pending[call_id] = fut
        try:
            with self.lock:
                self.conn.send((call_id, method, args, kwargs))
        except (OSError, BrokenPipeError):
            self.dead = True
            self.pending.pop(call_id, None)
            fut.set_exception(ActorDiedError(f"actor at {self.address} died"))
        return ObjectRef(fut)


_channels: dict[tuple[int, str], _Channel] = {}
_channels_lock = threading.Lock()


class _Method:
    def __init__(self, handle, name):
        self.handle, self.name = handle, name

    def remote(self, *args, **kwargs) -> ObjectRef:
        return self.handle._channel().call(self.name, args, kwargs)


class ActorHandle:
    def __init__(self, address: str, pid: int, name: str | None = None):
        self._address, self._pid, self._name = address, pid, name

    def _channel(self) -> _Channel:
        key = (os.getpid(), self._address)
        with _channels_lock:
            ch = _channels.get(key)
            if ch is None or ch.dead:
                try:
                    ch = _Channel(self._address, self._pid)
                except (FileNotFoundError, ConnectionRefusedError):
                    ch = _Channel.__new__(_Channel)
                    ch.address, ch.dead, ch.pending, ch.lock = self._address, True, {}, threading.Lock()
                _channels[key] = ch
            return ch

    def __getattr__(self, item):
        if item.startswith("_"):
            raise AttributeError(item)
        return _Method(self, item)

    def __reduce__(self):
        return (ActorHandle, (self._address, self._pid, self._name))

    def is_alive(self) -> bool:
        try:
            os.kill(self._pid, 0)
        except OSError:
            return False
        try:
            with open(f"/proc/{self._pid}/stat") as f:
                return f.read().split()[2] != "Z"
        except OSError:
            return False


class _Options:
    def __init__(self, cls, **opts):
        self.cls, self.opts = cls, opts

    def remote(self, *args, **kwargs) -> ActorHandle:
        return spawn_actor(self.cls, args, kwargs, **self.opts)


_processes: dict[int, mp.Process] = {}


def spawn_actor(cls, args=(), kwargs=None, *, name=None, env=None, max_concurrency=1, start_timeout=600.0) -> ActorHandle:
    ctx = mp.get_context("spawn")
    address = os.path.join(_SOCK_DIR, f"slb200-{uuid.uuid4().hex[:12]}.sock")
    ready = address + ".ready"
    proc = ctx.Process(target=_serve, args=(cls, args, kwargs or {}, address, env, ready, max_concurrency), daemon=False,
                       name=name or cls.__name__)  # fmt: skip
    proc.start()
    deadline = time.time() + start_timeout
    while not os.path.exists(ready):
        if not proc.is_alive():
            raise ActorDiedError(f"actor {cls.__name__} exited during start-up (exit code {proc.exitcode})")
        if time.time() > deadline:
            proc.kill()
            raise TimeoutError(f"actor {cls.__name__} did not start within {start_timeout}s")
        time.sleep(0.01)
    status = open(ready).read()
    os.unlink(ready)
    if status != "ok":
        proc.kill()
        raise RemoteError(f"constructor of {cls.__name__} failed:\n{status}")
    _processes[proc.pid] = proc
    return ActorHandle(address, proc.pid, name)


def remote(cls=None, **default_opts):
    """Decorator: ``@remote`` gives a class ``.remote(...)`` / ``.options(...).remote(...)`` constructors."""

    def wrap(c):
        c.remote = classmethod(lambda k, *a, **kw: spawn_actor(k, a, kw, **default_opts))
        c.options = classmethod(lambda k, **o: _Options(k, **{**default_opts, **o}))
        return c

    return wrap(cls) if cls is not None else wrap


def kill(handle: ActorHandle, graceful_timeout: float = 0.0):
    """Stop the actor's process. Only the exact PID this runtime started is signalled."""
    proc = _processes.pop(handle._pid, None)
    if graceful_timeout > 0:
        try:
            handle._channel().conn.send(("__exit__",))
        except Exception:  # noqa: BLE001
            pass
        if proc is not None:
            proc.join(graceful_timeout)
    if proc is not None:
        if proc.is_alive():
            proc.kill()
        proc.join(5)
    else:
        try:
            os.kill(handle._pid, 9)
        except OSError:
            pass
    for suffix in ("", ".ready"):
        try:
            os.unlink(handle._address + suffix)
        except OSError:
            pass


def shutdown():
    for pid in list(_processes):
        proc = _processes.pop(pid)
        if proc.is_alive():
            proc.kill()
        proc.join(5)


atexit.register(shutdown)


class Lock:
    """Mutual exclusion between actors (weight broadcasts to shared engines). Host it as an actor:
    ``lock = Lock.remote(); get(lock.acquire.remote()) ... get(lock.release.remote())``."""

    def __init__(self):
        self._held = False

    def acquire(self, blocking: bool = False) -> bool:
        if self._held:
            return False
        self._held = True
        return True

    def release(self):
        self._held = False


remote(Lock)


class LockClient:
    """Spin on a remote ``Lock`` actor with the ``acquire()/release()`` feel of a local lock."""

    def __init__(self, handle, poll=0.002):
        self.handle, self.poll = handle, poll

    def acquire(self):
        while not get(self.handle.acquire.remote()):
            time.sleep(self.poll)

    def release(self):
        get(self.handle.release.remote())

    __enter__ = lambda self: self.acquire()  # noqa: E731

    def __exit__(self, *exc):
        self.release()
