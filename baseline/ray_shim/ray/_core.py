"""A small stand-in for the parts of Ray that the reference uses, for images where Ray is not installed.

Ray gives the reference three things: actors (one ``PiperActor`` process per GPU, reached through
``handle.method.remote()``), tasks (one ``run_dp_rank`` driver per data-parallel replica) and named actors as a
key-value store.  This module provides the same surface over plain sockets on one host:

* every process of the job (one per GPU, started by ``torch.distributed.run`` or a single ``python``) runs a
  server thread; process ``r`` publishes its listening address in a rendezvous directory;
* ``Class.remote(...)`` asks a placement function which process should host the new actor (the default is the
  calling process) and sends it a ``create`` request; the host gives each actor a dedicated thread that executes
  its method calls in arrival order, as Ray does for a default actor;
* ``handle.method.remote(...)`` returns an ``ObjectRef`` backed by a future; arguments and results always cross
  a ``cloudpickle`` round trip, also for an actor in the same process, so the callee never shares objects with
  the caller (the reference relies on that: ``load_training_dag`` decorates the graph it is given);
* names of named actors live in a registry held by process 0.

Only what ``src/*.py`` and ``examples/test_llama.py`` of the reference call is implemented.
"""
from __future__ import annotations

import itertools
import os
import queue
import threading
import time
import traceback
from concurrent.futures import FIRST_COMPLETED, FIRST_EXCEPTION, Future
from concurrent.futures import wait as _fut_wait
from multiprocessing.connection import Client, Listener

import cloudpickle

_AUTH = b"piper-ray-shim"


class GetTimeoutError(TimeoutError):
    pass


class RayError(Exception):
    pass


class RayTaskError(RayError):
    pass


class RayActorError(RayError):
    pass


class ActorDiedError(RayActorError):
    pass


class ObjectRef:
    """Handle of a pending result."""

    __slots__ = ("_fut",)

    def __init__(self, fut: Future) -> None:
        self._fut = fut

    def __reduce__(self):
        # a reference that crosses a process boundary carries its value, as Ray resolves arguments before a call
        return (_resolved_ref, (self._fut.result(),))


def _resolved_ref(value):
    f: Future = Future()
    f.set_result(value)
    return ObjectRef(f)


def _dumps(obj) -> bytes:
    return cloudpickle.dumps(obj)


def _loads(data: bytes):
    return cloudpickle.loads(data)


def _pack_exception(exc: BaseException) -> bytes:
    text = "".join(traceback.format_exception(type(exc), exc, exc.__traceback__))
    try:
        return _dumps((exc, text))
    except Exception:
        return _dumps((RayTaskError(f"{type(exc).__name__}: {exc}"), text))


class _LocalActor:
    """An actor hosted by this process: the instance plus the thread that runs its calls one at a time."""

    def __init__(self, runtime: "Runtime", actor_id: str, instance) -> None:
        self.runtime, self.actor_id, self.instance = runtime, actor_id, instance
        self.calls: "queue.Queue" = queue.Queue()
        self.alive = True
        self.thread = threading.Thread(target=self._loop, name=f"actor-{actor_id}", daemon=True)
        self.thread.start()

    def _loop(self) -> None:
        while True:
            item = self.calls.get()
            if item is None:
                return
            fn, reply = item
            try:
                ok, payload = True, _dumps(fn(self.instance))
            except BaseException as exc:  # noqa: BLE001 - shipped to the caller
                ok, payload = False, _pack_exception(exc)
            reply(ok, payload)

    def submit(self, fn, reply) -> None:
        if not self.alive:
            reply(False, _pack_exception(ActorDiedError(f"actor {self.actor_id} was killed")))
            return
        self.calls.put((fn, reply))

    def kill(self) -> None:
        self.alive = False
        self.calls.put(None)


class _Peer:
    """Client side of the connection to another process: one socket, one reader thread, futures by call id."""

    def __init__(self, address) -> None:
        self.conn = Client(address, authkey=_AUTH)
        self.lock = threading.Lock()
        self.pending: dict[int, Future] = {}
        self.ids = itertools.count()
        threading.Thread(target=self._reader, daemon=True).start()

    def _reader(self) -> None:
        try:
            while True:
                call_id, ok, payload = self.conn.recv()
                fut = self.pending.pop(call_id, None)
                if fut is None:
                    continue
                _resolve(fut, ok, payload)
        except (EOFError, OSError):
            for fut in list(self.pending.values()):
                if not fut.done():
                    fut.set_exception(ActorDiedError("connection to the hosting process was lost"))

    def request(self, msg: tuple) -> Future:
        fut: Future = Future()
        with self.lock:
            call_id = next(self.ids)
            self.pending[call_id] = fut
            self.conn.send((call_id,) + msg)
        return fut


def _resolve(fut: Future, ok: bool, payload: bytes) -> None:
    if ok:
        fut.set_result(_loads(payload))
        return
    exc, text = _loads(payload)
    try:
        exc.add_note("remote traceback:\n" + text)
    except Exception:
        pass
    fut.set_exception(exc)


class Runtime:
    def __init__(self, rank: int, world: int, rendezvous_dir: str | None) -> None:
        self.rank, self.world, self.dir = rank, world, rendezvous_dir
        self.actors: dict[str, _LocalActor] = {}
        self.names: dict[str, tuple[int, str, list]] = {}       # process 0 only: name -> (rank, actor id, methods)
        self.names_lock = threading.Lock()
        self.peers: dict[int, _Peer] = {}
        self.peers_lock = threading.Lock()
        self.ids = itertools.count()
        self.shutdown_event = threading.Event()
        self.placement = None
        self.listener = None
        if world > 1:
            self.listener = Listener(("127.0.0.1", 0), authkey=_AUTH)
            os.makedirs(rendezvous_dir, exist_ok=True)
            tmp = os.path.join(rendezvous_dir, f".addr.{rank}.tmp")
            with open(tmp, "w") as f:
                f.write(f"{self.listener.address[0]}:{self.listener.address[1]}")
            os.replace(tmp, os.path.join(rendezvous_dir, f"addr.{rank}"))
            threading.Thread(target=self._accept_loop, daemon=True).start()

    # ---- server side -------------------------------------------------------------------------------------
    def _accept_loop(self) -> None:
        while not self.shutdown_event.is_set():
            try:
                conn = self.listener.accept()
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn) -> None:
        send_lock = threading.Lock()

        def replier(call_id):
            def reply(ok, payload):
                with send_lock:
                    try:
                        conn.send((call_id, ok, payload))
                    except OSError:
                        pass
            return reply

        try:
            while True:
                msg = conn.recv()
                call_id, kind, rest = msg[0], msg[1], msg[2:]
                self._handle(kind, rest, replier(call_id))
        except (EOFError, OSError):
            return

    def _handle(self, kind: str, rest: tuple, reply) -> None:
        try:
            if kind == "create":
                actor_id, blob = rest
                cls, args, kwargs = _loads(blob)
                self.actors[actor_id] = _LocalActor(self, actor_id, cls(*args, **kwargs))
                reply(True, _dumps(None))
            elif kind == "call":
                actor_id, method, blob = rest
                actor = self.actors.get(actor_id)
                if actor is None:
                    raise ActorDiedError(f"no actor {actor_id} in process {self.rank}")
                args, kwargs = _loads(blob)
                actor.submit(lambda inst: getattr(inst, method)(*args, **kwargs), reply)
            elif kind == "apply":
                actor_id, blob = rest
                actor = self.actors.get(actor_id)
                if actor is None:
                    raise ActorDiedError(f"no actor {actor_id} in process {self.rank}")
                fn, args, kwargs = _loads(blob)
                actor.submit(lambda inst: fn(inst, *args, **kwargs), reply)
            elif kind == "task":
                (blob,) = rest
                fn, args, kwargs = _loads(blob)

                def run():
                    try:
                        ok, payload = True, _dumps(fn(*args, **kwargs))
                    except BaseException as exc:  # noqa: BLE001
                        ok, payload = False, _pack_exception(exc)
                    reply(ok, payload)
                threading.Thread(target=run, daemon=True).start()
            elif kind == "kill":
                (actor_id,) = rest
                actor = self.actors.pop(actor_id, None)
                if actor is not None:
                    actor.kill()
                reply(True, _dumps(None))
            elif kind == "name_register":
                name, rank, actor_id, methods, if_absent = rest
                with self.names_lock:
                    if name in self.names and if_absent:
                        reply(True, _dumps(self.names[name]))
                        return
                    if name in self.names:
                        raise ValueError(f"an actor named {name!r} already exists")
                    self.names[name] = (rank, actor_id, methods)
                reply(True, _dumps(None))
            elif kind == "name_lookup":
                (name,) = rest
                with self.names_lock:
                    reply(True, _dumps(self.names.get(name)))
            elif kind == "name_remove":
                (actor_id,) = rest
                with self.names_lock:
                    for k in [k for k, v in self.names.items() if v[1] == actor_id]:
                        del self.names[k]
                reply(True, _dumps(None))
            elif kind == "shutdown":
                reply(True, _dumps(None))
                self.shutdown_event.set()
            else:
                raise ValueError(f"unknown request {kind!r}")
        except BaseException as exc:  # noqa: BLE001
            reply(False, _pack_exception(exc))

    # ---- client side -------------------------------------------------------------------------------------
    def _peer(self, rank: int) -> _Peer:
        with self.peers_lock:
            peer = self.peers.get(rank)
            if peer is None:
                path = os.path.join(self.dir, f"addr.{rank}")
                deadline = time.monotonic() + 600
                while not os.path.exists(path):
                    if time.monotonic() > deadline:
                        raise TimeoutError(f"process {rank} never published its address in {self.dir}")
                    time.sleep(0.02)
                host, port = open(path).read().split(":")
                peer = self.peers[rank] = _Peer((host, int(port)))
            return peer

    def request(self, rank: int, kind: str, *rest) -> Future:
        if rank == self.rank:
            fut: Future = Future()
            self._handle(kind, rest, lambda ok, payload: _resolve(fut, ok, payload))
            return fut
        return self._peer(rank).request((kind,) + rest)

    def new_id(self) -> str:
        return f"{self.rank}.{next(self.ids)}"

    def place(self, kind: str, target, args, kwargs, options) -> int:
        if self.placement is not None:
            r = self.placement(kind, target, args, kwargs, options)
            if r is not None:
                return int(r) % self.world
        return self.rank

    def serve_until_shutdown(self) -> None:
        self.shutdown_event.wait()

    def shutdown_all(self) -> None:
        for r in range(self.world):
            if r != self.rank:
                try:
                    self.request(r, "shutdown").result(timeout=10)
                except Exception:
                    pass
        self.shutdown_event.set()


_runtime: Runtime | None = None


def start(rank: int = 0, world: int = 1, rendezvous_dir: str | None = None) -> Runtime:
    global _runtime
    if _runtime is None:
        _runtime = Runtime(rank, world, rendezvous_dir)
    return _runtime


def runtime() -> Runtime:
    return start()


def set_placement(fn) -> None:
    """``fn(kind, target, args, kwargs, options) -> process index or None``; ``kind`` is "actor" or "task"."""
    runtime().placement = fn


# ---- the user-facing objects -------------------------------------------------------------------------------
class _MethodProxy:
    def __init__(self, handle: "ActorHandle", name: str) -> None:
        self._handle, self._name = handle, name

    def remote(self, *args, **kwargs) -> ObjectRef:
        h = self._handle
        if self._name == "__ray_terminate__":
            return ObjectRef(runtime().request(h._rank, "kill", h._actor_id))
        return ObjectRef(runtime().request(h._rank, "call", h._actor_id, self._name, _dumps((args, kwargs))))

    def options(self, **_):
        return self


class ActorHandle:
    def __init__(self, rank: int, actor_id: str, methods: list) -> None:
        self._rank, self._actor_id, self._methods = rank, actor_id, list(methods)

    def __getattr__(self, name: str):
        if name.startswith("_") and name not in self._methods and name != "__ray_terminate__":
            raise AttributeError(name)
        return _MethodProxy(self, name)

    def __reduce__(self):
        return (ActorHandle, (self._rank, self._actor_id, self._methods))


def apply_on_actor(handle: ActorHandle, fn, *args, **kwargs) -> ObjectRef:
    """Run ``fn(instance, *args, **kwargs)`` in the actor's own thread (not part of Ray: used for device timers)."""
    return ObjectRef(runtime().request(handle._rank, "apply", handle._actor_id, _dumps((fn, args, kwargs))))


class _ActorClass:
    def __init__(self, cls, options: dict | None = None) -> None:
        self._cls, self._options = cls, dict(options or {})
        self.__name__ = getattr(cls, "__name__", "Actor")

    def options(self, **kw) -> "_ActorClass":
        return _ActorClass(self._cls, {**self._options, **kw})

    def remote(self, *args, **kwargs) -> ActorHandle:
        rt = runtime()
        name = self._options.get("name")
        methods = [m for m in dir(self._cls) if callable(getattr(self._cls, m, None)) and not m.startswith("__")]
        if name is not None and self._options.get("get_if_exists", False):
            existing = rt.request(0, "name_lookup", name).result()
            if existing is not None:
                return ActorHandle(*existing)
        rank = rt.place("actor", self._cls, args, kwargs, self._options)
        actor_id = rt.new_id()
        rt.request(rank, "create", actor_id, _dumps((self._cls, args, kwargs))).result()
        if name is not None:
            # the name becomes visible only once the actor exists, so a lookup never returns a handle that
            # cannot be called yet
            existing = rt.request(0, "name_register", name, rank, actor_id, methods,
                                  bool(self._options.get("get_if_exists", False))).result()
            if existing is not None:                      # somebody else registered the name first
                rt.request(rank, "kill", actor_id).result()
                return ActorHandle(*existing)
        return ActorHandle(rank, actor_id, methods)

    def __call__(self, *a, **k):
        raise TypeError(f"actor class {self.__name__} cannot be instantiated directly; use .remote()")


class _RemoteFunction:
    def __init__(self, fn, options: dict | None = None) -> None:
        self._fn, self._options = fn, dict(options or {})
        self.__name__ = getattr(fn, "__name__", "task")

    def options(self, **kw) -> "_RemoteFunction":
        return _RemoteFunction(self._fn, {**self._options, **kw})

    def remote(self, *args, **kwargs) -> ObjectRef:
        rt = runtime()
        rank = rt.place("task", self._fn, args, kwargs, self._options)
        return ObjectRef(rt.request(rank, "task", _dumps((self._fn, args, kwargs))))

    def __call__(self, *a, **k):
        raise TypeError(f"remote function {self.__name__} cannot be called directly; use .remote()")


def remote(*args, **kwargs):
    def wrap(target):
        return _ActorClass(target, kwargs) if isinstance(target, type) else _RemoteFunction(target, kwargs)
    if len(args) == 1 and not kwargs and (isinstance(args[0], type) or callable(args[0])):
        return wrap(args[0])
    return wrap


def get(refs, timeout: float | None = None):
    """Values of one reference or a list.  A list fails as soon as any member has failed, so that a caller is not
    left waiting on a healthy actor that is itself blocked on the failed one."""
    single = isinstance(refs, ObjectRef)
    items = [refs] if single else list(refs)
    for r in items:
        if not isinstance(r, ObjectRef):
            raise TypeError(f"ray.get expects ObjectRef(s), got {type(r).__name__}")
    deadline = None if timeout is None else time.monotonic() + timeout
    pending = {r._fut for r in items}
    while pending:
        left = None if deadline is None else max(0.0, deadline - time.monotonic())
        done, pending = _fut_wait(pending, timeout=left, return_when=FIRST_EXCEPTION)
        for f in done:
            if f.exception() is not None:
                raise f.exception()
        if pending and deadline is not None and time.monotonic() >= deadline:
            raise GetTimeoutError(f"ray.get timed out after {timeout}s")
    out = [r._fut.result() for r in items]
    return out[0] if single else out


def wait(refs, num_returns: int = 1, timeout: float | None = None):
    refs = list(refs)
    deadline = None if timeout is None else time.monotonic() + timeout
    while True:
        done = [r for r in refs if r._fut.done()]
        if len(done) >= num_returns:
            done = done[:num_returns]
            return done, [r for r in refs if r not in done]
        left = None if deadline is None else deadline - time.monotonic()
        if left is not None and left <= 0:
            return done, [r for r in refs if r not in done]
        _fut_wait([r._fut for r in refs if not r._fut.done()], timeout=left, return_when=FIRST_COMPLETED)


def get_actor(name: str, namespace: str | None = None) -> ActorHandle:
    entry = runtime().request(0, "name_lookup", name).result()
    if entry is None:
        raise ValueError(f"Failed to look up actor with name {name!r}")
    return ActorHandle(*entry)


def kill(handle: ActorHandle, no_restart: bool = True) -> None:
    rt = runtime()
    rt.request(handle._rank, "kill", handle._actor_id).result()
    rt.request(0, "name_remove", handle._actor_id).result()


def put(value) -> ObjectRef:
    return _resolved_ref(value)
