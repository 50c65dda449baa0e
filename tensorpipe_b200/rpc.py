"""A small torch.distributed.rpc-style agent on top of pipes.

The reference library is the transport under PyTorch's TensorPipe RPC agent (that agent lives in
PyTorch, not in the reference tree); this module is the equivalent layer for this library so that a
user gets `rpc_sync` / `rpc_async` / `remote` with tensors travelling over the best channel
(GPU tensors device to device, CPU tensors over shared memory or TCP) without further plumbing.

    agent = rpc.init_rpc("worker1", rank=1, world_size=2, store=store)
    fut = agent.rpc_async("worker0", torch.add, args=(x, y))
    z = fut.result()
    agent.shutdown()

Rendezvous uses any object with `set(key, bytes)` / `get(key) -> bytes` that blocks until the key
exists (a `torch.distributed.TCPStore` or `FileStore` works). Calls are pickled; tensors found in
args / results are lifted out of the pickle and sent as message tensors.
"""
from __future__ import annotations

import io
import pickle
import threading
from concurrent.futures import Future
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from .core import Context, Pipe, default_context

_REQUEST, _RESPONSE, _ERROR = b"Q", b"R", b"E"


class _TensorPickler(pickle.Pickler):
    """Pickles everything except tensors, which are replaced by their index in `tensors`."""

    def __init__(self, file, tensors: List[torch.Tensor]):
        super().__init__(file, protocol=pickle.HIGHEST_PROTOCOL)
        self._tensors = tensors

    def persistent_id(self, obj):
        if isinstance(obj, torch.Tensor):
            self._tensors.append(obj.detach())
            return ("tensor", len(self._tensors) - 1)
        return None


class _TensorUnpickler(pickle.Unpickler):
    def __init__(self, file, tensors: List[torch.Tensor]):
        super().__init__(file)
        self._tensors = tensors

    def persistent_load(self, pid):
        kind, index = pid
        if kind != "tensor":
            raise pickle.UnpicklingError("unknown persistent id")
        return self._tensors[index]


def _dumps(obj: Any) -> Tuple[bytes, List[torch.Tensor]]:
    tensors: List[torch.Tensor] = []
    buf = io.BytesIO()
    _TensorPickler(buf, tensors).dump(obj)
    return buf.getvalue(), tensors


def _loads(data: bytes, tensors: List[torch.Tensor]) -> Any:
    return _TensorUnpickler(io.BytesIO(data), tensors).load()


def send_object(pipe: Pipe, obj: Any, target_device: Optional[str] = None) -> Future:
    """Send any picklable object over a pipe. Tensors inside it (at any depth) travel as message
    tensors over the best channel instead of through pickle; `target_device` ("cuda:1", "cpu")
    names where the receiver wants them, otherwise the receiver decides."""
    payload, tensors = _dumps(obj)
    targets = [target_device] * len(tensors) if target_device else None
    return pipe.send(tensors, [payload], b"O", target_devices=targets)


def recv_object(pipe: Pipe, device: Optional[str] = None) -> Future:
    """The counterpart of send_object: a future of the object, tensors rebuilt in place."""
    out: Future = Future()

    def done(fut: Future) -> None:
        try:
            msg = fut.result()
            out.set_result(_loads(bytes(msg.payloads[0]), msg.tensors))
        except Exception as exc:  # noqa: BLE001
            out.set_exception(exc)

    pipe.recv(device=device).add_done_callback(done)
    return out


class RRef:
    """Handle on a value that lives on its owner (what `remote` returns)."""

    def __init__(self, agent: "RpcAgent", owner: str, key: int):
        self._agent, self.owner_name, self._key = agent, owner, key

    def to_here(self) -> Any:
        return self._agent.rpc_sync(self.owner_name, _fetch_rref, args=(self._key,))

    def rpc_sync(self, method: str, *args, **kwargs) -> Any:
        return self._agent.rpc_sync(self.owner_name, _call_on_rref, args=(self._key, method, args, kwargs))

    def __reduce__(self):
        return (_rebuild_rref, (self.owner_name, self._key))


_current_agent: Optional["RpcAgent"] = None


def _rebuild_rref(owner: str, key: int) -> RRef:
    return RRef(_current_agent, owner, key)


def _fetch_rref(key: int) -> Any:
    return _current_agent._owned[key]


def _call_on_rref(key: int, method: str, args, kwargs) -> Any:
    return getattr(_current_agent._owned[key], method)(*args, **kwargs)


def _store_result(fn: Callable, args, kwargs) -> int:
    agent = _current_agent
    value = fn(*args, **kwargs)
    with agent._lock:
        agent._next_owned += 1
        key = agent._next_owned
        agent._owned[key] = value
    return key


class RpcAgent:
    def __init__(self, name: str, rank: int, world_size: int, store, context: Optional[Context] = None,
                 listen_urls=("uv://127.0.0.1", "shm://"), device: Optional[str] = None):
        global _current_agent
        self.name, self.rank, self.world_size = name, rank, world_size
        self.device = device  # where incoming CUDA tensors are placed (default: current device)
        self._ctx = context or default_context(name)
        self._listener = self._ctx.listen(list(listen_urls))
        self._lock = threading.Lock()
        self._pipes: Dict[str, Pipe] = {}
        self._accepted: List[Pipe] = []
        self._pending: Dict[int, Future] = {}
        self._next_id = 0
        self._owned: Dict[int, Any] = {}
        self._next_owned = 0
        self._closed = False
        self._store = store
        _current_agent = self
        self._arm_accept()
        store.set(f"tpb_rpc/name/{rank}", name.encode())
        store.set(f"tpb_rpc/url/{name}", self._listener.url("uv").encode())
        self._names = [store.get(f"tpb_rpc/name/{r}").decode() for r in range(world_size)]

    # ---- plumbing ----
    def _arm_accept(self) -> None:
        def on_accept(err: str, pipe: Optional[Pipe]) -> None:
            if err or pipe is None:
                return
            with self._lock:
                self._accepted.append(pipe)
            self._serve(pipe)
            self._arm_accept()

        self._listener.accept(on_accept)

    def _pipe_to(self, worker: str) -> Pipe:
        with self._lock:
            pipe = self._pipes.get(worker)
            if pipe is None:
                url = self._store.get(f"tpb_rpc/url/{worker}").decode()
                pipe = self._ctx.connect(url, remote_name=worker)
                self._pipes[worker] = pipe
                self._serve(pipe)  # responses come back on the same pipe
        return pipe

    def _serve(self, pipe: Pipe) -> None:
        """Keep one receive armed on the pipe; requests run on a worker thread, responses resolve futures."""

        def on_message(fut: Future) -> None:
            if self._closed:
                return
            try:
                msg = fut.result()
            except Exception as exc:  # pipe closed or peer gone: fail what is still waiting on it
                self._fail_pending(pipe, exc)
                return
            pipe.recv(device=self.device).add_done_callback(on_message)
            kind, call_id = msg.metadata[:1], int(msg.metadata[1:])
            if kind == _REQUEST:
                threading.Thread(target=self._run_request, args=(pipe, call_id, msg), daemon=True).start()
            else:
                with self._lock:
                    waiter = self._pending.pop(call_id, None)
                if waiter is None:
                    return
                try:
                    value = _loads(bytes(msg.payloads[0]), msg.tensors)
                except Exception as exc:  # noqa: BLE001
                    waiter.set_exception(exc)
                    return
                if kind == _ERROR:
                    waiter.set_exception(RuntimeError(f"remote call failed: {value}"))
                else:
                    waiter.set_result(value)

        pipe.recv(device=self.device).add_done_callback(on_message)

    def _fail_pending(self, pipe: Pipe, exc: Exception) -> None:
        with self._lock:
            doomed = [(k, f) for k, f in self._pending.items() if getattr(f, "_tpb_pipe", None) is pipe]
            for k, _ in doomed:
                self._pending.pop(k, None)
        for _, f in doomed:
            if not f.done():
                f.set_exception(RuntimeError(f"connection lost: {exc}"))

    def _run_request(self, pipe: Pipe, call_id: int, msg) -> None:
        try:
            fn, args, kwargs = _loads(bytes(msg.payloads[0]), msg.tensors)
            result = fn(*args, **(kwargs or {}))
            kind = _RESPONSE
        except Exception as exc:  # noqa: BLE001 - the error travels back to the caller
            result, kind = f"{type(exc).__name__}: {exc}", _ERROR
        payload, tensors = _dumps(result)
        pipe.send(tensors, [payload], kind + str(call_id).encode())

    # ---- user API ----
    def rpc_async(self, to: str, fn: Callable, args: tuple = (), kwargs: Optional[dict] = None) -> Future:
        if isinstance(to, int):
            to = self._names[to]
        fut: Future = Future()
        if to == self.name:  # local call: no wire
            try:
                fut.set_result(fn(*args, **(kwargs or {})))
            except Exception as exc:  # noqa: BLE001
                fut.set_exception(exc)
            return fut
        pipe = self._pipe_to(to)
        with self._lock:
            self._next_id += 1
            call_id = self._next_id
            fut._tpb_pipe = pipe
            self._pending[call_id] = fut
        payload, tensors = _dumps((fn, args, kwargs))
        sent = pipe.send(tensors, [payload], _REQUEST + str(call_id).encode())

        def on_sent(f: Future) -> None:
            exc = f.exception()
            if exc is not None:
                with self._lock:
                    self._pending.pop(call_id, None)
                if not fut.done():
                    fut.set_exception(exc)

        sent.add_done_callback(on_sent)
        return fut

    def rpc_sync(self, to: str, fn: Callable, args: tuple = (), kwargs: Optional[dict] = None,
                 timeout: Optional[float] = 120.0) -> Any:
        return self.rpc_async(to, fn, args, kwargs).result(timeout)

    def remote(self, to: str, fn: Callable, args: tuple = (), kwargs: Optional[dict] = None) -> RRef:
        if isinstance(to, int):
            to = self._names[to]
        key = self.rpc_sync(to, _store_result, args=(fn, args, kwargs or {}))
        return RRef(self, to, key)

    def worker_names(self) -> List[str]:
        return list(self._names)

    def barrier(self, tag: str = "barrier") -> None:
        """Store-based barrier (every rank must call it with the same tag, once per tag)."""
        self._store.set(f"tpb_rpc/{tag}/{self.rank}", b"1")
        for r in range(self.world_size):
            self._store.get(f"tpb_rpc/{tag}/{r}")

    def shutdown(self, graceful: bool = True) -> None:
        global _current_agent
        if graceful:
            self.barrier("shutdown")
        self._closed = True
        self._ctx.join()
        if _current_agent is self:
            _current_agent = None


def init_rpc(name: str, rank: int, world_size: int, store, **kwargs) -> RpcAgent:
    return RpcAgent(name, rank, world_size, store, **kwargs)
