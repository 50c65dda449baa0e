"""Torch-facing layer over the native module.

The reference's Python bindings only move CPU buffers (tensorpipe/python/tensorpipe.cc:103-130);
here a message carries torch tensors on CPU or CUDA, a receiver may ask for a dtype conversion
while the data moves, and 2-D strided views (e.g. a transposed matrix) are sent without first
being made contiguous when the selected channel can pack them on the fly.
"""
from __future__ import annotations

import atexit
import json
import threading
import weakref
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from . import _C

DTYPE_CODES = {
    torch.float32: 1,
    torch.bfloat16: 2,
    torch.float16: 3,
    torch.int64: 4,
    torch.int32: 5,
    torch.uint8: 6,
    torch.float64: 7,
    torch.int16: 8,
    torch.int8: 6,
    torch.bool: 6,
}
_CASTABLE = (torch.float32, torch.bfloat16, torch.float16)
_DTYPE_BY_NAME = {str(d).replace("torch.", ""): d for d in DTYPE_CODES}
_DTYPE_NAMES = {d: name for name, d in _DTYPE_BY_NAME.items()}


def kernel_launch_count() -> int:
    """Kernels launched by this library in this process so far."""
    return _C.kernel_launch_count()


def _parse_tensor_metadata(raw: bytes):
    """(dtype name, shape) out of the metadata this module attaches to tensors, or None for anything
    else (a foreign peer's metadata). The exact bytes `_add_tensor` writes are recognised without a
    JSON parser; anything that merely is JSON with those two keys still goes through json."""
    if raw.startswith(b'{"dtype": "') and raw.endswith(b']}'):
        try:
            end = raw.index(b'"', 11)
            if raw[end:end + 13] == b'", "shape": [':
                body = raw[end + 13:-2]
                shape = [int(x) for x in body.split(b",")] if body.strip() else []
                return raw[11:end].decode(), shape
        except ValueError:
            pass
    try:
        meta = json.loads(raw.decode())
    except (ValueError, UnicodeDecodeError):
        return None
    if isinstance(meta, dict) and isinstance(meta.get("shape"), list) and isinstance(meta.get("dtype"), str):
        return meta["dtype"], meta["shape"]
    return None


def _stream_handle(device: torch.device) -> int:
    if device.type != "cuda":
        return 0
    return torch.cuda.current_stream(device).cuda_stream


def _device_str(device: torch.device) -> str:
    if device.type == "cuda":
        index = device.index if device.index is not None else torch.cuda.current_device()
        return f"cuda:{index}"
    return "cpu:0"


@dataclass
class Message:
    """An outgoing message: metadata bytes, payloads (bytes-like) and torch tensors."""

    tensors: Sequence[torch.Tensor] = ()
    payloads: Sequence[bytes] = ()
    metadata: bytes = b""
    target_devices: Optional[Sequence[Optional[str]]] = None  # e.g. ["cuda:1", None]
    # Per-payload / per-tensor metadata strings. Tensor metadata defaults to a small JSON record
    # of dtype and shape, which is what lets the receiving side rebuild torch tensors; override it
    # only when talking to a peer that expects its own format (then tensors arrive as uint8).
    payload_metadata: Optional[Sequence[bytes]] = None
    tensor_metadata: Optional[Sequence[bytes]] = None


@dataclass
class ReceivedMessage:
    metadata: bytes = b""
    payloads: List[bytearray] = field(default_factory=list)
    tensors: List[torch.Tensor] = field(default_factory=list)
    payload_metadata: List[bytes] = field(default_factory=list)
    tensor_metadata: List[bytes] = field(default_factory=list)


class Pipe:
    """One end of a pipe. `write`/`read_descriptor`/`read` mirror the native one-shot callback
    API; `send`/`recv` are future-returning conveniences built on them."""

    def __init__(self, native: "_C.Pipe"):
        self._p = native
        self._lock = threading.Lock()
        self._layouts: Dict[tuple, bool] = {}

    @property
    def remote_name(self) -> str:
        return self._p.remote_name()

    def close(self) -> None:
        self._p.close()

    def set_timeouts(self, write: float = 0.0, read: float = 0.0, descriptor: float = 0.0) -> None:
        """Deadlines in seconds for operations issued from now on (0 = wait forever). A missed
        deadline fails the pipe: the late operation and all later ones report "timeout"."""
        self._p.set_timeouts(int(write * 1000), int(read * 1000), int(descriptor * 1000))

    # ---- native-shaped API ----
    def write(self, message: Message, callback: Callable[[str], None]) -> None:
        out = _C.OutgoingMessage(bytes(message.metadata))
        pmeta = message.payload_metadata or [b""] * len(message.payloads)
        for p, pm in zip(message.payloads, pmeta):
            out.add_payload(p if isinstance(p, (bytes, bytearray, memoryview)) else bytes(p), bytes(pm))
        targets = message.target_devices or [None] * len(message.tensors)
        tmeta = message.tensor_metadata or [None] * len(message.tensors)
        streams: Dict[torch.device, int] = {}  # one current-stream lookup per device and message
        for t, target, tm in zip(message.tensors, targets, tmeta):
            self._add_tensor(out, t, target, tm, streams)
        self._p.write(out, callback)

    def _supports_layouts(self, local: str, target: str) -> bool:
        # Fixed once the pipe is established: a yes is remembered per device pair. A no is asked
        # again next time, because a pipe that is still being set up answers no for every pair.
        key = (local, target)
        if self._layouts.get(key):
            return True
        known = bool(self._p.channel_supports_layouts(local, target))
        if known:
            self._layouts[key] = True
        return known

    def _add_tensor(self, out, t: torch.Tensor, target: Optional[str], metadata: Optional[bytes] = None,
                    streams: Optional[Dict[torch.device, int]] = None) -> None:
        local = _device_str(t.device)
        if (t.device.type == "cpu" and target is not None and target.startswith("cuda") and t.is_contiguous()
                and t.numel() > 0 and torch.cuda.is_available() and t.is_pinned()):
            # Pinned host memory bound for a GPU: handed to the device-to-device channel as a tensor
            # of the current GPU. A large one comes in through the copy engine: straight into a
            # receiver on the same GPU, in pieces that the channel's kernel forwards to another
            # GPU while the next piece is being copied (the host->device copy overlaps the
            # transfer). A small one the kernel reads in place. The message then says the tensor
            # comes from that GPU.
            gpu = torch.device("cuda", torch.cuda.current_device())
            if self._supports_layouts(_device_str(gpu), target):
                return self._add_raw(out, t, t.data_ptr(), gpu, target, metadata, streams, None)
        view = None
        if not t.is_contiguous():
            packable = (
                t.dim() == 2
                and t.numel() > 0
                and t.device.type == "cuda"
                and target is not None
                and self._supports_layouts(local, target)
            )
            if packable:
                view = (t.shape[0], t.shape[1], t.stride(0), t.stride(1))
            else:
                t = t.contiguous()
        self._add_raw(out, t, t.data_ptr(), t.device, target, metadata, streams, view)

    def _add_raw(self, out, t: torch.Tensor, ptr: int, device: torch.device, target: Optional[str],
                 metadata: Optional[bytes], streams: Optional[Dict[torch.device, int]], view) -> None:
        """Adds `t` as a tensor that the library reads at `ptr` on behalf of `device`."""
        meta = metadata if metadata is not None else (
            '{"dtype": "%s", "shape": %s}' % (_DTYPE_NAMES.get(t.dtype) or str(t.dtype).replace("torch.", ""),
                                              list(t.shape))).encode()
        dev_type, dev_index = _device_str(device).split(":")
        if streams is None:
            stream = _stream_handle(device)
        else:
            stream = streams.get(device)
            if stream is None:
                stream = streams[device] = _stream_handle(device)
        out.add_tensor(
            ptr,
            t.numel() * t.element_size(),
            dev_type,
            int(dev_index),
            stream,
            meta,
            DTYPE_CODES.get(t.dtype, 0),
            view,
            target,
            t,
        )

    def read_descriptor(self, callback: Callable[[str, dict], None]) -> None:
        self._p.read_descriptor(callback)

    def read(self, allocation: "_C.Allocation", callback: Callable[[str], None]) -> None:
        self._p.read(allocation, callback)

    # ---- conveniences ----
    def send(self, tensors: Sequence[torch.Tensor] = (), payloads: Sequence[bytes] = (), metadata: bytes = b"",
             target_devices: Optional[Sequence[Optional[str]]] = None,
             payload_metadata: Optional[Sequence[bytes]] = None,
             tensor_metadata: Optional[Sequence[bytes]] = None) -> Future:
        fut: Future = Future()

        def done(err: str) -> None:
            if err:
                fut.set_exception(RuntimeError(err))
            else:
                fut.set_result(None)

        self.write(Message(tensors, payloads, metadata, target_devices, payload_metadata, tensor_metadata), done)
        return fut

    def recv(self, device: Optional[str] = None, cast: Optional[Dict[int, torch.dtype]] = None,
             out: Optional[Sequence[torch.Tensor]] = None) -> Future:
        """Receive the next message. Tensors are allocated with torch on `device` (default: the
        device the sender asked for, else the sender's own device type), or written into `out`.
        `cast` maps a tensor index to the dtype this side wants it converted to on the way."""
        fut: Future = Future()
        cast = cast or {}
        # The descriptor arrives on a library thread, whose notion of "current device" and "current
        # stream" is not the caller's: both are taken here, on the caller's thread, and the
        # allocation below happens under them. The received tensors are then ordered on the stream
        # the caller was working on, and belong to it as far as torch's allocator is concerned.
        # Only devices the caller already works with are asked for their stream: asking a GPU that
        # this process has not touched would create a context on it, and a GPU that serves several
        # processes' contexts time-slices between them.
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            caller_device = torch.cuda.current_device()
            wanted = {caller_device}
            if device is not None and str(device).startswith("cuda"):
                wanted.add(torch.device(device).index if torch.device(device).index is not None else caller_device)
            for t in out or ():
                if t.device.type == "cuda":
                    wanted.add(t.device.index)
            caller_streams = {i: torch.cuda.current_stream(i) for i in wanted}
        else:
            caller_device, caller_streams = None, {}

        def stream_of(dev: torch.device):
            if dev.type != "cuda":
                return None
            index = dev.index if dev.index is not None else caller_device
            return caller_streams.get(index) or torch.cuda.current_stream(dev)

        def on_descriptor(err: str, desc: dict) -> None:
            if err:
                fut.set_exception(RuntimeError(err))
                return
            try:
                msg = ReceivedMessage(metadata=desc["metadata"])
                alloc = _C.Allocation()
                for p in desc["payloads"]:
                    buf = bytearray(p["length"])
                    msg.payloads.append(buf)
                    msg.payload_metadata.append(p["metadata"])
                    alloc.add_payload(buf)
                for i, td in enumerate(desc["tensors"]):
                    msg.tensor_metadata.append(td["metadata"])
                    meta = _parse_tensor_metadata(td["metadata"])
                    if meta is not None and meta[0] not in _DTYPE_BY_NAME:
                        meta = None  # a foreign peer's metadata: deliver the bytes as they are
                    src_dtype = _DTYPE_BY_NAME[meta[0]] if meta else torch.uint8
                    shape = meta[1] if meta else [td["length"]]
                    want = cast.get(i)
                    dst_dtype = want if want is not None else src_dtype
                    here = caller_device if caller_device is not None else 0
                    where = td["target_device"] or device or (
                        f"cuda:{here}" if td["source_device"].startswith("cuda") else "cpu")
                    if out is not None:
                        t = out[i]
                        stream = stream_of(t.device)
                    else:
                        where_dev = torch.device(where.replace("cpu:0", "cpu"))
                        stream = stream_of(where_dev)
                        if stream is not None:
                            with torch.cuda.stream(stream):
                                t = torch.empty(shape, dtype=dst_dtype, device=where_dev)
                        else:
                            t = torch.empty(shape, dtype=dst_dtype, device=where_dev)
                    msg.tensors.append(t)
                    dev_type, _, dev_index = _device_str(t.device).partition(":")
                    cast_code = None
                    if want is not None and want != src_dtype:
                        if want not in _CASTABLE or src_dtype not in _CASTABLE:
                            raise ValueError(f"cannot convert {src_dtype} to {want} in flight")
                        cast_code = DTYPE_CODES[want]
                    alloc.add_tensor(t.data_ptr(), dev_type, int(dev_index),
                                     stream.cuda_stream if stream is not None else 0, cast_code,
                                     DTYPE_CODES.get(src_dtype, 0), t)

                def on_read(err2: str) -> None:
                    if err2:
                        fut.set_exception(RuntimeError(err2))
                    else:
                        fut.set_result(msg)

                self._p.read(alloc, on_read)
            except Exception as exc:  # surface allocation problems to the waiter
                fut.set_exception(exc)

        self._p.read_descriptor(on_descriptor)
        return fut


class Listener:
    def __init__(self, native: "_C.Listener"):
        self._l = native

    def accept(self, callback: Callable[[str, Optional[Pipe]], None]) -> None:
        self._l.accept(lambda err, p: callback(err, Pipe(p) if p is not None else None))

    def accept_future(self) -> Future:
        fut: Future = Future()

        def done(err: str, pipe: Optional[Pipe]) -> None:
            if err:
                fut.set_exception(RuntimeError(err))
            else:
                fut.set_result(pipe)

        self.accept(done)
        return fut

    def url(self, transport: str = "uv") -> str:
        return self._l.url(transport)

    def addresses(self) -> Dict[str, str]:
        return self._l.addresses()

    def close(self) -> None:
        self._l.close()


_live_contexts: "weakref.WeakSet[Context]" = weakref.WeakSet()


def _join_live_contexts() -> None:
    """At interpreter exit: contexts the program never joined are joined here, on the main
    thread and before modules are torn down, so that operations still pending end with an error
    callback while Python can still run one, and no library thread outlives the interpreter."""
    for ctx in list(_live_contexts):
        try:
            ctx.join()
        except Exception:  # noqa: BLE001 - nothing to report to at exit
            pass


atexit.register(_join_live_contexts)


class Context:
    def __init__(self, name: str = ""):
        self._c = _C.Context(name)
        self._joined = False
        _live_contexts.add(self)

    def register_transport(self, priority: int, name: str, transport) -> None:
        self._c.register_transport(priority, name, transport)

    def register_channel(self, priority: int, name: str, channel) -> None:
        self._c.register_channel(priority, name, channel)

    def listen(self, urls: Sequence[str]) -> Listener:
        return Listener(self._c.listen(list(urls)))

    def connect(self, url: str, remote_name: str = "") -> Pipe:
        return Pipe(self._c.connect(url, remote_name))

    def stats(self) -> dict:
        return self._c.stats()

    def close(self) -> None:
        self._c.close()

    def join(self) -> None:
        if not self._joined:
            self._joined = True
            self._c.join()

    def __enter__(self) -> "Context":
        return self

    def __exit__(self, *exc) -> None:
        self.join()


def default_context(name: str = "", shm: bool = True, cuda: Optional[bool] = None, mpt_lanes: int = 0,
                    **cuda_p2p_options) -> Context:
    """A context with every sensible backend registered, best first:
    transports shm (same host) > uv (TCP); channels cuda_p2p (GPU<->GPU over NVLink / same GPU) >
    cuda_basic (anything involving a GPU, staged through pinned memory) > xth (CPU, same process)
    > cma (CPU, same host) > mpt (CPU, striped over TCP lanes, optional) > basic (CPU, anywhere).
    Backends that cannot work on this machine drop out silently. Keyword arguments go to the
    device-to-device channel: eager_threshold, inbox_bytes, max_ctas, wait_with_kernel,
    use_bulk_copy, send_order_min_bytes, host_copy_min_bytes (see channel::cuda_p2p::Options)."""
    ctx = Context(name)
    ctx.register_transport(0, "uv", _C.create_uv_transport())
    if shm:
        ctx.register_transport(10, "shm", _C.create_shm_transport())
    ctx.register_channel(0, "basic", _C.create_basic_channel())
    if mpt_lanes > 0:
        ctx.register_channel(5, "mpt_uv", _C.create_mpt_channel(mpt_lanes))
    ctx.register_channel(10, "cma", _C.create_cma_channel())
    ctx.register_channel(20, "xth", _C.create_xth_channel())
    if cuda is None:
        cuda = torch.cuda.is_available()
    if cuda:
        ctx.register_channel(50, "cuda_basic", _C.create_cuda_basic_channel(_C.create_basic_channel()))
        ctx.register_channel(100, "cuda_p2p", _C.create_cuda_p2p_channel(**cuda_p2p_options))
    return ctx
