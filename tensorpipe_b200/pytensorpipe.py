"""Drop-in for the reference's experimental Python module.

Same names and call shapes as ``pytensorpipe`` (tensorpipe/python/tensorpipe.cc:229-453): callers
register transports and channels on a ``Context``, ``Listener.listen(cb)`` hands over pipes, and
pipes ``write`` / ``read_descriptor`` / ``read`` objects that wrap Python buffers (anything with the
buffer protocol; CPU memory only, as in the reference). Callbacks take no error argument: as in the
reference a failed operation logs and never calls back. For torch tensors, CUDA memory, strided
views and futures use ``tensorpipe_b200.Pipe`` instead.
"""
import sys

import numpy as np

from . import _C

__all__ = [
    "Context", "Listener", "Pipe", "OutgoingPayload", "OutgoingTensor", "OutgoingMessage", "IncomingPayload",
    "IncomingTensor", "IncomingMessage", "create_uv_transport", "create_shm_transport", "create_basic_channel",
    "create_cma_channel", "create_xth_channel", "create_mpt_channel",
]

create_uv_transport = _C.create_uv_transport
create_shm_transport = _C.create_shm_transport
create_basic_channel = _C.create_basic_channel
create_cma_channel = _C.create_cma_channel
create_xth_channel = _C.create_xth_channel
create_mpt_channel = _C.create_mpt_channel


def _log(what):
    print(f"pytensorpipe: {what}", file=sys.stderr)


def _address_of(buffer, writable):
    view = memoryview(buffer)
    if writable and view.readonly:
        raise TypeError("a writable buffer is required")
    if not view.contiguous:
        raise TypeError("a contiguous buffer is required")
    flat = np.frombuffer(view, dtype=np.uint8) if view.nbytes else np.empty(0, dtype=np.uint8)
    return flat.ctypes.data, view.nbytes, (flat, view)


class OutgoingPayload:
    def __init__(self, buffer, metadata):
        self.buffer, self.metadata = buffer, bytes(metadata)


class OutgoingTensor:
    def __init__(self, buffer, metadata):
        self.buffer, self.metadata = buffer, bytes(metadata)


class OutgoingMessage:
    def __init__(self, metadata, payloads, tensors):
        self.metadata, self.payloads, self.tensors = bytes(metadata), list(payloads), list(tensors)


class _Incoming:
    def __init__(self, length, metadata):
        self.length = length
        self.metadata = bytearray(metadata)
        self._buffer = None

    @property
    def buffer(self):
        if self._buffer is None:
            raise ValueError("No buffer")
        return self._buffer

    @buffer.setter
    def buffer(self, value):
        if memoryview(value).nbytes != self.length:
            raise ValueError("Bad length")
        self._buffer = value


class IncomingPayload(_Incoming):
    pass


class IncomingTensor(_Incoming):
    pass


class IncomingMessage:
    def __init__(self, descriptor):
        self.metadata = bytearray(descriptor["metadata"])
        self.payloads = [IncomingPayload(p["length"], p["metadata"]) for p in descriptor["payloads"]]
        self.tensors = [IncomingTensor(t["length"], t["metadata"]) for t in descriptor["tensors"]]


class Pipe:
    def __init__(self, pipe):
        self._pipe = pipe

    def write(self, message, callback):
        out = _C.OutgoingMessage(message.metadata)
        for p in message.payloads:
            out.add_payload(p.buffer, p.metadata)
        for t in message.tensors:
            ptr, nbytes, keep = _address_of(t.buffer, writable=False)
            out.add_tensor(ptr, nbytes, "cpu", 0, metadata=t.metadata, target_device="cpu:0", keep=(keep, t.buffer))

        def done(error):
            if error:
                _log(error)
            else:
                callback()

        self._pipe.write(out, done)

    def read_descriptor(self, callback):
        def done(error, descriptor):
            if error:
                _log(error)
            else:
                callback(IncomingMessage(descriptor))

        self._pipe.read_descriptor(done)

    def read(self, message, callback):
        alloc = _C.Allocation()
        for p in message.payloads:
            alloc.add_payload(p.buffer)
        for t in message.tensors:
            ptr, _, keep = _address_of(t.buffer, writable=True)
            alloc.add_tensor(ptr, "cpu", 0, keep=(keep, t.buffer))

        def done(error):
            if error:
                _log(error)
            else:
                callback()

        self._pipe.read(alloc, done)

    def close(self):
        self._pipe.close()


class Listener:
    def __init__(self, listener):
        self._listener = listener

    def listen(self, callback):
        """Calls ``callback(pipe)`` for every incoming connection until the listener closes."""
        def accepted(error, pipe):
            if error:
                return  # closed
            self._listener.accept(accepted)
            callback(Pipe(pipe))

        self._listener.accept(accepted)

    def get_url(self, transport):
        return self._listener.url(transport)

    def close(self):
        self._listener.close()


class Context:
    def __init__(self):
        self._context = _C.Context("")

    def register_transport(self, priority, name, transport):
        self._context.register_transport(priority, name, transport)

    def register_channel(self, priority, name, channel):
        self._context.register_channel(priority, name, channel)

    def listen(self, urls):
        return Listener(self._context.listen(list(urls)))

    def connect(self, url):
        return Pipe(self._context.connect(url))

    def join(self):
        self._context.join()
