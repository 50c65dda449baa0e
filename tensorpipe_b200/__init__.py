"""tensorpipe_b200: a Blackwell-native tensor pipe.

Point-to-point, asynchronous, message-oriented transport for messages made of a small CPU core
(metadata + payloads) and tensors on any device, with the capabilities and API shape of
pytorch/tensorpipe (Context / Listener / Pipe / Message; write, read_descriptor, read with
one-shot callbacks) and PyTorch as the framework layer: messages carry torch tensors.

    ctx = tensorpipe_b200.default_context("worker0")
    listener = ctx.listen(["uv://127.0.0.1", "shm://"])
    pipe = ctx.connect(url)
    pipe.send([tensor]).result()          # or pipe.write(message, callback)
    msg = pipe.recv().result()
"""
import torch  # noqa: F401  (loaded first so both extensions share one C++ runtime)

from . import _C  # the native module; importing it fails loudly if it was not built
from .core import (
    Context,
    Listener,
    Pipe,
    Message,
    ReceivedMessage,
    default_context,
    DTYPE_CODES,
    kernel_launch_count,
)

__all__ = [
    "Context",
    "Listener",
    "Pipe",
    "Message",
    "ReceivedMessage",
    "default_context",
    "DTYPE_CODES",
    "kernel_launch_count",
    "_C",
]
