"""The reference's Python module, as served by this library: the scenario of the reference's own
test (tensorpipe/test/python/tensorpipe.py:14-83) plus several connections on one listener."""
import threading

import pytensorpipe as tp


def make_context():
    context = tp.Context()
    context.register_transport(0, "tcp", tp.create_uv_transport())
    context.register_transport(-1, "shm", tp.create_shm_transport())
    context.register_channel(0, "basic", tp.create_basic_channel())
    context.register_channel(-1, "cma", tp.create_cma_channel())
    return context


def test_read_write_with_the_reference_module_names():
    context = make_context()
    pipes = []
    listener = context.listen(["tcp://127.0.0.1"])
    write_completed = threading.Event()

    def on_connection(pipe):
        payload = tp.OutgoingPayload(b"Hello ", b"a greeting")
        tensor = tp.OutgoingTensor(b"World!", b"a place")
        pipe.write(tp.OutgoingMessage(b"metadata", [payload], [tensor]), write_completed.set)
        pipes.append(pipe)

    listener.listen(on_connection)
    client_pipe = context.connect(listener.get_url("tcp"))

    received_payloads, received_tensors = [], []
    read_completed = threading.Event()
    seen = {}

    def on_read_descriptor(message):
        seen["metadata"] = message.metadata
        for payload in message.payloads:
            seen["payload_metadata"] = payload.metadata
            received_payloads.append(bytearray(payload.length))
            payload.buffer = received_payloads[-1]
        for tensor in message.tensors:
            seen["tensor_metadata"] = tensor.metadata
            received_tensors.append(bytearray(tensor.length))
            tensor.buffer = received_tensors[-1]
        client_pipe.read(message, read_completed.set)

    client_pipe.read_descriptor(on_read_descriptor)
    assert write_completed.wait(30)
    assert read_completed.wait(30)
    assert seen == {"metadata": bytearray(b"metadata"), "payload_metadata": bytearray(b"a greeting"),
                    "tensor_metadata": bytearray(b"a place")}
    assert received_payloads == [bytearray(b"Hello ")]
    assert received_tensors == [bytearray(b"World!")]
    context.join()


def test_listener_keeps_accepting():
    context = make_context()
    listener = context.listen(["tcp://127.0.0.1"])
    accepted = []
    three = threading.Event()

    def on_connection(pipe):
        accepted.append(pipe)
        if len(accepted) == 3:
            three.set()

    listener.listen(on_connection)
    clients = [context.connect(listener.get_url("tcp")) for _ in range(3)]
    assert three.wait(30)
    assert len(clients) == 3
    context.join()


def test_incoming_buffer_must_match_the_length():
    msg = tp.IncomingMessage({"metadata": b"", "payloads": [{"length": 4, "metadata": b""}], "tensors": []})
    try:
        msg.payloads[0].buffer = bytearray(3)
    except ValueError:
        pass
    else:
        raise AssertionError("a buffer of the wrong length was accepted")
    try:
        msg.payloads[0].buffer
    except ValueError:
        pass
    else:
        raise AssertionError("reading an unset buffer did not raise")
