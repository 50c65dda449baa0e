"""The allocation-free C entry point (include/tpb/noalloc.h) against the library's ordinary push kernel.

Some callers of this library cannot call cudaMalloc: a serving loop that must not trigger the
device-wide synchronisation an allocation implies, a plugin living inside a fixed memory budget, a
process whose framework already owns all device memory. For them the library exports
`tpb_noalloc_push`, whose scratch memory is a fixed array inside the library image. This test calls
it through its exported C symbol (ctypes, no Python binding in between) and checks that it moves
exactly the bytes the ordinary entry point moves, twice in a row, because the second call finds the
first call's table and counter still in the shared array.

This file is collected last on purpose: should it fail, a run that stops at the first failure has
already run every other test.
"""
import ctypes

import pytest
import torch

import tensorpipe_b200 as tpb
from tensorpipe_b200 import _C

MAX_ITEMS = 256


class Item(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst", ctypes.c_void_p), ("bytes", ctypes.c_uint64)]


def load_symbol():
    lib = ctypes.CDLL(_C.__file__)
    fn = lib.tpb_noalloc_push
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(Item), ctypes.c_size_t, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p]
    err = lib.tpb_noalloc_strerror
    err.restype = ctypes.c_char_p
    err.argtypes = [ctypes.c_int]
    return fn, err


def ranges(rng_seed):
    """(source offset, destination offset, length) triples: empty, tiny, ragged, odd offsets, several tiles."""
    g = torch.Generator().manual_seed(rng_seed)
    sizes = [0, 1, 15, 16, 17, 4096, 8191, 8192, 8193, 70001, (1 << 20) + 3]
    out, src_off, dst_off = [], 0, 0
    for i, n in enumerate(sizes):
        skew_s = int(torch.randint(0, 16, (1,), generator=g)) if i % 2 else 0
        skew_d = int(torch.randint(0, 16, (1,), generator=g)) if i % 3 else skew_s
        out.append((src_off + skew_s, dst_off + skew_d, n))
        src_off += n + 64
        dst_off += n + 64
    return out, src_off, dst_off


@pytest.mark.gpu
def test_no_alloc_entry_point_matches_the_ordinary_kernel(built):
    fn, strerror = load_symbol()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    for round_index in range(2):  # the second call reuses the scratch the first one left behind
        triples, src_total, dst_total = ranges(100 + round_index)
        src = torch.randint(0, 256, (src_total,), dtype=torch.uint8, device="cuda")
        expect = torch.full((dst_total,), 0xCD, dtype=torch.uint8, device="cuda")
        got = torch.full((dst_total,), 0xCD, dtype=torch.uint8, device="cuda")
        flags = torch.zeros(4, dtype=torch.int32, device="cuda")  # [0] ordinary flag, [1] its counter, [2] new flag

        # the existing entry point
        items = [(src.data_ptr() + s, expect.data_ptr() + d, n) for s, d, n in triples]
        _C.launch_push(items, stream, True, flags.data_ptr(), 7 + round_index, flags.data_ptr() + 4)

        # the allocation-free entry point, through its C symbol
        arr = (Item * len(triples))(*[Item(src.data_ptr() + s, got.data_ptr() + d, n) for s, d, n in triples])
        rc = fn(arr, len(triples), flags.data_ptr() + 8, 7 + round_index, stream)
        assert rc == 0, strerror(rc).decode()
        torch.cuda.synchronize()

        assert torch.equal(got, expect), "the two entry points moved different bytes"
        for s, d, n in triples:
            assert torch.equal(got[d:d + n], src[s:s + n])
        assert int(flags[0]) == 7 + round_index and int(flags[2]) == 7 + round_index
        assert int(flags[1]) == 0  # the ordinary kernel leaves its counter cleared

    # requests beyond the fixed scratch are refused, with a message, and nothing is launched
    too_many = (Item * (MAX_ITEMS + 1))()
    rc = fn(too_many, MAX_ITEMS + 1, None, 0, stream)
    assert rc == -1 and b"split" in strerror(rc)
    # an empty request still publishes the flag
    rc = fn(None, 0, flags.data_ptr() + 12, 99, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(flags[3]) == 99
