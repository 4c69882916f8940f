"""The allocation-free entry point against the ordinary one.

Some hosts cannot let a library allocate device memory while attention runs:
their device memory is carved up once by their own arena, or an allocation's
device-wide synchronisation would stall a serving loop.  For them
``tx_sdpa_fp16_static_scratch`` keeps the tensor-core kernel's scratch (status
word, device copy of the key lengths) in an array that is part of the library
image instead of in cudaMalloc'ed memory.  It must give exactly what
``tx_sdpa_forward`` gives -- same kernel, same inputs -- on consecutive calls,
since every call reuses the same array and finds the previous call's contents
there.  This file is collected last so that a failure here cannot hide another
test's result in a stop-at-first-failure run; it passes alone in a fresh
process (first call = address look-up) and after the other tests.
"""
import ctypes

import numpy as np
import pytest

from conftest import seeded
from gpu_util import sdpa_device
from tensorax_b200 import _lib

pytestmark = pytest.mark.gpu


def static_call(q, k, v, causal, lens):
    lib = _lib.load()
    B, Hq, Sq, d = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    bufs = [_lib.to_device(x) for x in (q, k, v)]          # inputs and output stay the caller's business
    out = _lib.DeviceBuffer(B * Hq * Sq * d * 4)
    out.upload(np.full(B * Hq * Sq * d, -3.0, np.float32))
    lens_arr = None if lens is None else np.ascontiguousarray(lens, dtype=np.int32)
    rc = lib.tx_sdpa_fp16_static_scratch(
        bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, out.ptr, B, Hq, Hkv, Sq, Sk, d, int(causal),
        None if lens_arr is None else lens_arr.ctypes.data_as(ctypes.c_void_p), None)
    _lib.check(rc)
    return out.download((B, Hq, Sq, d), np.float32)


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    # two different problems back to back: the second call finds the first call's
    # key lengths and status word in the shared array and must not be affected by them
    cases = [
        (2, 4, 2, 300, 64, True, [300, 123]),
        (3, 2, 2, 257, 128, False, [5, 257, 100]),
        (2, 4, 2, 300, 64, True, None),
        (1, 2, 1, 200, 256, True, [150]),          # wide heads: one query tile per CTA, Q in tensor memory
        (1, 1, 1, 130, 512, False, None),          # two CTAs per query tile, each with half of the value columns
    ]
    for n, (B, Hq, Hkv, S, d, causal, lens) in enumerate(cases):
        q = seeded(700 + n, B, Hq, S, d).astype(np.float16)
        k = seeded(710 + n, B, Hkv, S, d).astype(np.float16)
        v = seeded(720 + n, B, Hkv, S, d).astype(np.float16)
        ref, used_tc = sdpa_device(q, k, v, causal=causal, kv_lens=lens)
        assert used_tc
        for _ in range(2):
            got = static_call(q, k, v, causal, lens)
            # same kernel, same inputs: the tolerance is zero
            assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_static_scratch_entry_point_refuses_what_it_cannot_hold():
    lib = _lib.load()
    one = _lib.DeviceBuffer(1 << 20)
    too_many = np.ones(5000, np.int32)
    rc = lib.tx_sdpa_fp16_static_scratch(one.ptr, one.ptr, one.ptr, one.ptr, 5000, 1, 1, 1, 1, 64, 0,
                                         too_many.ctypes.data_as(ctypes.c_void_p), None)
    assert rc == 1 and b"exceeds" in lib.tx_last_error()
    rc = lib.tx_sdpa_fp16_static_scratch(one.ptr, one.ptr, one.ptr, one.ptr, 1, 1, 1, 8, 8, 48, 0, None, None)
    assert rc == 5 and b"tensor-core shapes" in lib.tx_last_error()
