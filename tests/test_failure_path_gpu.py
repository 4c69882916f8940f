"""The give-up path of the tensor-core kernel on a real GPU, without faulting, trapping or hanging anything:
a self-test instantiation of the production d = 64 kernel whose waits give up after 2 ms and whose TMA producer
leaves one K tile out (tx_selftest_wait_timeout).  The kernel must return by itself, report through the status
word, mark its rows, free its tensor memory, and leave the context fit for the next launch.  Plus canary rows
around every output buffer of the edge-shape calls: the kernels write what they own and nothing else."""
import ctypes

import numpy as np
import pytest

import oracle
from conftest import FP16_ATOL, seeded
from tensorax_b200 import _lib

pytestmark = pytest.mark.gpu


def _desc(bq, bk, bv, bo, B, Hq, Hkv, Sq, Sk, d, causal=0, lens=None, lse=None, flags=0, out_off=0, lse_off=0):
    return _lib.SdpaDesc(q=bq.ptr, k=bk.ptr, v=bv.ptr, mask=None, kv_lens=lens.ptr if lens else None, out=bo.ptr + out_off,
                         batch=B, q_heads=Hq, kv_heads=Hkv, seq_q=Sq, seq_k=Sk, d_k=d, d_v=d, dtype=_lib.TX_DTYPE_F16,
                         causal=causal, flags=flags, stream=None, lse=(lse.ptr + lse_off) if lse else None)


def test_wait_runs_out_and_the_context_survives():
    lib = _lib.load()
    B, H, S, d = 1, 1, 256, 64                      # one CTA, two query tiles, two key tiles
    q, k, v = (seeded(70 + i, B, H, S, d).astype(np.float16) for i in range(3))
    bq, bk, bv = (_lib.to_device(x) for x in (q, k, v))
    bo = _lib.DeviceBuffer(B * H * S * d * 4)
    desc = _desc(bq, bk, bv, bo, B, H, H, S, S, d)
    # reference bits from the production kernel
    _lib.check(lib.tx_sdpa_forward(ctypes.byref(desc)))
    _lib.check(lib.tx_sdpa_finish(None))
    good = bo.download((B, H, S, d), np.float32)
    ref = oracle.sdpa_structured(q, k, v)
    assert float(np.abs(good - ref).max()) <= FP16_ATOL
    # the self-test instantiation with nothing left out is an ordinary forward pass
    assert lib.tx_selftest_wait_timeout(ctypes.byref(desc), -1) == _lib.TX_OK, lib.tx_last_error()
    assert np.array_equal(bo.download((B, H, S, d), np.float32).view(np.uint32), good.view(np.uint32))
    # K tile 1 never arrives: the MMA warp's wait runs out after 2 ms
    rc = lib.tx_selftest_wait_timeout(ctypes.byref(desc), 1)
    msg = lib.tx_last_error().decode()
    assert rc == 4, (rc, msg)                        # TX_ERR_KERNEL
    assert "stage code 3" in msg, msg                # TC_ERR_MMA: the MMA warp is the one that waited for the tile
    marked = bo.download((B, H, S, d), np.float32)
    assert np.isnan(marked).all(), "rows of a CTA that gave up must read NaN"
    # the status word was cleared by the failed call; the next launches are clean and bit-identical
    for _ in range(2):
        _lib.check(lib.tx_sdpa_forward(ctypes.byref(desc)))
        _lib.check(lib.tx_sdpa_finish(None))
        again = bo.download((B, H, S, d), np.float32)
        assert np.array_equal(again.view(np.uint32), good.view(np.uint32))


def test_a_failed_launch_stops_later_ctas_and_marks_their_rows():
    """Several CTAs: the first to give up sets the device status word, CTAs that start afterwards return at once;
    every row of the launch reads NaN or a finished result, never stale memory."""
    lib = _lib.load()
    B, H, S, d = 1, 2, 512, 64
    q, k, v = (seeded(80 + i, B, H, S, d).astype(np.float16) for i in range(3))
    bq, bk, bv = (_lib.to_device(x) for x in (q, k, v))
    bo = _lib.to_device(np.full((B, H, S, d), 7.0, np.float32))
    desc = _desc(bq, bk, bv, bo, B, H, H, S, S, d)
    assert lib.tx_selftest_wait_timeout(ctypes.byref(desc), 2) == 4
    out = bo.download((B, H, S, d), np.float32)
    assert np.isnan(out).all()
    _lib.check(lib.tx_sdpa_forward(ctypes.byref(desc)))
    _lib.check(lib.tx_sdpa_finish(None))
    ref = oracle.sdpa_structured(q, k, v)
    assert float(np.abs(bo.download((B, H, S, d), np.float32) - ref).max()) <= FP16_ATOL


CANARY = np.float32(-12345.5)


@pytest.mark.parametrize("shape", [
    (1, 2, 2, 129, 129, 64, True),       # one row past a tile
    (2, 4, 2, 300, 300, 64, True),       # grouped heads, ragged tail
    (1, 1, 1, 100, 900, 128, False),     # Sq != Sk, second query tile of the pair does not exist
    (1, 2, 2, 257, 257, 128, True),
    (1, 1, 1, 130, 200, 256, False),
    (1, 1, 1, 70, 130, 512, False),
])
def test_canary_rows_around_out_and_lse(shape):
    """`out` and `lse` sit between guard rows filled with a sentinel; after the call the guards are untouched and
    everything between them was written."""
    lib = _lib.load()
    B, Hq, Hkv, Sq, Sk, d, causal = shape
    q = seeded(60, B, Hq, Sq, d).astype(np.float16)
    k = seeded(61, B, Hkv, Sk, d).astype(np.float16)
    v = seeded(62, B, Hkv, Sk, d).astype(np.float16)
    bq, bk, bv = (_lib.to_device(x) for x in (q, k, v))
    n_out, n_lse, guard = B * Hq * Sq * d, B * Hq * Sq, 1024            # guard: 1024 floats = 4 KiB either side
    host_out = np.full(n_out + 2 * guard, CANARY, np.float32)
    host_lse = np.full(n_lse + 2 * guard, CANARY, np.float32)
    bo, bl = _lib.to_device(host_out), _lib.to_device(host_lse)
    desc = _desc(bq, bk, bv, bo, B, Hq, Hkv, Sq, Sk, d, causal=int(causal), lse=bl, out_off=guard * 4, lse_off=guard * 4)
    assert lib.tx_sdpa_uses_tensor_cores(ctypes.byref(desc)) == 1
    _lib.check(lib.tx_sdpa_forward(ctypes.byref(desc)))
    _lib.check(lib.tx_sdpa_finish(None))
    got_out = bo.download((n_out + 2 * guard,), np.float32)
    got_lse = bl.download((n_lse + 2 * guard,), np.float32)
    for arr, n in ((got_out, n_out), (got_lse, n_lse)):
        assert (arr[:guard] == CANARY).all() and (arr[guard + n:] == CANARY).all(), "a guard row was written"
        assert not (arr[guard:guard + n] == CANARY).any(), "part of the buffer was left unwritten"
    ref = oracle.sdpa_structured(q, k, v, causal=causal)
    assert float(np.abs(got_out[guard:guard + n_out].reshape(B, Hq, Sq, d) - ref).max()) <= FP16_ATOL


def test_canary_rows_around_backward_outputs():
    lib = _lib.load()
    B, Hq, Hkv, S, d = 1, 4, 2, 200, 64
    q = seeded(50, B, Hq, S, d).astype(np.float16)
    k = seeded(51, B, Hkv, S, d).astype(np.float16)
    v = seeded(52, B, Hkv, S, d).astype(np.float16)
    g = seeded(53, B, Hq, S, d)
    bq, bk, bv, bg = (_lib.to_device(x) for x in (q, k, v, g))
    bo, bl = _lib.DeviceBuffer(q.size * 4), _lib.DeviceBuffer(B * Hq * S * 4)
    fwd = _desc(bq, bk, bv, bo, B, Hq, Hkv, S, S, d, causal=1, lse=bl)
    _lib.check(lib.tx_sdpa_forward(ctypes.byref(fwd)))
    _lib.check(lib.tx_sdpa_finish(None))
    guard = 1024
    bufs = [_lib.to_device(np.full(n + 2 * guard, CANARY, np.float32)) for n in (q.size, k.size, v.size)]
    bwd = _lib.SdpaBwdDesc(q=bq.ptr, k=bk.ptr, v=bv.ptr, out=bo.ptr, dout=bg.ptr, lse=bl.ptr, kv_lens=None,
                           dq=bufs[0].ptr + guard * 4, dk=bufs[1].ptr + guard * 4, dv=bufs[2].ptr + guard * 4,
                           batch=B, q_heads=Hq, kv_heads=Hkv, seq_q=S, seq_k=S, d=d, causal=1, flags=0, stream=None)
    _lib.check(lib.tx_sdpa_backward(ctypes.byref(bwd)))
    _lib.check(lib.tx_sdpa_finish(None))
    for buf, n in zip(bufs, (q.size, k.size, v.size)):
        arr = buf.download((n + 2 * guard,), np.float32)
        assert (arr[:guard] == CANARY).all() and (arr[guard + n:] == CANARY).all(), "a guard row was written"
        assert not (arr[guard:guard + n] == CANARY).any()
