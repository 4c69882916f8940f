"""GPU parity of the fp32 tensor-core path (fp32 operands carried as hi + lo fp16 pairs, three tcgen05 MMAs per
product, csrc/sdpa_tc_x3.cuh) against the oracle -- the restatement of the reference's sdpa_cpu
(csrc/cpu/tensor_cpu.cpp:464-529) -- and against the exact CUDA-core kernel it stands in front of.
Tolerance against the oracle: max-abs 1e-5, the fp32 figure; against the exact kernel 4e-6."""
import ctypes

import numpy as np
import pytest

import oracle
from conftest import assert_close_fp32, seeded
from gpu_util import sdpa_device
from tensorax_b200 import _lib

pytestmark = pytest.mark.gpu

CASES = [
    # B, Hq, Hkv, Sq, Sk, causal, kv_lens
    (1, 2, 2, 300, 300, True, None),
    (2, 4, 2, 320, 320, True, [320, 133]),
    (1, 1, 1, 128, 128, False, None),
    (1, 1, 1, 129, 129, True, None),
    (1, 2, 1, 200, 700, False, None),
    (2, 2, 2, 256, 256, False, [0, 256]),          # batch 0 sees no key: NaN rows, as the reference
    (1, 1, 1, 100, 900, True, None),
    (2, 100, 100, 257, 257, False, [257, 77]),     # more work items than SMs
]


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_parity_with_oracle_and_exact_kernel(d, case):
    B, Hq, Hkv, Sq, Sk, causal, lens = CASES[case]
    q, k, v = seeded(100 + case, B, Hq, Sq, d), seeded(200 + case, B, Hkv, Sk, d), seeded(300 + case, B, Hkv, Sk, d)
    got, tc = sdpa_device(q, k, v, causal=causal, kv_lens=lens)
    assert tc
    ref = oracle.sdpa_structured(q, k, v, causal=causal, kv_lens=lens, threads=8)
    assert_close_fp32(got, ref)                                     # NaN rows must match too
    exact, tc_exact = sdpa_device(q, k, v, causal=causal, kv_lens=lens, flags=_lib.TX_SDPA_FORCE_SIMT)
    assert not tc_exact
    ok = np.isfinite(exact)
    assert np.array_equal(ok, np.isfinite(got))
    assert float(np.abs(got[ok] - exact[ok]).max(initial=0.0)) <= 4e-6


@pytest.mark.parametrize("d", [64, 128])
def test_long_sequence_stays_fp32_grade(d):
    """8192 keys = 128 key tiles: the per-tile sums are added in fp32 registers, so the error does not grow with
    the sequence (the tensor core's own accumulator truncates).  One flat head and one peaked head."""
    S = 8192
    q, k, v = seeded(1, 1, 2, S, d), seeded(2, 1, 2, S, d), seeded(3, 1, 2, S, d)
    q[0, 1] *= 0.05
    outs, tc = sdpa_device(q, k, v, repeats=2)
    assert tc
    assert np.array_equal(outs[0], outs[1])                         # run-to-run bitwise
    rows = (S - 256, S)
    ref = oracle.sdpa_structured(q, k, v, rows=rows, threads=2)
    err = np.abs(outs[0][:, :, rows[0]:rows[1]] - ref[:, :, rows[0]:rows[1]]).max()
    assert float(err) <= 2e-6, f"max-abs {float(err):.2e}"


def test_full_size_parity_shape_sampled():
    """The fp32 shape of MultiHeadAttention's parity configuration (B4 H16 S4096 d128, causal) at full size: sampled
    heads and row blocks (first, diagonal-crossing middle, last) against the oracle."""
    B, H, S, d = 4, 16, 4096, 128
    q, k, v = seeded(41, B, H, S, d), seeded(42, B, H, S, d), seeded(43, B, H, S, d)
    got, tc = sdpa_device(q, k, v, causal=True)
    assert tc
    worst = 0.0
    for bh in (0, 21, 42, 63):
        for r0 in (0, 1984, S - 128):
            ref = oracle.sdpa_structured(q, k, v, causal=True, heads=[bh], rows=(r0, r0 + 128))
            b, h = divmod(bh, H)
            worst = max(worst, float(np.abs(got[b, h, r0:r0 + 128] - ref[b, h, r0:r0 + 128]).max()))
    assert worst <= 5e-6, f"max-abs {worst:.2e}"


@pytest.mark.parametrize("bad", [1.0e6, -4.0e4, np.inf, np.nan])
def test_value_outside_the_pairs_range_goes_to_the_exact_kernel(bad):
    d = 64
    q, k, v = seeded(11, 1, 2, 300, d), seeded(12, 1, 2, 300, d), seeded(13, 1, 2, 300, d)
    v[0, 1, 17, 3] = bad
    got, tc = sdpa_device(q, k, v, causal=True)
    assert tc                                                       # by shape; the data decides on the device
    exact, _ = sdpa_device(q, k, v, causal=True, flags=_lib.TX_SDPA_FORCE_SIMT)
    assert np.array_equal(got, exact, equal_nan=True)


def test_launches_and_shape_rule():
    lib = _lib.load()
    d = 128
    q, k, v = seeded(21, 1, 2, 256, d), seeded(22, 1, 2, 256, d), seeded(23, 1, 2, 256, d)
    n0 = lib.tx_kernel_launch_count()
    _, tc = sdpa_device(q, k, v)
    assert tc and lib.tx_kernel_launch_count() - n0 == 3            # split pass, tensor-core kernel, stand-in
    m = np.zeros((1, 2, 256, 256), np.float32)
    _, tc_mask = sdpa_device(q, k, v, mask=m)
    assert not tc_mask                                              # dense masks stay on the exact kernel
    q32 = seeded(24, 1, 2, 256, 32)
    _, tc_small = sdpa_device(q32, q32, q32)
    assert not tc_small


def test_five_reference_names_share_the_path():
    from test_sdpa_fp32_gpu import F32_ENTRY_POINTS, call_reference_signature
    q, k, v = seeded(31, 2, 3, 260, 64), seeded(32, 2, 3, 260, 64), seeded(33, 2, 3, 260, 64)
    ref = oracle.sdpa_f32(q, k, v)
    outs = [call_reference_signature(name, q, k, v) for name in F32_ENTRY_POINTS]
    for o in outs:
        assert_close_fp32(o, ref)
        assert np.array_equal(o, outs[0])
