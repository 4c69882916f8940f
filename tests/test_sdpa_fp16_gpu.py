"""GPU parity of the fp16 path (fp16 operands, fp32 accumulation) against the
reference CPU SDPA on the same fp16-rounded inputs.  Tolerance: max-abs 2e-3
and relative 1e-2 (conftest.assert_close_fp16)."""
import ctypes
import hashlib

import numpy as np
import pytest

import oracle
import tensorax_b200 as ts
import tensorax_b200.functional as F
from conftest import assert_close_fp16, seeded
from gpu_util import sample_rows, sdpa_device
from tensorax_b200 import _lib

pytestmark = pytest.mark.gpu

TS, SS = 0, _lib.TX_SDPA_P_IN_SMEM


def widen(x):
    return x.astype(np.float32)


def check_sampled(got, q, k, v, heads, rows, causal=False, kv_lens=None, threads=8):
    """Oracle on selected (flattened b*Hq+h) heads and query rows only."""
    Sq = q.shape[2]
    for r0 in rows:
        r1 = min(r0 + 2, Sq)
        ref = oracle.sdpa_structured(widen(q), widen(k), widen(v), causal=causal, kv_lens=kv_lens,
                                     heads=heads, rows=(r0, r1), threads=threads)
        flat_ref = ref.reshape(-1, Sq, ref.shape[-1])[heads, r0:r1]
        flat_got = got.reshape(-1, Sq, got.shape[-1])[heads, r0:r1]
        assert_close_fp16(flat_got, flat_ref)


@pytest.mark.parametrize("i", range(7))
def test_golden_fp16_shapes(golden, i):
    """Small shapes of the reference's tests/test_sdpa_fp16.py:41-60, outputs from sdpa_cpu."""
    B, H, Sq, Sk, dk, dv = (int(x) for x in golden["f16_shapes"][i])
    q = seeded(400 + i, B, H, Sq, dk).astype(np.float16)
    k = seeded(420 + i, B, H, Sk, dk).astype(np.float16)
    v = seeded(440 + i, B, H, Sk, dv).astype(np.float16)
    h = hashlib.sha256()
    for a in (q, k, v):
        h.update(a.tobytes())
    assert np.array_equal(np.frombuffer(h.digest()[:8], dtype=np.uint64), golden[f"f16_{i}_digest"])
    rows = golden[f"f16_{i}_rows"]
    lib = _lib.load()
    bufs = [_lib.to_device(x) for x in (q, k, v)]
    out = _lib.DeviceBuffer(B * H * Sq * dv * 4)
    _lib.check(lib.tx_sdpa_mma_fp16_cuda(bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, out.ptr, B, H, Sq, Sk, dk, dv))
    got = out.download((B, H, Sq, dv), np.float32)
    assert_close_fp16(got[:, :, rows, :], golden[f"f16_{i}_out"])


def test_golden_grouped_heads_causal_key_lengths(golden):
    for flags in (SS, TS):
        got, tc = sdpa_device(golden["gqa_q"], golden["gqa_k"], golden["gqa_v"], causal=True,
                              kv_lens=golden["gqa_lens"], flags=flags)
        assert tc
        assert_close_fp16(got, golden["gqa_out"])
    got, tc = sdpa_device(golden["gqa_q"], golden["gqa_k"], golden["gqa_v"], causal=True,
                          kv_lens=golden["gqa_lens"], flags=_lib.TX_SDPA_FORCE_SIMT)
    assert not tc
    assert_close_fp16(got, golden["gqa_out"], atol=1e-5)


@pytest.mark.parametrize("flags", [SS, TS])
@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 64), (1, 2, 127, 129, 64), (2, 2, 128, 128, 128),
                                   (1, 3, 300, 555, 128), (2, 1, 513, 64, 64), (1, 1, 80, 80, 64),
                                   (1, 2, 200, 333, 256), (2, 1, 129, 97, 512), (1, 1, 1, 31, 512)])
def test_tensor_core_kernel_edge_shapes(flags, shape):
    B, H, Sq, Sk, d = shape
    q, k, v = (seeded(30 + j, B, H, S, d).astype(np.float16) for j, S in enumerate((Sq, Sk, Sk)))
    got, tc = sdpa_device(q, k, v, flags=flags)
    assert tc
    assert_close_fp16(got, oracle.sdpa_f32(widen(q), widen(k), widen(v)))


@pytest.mark.parametrize("d", [64, 128, 256, 512])
def test_tensor_core_kernel_masks(d):
    B, Hq, Hkv, S = 3, 6, 2, 450
    q = seeded(40, B, Hq, S, d).astype(np.float16)
    k = (0.5 * seeded(41, B, Hkv, S, d)).astype(np.float16)
    v = (0.5 * seeded(42, B, Hkv, S, d)).astype(np.float16)
    for causal, lens in ((True, None), (False, [450, 1, 200]), (True, [129, 450, 128])):
        got, tc = sdpa_device(q, k, v, causal=causal, kv_lens=lens)
        assert tc
        assert_close_fp16(got, oracle.sdpa_structured(widen(q), widen(k), widen(v), causal=causal, kv_lens=lens))
    empty, _ = sdpa_device(q, k, v, kv_lens=[0, 10, 450])      # batch 0 sees no key: NaN rows like the reference
    assert np.isnan(empty[0]).all() and np.isfinite(empty[1:]).all()


def test_fp16_with_dense_mask_runs_on_cuda_cores():
    B, H, S, d = 1, 2, 100, 64
    q, k, v = (seeded(50 + j, B, H, S, d).astype(np.float16) for j in range(3))
    m = seeded(53, B, H, S, S)
    m[m > 0.8] = -np.inf
    m[:, :, :, 0] = 0.0
    got, tc = sdpa_device(q, k, v, mask=m)
    assert not tc
    assert_close_fp16(got, oracle.sdpa_f32(widen(q), widen(k), widen(v), m), atol=1e-5)


LARGE = [  # (B, Hq, Hkv, S, d, causal, with_lens, scale_kv)   -- BASELINE configs 2-5 and the reference's long shapes
    (4, 8, 8, 8192, 64, False, False, 1.0),     # config 2 (tests/test_sdpa_fp16.py:56)
    (1, 8, 8, 8192, 64, False, False, 1.0),
    (4, 8, 8, 2048, 128, False, False, 1.0),
    (4, 8, 8, 4096, 128, False, False, 1.0),
    (4, 16, 16, 4096, 128, True, True, 1.0),    # config 3
    (8, 32, 8, 8192, 128, True, False, 0.5),    # config 4
]


@pytest.mark.parametrize("cfg", LARGE, ids=lambda c: "B%d_Hq%d_Hkv%d_S%d_d%d_c%d_l%d" % c[:7])
def test_full_size_configs_sampled_against_oracle(cfg):
    B, Hq, Hkv, S, d, causal, with_lens, kv_scale = cfg
    rng = np.random.Generator(np.random.PCG64(7))
    q = rng.standard_normal((B, Hq, S, d), dtype=np.float32).astype(np.float16)
    k = (kv_scale * rng.standard_normal((B, Hkv, S, d), dtype=np.float32)).astype(np.float16)
    v = (kv_scale * rng.standard_normal((B, Hkv, S, d), dtype=np.float32)).astype(np.float16)
    lens = rng.integers(S // 2, S, size=B, endpoint=True).astype(np.int32) if with_lens else None
    got, tc = sdpa_device(q, k, v, causal=causal, kv_lens=lens)
    assert tc
    assert np.isfinite(got).all()
    heads = sorted({0, B * Hq - 1, (B * Hq) // 2 + 1})
    extra = [127, 128, S // 2 - 1, S // 2] + ([int(lens[0]) - 1, int(lens[0])] if with_lens else [])
    check_sampled(got, q, k, v, heads, sample_rows(S, 5, extra), causal=causal, kv_lens=lens)
    # size-independent properties on the whole tensor: rows are convex combinations of V rows ...
    group = Hq // Hkv
    vmax = np.repeat(widen(v).max(axis=2), group, axis=1)[:, :, None, :]
    vmin = np.repeat(widen(v).min(axis=2), group, axis=1)[:, :, None, :]
    assert (got <= vmax + 2e-3).all() and (got >= vmin - 2e-3).all()
    # ... and under a causal mask row 0 of every head is exactly V row 0
    if causal:
        v0 = np.repeat(widen(v)[:, :, 0, :], group, axis=1)
        assert np.abs(got[:, :, 0, :] - v0).max() <= 2e-3


@pytest.mark.parametrize("cfg", [(4, 8, 256, 512), (2, 4, 1024, 256)])
def test_remaining_reference_accuracy_configs_in_full(cfg):
    """The two ACCURACY_CONFIGS of tests/test_sdpa_fp16.py:41-60 that neither the golden file (its first seven)
    nor the sampled full-size runs cover: every output element against the oracle."""
    B, H, S, d = cfg
    rng = np.random.Generator(np.random.PCG64(11))
    q, k, v = (rng.standard_normal((B, H, S, d), dtype=np.float32).astype(np.float16) for _ in range(3))
    got, tc = sdpa_device(q, k, v)
    assert tc
    assert_close_fp16(got, oracle.sdpa_structured(widen(q), widen(k), widen(v), threads=8))


@pytest.mark.parametrize("d", [256, 512])
def test_config5_large_head_dims(d):
    B, H, S = 4, 8, 4096
    rng = np.random.Generator(np.random.PCG64(8))
    q, k, v = ((rng.standard_normal((B, H, S, d), dtype=np.float32) / np.sqrt(d)).astype(np.float16) for _ in range(3))
    got, tc = sdpa_device(q, k, v)
    assert tc
    assert np.isfinite(got).all()
    check_sampled(got, q, k, v, [0, 17, B * H - 1], sample_rows(S, 4))
    simt, tc = sdpa_device(q[:1, :2], k[:1, :2], v[:1, :2], flags=_lib.TX_SDPA_FORCE_SIMT)
    assert not tc
    assert np.abs(simt - got[:1, :2]).max() <= 2e-3


def test_linearity_in_v_at_config2_size():
    """sdpa(Q,K,a*V1+b*V2) == a*sdpa(Q,K,V1) + b*sdpa(Q,K,V2): holds for the exact
    operator at any size, so it checks the full-size run without an oracle."""
    B, H, S, d = 2, 8, 8192, 64
    rng = np.random.Generator(np.random.PCG64(9))
    q, k, v1, v2 = (rng.standard_normal((B, H, S, d), dtype=np.float32).astype(np.float16) for _ in range(4))
    vsum = (0.5 * widen(v1) - 0.25 * widen(v2)).astype(np.float16)
    o1, _ = sdpa_device(q, k, v1)
    o2, _ = sdpa_device(q, k, v2)
    os_, _ = sdpa_device(q, k, vsum)
    assert np.abs(os_ - (0.5 * o1 - 0.25 * o2)).max() <= 2e-3


DETERMINISM = [(4, 8, 2048, 128), (4, 8, 4096, 128), (4, 8, 8192, 64), (1, 8, 8192, 64),
               (4, 8, 4096, 256)]   # tests/test_sdpa_fp16.py:111-117


@pytest.mark.parametrize("cfg", DETERMINISM)
def test_bitwise_determinism_over_four_runs(cfg):
    B, H, S, d = cfg
    rng = np.random.Generator(np.random.PCG64(10))
    q, k, v = (rng.standard_normal((B, H, S, d), dtype=np.float32).astype(np.float16) for _ in range(3))
    outs, tc = sdpa_device(q, k, v, repeats=4)
    assert tc
    for o in outs[1:]:
        assert np.array_equal(o.view(np.uint32), outs[0].view(np.uint32))


def test_python_fp16_pipeline_like_the_reference_test():
    """tests/test_sdpa_fp16.py:70-81: fp32 numpy -> Tensor(cuda) -> cast_to_fp16 -> mma_fp16."""
    B, H, S, d = 2, 4, 256, 64
    q, k, v = (seeded(60 + j, B, H, S, d) for j in range(3))
    qh, kh, vh = (F.cast_to_fp16(ts.Tensor(x, dtype="float32", device="cuda")) for x in (q, k, v))
    out = F.scaled_dot_product_attention_mma_fp16(qh, kh, vh)
    assert out.dtype == "float32" and out.device == "cuda" and out.shape == (B, H, S, d)
    ref = oracle.sdpa_f32(*(widen(x.astype(np.float16)) for x in (q, k, v)))
    assert_close_fp16(out.numpy(), ref)
    # generic entry points take fp16 too and give float32 (the reference reinterprets the bytes)
    assert_close_fp16(F.scaled_dot_product_attention(qh, kh, vh).numpy(), ref)
    # structured masks + grouped heads through the additive entry point
    kg, vg = (F.cast_to_fp16(ts.Tensor(x[:, :2], device="cuda")) for x in (k, v))
    got = F.scaled_dot_product_attention_ex(qh, kg, vg, causal=True, kv_lens=[200, 256]).numpy()
    ref = oracle.sdpa_structured(widen(q.astype(np.float16)), widen(k[:, :2].astype(np.float16)),
                                 widen(v[:, :2].astype(np.float16)), causal=True, kv_lens=[200, 256])
    assert_close_fp16(got, ref)


def test_host_buffer_entry_point():
    B, Hq, Hkv, S, d = 2, 4, 2, 700, 128
    q = seeded(70, B, Hq, S, d).astype(np.float16)
    k, v = (seeded(71 + j, B, Hkv, S, d).astype(np.float16) for j in range(2))
    lens = np.asarray([700, 333], np.int32)
    out = np.empty((B, Hq, S, d), np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    desc = _lib.SdpaDesc(q=p(q), k=p(k), v=p(v), mask=None, kv_lens=p(lens), out=p(out), batch=B,
                         q_heads=Hq, kv_heads=Hkv, seq_q=S, seq_k=S, d_k=d, d_v=d,
                         dtype=_lib.TX_DTYPE_F16, causal=1, flags=0, stream=None)
    for _ in range(2):   # second call reuses the cached staging buffer
        out[:] = 0
        _lib.check(_lib.load().tx_sdpa_forward_host(ctypes.byref(desc)))
        dev, _ = sdpa_device(q, k, v, causal=True, kv_lens=lens)
        assert np.array_equal(out.view(np.uint32), dev.view(np.uint32))
    # fp16 result through the host form: half the bytes come back
    out16 = np.empty((B, Hq, S, d), np.float16)
    desc.out, desc.flags = p(out16), _lib.TX_SDPA_OUT_F16
    _lib.check(_lib.load().tx_sdpa_forward_host(ctypes.byref(desc)))
    assert np.array_equal(out16, dev.astype(np.float16))
    lse = np.empty((B, Hq, S), np.float32)
    desc.lse = p(lse)
    assert _lib.load().tx_sdpa_forward_host(ctypes.byref(desc)) == 5          # TX_ERR_UNSUPPORTED, nothing ran


def test_host_buffer_entry_point_with_pinned_buffers():
    """Pinned buffers: the call is cut into chunks (the problem is above the 8 MiB it takes) and every chunk's result is
    written into the caller's buffer by a kernel.  Same bits as the device-resident call."""
    lib = _lib.load()
    B, Hq, Hkv, S, d = 3, 4, 2, 2048, 64
    q = seeded(75, B, Hq, S, d).astype(np.float16)
    k, v = (seeded(76 + j, B, Hkv, S, d).astype(np.float16) for j in range(2))
    n_out = B * Hq * S * d
    sizes = [q.nbytes, k.nbytes, v.nbytes, n_out * 4]
    ptrs = [lib.tx_host_alloc_pinned(n) for n in sizes]
    assert all(ptrs)
    try:
        for ptr, a in zip(ptrs[:3], (q, k, v)):
            ctypes.memmove(ptr, a.ctypes.data, a.nbytes)
        ctypes.memset(ptrs[3], 0xFF, sizes[3])
        desc = _lib.SdpaDesc(q=ptrs[0], k=ptrs[1], v=ptrs[2], mask=None, kv_lens=None, out=ptrs[3], batch=B, q_heads=Hq,
                             kv_heads=Hkv, seq_q=S, seq_k=S, d_k=d, d_v=d, dtype=_lib.TX_DTYPE_F16, causal=1, flags=0,
                             stream=None)
        n0 = lib.tx_kernel_launch_count()
        _lib.check(lib.tx_sdpa_forward_host(ctypes.byref(desc)))
        launches = lib.tx_kernel_launch_count() - n0
        out = np.ctypeslib.as_array((ctypes.c_float * n_out).from_address(ptrs[3])).reshape(B, Hq, S, d).copy()
    finally:
        for ptr in ptrs:
            lib.tx_host_free_pinned(ptr)
    dev, _ = sdpa_device(q, k, v, causal=True)
    assert np.array_equal(out.view(np.uint32), dev.view(np.uint32))
    assert launches >= 4 and launches % 2 == 0          # per chunk: one attention launch and one write-back launch


def test_sharded_runs_equal_the_single_device_run_bitwise():
    """Each rank's slab through the same kernel, reassembled: identical bits."""
    from tensorax_b200 import sharding
    B, Hq, Hkv, S, d = 4, 8, 2, 512, 128
    q = seeded(80, B, Hq, S, d).astype(np.float16)
    k, v = (seeded(81 + j, B, Hkv, S, d).astype(np.float16) for j in range(2))
    lens = [512, 100, 300, 511]
    full, _ = sdpa_device(q, k, v, causal=True, kv_lens=lens)
    for world in (2, 8):
        out = np.zeros_like(full)
        for r in range(world):
            sh = sharding.partition(B, Hkv, Hq, world, r)
            qs, ks, vs, ls = sharding.shard_arrays(sh, q, k, v, lens)
            loc, _ = sdpa_device(qs, ks, vs, causal=True, kv_lens=ls)
            sharding.place_output(sh, out, loc)
        assert np.array_equal(out.view(np.uint32), full.view(np.uint32))


def test_section_profile_entry_point():
    """Section profile of the tensor-core kernels (the fp16 counterpart of the reference's profile_sections_sdpa_*,
    csrc/tensor_ops.cpp:1434-1507): 64 counters, sane values for both query tiles and the MMA lane."""
    from tensorax_b200 import _C
    B, H, S, d = 1, 2, 1024, 64
    q, k, v = (_C.from_numpy(seeded(90 + j, B, H, S, d).astype(np.float16), "cuda") for j in range(3))
    t = _C.profile_sections_sdpa(q, k, v)
    assert len(t) == 64 and t[10] == S // 128 and t[42] == S // 128     # key tiles walked by either query tile of CTA (0,0,0)
    assert t[0] > 0 and t[32] > 0 and t[16] > 0                          # both softmax lanes and the MMA lane reported
    assert t[5] > t[7] > 0 and t[37] > t[39] > 0                         # exponentials cost more than the P hand-over
    assert sum(t[1:9]) <= t[0] * 1.05 and sum(t[33:41]) <= t[32] * 1.05


@pytest.mark.parametrize("d", [256, 512])
def test_section_profile_wide_heads(d):
    """One query tile per CTA at d = 256 / 512: softmax, MMA and producer lanes report."""
    from tensorax_b200 import _C
    B, H, S = 1, 1, 512
    q, k, v = (_C.from_numpy(seeded(95 + j, B, H, S, d).astype(np.float16), "cuda") for j in range(3))
    t = _C.profile_sections_sdpa(q, k, v)
    assert len(t) == 64 and t[10] == S // 64
    assert t[0] > 0 and t[16] > 0 and t[24] > 0


@pytest.mark.parametrize("name", ["naive", "tiled", "flash", "mma", "flash_optimized"])
def test_fp32_section_profiles_by_reference_name(name):
    """profile_sections_sdpa_{naive,tiled,flash,mma,flash_optimized} (csrc/tensor_ops.cpp:1434-1507,1622-1636):
    32 clock64 stamps, non-decreasing over the eight sections the exact-fp32 kernel reports, the rest zero."""
    from tensorax_b200 import _C
    q, k, v = (_C.from_numpy(seeded(97 + j, 1, 2, 256, 64), "cuda") for j in range(3))
    t = getattr(_C, f"profile_sections_sdpa_{name}")(q, k, v)
    assert len(t) == 32 and all(x > 0 for x in t[:8]) and all(b >= a for a, b in zip(t[:8], t[1:8]))
    assert all(x == 0 for x in t[8:])


def test_non_blocking_python_calls_are_stream_ordered():
    """sync=False returns after the launch; a burst of such calls followed by one synchronize() gives
    the same bits as blocking calls (each call's temporaries go back to the pool in stream order)."""
    q, k, v = (seeded(i, 2, 4, 640, 64).astype(np.float16) for i in (110, 111, 112))
    tq, tk, tv = (ts.Tensor(x, dtype="float16", device="cuda") for x in (q, k, v))
    blocking = F.scaled_dot_product_attention_ex(tq, tk, tv, causal=True, kv_lens=[640, 333]).numpy()
    outs = [F.scaled_dot_product_attention_ex(tq, tk, tv, causal=True, kv_lens=[640, 333], sync=False) for _ in range(8)]
    ts.synchronize()
    for o in outs:
        assert np.array_equal(o.numpy().view(np.uint32), blocking.view(np.uint32))


def test_fp32_tensors_on_the_tensor_cores_by_request():
    """TX_SDPA_F32_VIA_F16 / fp16_compute=True: fp32 inputs, operands rounded to fp16 on the device, tensor-core
    kernel, fp32 result -- equal to running the fp16-rounded inputs through the fp16 path, bit for bit; without
    the flag the same call keeps exact fp32 arithmetic."""
    from conftest import assert_close_fp32
    q, k, v = (seeded(i, 2, 4, 384, 128) for i in (130, 131, 132))
    via, tc_flagged = sdpa_device(q, k, v, causal=True, flags=_lib.TX_SDPA_F32_VIA_F16)
    direct, tc = sdpa_device(q.astype(np.float16), k.astype(np.float16), v.astype(np.float16), causal=True)
    assert tc and tc_flagged and np.array_equal(via.view(np.uint32), direct.view(np.uint32))
    exact, _ = sdpa_device(q, k, v, causal=True)
    assert_close_fp32(exact, oracle.sdpa_structured(q, k, v, causal=True))
    tq, tk, tv = (ts.Tensor(x, device="cuda") for x in (q, k, v))
    out = F.scaled_dot_product_attention_ex(tq, tk, tv, causal=True, fp16_compute=True)
    assert out.dtype == "float32" and np.array_equal(out.numpy().view(np.uint32), direct.view(np.uint32))
    # shapes the tensor-core kernel does not take keep exact fp32 arithmetic even with the flag
    q2, k2, v2 = (seeded(i, 1, 2, 50, 40) for i in (133, 134, 135))
    got, _ = sdpa_device(q2, k2, v2, flags=_lib.TX_SDPA_F32_VIA_F16)
    assert_close_fp32(got, oracle.sdpa_f32(q2, k2, v2))
