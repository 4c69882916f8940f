"""GPU parity of the fp16 output option, the saved row statistics and the SDPA backward kernels
against the CPU oracle (oracle.sdpa_backward: the reference's autograd rule, tensorax/tensor.py:806-827,
in float64 on the same fp16-rounded inputs).

Tolerances.  Forward fp16 output: the fp32-output result rounded to fp16, within one fp16 ulp.
Backward (fp16 operands, P and dS rounded to fp16 before their MMAs, fp32 accumulation):
||got - ref|| / ||ref|| <= 1e-2 per gradient and max-abs error <= 2e-2 * max|ref|; a gradient whose
max-abs error is inside the forward's absolute fp16 bound (2e-3) passes as well, which is what a
gradient that is exactly zero in exact arithmetic (one visible key per row) is measured by."""
import ctypes

import numpy as np
import pytest

import oracle
import tensorax_b200 as ts
import tensorax_b200.functional as F
from conftest import assert_close_fp16, seeded
from gpu_util import sdpa_device
from tensorax_b200 import _lib

pytestmark = pytest.mark.gpu


def widen(x):
    return x.astype(np.float32)


def backward_device(q, k, v, dout, causal=False, kv_lens=None, out_f16=False, repeats=1):
    """Forward (with lse) + tx_sdpa_backward through the C ABI.  Returns (out, lse, dq, dk, dv)."""
    lib = _lib.load()
    B, Hq, Sq, d = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    flags = _lib.TX_SDPA_OUT_F16 if out_f16 else 0
    dq_, dk_, dv_ = (_lib.to_device(np.ascontiguousarray(x, dtype=np.float16)) for x in (q, k, v))
    out = _lib.DeviceBuffer(B * Hq * Sq * d * (2 if out_f16 else 4))
    lse = _lib.DeviceBuffer(B * Hq * Sq * 4)
    dl = _lib.to_device(np.ascontiguousarray(kv_lens, dtype=np.int32)) if kv_lens is not None else None
    fwd = _lib.SdpaDesc(q=dq_.ptr, k=dk_.ptr, v=dv_.ptr, mask=None, kv_lens=dl.ptr if dl else None, out=out.ptr,
                        batch=B, q_heads=Hq, kv_heads=Hkv, seq_q=Sq, seq_k=Sk, d_k=d, d_v=d, dtype=_lib.TX_DTYPE_F16,
                        causal=int(causal), flags=flags, stream=None, lse=lse.ptr)
    _lib.check(lib.tx_sdpa_forward(ctypes.byref(fwd)))
    _lib.check(lib.tx_sdpa_finish(None))
    g = _lib.to_device(np.ascontiguousarray(dout, dtype=np.float32))
    gq = _lib.DeviceBuffer(B * Hq * Sq * d * 4)
    gk = _lib.DeviceBuffer(B * Hkv * Sk * d * 4)
    gv = _lib.DeviceBuffer(B * Hkv * Sk * d * 4)
    bwd = _lib.SdpaBwdDesc(q=dq_.ptr, k=dk_.ptr, v=dv_.ptr, out=out.ptr, dout=g.ptr, lse=lse.ptr,
                           kv_lens=dl.ptr if dl else None, dq=gq.ptr, dk=gk.ptr, dv=gv.ptr, batch=B, q_heads=Hq,
                           kv_heads=Hkv, seq_q=Sq, seq_k=Sk, d=d, causal=int(causal), flags=flags, stream=None)
    res = []
    for _ in range(repeats):
        _lib.check(lib.tx_sdpa_backward(ctypes.byref(bwd)))
        _lib.check(lib.tx_sdpa_finish(None))
        res.append((gq.download((B, Hq, Sq, d), np.float32), gk.download((B, Hkv, Sk, d), np.float32),
                    gv.download((B, Hkv, Sk, d), np.float32)))
    o = out.download((B, Hq, Sq, d), np.float16 if out_f16 else np.float32)
    l = lse.download((B, Hq, Sq), np.float32)
    return (o, l) + res[0] if repeats == 1 else (o, l, res)


def assert_grad_close(got, ref, name):
    ref = np.asarray(ref, dtype=np.float64)
    assert np.isfinite(got).all(), name
    rel = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
    mx = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    if np.abs(got - ref).max() <= 2e-3:
        return
    assert rel <= 1e-2 and mx <= 2e-2, f"{name}: rel {rel:.3e}, max-abs/max|ref| {mx:.3e}"


# ------------------------------------------------------------------ fp16 output
@pytest.mark.parametrize("d", [64, 128, 256, 512, 32])
def test_fp16_output_is_the_fp32_result_rounded(d):
    B, Hq, Hkv, S = 2, 4, 2, 300
    q = seeded(70, B, Hq, S, d).astype(np.float16)
    k = seeded(71, B, Hkv, S, d).astype(np.float16)
    v = seeded(72, B, Hkv, S, d).astype(np.float16)
    o32, tc = sdpa_device(q, k, v, causal=True, kv_lens=[300, 177])
    o16, tc16 = sdpa_device(q, k, v, causal=True, kv_lens=[300, 177], flags=_lib.TX_SDPA_OUT_F16)
    assert tc == tc16 == (d != 32) and o16.dtype == np.float16
    assert np.array_equal(o16, o32.astype(np.float16))       # same arithmetic, one rounding at the store
    assert_close_fp16(o16.astype(np.float32), oracle.sdpa_structured(widen(q), widen(k), widen(v), causal=True,
                                                                    kv_lens=[300, 177]))


def test_python_api_fp16_output():
    q, k, v = (seeded(i, 1, 2, 256, 64).astype(np.float16) for i in (73, 74, 75))
    tq, tk, tv = (ts.Tensor(x, dtype="float16", device="cuda") for x in (q, k, v))
    out = F.scaled_dot_product_attention_ex(tq, tk, tv, causal=True, out_dtype="float16")
    assert out.dtype == "float16" and out.shape == (1, 2, 256, 64)
    ref = oracle.sdpa_structured(widen(q), widen(k), widen(v), causal=True)
    assert_close_fp16(out.numpy().astype(np.float32), ref)


# ------------------------------------------------------------------ row statistics
@pytest.mark.parametrize("d", [64, 128, 256, 512])
def test_saved_row_statistic_matches_oracle(d):
    B, Hq, Hkv, Sq, Sk = 2, 4, 2, 200, 333
    q = seeded(76, B, Hq, Sq, d).astype(np.float16)
    k = (0.5 * seeded(77, B, Hkv, Sk, d)).astype(np.float16)
    v = seeded(78, B, Hkv, Sk, d).astype(np.float16)
    for causal, lens in ((False, None), (True, [333, 150])):
        _, lse, tc = sdpa_device(q, k, v, causal=causal, kv_lens=lens, want_lse=True)
        assert tc
        ref = oracle.sdpa_backward(widen(q), widen(k), widen(v), np.zeros((B, Hq, Sq, d)), causal=causal, kv_lens=lens)[3]
        np.testing.assert_allclose(lse, ref, atol=2e-3)       # log2 units; exp2 of the error is 0.14 %


def test_lse_is_refused_where_no_kernel_writes_it():
    q = seeded(79, 1, 1, 16, 32).astype(np.float16)
    with pytest.raises(_lib.BackendError, match="log-sum-exp"):
        sdpa_device(q, q, q, want_lse=True)


# ------------------------------------------------------------------ backward
CASES = [
    # B, Hq, Hkv, Sq, Sk, d, causal, lens
    (1, 1, 1, 128, 128, 64, False, None),
    (2, 2, 2, 256, 256, 64, True, None),
    (2, 4, 2, 300, 555, 64, False, [555, 301]),
    (1, 4, 1, 450, 450, 64, True, [129]),
    (1, 2, 2, 1, 1, 64, False, None),
    (1, 2, 1, 77, 130, 128, False, None),
    (2, 2, 2, 384, 384, 128, True, [384, 200]),
    (1, 8, 2, 513, 640, 128, False, [600]),
    (1, 2, 2, 700, 64, 64, True, None),
    (1, 2, 1, 200, 333, 256, False, None),
    (2, 4, 2, 300, 300, 256, True, [300, 129]),
    (1, 1, 1, 1, 1, 256, False, None),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "B%d_Hq%d_Hkv%d_Sq%d_Sk%d_d%d_c%d" % (c[:6] + (int(c[6]),)))
def test_backward_matches_oracle(case):
    B, Hq, Hkv, Sq, Sk, d, causal, lens = case
    q = seeded(80, B, Hq, Sq, d).astype(np.float16)
    k = seeded(81, B, Hkv, Sk, d).astype(np.float16)
    v = seeded(82, B, Hkv, Sk, d).astype(np.float16)
    g = seeded(83, B, Hq, Sq, d).astype(np.float32)
    out, lse, dq, dk, dv = backward_device(q, k, v, g, causal=causal, kv_lens=lens)
    rq, rk, rv, _ = oracle.sdpa_backward(widen(q), widen(k), widen(v), g, causal=causal, kv_lens=lens)
    assert_close_fp16(out, oracle.sdpa_structured(widen(q), widen(k), widen(v), causal=causal, kv_lens=lens))
    assert_grad_close(dq, rq, "dq")
    assert_grad_close(dk, rk, "dk")
    assert_grad_close(dv, rv, "dv")
    if lens is not None:                                     # keys past the valid length get exactly zero
        for b, n in enumerate(lens):
            assert not dk[b, :, n:].any() and not dv[b, :, n:].any()


def test_backward_from_fp16_output_and_bitwise_determinism():
    B, Hq, Hkv, S, d = 2, 4, 2, 512, 64
    q, k, v = (seeded(i, B, h, S, d).astype(np.float16) for i, h in ((84, Hq), (85, Hkv), (86, Hkv)))
    g = seeded(87, B, Hq, S, d).astype(np.float32)
    out, lse, runs = backward_device(q, k, v, g, causal=True, out_f16=True, repeats=3)
    assert out.dtype == np.float16
    rq, rk, rv, _ = oracle.sdpa_backward(widen(q), widen(k), widen(v), g, causal=True)
    for got, ref, name in zip(runs[0], (rq, rk, rv), ("dq", "dk", "dv")):
        assert_grad_close(got, ref, name)
    for other in runs[1:]:
        for a, b in zip(runs[0], other):
            assert np.array_equal(a, b)                       # no atomics anywhere: same bits every run


def test_backward_is_linear_in_the_upstream_gradient_at_a_large_size():
    """Size-independent property at a size the oracle cannot reach: grads(a*g1 + g2) = a*grads(g1) + grads(g2)."""
    B, H, S, d = 1, 4, 4096, 128
    q, k, v = (seeded(i, B, H, S, d).astype(np.float16) for i in (88, 89, 90))
    g1 = seeded(91, B, H, S, d).astype(np.float32)
    g2 = seeded(92, B, H, S, d).astype(np.float32)
    r1 = backward_device(q, k, v, g1, causal=True)[2:]
    r2 = backward_device(q, k, v, g2, causal=True)[2:]
    r3 = backward_device(q, k, v, 2.0 * g1 + g2, causal=True)[2:]
    for a, b, c, name in zip(r1, r2, r3, ("dq", "dk", "dv")):
        assert_grad_close(c, 2.0 * a.astype(np.float64) + b, name)
    # a sampled head against the oracle
    rq, rk, rv, _ = oracle.sdpa_backward(widen(q[:, :1, :1024]), widen(k[:, :1, :1024]), widen(v[:, :1, :1024]),
                                         g1[:, :1, :1024], causal=True)
    small = backward_device(q[:, :1, :1024], k[:, :1, :1024], v[:, :1, :1024], g1[:, :1, :1024], causal=True)[2:]
    for got, ref, name in zip(small, (rq, rk, rv), ("dq", "dk", "dv")):
        assert_grad_close(got, ref, name)


def test_autograd_through_the_python_api():
    """The reference's usage: requires_grad inputs, out.backward(grad), .grad on the leaves
    (tensorax/functional.py:312-319, tensorax/tensor.py:604-620,806-827)."""
    B, Hq, Hkv, S, d = 1, 4, 2, 320, 64
    q, k, v = (seeded(i, B, h, S, d).astype(np.float16) for i, h in ((93, Hq), (94, Hkv), (95, Hkv)))
    g = seeded(96, B, Hq, S, d).astype(np.float32)
    tq, tk, tv = (ts.Tensor(x, dtype="float16", device="cuda", requires_grad=True) for x in (q, k, v))
    out = F.scaled_dot_product_attention_ex(tq, tk, tv, causal=True, kv_lens=[300])
    assert out.requires_grad and out._grad_fn[0] == "scaled_dot_product_attention"
    out.backward(ts.Tensor(g, device="cuda"))
    rq, rk, rv, _ = oracle.sdpa_backward(widen(q), widen(k), widen(v), g, causal=True, kv_lens=[300])
    assert_grad_close(tq.grad.numpy(), rq, "dq")
    assert_grad_close(tk.grad.numpy(), rk, "dk")
    assert_grad_close(tv.grad.numpy(), rv, "dv")
    # a forward without a backward kernel still records the reference's tuple and fails loudly on backward
    f32 = [ts.Tensor(widen(x[:, :, :16, :16]), device="cuda", requires_grad=True) for x in (q, q, q)]
    o2 = F.scaled_dot_product_attention(*f32)
    assert o2.requires_grad
    with pytest.raises(RuntimeError, match="kept no row statistics"):
        o2.backward(ts.Tensor(np.ones((1, 4, 16, 16), np.float32), device="cuda"))


def test_sharded_backward_equals_the_single_device_run_bitwise():
    """The forward's partition (whole (batch, K/V-head) units per rank, no collective) carries over to the
    backward: a unit's dK/dV sum only over its own query heads.  Each rank's slab through the same kernels,
    reassembled: identical bits."""
    from tensorax_b200 import sharding
    B, Hq, Hkv, S, d = 2, 8, 2, 384, 64
    q = seeded(97, B, Hq, S, d).astype(np.float16)
    k, v = (seeded(98 + j, B, Hkv, S, d).astype(np.float16) for j in range(2))
    g = seeded(100, B, Hq, S, d).astype(np.float32)
    lens = [384, 200]
    _, _, fq, fk, fv = backward_device(q, k, v, g, causal=True, kv_lens=lens)
    for world in (2, 4):
        dq, dk, dv = np.zeros_like(fq), np.zeros_like(fk), np.zeros_like(fv)
        for r in range(world):
            sh = sharding.partition(B, Hkv, Hq, world, r)
            qs, ks, vs, ls = sharding.shard_arrays(sh, q, k, v, lens)
            _, _, lq, lk, lv = backward_device(qs, ks, vs, sharding.shard_grad(sh, g), causal=True, kv_lens=ls)
            sharding.place_output(sh, dq, lq)
            sharding.place_kv_grad(sh, dk, lk)
            sharding.place_kv_grad(sh, dv, lv)
        for a, b in ((dq, fq), (dk, fk), (dv, fv)):
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes_forward_and_backward(seed):
    """Seeded random ragged shapes, masks and head groupings: forward (all tensor-core head dims, fp32 or fp16
    result) and, where the backward kernels exist, all three gradients."""
    rng = np.random.default_rng(1000 + seed)
    d = int(rng.choice([64, 128, 256, 512]))
    Hkv = int(rng.integers(1, 4))
    Hq = Hkv * int(rng.integers(1, 4))
    B = int(rng.integers(1, 4))
    Sq = int(rng.integers(1, 700 if d <= 128 else 400))
    Sk = int(rng.integers(1, 700 if d <= 128 else 400))
    causal = bool(rng.integers(0, 2))
    lens = [int(x) for x in rng.integers(1, Sk + 1, size=B)] if rng.integers(0, 2) else None
    out_f16 = bool(rng.integers(0, 2))
    q = seeded(2000 + seed, B, Hq, Sq, d).astype(np.float16)
    k = seeded(3000 + seed, B, Hkv, Sk, d).astype(np.float16)
    v = seeded(4000 + seed, B, Hkv, Sk, d).astype(np.float16)
    ref = oracle.sdpa_structured(widen(q), widen(k), widen(v), causal=causal, kv_lens=lens)
    if d > 256:
        got, tc = sdpa_device(q, k, v, causal=causal, kv_lens=lens, flags=_lib.TX_SDPA_OUT_F16 if out_f16 else 0)
        assert tc
        assert_close_fp16(got.astype(np.float32), ref)
        return
    g = seeded(5000 + seed, B, Hq, Sq, d).astype(np.float32)
    out, lse, dq, dk, dv = backward_device(q, k, v, g, causal=causal, kv_lens=lens, out_f16=out_f16)
    assert_close_fp16(out.astype(np.float32), ref)
    rq, rk, rv, _ = oracle.sdpa_backward(widen(q), widen(k), widen(v), g, causal=causal, kv_lens=lens)
    for got, r, name in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
        assert_grad_close(got, r, f"{name} {(B, Hq, Hkv, Sq, Sk, d, causal, lens, out_f16)}")


def test_batch_element_without_valid_keys_propagates_nan_like_the_reference_rule():
    """kv_lens[b] = 0: the forward rows of that batch element are 0/0 (NaN, as the reference), and the
    autograd rule (tensorax/tensor.py:806-827) then yields NaN for all of its gradients; the other batch
    elements are unaffected."""
    B, Hq, Hkv, S, d = 2, 2, 1, 200, 64
    q, k, v = (seeded(i, B, h, S, d).astype(np.float16) for i, h in ((120, Hq), (121, Hkv), (122, Hkv)))
    g = seeded(123, B, Hq, S, d).astype(np.float32)
    out, lse, dq, dk, dv = backward_device(q, k, v, g, kv_lens=[0, 150])
    with np.errstate(all="ignore"):
        rq, rk, rv, _ = oracle.sdpa_backward(widen(q), widen(k), widen(v), g, kv_lens=[0, 150])
    assert np.isnan(rq[0]).all() and np.isnan(rk[0]).all() and np.isnan(rv[0]).all()
    assert np.isnan(out[0]).all() and np.isnan(dq[0]).all() and np.isnan(dk[0]).all() and np.isnan(dv[0]).all()
    for got, ref, name in ((dq[1:], rq[1:], "dq"), (dk[1:], rk[1:], "dk"), (dv[1:], rv[1:], "dv")):
        assert_grad_close(got, ref, name)


@pytest.mark.parametrize("d", [64, 128, 256])
def test_peaked_attention_rows_forward_and_backward(d):
    """Large logits (softmax close to one-hot, running max growing by far more than the lazy-rescale
    threshold from tile to tile): the rescale path of the forward and the saved statistics stay exact enough
    for the gradients."""
    B, H, S = 1, 2, 520
    rng = np.random.default_rng(77)
    q = (3.0 * rng.standard_normal((B, H, S, d))).astype(np.float16)
    k = (3.0 * rng.standard_normal((B, H, S, d))).astype(np.float16)
    k[:, :, 300:] *= 2.0                                     # later key tiles carry the larger scores
    v = rng.standard_normal((B, H, S, d)).astype(np.float16)
    g = rng.standard_normal((B, H, S, d)).astype(np.float32)
    out, lse, dq, dk, dv = backward_device(q, k, v, g)
    assert_close_fp16(out, oracle.sdpa_structured(widen(q), widen(k), widen(v)))
    rq, rk, rv, rl = oracle.sdpa_backward(widen(q), widen(k), widen(v), g)
    np.testing.assert_allclose(lse, rl, rtol=2e-5, atol=2e-3)
    for got, r, name in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
        assert_grad_close(got, r, name)


# ------------------------------------------------------------------ launch order
def test_launch_order_never_changes_a_result():
    """Causal calls walk their (batch, head) slabs in groups, longest work items first (tx_sdpa_set_group_l2_bytes).
    A group is never smaller than two waves of CTAs, so the call has many slabs: 117 (batch, query head) slabs of three
    query pairs fall into two groups of 60 and 57 (whole K/V heads of three query heads each) under a small budget and
    into one under the default.  Every CTA computes what it always computes:
    forward (fp16 at d = 64, 128, 256; fp32 on the tensor cores) and backward are bitwise the same either way, and right."""
    lib = _lib.load()
    B, Hq, Hkv, S = 3, 39, 13, 700
    lens = [700, 333, 512]
    try:
        for d in (64, 128, 256):
            q = seeded(500 + d, B, Hq, S, d).astype(np.float16)
            k, v = (seeded(501 + d + j, B, Hkv, S, d).astype(np.float16) for j in range(2))
            g = seeded(510 + d, B, Hq, S, d)
            res = []
            for budget in (0, 1 << 20, 300 << 10):
                _lib.check(lib.tx_sdpa_set_group_l2_bytes(budget))
                res.append(backward_device(q, k, v, g, causal=True, kv_lens=lens))
            for other in res[1:]:
                for a, b in zip(res[0], other):
                    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
            ref = oracle.sdpa_structured(widen(q), widen(k), widen(v), causal=True, kv_lens=lens, threads=8)
            assert_close_fp16(res[0][0], ref)
            if d <= 128:
                q32, k32, v32 = seeded(520 + d, B, Hq, S, d), seeded(521 + d, B, Hkv, S, d), seeded(522 + d, B, Hkv, S, d)
                outs = []
                for budget in (0, 1 << 20):
                    _lib.check(lib.tx_sdpa_set_group_l2_bytes(budget))
                    o32, tc = sdpa_device(q32, k32, v32, causal=True, kv_lens=lens)
                    assert tc
                    outs.append(o32)
                assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    finally:
        _lib.check(lib.tx_sdpa_set_group_l2_bytes(0))
