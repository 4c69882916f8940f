"""CPU suite: the oracle restatement against the golden vectors written by the
reference's own sdpa_cpu, against the reference library itself where it was
built (oracle/_ref), and against an independent float64 numpy evaluation."""
import hashlib

import numpy as np
import pytest

import oracle
from conftest import seeded


def np_sdpa64(q, k, v, mask=None):
    """float64 evaluation in the style of the reference tests' own pure-Python
    oracle (tests/test_attention.py:8-36)."""
    q, k, v = (x.astype(np.float64) for x in (q, k, v))
    s = np.einsum("bhid,bhjd->bhij", q, k) / np.sqrt(q.shape[-1])
    if mask is not None:
        s = s + mask.astype(np.float64)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("bhij,bhjd->bhid", p, v)


def bit_equal(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_config1_bit_exact(golden):
    out = oracle.sdpa_f32(golden["c1_q"], golden["c1_k"], golden["c1_v"])
    assert bit_equal(out, golden["c1_out"])
    assert np.abs(out - np_sdpa64(golden["c1_q"], golden["c1_k"], golden["c1_v"])).max() < 1e-5


@pytest.mark.parametrize("name", ["single_query", "pattern", "manual2x2", "const100"])
def test_hand_written_cases(golden, name):
    q, k, v = (golden[f"hand_{name}_{t}"] for t in "qkv")
    out = oracle.sdpa_f32(q, k, v)
    assert bit_equal(out, golden[f"hand_{name}_out"])
    assert np.abs(out - np_sdpa64(q, k, v)).max() < 1e-4      # tolerance of test_attention.py:54
    if name == "pattern":
        assert out.ravel()[0] > 3.0                            # test_attention.py:132
    if name == "const100":
        assert np.isfinite(out).all()                          # test_attention.py:198-199


@pytest.mark.parametrize("kind", ["1e9", "inf", "row", "rand"])
def test_dense_masks(golden, kind):
    q, k, v = golden["mask_q"], golden["mask_k"], golden["mask_v"]
    out = oracle.sdpa_f32(q, k, v, golden[f"mask_m{kind}"])
    assert bit_equal(out, golden[f"mask_out{kind}"])
    if kind == "row":
        assert np.isnan(out[0, 1, 3]).all() and np.isfinite(out[0, 0]).all()


@pytest.mark.parametrize("i", range(5))
def test_ragged_shapes(golden, i):
    q, k, v = (golden[f"ragged{i}_{t}"] for t in "qkv")
    assert bit_equal(oracle.sdpa_f32(q, k, v), golden[f"ragged{i}_out"])


def _digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest()[:8], dtype=np.uint64)


def f16_inputs(i, shape):
    B, H, Sq, Sk, dk, dv = (int(x) for x in shape)
    q = seeded(400 + i, B, H, Sq, dk).astype(np.float16)
    k = seeded(420 + i, B, H, Sk, dk).astype(np.float16)
    v = seeded(440 + i, B, H, Sk, dv).astype(np.float16)
    return q, k, v


@pytest.mark.parametrize("i", range(5))
def test_fp16_shapes_sampled_rows(golden, i):
    q, k, v = f16_inputs(i, golden["f16_shapes"][i])
    assert np.array_equal(_digest(q, k, v), golden[f"f16_{i}_digest"]), "seeded inputs drifted"
    rows = golden[f"f16_{i}_rows"]
    out = oracle.sdpa_f32(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32))
    assert bit_equal(np.ascontiguousarray(out[:, :, rows, :]), golden[f"f16_{i}_out"])


def test_structured_form_equals_reference_dense_form(golden):
    q, k, v = (golden[f"gqa_{t}"].astype(np.float32) for t in "qkv")
    out = oracle.sdpa_structured(q, k, v, causal=True, kv_lens=golden["gqa_lens"])
    assert bit_equal(out, golden["gqa_out"])
    # restricted evaluation writes only what was asked for
    part = oracle.sdpa_structured(q, k, v, causal=True, kv_lens=golden["gqa_lens"], heads=[5], rows=(10, 20))
    assert bit_equal(np.ascontiguousarray(part[1, 1, 10:20]), np.ascontiguousarray(out[1, 1, 10:20]))
    assert np.isnan(part[0]).all() and np.isnan(part[1, 1, :10]).all()
    threaded = oracle.sdpa_structured(q, k, v, causal=True, kv_lens=golden["gqa_lens"], threads=4)
    assert bit_equal(threaded, out)


@pytest.mark.skipif(not oracle.have_reference(), reason="reference CPU library not built on this machine")
def test_restatement_equals_reference_library():
    for seed, (B, H, Sq, Sk, dk, dv) in enumerate([(1, 2, 128, 128, 64, 64), (2, 2, 33, 70, 48, 20)]):
        q, k, v = seeded(900 + seed, B, H, Sq, dk), seeded(910 + seed, B, H, Sk, dk), seeded(920 + seed, B, H, Sk, dv)
        m = seeded(930 + seed, B, H, Sq, Sk)
        m[m > 1.2] = -np.inf
        assert bit_equal(oracle.sdpa_f32(q, k, v), oracle.ref_sdpa_cpu(q, k, v))
        assert bit_equal(oracle.sdpa_f32(q, k, v, m), oracle.ref_sdpa_cpu(q, k, v, m))


def test_linear_and_mha_forward_restatements(golden):
    x, w, b = golden["lin_x"], golden["lin_w"], golden["lin_b"]
    assert bit_equal(oracle.linear_f32(x, w, b), golden["lin_out"])
    assert bit_equal(oracle.linear_f32(x, w), golden["lin_out_nobias"])
    params = {n: golden[f"mha_{n}"] for n in ("q_weight", "k_weight", "v_weight", "out_weight",
                                               "q_bias", "k_bias", "v_bias", "out_bias")}
    out = oracle.mha_forward_f32(golden["mha_xq"], golden["mha_xk"], golden["mha_xv"], params, num_heads=4)
    assert bit_equal(out, golden["mha_out"])


# ------------------------------------------------------------------ backward oracle
@pytest.mark.parametrize("causal,lens,hkv", [(False, None, 2), (True, None, 1), (True, [9, 5], 2), (False, [4, 11], 1)])
def test_backward_oracle_matches_central_differences_of_the_forward_oracle(causal, lens, hkv):
    """The backward restatement (tensorax/tensor.py:806-827) is the gradient of the pinned forward
    oracle: d/dx sum(out * g) by central differences, every input element of small tensors."""
    rng = np.random.default_rng(7)
    B, Hq, Sq, Sk, d = 2, 2, 6, 11, 4
    q = rng.standard_normal((B, Hq, Sq, d))
    k = rng.standard_normal((B, hkv, Sk, d))
    v = rng.standard_normal((B, hkv, Sk, d))
    g = rng.standard_normal((B, Hq, Sq, d))
    dq, dk, dv, lse2 = oracle.sdpa_backward(q, k, v, g, causal=causal, kv_lens=lens)

    def loss(q_, k_, v_):
        # float64 forward with the same masks; checked against the C oracle below
        out = np.zeros((B, Hq, Sq, d))
        for b in range(B):
            vis = oracle._visible(Sq, Sk, causal, None if lens is None else lens[b])
            for h in range(Hq):
                s = np.where(vis, (q_[b, h] @ k_[b, h // (Hq // hkv)].T) / np.sqrt(d), -np.inf)
                p = np.exp(s - s.max(-1, keepdims=True))
                out[b, h] = (p / p.sum(-1, keepdims=True)) @ v_[b, h // (Hq // hkv)]
        return out

    ref_out = oracle.sdpa_structured(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32),
                                     causal=causal, kv_lens=lens)
    np.testing.assert_allclose(loss(q, k, v), ref_out, atol=2e-6)
    eps = 1e-5
    for name, x, gx in (("q", q, dq), ("k", k, dk), ("v", v, dv)):
        num = np.zeros_like(x)
        it = np.nditer(x, flags=["multi_index"])
        for _ in it:
            i = it.multi_index
            old = x[i]
            x[i] = old + eps
            up = (loss(q, k, v) * g).sum()
            x[i] = old - eps
            dn = (loss(q, k, v) * g).sum()
            x[i] = old
            num[i] = (up - dn) / (2 * eps)
        np.testing.assert_allclose(gx, num, atol=1e-7, rtol=1e-6, err_msg=name)
    # the saved row statistic reproduces the probabilities
    s2 = np.einsum("bhid,bhjd->bhij", q, np.repeat(k, Hq // hkv, axis=1)) / np.sqrt(d) * np.log2(np.e)
    p = np.exp2(s2 - lse2[..., None])
    for b in range(B):
        vis = oracle._visible(Sq, Sk, causal, None if lens is None else lens[b])
        np.testing.assert_allclose((p[b] * vis).sum(-1), 1.0, rtol=1e-12)
