"""GPU parity of the fp32 path against the golden vectors written by the
reference's sdpa_cpu and against the oracle, through the C ABI and through the
Python mirror of the reference API.  Tolerance: max-abs 1e-5."""
import ctypes

import numpy as np
import pytest

import oracle
import tensorax_b200 as ts
import tensorax_b200.functional as F
from conftest import assert_close_fp32, seeded
from gpu_util import sdpa_device
from tensorax_b200 import _lib
from tensorax_b200.nn.attention import (GroupedQueryAttention, ScaledDotProductAttention,
                                        create_causal_mask, create_padding_mask)

pytestmark = pytest.mark.gpu

F32_ENTRY_POINTS = ["tx_sdpa_naive_cuda", "tx_sdpa_tiled_cuda", "tx_sdpa_flash_cuda",
                    "tx_sdpa_optimized_flash_cuda", "tx_sdpa_mma_cuda"]
F32_FUNCTIONS = [F.scaled_dot_product_attention, F.scaled_dot_product_attention_tiled,
                 F.scaled_dot_product_attention_flash, F.scaled_dot_product_attention_mma,
                 F.scaled_dot_product_attention_flash_optimized]


def call_reference_signature(name, q, k, v, mask=None):
    lib = _lib.load()
    B, H, Sq, dk = q.shape
    Sk, dv = k.shape[2], v.shape[3]
    bufs = [_lib.to_device(x) for x in (q, k, v)]
    m = _lib.to_device(mask) if mask is not None else None
    out = _lib.DeviceBuffer(B * H * Sq * dv * 4)
    _lib.check(getattr(lib, name)(bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, m.ptr if m else None, out.ptr,
                                  B, H, Sq, Sk, dk, dv))
    return out.download((B, H, Sq, dv), np.float32)


@pytest.mark.parametrize("name", F32_ENTRY_POINTS)
def test_config1_every_fp32_entry_point(golden, name):
    got = call_reference_signature(name, golden["c1_q"], golden["c1_k"], golden["c1_v"])
    assert_close_fp32(got, golden["c1_out"])


@pytest.mark.parametrize("case", ["single_query", "pattern", "manual2x2", "const100"])
def test_hand_written_cases(golden, case):
    q, k, v = (golden[f"hand_{case}_{t}"] for t in "qkv")
    got, tc = sdpa_device(q, k, v)
    assert not tc
    assert_close_fp32(got, golden[f"hand_{case}_out"])


@pytest.mark.parametrize("kind", ["1e9", "inf", "row", "rand"])
def test_dense_masks_including_a_fully_masked_row(golden, kind):
    got = call_reference_signature("tx_sdpa_flash_cuda", golden["mask_q"], golden["mask_k"],
                                   golden["mask_v"], golden[f"mask_m{kind}"])
    assert_close_fp32(got, golden[f"mask_out{kind}"])     # also checks NaN rows match


@pytest.mark.parametrize("i", range(5))
def test_ragged_shapes(golden, i):
    q, k, v = (golden[f"ragged{i}_{t}"] for t in "qkv")
    got, _ = sdpa_device(q, k, v)
    assert_close_fp32(got, golden[f"ragged{i}_out"])


def test_medium_random_with_mask_against_oracle():
    B, H, Sq, Sk, dk, dv = 2, 3, 200, 333, 72, 136
    q, k, v = seeded(1, B, H, Sq, dk), seeded(2, B, H, Sk, dk), seeded(3, B, H, Sk, dv)
    m = seeded(4, B, H, Sq, Sk)
    m[m > 1.0] = -np.inf
    got, _ = sdpa_device(q, k, v, mask=m)
    assert_close_fp32(got, oracle.sdpa_f32(q, k, v, m))


def test_structured_masks_equal_dense_masks_on_fp32():
    B, Hq, Hkv, S, d = 2, 4, 2, 150, 32
    q, k, v = seeded(5, B, Hq, S, d), seeded(6, B, Hkv, S, d), seeded(7, B, Hkv, S, d)
    lens = [150, 77]
    got, _ = sdpa_device(q, k, v, causal=True, kv_lens=lens)
    assert_close_fp32(got, oracle.sdpa_structured(q, k, v, causal=True, kv_lens=lens))
    empty, _ = sdpa_device(q, k, v, kv_lens=[0, 5])        # no visible key -> NaN rows, as the reference
    assert np.isnan(empty[0]).all() and np.isfinite(empty[1]).all()


@pytest.mark.parametrize("fn", F32_FUNCTIONS)
def test_python_api_on_cuda_tensors(golden, fn):
    """The reference's own unit tests (tests/test_attention.py:48-148) on device='cuda'."""
    q, k, v = (ts.Tensor(golden[f"ragged0_{t}"], device="cuda") for t in "qkv")
    out = fn(q, k, v)
    assert out.shape == (2, 2, 4, 8) and out.device == "cuda" and out.dtype == "float32"
    assert_close_fp32(out.numpy(), golden["ragged0_out"])
    mask = ts.Tensor(golden["mask_m1e9"], device="cuda")
    q, k, v = (ts.Tensor(golden[f"mask_{t}"], device="cuda") for t in "qkv")
    assert_close_fp32(fn(q, k, v, mask).numpy(), golden["mask_out1e9"])
    assert fn(q, k, v).tolist()[0][0] != fn(q, k, v).tolist()[0][1]      # head independence


def test_layers_and_mask_builders_on_cuda(golden):
    q, k, v = (ts.Tensor(golden[f"mask_{t}"], device="cuda") for t in "qkv")
    S = q.shape[2]
    mask = create_causal_mask(S, batch_size=2, num_heads=2, device="cuda")
    out = ScaledDotProductAttention()(q, k, v, mask)
    assert_close_fp32(out.numpy(), golden["mask_outinf"])
    # padding mask has shape [B,H,1,L]: accepted only for a single query row, as in the reference
    pm = create_padding_mask([5, 12], S, num_heads=2, device="cuda")
    with pytest.raises(RuntimeError, match="Mask shape must be"):
        F.scaled_dot_product_attention(q, k, v, pm)
    q1 = ts.Tensor(golden["mask_q"][:, :, :1, :], device="cuda")
    got = F.scaled_dot_product_attention(q1, k, v, pm).numpy()
    ref = oracle.sdpa_structured(golden["mask_q"][:, :, :1, :], golden["mask_k"], golden["mask_v"], kv_lens=[5, 12])
    assert_close_fp32(got, ref)
    # GQA layer: the reference replicates along dim 2 and passes the result on unchanged
    gqa = GroupedQueryAttention(4, 2)
    x = seeded(9, 1, 3, 4, 8)
    kv = seeded(10, 1, 3, 2, 8)
    got = gqa(ts.Tensor(x, device="cuda"), ts.Tensor(kv, device="cuda"), ts.Tensor(kv, device="cuda"))
    rep = np.repeat(kv, 2, axis=2)
    assert got.shape == (1, 3, 4, 8)
    assert_close_fp32(got.numpy(), oracle.sdpa_f32(x, rep, rep))
    # the same sharing in the [B,H,S,d] layout needs no copy
    qh, kh = seeded(11, 2, 4, 20, 16), seeded(12, 2, 2, 20, 16)
    got = gqa.forward_bhsd(ts.Tensor(qh, device="cuda"), ts.Tensor(kh, device="cuda"), ts.Tensor(kh, device="cuda"))
    assert_close_fp32(got.numpy(), oracle.sdpa_f32(qh, np.repeat(kh, 2, axis=1), np.repeat(kh, 2, axis=1)))


def test_cast_and_repeat_interleave_on_device():
    x = seeded(20, 3, 5, 7, 11)
    t = ts.Tensor(x, device="cuda")
    h = F.cast_to_fp16(t)
    assert h.dtype == "float16" and h.shape == t.shape
    assert np.array_equal(h.numpy(), x.astype(np.float16))
    assert F.cast_to_fp16(h) is h
    for dim in (0, 1, 2, 3, -1):
        assert np.array_equal(t.repeat_interleave(3, dim=dim).numpy(), np.repeat(x, 3, axis=dim))
    assert np.array_equal(h.repeat_interleave(2, dim=1).numpy(), np.repeat(x.astype(np.float16), 2, axis=1))
    assert t.cpu().tolist() == x.astype(np.float64).tolist()


def test_allocation_pool_reuses_and_trims():
    """cuda_malloc / cuda_free replacements (csrc/cuda/tensor_cuda.cu:13-21) on the stream-ordered pool."""
    lib = _lib.load()
    x = seeded(30, 1 << 16)
    ptrs = set()
    for _ in range(20):
        buf = _lib.to_device(x)
        assert np.array_equal(buf.download(x.shape, np.float32), x)
        ptrs.add(buf.ptr)
        del buf
    assert len(ptrs) < 20          # freed blocks come back from the pool
    _lib.check(lib.tx_cuda_pool_trim())
    buf = _lib.to_device(x)
    assert np.array_equal(buf.download(x.shape, np.float32), x)
