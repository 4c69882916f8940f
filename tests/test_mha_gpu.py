"""GPU parity of the linear layers and of MultiHeadAttention.forward against the
reference's matmul_cpu / sdpa_cpu compositions.  fp32 throughout, tolerance 1e-5."""
import numpy as np
import pytest

import oracle
import tensorax_b200 as ts
import tensorax_b200.functional as F
from conftest import assert_close_fp32, seeded
from tensorax_b200 import _C
from tensorax_b200.nn.attention import MultiHeadAttention

pytestmark = pytest.mark.gpu


def test_linear_golden(golden):
    x, w, b = (ts.Tensor(golden[f"lin_{n}"], device="cuda") for n in ("x", "w", "b"))
    assert_close_fp32(F.linear(x, w, b).numpy(), golden["lin_out"])
    assert_close_fp32(F.linear(x, w).numpy(), golden["lin_out_nobias"])
    x2 = ts.Tensor(golden["lin_x"][0], device="cuda")          # 2-D input
    assert_close_fp32(F.linear(x2, w, b).numpy(), golden["lin_out"][0])


@pytest.mark.parametrize("B,S,K,N,H", [(2, 70, 96, 64, 4), (1, 129, 130, 66, 2), (3, 5, 33, 260, 1)])
def test_linear_with_head_split_and_merge(B, S, K, N, H):
    x, w, b = seeded(1, B, S, K), seeded(2, N, K) / np.sqrt(K), seeded(3, N)
    ref = oracle.linear_f32(x, w, b)
    xt, wt, bt = (ts.Tensor(a, device="cuda") for a in (x, w, b))
    plain = _C.to_numpy(_C.linear(xt._c_tensor, wt._c_tensor, bt._c_tensor))
    assert_close_fp32(plain, ref)
    split = _C.to_numpy(_C.linear(xt._c_tensor, wt._c_tensor, bt._c_tensor, heads_out=H))
    assert split.shape == (B, H, S, N // H)
    assert np.array_equal(split, plain.reshape(B, S, H, N // H).transpose(0, 2, 1, 3))
    if K % H == 0:
        xs = np.ascontiguousarray(x.reshape(B, S, H, K // H).transpose(0, 2, 1, 3))     # what a head-split producer leaves
        merged = _C.to_numpy(_C.linear(ts.Tensor(xs, device="cuda")._c_tensor, wt._c_tensor, bt._c_tensor, heads_in=H))
        assert np.array_equal(merged, plain)


def test_multi_head_attention_forward_golden(golden):
    mha = MultiHeadAttention(32, 4, device="cuda")
    for n in ("q_weight", "k_weight", "v_weight", "out_weight", "q_bias", "k_bias", "v_bias", "out_bias"):
        mha._parameters[n] = ts.Tensor(golden[f"mha_{n}"], device="cuda")
    xq, xk, xv = (ts.Tensor(golden[f"mha_{n}"], device="cuda") for n in ("xq", "xk", "xv"))
    out = mha(xq, xk, xv)
    assert out.shape == (2, 10, 32) and out.device == "cuda"
    assert_close_fp32(out.numpy(), golden["mha_out"])


def test_multi_head_attention_forward_with_mask_and_no_bias():
    B, S, E, H = 2, 150, 256, 8
    mha = MultiHeadAttention(E, H, bias=False).cuda()
    params = {n: p.numpy() for n, p in mha._parameters.items() if p is not None}
    x = seeded(7, B, S, E)
    mask = np.where(np.tril(np.ones((S, S), bool)), 0.0, -np.inf).astype(np.float32)
    mask = np.ascontiguousarray(np.broadcast_to(mask, (B, H, S, S)))
    xt = ts.Tensor(x, device="cuda")
    got = mha(xt, xt, xt, ts.Tensor(mask, device="cuda")).numpy()
    ref = oracle.mha_forward_f32(x, x, x, params, H, mask)
    assert_close_fp32(got, ref, atol=2e-5)     # four chained fp32 stages
