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


LINEAR_SHAPES = [
    (2, 70, 96, 64, 4),       # ragged rows, 16-wide heads: CUDA-core kernel for the head-split forms
    (1, 129, 130, 66, 2),     # nothing is a multiple of 32: CUDA-core kernel
    (3, 5, 33, 260, 1),
    (2, 200, 128, 256, 4),    # multiples of 32 throughout: split-TF32 tensor-core kernel
    (1, 384, 512, 384, 6),
    (2, 128, 64, 128, 2),
]


@pytest.mark.parametrize("cuda_cores_only", [False, True])
@pytest.mark.parametrize("B,S,K,N,H", LINEAR_SHAPES)
def test_linear_with_head_split_and_merge(B, S, K, N, H, cuda_cores_only):
    from tensorax_b200 import _lib
    lib = _lib.load()
    x, w, b = seeded(1, B, S, K), seeded(2, N, K) / np.sqrt(K), seeded(3, N)
    ref = oracle.linear_f32(x, w, b)
    xt, wt, bt = (ts.Tensor(a, device="cuda") for a in (x, w, b))
    lib.tx_linear_set_cuda_cores_only(int(cuda_cores_only))
    try:
        launches = lib.tx_kernel_launch_count()
        plain = _C.to_numpy(_C.linear(xt._c_tensor, wt._c_tensor, bt._c_tensor))
        assert lib.tx_kernel_launch_count() == launches + 1
        assert_close_fp32(plain, ref)
        split = _C.to_numpy(_C.linear(xt._c_tensor, wt._c_tensor, bt._c_tensor, heads_out=H))
        assert split.shape == (B, H, S, N // H)
        assert_close_fp32(split, ref.reshape(B, S, H, N // H).transpose(0, 2, 1, 3))
        if K % H == 0:
            xs = np.ascontiguousarray(x.reshape(B, S, H, K // H).transpose(0, 2, 1, 3))   # what a head-split producer leaves
            merged = _C.to_numpy(_C.linear(ts.Tensor(xs, device="cuda")._c_tensor, wt._c_tensor, bt._c_tensor, heads_in=H))
            assert_close_fp32(merged, ref)
        nobias = _C.to_numpy(_C.linear(xt._c_tensor, wt._c_tensor, None))
        assert_close_fp32(nobias, oracle.linear_f32(x, w))
    finally:
        lib.tx_linear_set_cuda_cores_only(0)


def test_split_tf32_keeps_fp32_accuracy_on_hard_inputs():
    """Values whose low mantissa bits matter: a plain TF32 product would be off by ~1e-3 here."""
    B, S, K, N = 1, 256, 1024, 128
    x = (1.0 + seeded(40, B, S, K) * 1e-3).astype(np.float32)        # 1.000xxx: the information sits below TF32's 10 bits
    w = (seeded(41, N, K) / K).astype(np.float32)
    got = _C.to_numpy(_C.linear(ts.Tensor(x, device="cuda")._c_tensor, ts.Tensor(w, device="cuda")._c_tensor, None))
    ref64 = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(got - ref64).max() <= 2e-6
    assert_close_fp32(got, oracle.linear_f32(x, w))


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


def test_multi_head_attention_with_fp16_attention_step_and_implicit_causal_mask():
    """attention_dtype='float16': projections in fp32, heads rounded to fp16, attention on the tensor-core
    kernel (head_dim 64), output projection in fp32; causal= instead of the dense mask.  Against the fp32
    composition of the reference's CPU ops with the dense causal mask, at the fp16 tolerance."""
    from conftest import assert_close_fp16
    B, S, E, H = 2, 300, 256, 4
    mha = MultiHeadAttention(E, H, attention_dtype="float16").cuda()
    params = {n: p.numpy() for n, p in mha._parameters.items() if p is not None}
    x = seeded(9, B, S, E)
    mask = np.where(np.tril(np.ones((S, S), bool)), 0.0, -np.inf).astype(np.float32)
    mask = np.ascontiguousarray(np.broadcast_to(mask, (B, H, S, S)))
    xt = ts.Tensor(x, device="cuda")
    got = mha(xt, xt, xt, causal=True).numpy()
    ref = oracle.mha_forward_f32(x, x, x, params, H, mask)
    assert_close_fp16(got, ref)
    same = MultiHeadAttention(E, H).cuda()
    same._parameters = mha._parameters
    assert_close_fp32(same(xt, xt, xt, causal=True).numpy(), ref, atol=2e-5)   # fp32 path, implicit mask
    with pytest.raises(ValueError):
        MultiHeadAttention(E, H, attention_dtype="bfloat16")
