"""CPU suite for the host side: the C-ABI library loads and exports every symbol
the header declares, the Python mirror of the reference API keeps its error
contracts, and nothing computes without a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

import tensorax_b200 as ts
import tensorax_b200.functional as F
from tensorax_b200 import _C, _lib
from tensorax_b200.nn.attention import (GroupedQueryAttention, MultiHeadAttention,
                                        ScaledDotProductAttention, create_causal_mask,
                                        create_padding_mask)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "tensorax_b200.h")).read()
    return sorted(set(re.findall(r"TX_API\s+[\w\s\*]+?\b(tx_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = header_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/tensorax_b200.h but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == names


def test_desc_struct_layout_matches_header():
    # 6 pointers + 7 int64 + 4 int32 + 2 pointers, no padding surprises
    assert ctypes.sizeof(_lib.SdpaDesc) == 6 * 8 + 7 * 8 + 4 * 4 + 2 * 8
    assert _lib.SdpaDesc.lse.offset == 6 * 8 + 7 * 8 + 4 * 4 + 8
    # backward: 10 pointers + 6 int64 + 2 int32 + 1 pointer
    assert ctypes.sizeof(_lib.SdpaBwdDesc) == 10 * 8 + 6 * 8 + 2 * 4 + 8


@pytest.mark.skipif(_lib.cuda_is_available(), reason="checks the no-device behaviour")
def test_no_device_means_loud_failure_not_fallback():
    lib = _lib.load()
    buf = (ctypes.c_float * 16)()
    rc = lib.tx_sdpa_naive_cuda(buf, buf, buf, None, buf, 1, 1, 2, 2, 2, 2)
    assert rc == 2 and b"no CUDA device" in lib.tx_last_error()
    with pytest.raises(RuntimeError):
        ts.Tensor(np.zeros((1, 1, 2, 2), np.float32), device="cuda")
    q = ts.Tensor.randn((1, 1, 2, 2))
    with pytest.raises(RuntimeError, match="CUDA path only"):
        F.scaled_dot_product_attention(q, q, q)


def test_backward_rejects_bad_descriptors_before_any_launch():
    lib = _lib.load()
    assert lib.tx_sdpa_backward(None) == 1
    d = _lib.SdpaBwdDesc(q=16, k=16, v=16, out=16, dout=16, lse=16, dq=16, dk=16, dv=16, batch=1, q_heads=2,
                         kv_heads=2, seq_q=8, seq_k=8, d=32)
    assert lib.tx_sdpa_backward(ctypes.byref(d)) == 5 and b"d in {64, 128, 256}" in lib.tx_last_error()
    d.d = 64
    d.kv_heads = 3
    assert lib.tx_sdpa_backward(ctypes.byref(d)) == 1
    d.kv_heads = 2
    d.lse = None
    assert lib.tx_sdpa_backward(ctypes.byref(d)) == 1 and b"must not be null" in lib.tx_last_error()


def test_backward_of_unsupported_forward_raises():
    """A result recorded for autograd whose shapes have no backward kernel fails loudly."""
    t = ts.Tensor.__new__(ts.Tensor)
    t.requires_grad, t.grad, t._grad_fn, t._shape, t._size = True, None, ("scaled_dot_product_attention", t, t, t, None), (2,), 2
    with pytest.raises(RuntimeError, match="grad must be specified"):
        t.backward()
    g = ts.Tensor.randn((2,))
    with pytest.raises(RuntimeError, match="kept no row statistics"):
        t.backward(g)


def test_invalid_arguments_are_rejected_before_any_launch():
    lib = _lib.load()
    buf = (ctypes.c_float * 16)()
    assert lib.tx_sdpa_naive_cuda(None, buf, buf, None, buf, 1, 1, 2, 2, 2, 2) == 1
    assert lib.tx_sdpa_naive_cuda(buf, buf, buf, None, buf, 1, 0, 2, 2, 2, 2) == 1
    d = _lib.SdpaDesc(q=1, k=1, v=1, out=1, batch=1, q_heads=3, kv_heads=2, seq_q=1, seq_k=1, d_k=1, d_v=1)
    assert lib.tx_sdpa_forward(ctypes.byref(d)) == 1
    assert b"Key dimensions don't match Query" in lib.tx_last_error()


def test_error_contracts_of_the_functional_api():
    """tests/test_attention.py:172-184,327-388 of the reference."""
    with pytest.raises((ValueError, RuntimeError)):
        t = ts.Tensor.randn((4, 8))
        F.scaled_dot_product_attention(t, t, t)
    q = ts.Tensor.randn((1, 1, 4, 8))
    for fn in (F.scaled_dot_product_attention, F.scaled_dot_product_attention_tiled,
               F.scaled_dot_product_attention_flash, F.scaled_dot_product_attention_mma,
               F.scaled_dot_product_attention_flash_optimized):
        with pytest.raises(ValueError, match="must be 4D tensors"):
            fn(ts.Tensor.randn((4, 8)), q, q)
        other = ts.Tensor.randn((1, 1, 4, 8))
        other.device = "cuda"                      # the reference tests fake devices the same way
        with pytest.raises(ValueError, match="same device"):
            fn(q, other, q)
        with pytest.raises(ValueError, match="Mask must be on the same device"):
            fn(q, q, q, other)
    with pytest.raises(ValueError, match="must be float16"):
        F.scaled_dot_product_attention_mma_fp16(q, q, q)
    with pytest.raises(ValueError, match="only CUDA tensors"):
        F.cast_to_fp16(q)


def test_backend_missing_message(monkeypatch):
    monkeypatch.setattr(F, "_C", None)             # tests/test_attention.py:350-361
    q = ts.Tensor.randn((1, 1, 2, 2))
    with pytest.raises(RuntimeError, match=r"C\+\+ backend not available"):
        F.scaled_dot_product_attention(q, q, q)


def test_backend_validation_messages():
    def t(*shape, device="cuda"):
        x = _C.TensorImpl.__new__(_C.TensorImpl)
        x._shape, x._size, x._dtype, x._device, x._buf, x._host = list(shape), 1, "float32", device, None, None
        return x
    with pytest.raises(RuntimeError, match="must be 4D"):
        _C.scaled_dot_product_attention(t(4, 8), t(4, 8), t(4, 8))
    with pytest.raises(RuntimeError, match="Key dimensions don't match Query"):
        _C.scaled_dot_product_attention(t(1, 1, 4, 8), t(1, 1, 4, 16), t(1, 1, 4, 8))
    with pytest.raises(RuntimeError, match="Value dimensions don't match Key"):
        _C.scaled_dot_product_attention(t(1, 1, 4, 8), t(1, 1, 4, 8), t(1, 1, 5, 8))
    with pytest.raises(RuntimeError, match="Mask shape must be"):
        _C.scaled_dot_product_attention(t(2, 1, 4, 8), t(2, 1, 6, 8), t(2, 1, 6, 8), t(2, 1, 1, 6))
    with pytest.raises(RuntimeError, match="all tensors must be on CUDA"):
        _C.scaled_dot_product_attention_mma_fp16(t(1, 1, 4, 8, device="cpu"), t(1, 1, 4, 8), t(1, 1, 4, 8))
    with pytest.raises(RuntimeError, match="dtype float16"):
        _C.scaled_dot_product_attention_mma_fp16(t(1, 1, 4, 8), t(1, 1, 4, 8), t(1, 1, 4, 8))


def test_mask_builders_values_and_shapes():
    """tests/test_attention.py:288-311 of the reference."""
    m = create_causal_mask(4, batch_size=2, num_heads=3)
    assert m.shape == (2, 3, 4, 4)
    a = m.numpy()
    for i in range(4):
        for j in range(4):
            assert a[1, 2, i, j] == (0.0 if j <= i else -np.inf)
    p = create_padding_mask([3, 5], 5, num_heads=2)
    assert p.shape == (2, 2, 1, 5)
    b = p.numpy()
    assert list(b[0, 1, 0]) == [0.0, 0.0, 0.0, -np.inf, -np.inf] and (b[1] == 0).all()


def test_layers_construct_and_print_like_the_reference():
    assert repr(ScaledDotProductAttention()) == "ScaledDotProductAttention()"
    g = GroupedQueryAttention(8, 2)
    assert g.num_queries_per_kv == 4 and repr(g) == "GroupedQueryAttention(num_heads=8, num_kv_heads=2)"
    with pytest.raises(AssertionError):
        GroupedQueryAttention(6, 4)
    mha = MultiHeadAttention(64, 4)
    assert repr(mha) == "MultiHeadAttention(embed_dim=64, num_heads=4, head_dim=16, dropout=0.0)"
    assert len(mha.parameters()) == 8 and len(MultiHeadAttention(64, 4, bias=False).parameters()) == 4
    with pytest.raises(ValueError):
        MultiHeadAttention(10, 3)


def test_tensor_round_trip_and_repeat_interleave_on_host():
    x = ts.Tensor(np.arange(24, dtype=np.float32).reshape(1, 2, 3, 4))
    assert x.shape == (1, 2, 3, 4) and x.tolist()[0][1][2][3] == 23.0
    r = x.repeat_interleave(2, dim=1).numpy()
    assert r.shape == (1, 4, 3, 4)
    assert np.array_equal(r[0, 0], r[0, 1]) and np.array_equal(r[0, 2], x.numpy()[0, 1])
    with pytest.raises(ValueError):
        ts.Tensor([1.0], device="tpu")


@pytest.mark.skipif(_lib.cuda_is_available(), reason="checks the no-device behaviour")
def test_workloads_cli_refuses_to_run_without_a_device():
    from tensorax_b200 import workloads
    with pytest.raises(RuntimeError, match="no CPU compute path"):
        workloads.main(["bwd", "--batch", "1", "--heads", "1", "--seq", "128", "--d", "64", "--iters", "1"])


def test_header_is_plain_c_and_links_from_a_c_program(tmp_path):
    """include/tensorax_b200.h compiles as C99 and a C program can link against the library."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    src = tmp_path / "probe.c"
    src.write_text(
        '#include <stdio.h>\n#include "tensorax_b200.h"\n'
        "int main(void) {\n"
        "    tx_sdpa_desc d = {0};\n    tx_sdpa_bwd_desc g = {0};\n"
        "    int rc = tx_sdpa_forward(&d);              /* null pointers: rejected before any device work */\n"
        "    int rb = tx_sdpa_backward(&g);\n"
        '    printf("%d %d %d %d\\n", tx_version() > 0, rc, rb, (int)sizeof(d));\n'
        "    return 0;\n}\n")
    exe = tmp_path / "probe"
    libdir = os.path.join(ROOT, "tensorax_b200", "csrc")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), str(src),
                    "-L", libdir, "-ltensorax_b200", "-Wl,-rpath," + libdir, "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out == ["1", "1", "1", str(ctypes.sizeof(_lib.SdpaDesc))]
