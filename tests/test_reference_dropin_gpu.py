"""The reference's own Python package on top of this library.

``integration/Makefile`` builds the reference's unmodified pybind11 module (``csrc/tensor_ops.cpp``:
``TensorImpl``, the six SDPA dispatchers, ``cast_to_fp16``, the ``profile_sections_sdpa_*`` bindings)
with ``integration/shim.cpp`` in place of its attention kernels and CUDA glue, and lays the reference's
Python package out next to it under ``integration/_ref/`` (a built artefact, like an installed wheel).
These tests import THAT package -- the reference's ``Tensor``, ``functional`` and pybind dispatchers --
and run the reference's own call sequences (tests/test_sdpa_fp16.py:70-81, tests/test_attention.py), so
every result below went: reference Python -> reference pybind dispatcher -> shim -> this library's kernels.
Results are compared with the CPU oracle / the golden vectors written from the reference's ``sdpa_cpu``.
"""
import glob
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import FP16_ATOL, FP16_REL, FP32_ATOL, ROOT, seeded

REF_PKG_DIR = os.path.join(ROOT, "integration", "_ref")


def _module_built():
    return bool(glob.glob(os.path.join(REF_PKG_DIR, "tensorax", "_C*.so")))


def test_recipe_and_shim_are_committed():
    assert os.path.isfile(os.path.join(ROOT, "integration", "Makefile"))
    src = open(os.path.join(ROOT, "integration", "shim.cpp")).read()
    for name in ("sdpa_naive_cuda", "sdpa_tiled_cuda", "sdpa_flash_cuda", "sdpa_optimized_flash_cuda", "sdpa_mma_cuda",
                 "sdpa_mma_fp16_cuda", "cast_f32_to_f16_cuda", "cuda_malloc", "cuda_free", "cuda_memcpy_h2d",
                 "cuda_memcpy_d2h", "cuda_is_available", "sdpa_naive_profile_sections_cuda",
                 "sdpa_optimized_flash_profile_sections_cuda"):
        assert name in src, name


@pytest.mark.skipif(not _module_built(), reason="integration/_ref not built (needs the reference checkout: make -C integration REF=...)")
def test_reference_module_links_against_this_library():
    """CPU check: the built module's dynamic dependencies name libtensorax_b200.so, and every tensorax::
    launcher the dispatchers call is defined (the module imports without unresolved symbols)."""
    so = glob.glob(os.path.join(REF_PKG_DIR, "tensorax", "_C*.so"))[0]
    out = subprocess.run(["ldd", so], capture_output=True, text=True).stdout
    assert "libtensorax_b200.so" in out
    code = ("import sys; sys.path.insert(0, %r); import tensorax; from tensorax import _C; "
            "print(sorted(n for n in dir(_C) if 'sdpa' in n or 'scaled_dot' in n or n == 'cast_to_fp16'))" % REF_PKG_DIR)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr[-2000:]
    for name in ("scaled_dot_product_attention", "scaled_dot_product_attention_tiled", "scaled_dot_product_attention_flash",
                 "scaled_dot_product_attention_mma", "scaled_dot_product_attention_flash_optimized",
                 "scaled_dot_product_attention_mma_fp16", "cast_to_fp16", "profile_sections_sdpa_naive",
                 "profile_sections_sdpa_tiled", "profile_sections_sdpa_flash", "profile_sections_sdpa_mma",
                 "profile_sections_sdpa_flash_optimized"):
        assert name in proc.stdout, name


@pytest.fixture(scope="module")
def ref_ts():
    if not _module_built():
        pytest.fail("integration/_ref/tensorax/_C*.so is missing: build it with `make -C integration REF=<tensorax checkout>`")
    sys.path.insert(0, REF_PKG_DIR)
    try:
        import tensorax as ts
        import tensorax.functional as F
    finally:
        sys.path.remove(REF_PKG_DIR)
    assert os.path.realpath(ts.__file__).startswith(os.path.realpath(REF_PKG_DIR))
    assert ts.cuda_is_available(), "the reference package sees no CUDA device through the shim"
    return ts, F


def _to_np(t, shape):
    return np.asarray(t.cpu().tolist(), dtype=np.float32).reshape(shape)


@pytest.mark.gpu
@pytest.mark.parametrize("fn_name", ["scaled_dot_product_attention", "scaled_dot_product_attention_tiled",
                                     "scaled_dot_product_attention_flash", "scaled_dot_product_attention_mma",
                                     "scaled_dot_product_attention_flash_optimized"])
def test_reference_fp32_functions_on_config1(ref_ts, golden, fn_name):
    ts, F = ref_ts
    q, k, v = (ts.Tensor(golden[f"c1_{n}"], dtype="float32", device="cuda") for n in "qkv")
    out = getattr(F, fn_name)(q, k, v)
    assert out.device == "cuda" and tuple(out.shape) == golden["c1_out"].shape
    got = _to_np(out, golden["c1_out"].shape)
    assert float(np.abs(got - golden["c1_out"]).max()) <= FP32_ATOL


@pytest.mark.gpu
def test_reference_fp32_with_dense_mask(ref_ts, golden):
    ts, F = ref_ts
    q, k, v = (ts.Tensor(golden[f"mask_{n}"], dtype="float32", device="cuda") for n in "qkv")
    for mkey, okey in (("mask_m1e9", "mask_out1e9"), ("mask_mrand", "mask_outrand")):
        m = ts.Tensor(golden[mkey], dtype="float32", device="cuda")
        got = _to_np(F.scaled_dot_product_attention(q, k, v, mask=m), golden[okey].shape)
        assert float(np.abs(got - golden[okey]).max()) <= FP32_ATOL


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1, 1, 64, 64, 64, 64), (2, 4, 128, 128, 64, 64), (1, 2, 256, 256, 128, 128),
                                   (1, 1, 100, 164, 64, 64), (1, 1, 128, 128, 256, 256), (1, 1, 64, 128, 512, 512)])
def test_reference_fp16_flow(ref_ts, shape):
    """Tensor(..., device='cuda') -> F.cast_to_fp16 -> F.scaled_dot_product_attention_mma_fp16, the sequence of the
    reference's tests/test_sdpa_fp16.py:70-81, against the oracle on the fp16-rounded inputs."""
    import oracle
    ts, F = ref_ts
    B, H, Sq, Sk, dk, dv = shape
    q, k, v = seeded(21, B, H, Sq, dk), seeded(22, B, H, Sk, dk), seeded(23, B, H, Sk, dv)
    qh, kh, vh = (F.cast_to_fp16(ts.Tensor(x, dtype="float32", device="cuda")) for x in (q, k, v))
    assert qh.dtype == "float16"
    out = F.scaled_dot_product_attention_mma_fp16(qh, kh, vh)
    assert out.dtype == "float32" and out.device == "cuda"
    got = _to_np(out, (B, H, Sq, dv))
    r16 = lambda x: x.astype(np.float16).astype(np.float32)
    ref = oracle.sdpa_f32(r16(q), r16(k), r16(v))
    err = np.abs(got.astype(np.float64) - ref)
    assert float(err.max()) <= FP16_ATOL
    assert float(np.linalg.norm(err) / np.linalg.norm(ref)) <= FP16_REL


@pytest.mark.gpu
def test_reference_dispatcher_errors_survive(ref_ts):
    """Validation stays the reference's: its dispatcher rejects mismatched shapes before the shim is reached."""
    ts, F = ref_ts
    q = ts.Tensor(seeded(1, 1, 2, 8, 16), dtype="float32", device="cuda")
    k = ts.Tensor(seeded(2, 1, 2, 8, 32), dtype="float32", device="cuda")
    with pytest.raises(RuntimeError):
        F.scaled_dot_product_attention(q, k, k)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["naive", "tiled", "flash", "mma", "flash_optimized"])
def test_reference_profile_sections_bindings(ref_ts, name):
    """profile_sections_sdpa_* (csrc/tensor_ops.cpp:1434-1507): 32 clock64 stamps, increasing over the sections
    the kernel went through."""
    ts, F = ref_ts
    sys.path.insert(0, REF_PKG_DIR)
    try:
        from tensorax import _C
    finally:
        sys.path.remove(REF_PKG_DIR)
    q, k, v = (ts.Tensor(seeded(30 + i, 1, 2, 128, 64), dtype="float32", device="cuda") for i in range(3))
    ticks = getattr(_C, f"profile_sections_sdpa_{name}")(q._c_tensor, k._c_tensor, v._c_tensor)
    assert len(ticks) == 32
    used = ticks[:8]
    assert all(t > 0 for t in used) and all(b >= a for a, b in zip(used, used[1:])), used
    assert all(t == 0 for t in ticks[8:])
