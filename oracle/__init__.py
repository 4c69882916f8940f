"""ctypes front end of the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Two shared objects live beside this file, both built by ``oracle/Makefile``:

* ``liboracle.so`` -- the plain-C restatement of the reference CPU SDPA
  (``oracle/sdpa_oracle.c``, which cites tensorax ``csrc/cpu/tensor_cpu.cpp:464-529``).
* ``_ref/libtensorax_ref_cpu.so`` -- the reference's own ``sdpa_cpu`` compiled from
  the reference checkout, when that build was possible.

Nothing in the product package imports this module: it is used by the tests,
by the smoke check and by the benchmark's CPU legs, always as the checker or
as the CPU baseline, never as the thing being shipped or measured as "ours".
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libtensorax_ref_cpu.so")

_i64 = ctypes.c_int64
_fp = ctypes.c_void_p


def reference_root() -> str | None:
    """Where the reference checkout lies: $TENSORAX_REF, else a directory named `reference` beside this
    repository.  None when neither holds the reference's CPU source."""
    cands = [os.environ.get("TENSORAX_REF"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "csrc", "cpu", "tensor_cpu.cpp")):
            return c
    return None


def build(with_ref: bool | None = None, ref_root: str | None = None) -> None:
    """Compile the checkers.  ``with_ref=None`` builds the reference copy only
    when the reference checkout is present on this machine."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    ref_root = ref_root or reference_root()
    if with_ref is None:
        with_ref = ref_root is not None
    if with_ref:
        if ref_root is None:
            raise RuntimeError("reference checkout not found: set TENSORAX_REF")
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={ref_root}"], check=True,
                       capture_output=True)


_lib = None
_ref = None


def _oracle():
    global _lib
    if _lib is None:
        if not os.path.isfile(_ORACLE_SO):
            build(with_ref=False)
        _lib = ctypes.CDLL(_ORACLE_SO)
        _lib.oracle_sdpa_f32.argtypes = [_fp] * 5 + [_i64] * 6
        _lib.oracle_sdpa_f32.restype = None
        _lib.oracle_sdpa_structured.argtypes = (
            [_fp] * 4 + [_i64] * 7 + [ctypes.c_int, _fp] + [_i64] * 4)
        _lib.oracle_sdpa_structured.restype = None
        _lib.oracle_linear_f32.argtypes = [_fp] * 4 + [_i64] * 3
        _lib.oracle_linear_f32.restype = None
    return _lib


def have_reference() -> bool:
    return os.path.isfile(_REF_SO)


def _reference():
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(_REF_SO)
        _ref.ref_sdpa_cpu.argtypes = [_fp] * 5 + [_i64] * 6
        _ref.ref_sdpa_cpu.restype = None
        _ref.ref_matmul_cpu.argtypes = [_fp] * 3 + [_i64] * 4
        _ref.ref_matmul_cpu.restype = None
    return _ref


def _f32c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _dense(fn, q, k, v, mask):
    q, k, v = _f32c(q), _f32c(k), _f32c(v)
    B, H, Sq, dk = q.shape
    Sk, dv = k.shape[2], v.shape[3]
    m = None if mask is None else _f32c(mask)
    if m is not None:
        assert m.shape == (B, H, Sq, Sk), "dense mask must be [B,H,Sq,Sk] as the reference requires"
    out = np.empty((B, H, Sq, dv), dtype=np.float32)
    fn(_ptr(q), _ptr(k), _ptr(v), _ptr(m), _ptr(out), B, H, Sq, Sk, dk, dv)
    return out


def sdpa_f32(q, k, v, mask=None):
    """Restated oracle, same contract as the reference ``sdpa_cpu``."""
    return _dense(_oracle().oracle_sdpa_f32, q, k, v, mask)


def ref_sdpa_cpu(q, k, v, mask=None):
    """The reference's own ``sdpa_cpu`` (only where ``have_reference()``)."""
    return _dense(_reference().ref_sdpa_cpu, q, k, v, mask)


def sdpa_structured(q, k, v, causal=False, kv_lens=None, heads=None, rows=None, out=None,
                    threads: int = 1):
    """Oracle with implicit causal / key-length masks and grouped K/V heads.

    q: [B,Hq,Sq,dk]; k: [B,Hkv,Sk,dk]; v: [B,Hkv,Sk,dv] (any float dtype, widened
    to fp32 exactly).  ``heads`` = iterable of flattened b*Hq+h indices to evaluate
    (default all), ``rows`` = (begin, end) query-row range (default all).  Rows that
    are not evaluated are left as NaN in the returned array.
    """
    q, k, v = _f32c(q), _f32c(k), _f32c(v)
    B, Hq, Sq, dk = q.shape
    Hkv, Sk, dv = k.shape[1], k.shape[2], v.shape[3]
    assert Hq % Hkv == 0
    lens = None if kv_lens is None else np.ascontiguousarray(kv_lens, dtype=np.int32)
    if out is None:
        out = np.full((B, Hq, Sq, dv), np.nan, dtype=np.float32)
    r0, r1 = (0, Sq) if rows is None else rows
    head_list = list(range(B * Hq)) if heads is None else list(heads)
    lib = _oracle()

    def one(bh):
        lib.oracle_sdpa_structured(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, Hq, Hkv, Sq, Sk, dk,
                                   dv, int(bool(causal)), _ptr(lens), bh, bh + 1, r0, r1)

    if threads <= 1 or len(head_list) <= 1:
        for bh in head_list:
            one(bh)
    else:
        with ThreadPoolExecutor(max_workers=threads) as ex:
            list(ex.map(one, head_list))
    return out


def linear_f32(x, w, bias=None):
    """Restated F.linear: x [..., K] @ w[N, K].T + bias, reference accumulation order."""
    x, w = _f32c(x), _f32c(w)
    K, N = x.shape[-1], w.shape[0]
    rows = x.size // K
    b = None if bias is None else _f32c(bias)
    out = np.empty(x.shape[:-1] + (N,), dtype=np.float32)
    _oracle().oracle_linear_f32(_ptr(x), _ptr(w), _ptr(b), _ptr(out), rows, K, N)
    return out


def ref_linear(x, w, bias=None):
    """F.linear through the reference's own matmul_cpu (x @ w.T, then + bias)."""
    x, w = _f32c(x), _f32c(w)
    K, N = x.shape[-1], w.shape[0]
    rows = x.size // K
    wt = np.ascontiguousarray(w.T)
    out = np.empty(x.shape[:-1] + (N,), dtype=np.float32)
    _reference().ref_matmul_cpu(_ptr(x), _ptr(wt), _ptr(out), 1, rows, N, K)
    return out if bias is None else out + _f32c(bias)


def mha_forward_f32(query, key, value, params, num_heads, mask=None):
    """MultiHeadAttention.forward as the reference writes it (tensorax/nn/attention/layers.py:96-129),
    composed from the restated pieces: three projections, head split, SDPA, head merge, output
    projection.  `params` maps q/k/v/out _weight and _bias names to arrays (bias may be None)."""
    B, Sq, E = query.shape
    Sk = key.shape[1]
    dh = E // num_heads

    def split(t, S):
        return np.ascontiguousarray(t.reshape(B, S, num_heads, dh).transpose(0, 2, 1, 3))

    q = split(linear_f32(query, params["q_weight"], params.get("q_bias")), Sq)
    k = split(linear_f32(key, params["k_weight"], params.get("k_bias")), Sk)
    v = split(linear_f32(value, params["v_weight"], params.get("v_bias")), Sk)
    a = sdpa_f32(q, k, v, mask)
    merged = np.ascontiguousarray(a.transpose(0, 2, 1, 3)).reshape(B, Sq, E)
    return linear_f32(merged, params["out_weight"], params.get("out_bias"))


# ------------------------------------------------------------------ SDPA backward (numpy, float64)
# PARITY UNPINNED against the reference itself: its autograd rule (tensorax/tensor.py:806-827)
# cannot run there -- `key.transpose(-2, -1)` raises ValueError for negative dims
# (tensorax/tensor.py:963-964) and `_C.transpose_dims` is not bound -- and its tests hold no vector
# for it.  The restatement below follows that rule line by line in float64; tests/test_oracle.py pins
# it from the other side, against central differences of the (pinned) forward oracle.
def _visible(Sq, Sk, causal, kv_len):
    vis = np.ones((Sq, Sk), dtype=bool)
    if kv_len is not None:
        vis[:, max(int(kv_len), 0):] = False
    if causal:
        vis &= np.arange(Sk)[None, :] <= np.arange(Sq)[:, None]
    return vis


def sdpa_backward(q, k, v, dout, causal=False, kv_lens=None):
    """(dq, dk, dv, lse2) for out = softmax(q k^T / sqrt(d) + implicit mask) v.

    tensorax/tensor.py:811-827: scores = q k^T * scale (+ mask); attn = softmax(scores);
    dv = attn^T grad; d_attn = grad v^T; dot = sum(d_attn * attn, -1);
    d_scores = attn * (d_attn - dot) * scale; dq = d_scores k; dk = d_scores^T q.
    Grouped K/V heads: the gradients of one K/V head are summed over its query heads.
    lse2[b,h,i] = log2(sum_j 2^(scores_ij * log2(e))), the row statistic the device forward saves."""
    q, k, v, dout = (np.asarray(x, dtype=np.float64) for x in (q, k, v, dout))
    B, Hq, Sq, d = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    group = Hq // Hkv
    scale = 1.0 / np.sqrt(np.float64(d))
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    lse2 = np.zeros((B, Hq, Sq))
    for b in range(B):
        vis = _visible(Sq, Sk, causal, None if kv_lens is None else kv_lens[b])
        for h in range(Hq):
            g = h // group
            scores = (q[b, h] @ k[b, g].T) * scale
            scores = np.where(vis, scores, -np.inf)
            with np.errstate(invalid="ignore", divide="ignore"):
                m = scores.max(axis=-1, keepdims=True)
                e = np.exp(scores - m)
                s = e.sum(axis=-1, keepdims=True)
                attn = e / s
                lse2[b, h] = ((m + np.log(s)) * np.log2(np.e))[:, 0]
            dv[b, g] += attn.T @ dout[b, h]
            d_attn = dout[b, h] @ v[b, g].T
            dot = (d_attn * attn).sum(axis=-1, keepdims=True)
            d_scores = attn * (d_attn - dot) * scale
            dq[b, h] = d_scores @ k[b, g]
            dk[b, g] += d_scores.T @ q[b, h]
    return dq, dk, dv, lse2
