"""Helpers of the GPU tests: call the C ABI with numpy inputs."""
import ctypes

import numpy as np

from tensorax_b200 import _lib


def sdpa_device(q, k, v, mask=None, causal=False, kv_lens=None, flags=0, dtype=None, repeats=1, want_lse=False):
    """Upload, run tx_sdpa_forward (+ tx_sdpa_finish), download.  q/k/v dtype picks
    the kernel family unless `dtype` says otherwise.  Returns (out, used_tensor_cores), or
    (out, lse, used_tensor_cores) with want_lse; TX_SDPA_OUT_F16 in flags gives a float16 `out`."""
    lib = _lib.load()
    if dtype is None:
        dtype = np.float16 if q.dtype == np.float16 else np.float32
    B, Hq, Sq, dk = q.shape
    Hkv, Sk, dv = k.shape[1], k.shape[2], v.shape[3]
    dq, dk_, dv_ = (_lib.to_device(np.ascontiguousarray(x, dtype=dtype)) for x in (q, k, v))
    out_np = np.float16 if flags & _lib.TX_SDPA_OUT_F16 else np.float32
    out = _lib.DeviceBuffer(B * Hq * Sq * dv * np.dtype(out_np).itemsize)
    lse = _lib.DeviceBuffer(B * Hq * Sq * 4) if want_lse else None
    dm = _lib.to_device(np.ascontiguousarray(mask, dtype=np.float32)) if mask is not None else None
    dl = _lib.to_device(np.ascontiguousarray(kv_lens, dtype=np.int32)) if kv_lens is not None else None
    desc = _lib.SdpaDesc(q=dq.ptr, k=dk_.ptr, v=dv_.ptr, mask=dm.ptr if dm else None,
                         kv_lens=dl.ptr if dl else None, out=out.ptr, batch=B, q_heads=Hq,
                         kv_heads=Hkv, seq_q=Sq, seq_k=Sk, d_k=dk, d_v=dv,
                         dtype=_lib.TX_DTYPE_F16 if dtype == np.float16 else _lib.TX_DTYPE_F32,
                         causal=int(causal), flags=flags, stream=None, lse=lse.ptr if lse else None)
    uses_tc = bool(lib.tx_sdpa_uses_tensor_cores(ctypes.byref(desc)))
    outs = []
    for _ in range(repeats):
        _lib.check(lib.tx_sdpa_forward(ctypes.byref(desc)))
        _lib.check(lib.tx_sdpa_finish(None))
        outs.append(out.download((B, Hq, Sq, dv), out_np))
    if want_lse:
        return outs[0], lse.download((B, Hq, Sq), np.float32), uses_tc
    return (outs[0] if repeats == 1 else outs), uses_tc


def sample_rows(Sq, n=6, extra=()):
    rows = set(np.linspace(0, Sq - 1, n).astype(int).tolist()) | {r for r in extra if 0 <= r < Sq}
    return sorted(rows)
