"""Run one named SDPA workload through the C ABI on synthetic device-resident data and print its time.

    python -m tensorax_b200.workloads fwd --batch 4 --heads 8 --seq 4096 --d 256
    python -m tensorax_b200.workloads bwd --batch 2 --heads 8 --seq 4096 --d 128 --iters 2 --warmup 2

For shapes other than the benchmark's (bench.py measures BASELINE config 2 only) and for profiler
captures of one kernel: `--iters/--warmup` fix the number of launches, nothing else runs on the GPU.
Timing is host wall-clock around `iters` back-to-back launches and one `tx_sdpa_finish`.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import time

import numpy as np

from . import _lib


def _randn_f16(rng, n):
    return _lib.to_device(rng.standard_normal(n, dtype=np.float32).astype(np.float16))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["fwd", "bwd"])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=0, help="K/V heads (default: same as --heads)")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--out-f16", action="store_true", help="fp16 result (TX_SDPA_OUT_F16)")
    ap.add_argument("--fp32", action="store_true", help="float32 inputs: the exact-fp32 CUDA-core kernel (forward only)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    B, H, S, D = a.batch, a.heads, a.seq, a.d
    Hkv = a.kv_heads or H
    lib = _lib.load()
    if not lib.tx_cuda_is_available():
        raise RuntimeError("no CUDA device: this package has no CPU compute path")
    rng = np.random.default_rng(a.seed)
    nq, nk = B * H * S * D, B * Hkv * S * D
    if a.fp32:
        if a.what != "fwd":
            raise SystemExit("--fp32 is a forward workload")
        q, k, v = (_lib.to_device(rng.standard_normal(n, dtype=np.float32)) for n in (nq, nk, nk))
    else:
        q, k, v = _randn_f16(rng, nq), _randn_f16(rng, nk), _randn_f16(rng, nk)
    flags = _lib.TX_SDPA_OUT_F16 if a.out_f16 else 0
    out = _lib.DeviceBuffer(nq * (2 if a.out_f16 else 4))
    lse = _lib.DeviceBuffer(B * H * S * 4)
    fwd = _lib.SdpaDesc(q=q.ptr, k=k.ptr, v=v.ptr, mask=None, kv_lens=None, out=out.ptr, batch=B, q_heads=H,
                        kv_heads=Hkv, seq_q=S, seq_k=S, d_k=D, d_v=D,
                        dtype=_lib.TX_DTYPE_F32 if a.fp32 else _lib.TX_DTYPE_F16, causal=int(a.causal),
                        flags=flags, stream=None, lse=lse.ptr if a.what == "bwd" else None)
    visible = 0.5 * S * (S + 1) if a.causal else float(S) * S
    if a.what == "fwd":
        def launch():
            _lib.check(lib.tx_sdpa_forward(ctypes.byref(fwd)))
        flops = 4.0 * B * H * visible * D
    else:
        _lib.check(lib.tx_sdpa_forward(ctypes.byref(fwd)))
        _lib.check(lib.tx_sdpa_finish(None))
        g = _lib.to_device(rng.standard_normal(nq, dtype=np.float32))
        dq, dk, dv = _lib.DeviceBuffer(nq * 4), _lib.DeviceBuffer(nk * 4), _lib.DeviceBuffer(nk * 4)
        bwd = _lib.SdpaBwdDesc(q=q.ptr, k=k.ptr, v=v.ptr, out=out.ptr, dout=g.ptr, lse=lse.ptr, kv_lens=None,
                               dq=dq.ptr, dk=dk.ptr, dv=dv.ptr, batch=B, q_heads=H, kv_heads=Hkv, seq_q=S, seq_k=S,
                               d=D, causal=int(a.causal), flags=flags, stream=None)

        def launch():
            _lib.check(lib.tx_sdpa_backward(ctypes.byref(bwd)))
        flops = 10.0 * B * H * visible * D           # the rule's five GEMMs
    for _ in range(a.warmup):
        launch()
    _lib.check(lib.tx_sdpa_finish(None))
    t0 = time.perf_counter()
    for _ in range(a.iters):
        launch()
    _lib.check(lib.tx_sdpa_finish(None))
    ms = (time.perf_counter() - t0) / max(a.iters, 1) * 1e3
    print(json.dumps({"workload": f"{a.what} {'fp32' if a.fp32 else 'fp16'} B{B} Hq{H} Hkv{Hkv} S{S} d{D}" + (" causal" if a.causal else ""),
                      "ms": ms, "tflops_algorithmic": flops / (ms * 1e-3) / 1e12, "iters": a.iters,
                      "kernels_launched": int(lib.tx_kernel_launch_count())}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
