"""Generates tests/golden/sdpa_golden.npz by running the REFERENCE's own CPU SDPA.

Run in a container that has the reference checkout (TENSORAX_REF=<path to it>):

    make -C oracle ref REF=$TENSORAX_REF && python tests/golden/make_golden.py

It calls ``tensorax::sdpa_cpu`` (csrc/cpu/tensor_cpu.cpp:464-529) through
oracle/_ref/libtensorax_ref_cpu.so -- the reference's source compiled where it
lies -- on seeded inputs, and stores inputs (or their seeds + checksums) and
outputs.  The GPU box has no reference checkout; the tests there read this file.

Cases
  c1_*          BASELINE config 1: B1 H2 S128 d64 fp32, N(0,1), no mask
  hand_*        the hand-written known-answer inputs of the reference's
                tests/test_attention.py:104-132,186-217 (values restated, outputs from sdpa_cpu)
  mask_*        dense additive masks: -1e9 causal (test_attention.py:79-102), -inf causal,
                a fully masked row (NaN row), random finite mask
  ragged_*      Sq != Sk, d_k != d_v, sizes that are no multiple of any tile
  f16_*         the small fp16 accuracy shapes of tests/test_sdpa_fp16.py:41-60; inputs are
                fp16-rounded N(0,1) widened to fp32, so the file pins what the fp16 kernels
                must reproduce within their tolerance
  gqa_*         grouped K/V heads + causal + key lengths, expressed the only way the
                reference can: K/V replicated head-wise (repeat_interleave semantics,
                csrc/tensor_ops.cpp:145-154) and a dense 0/-inf mask
  lin_*, mha_*  F.linear (tensorax/functional.py:105-110) through the reference's matmul_cpu, and
                MultiHeadAttention.forward (tensorax/nn/attention/layers.py:112-128) composed from the
                reference's matmul_cpu + sdpa_cpu (the reference cannot run that forward itself)
Large outputs are stored as sampled rows (`*_rows` gives the row indices).
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402


def seeded(seed, *shape):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal(shape, dtype=np.float32)


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest()[:8], dtype=np.uint64).copy()


def main():
    assert oracle.have_reference(), "build the reference copy first: make -C oracle ref"
    ref = oracle.ref_sdpa_cpu
    g = {}

    # ---- config 1
    q, k, v = seeded(101, 1, 2, 128, 64), seeded(102, 1, 2, 128, 64), seeded(103, 1, 2, 128, 64)
    g.update(c1_q=q, c1_k=k, c1_v=v, c1_out=ref(q, k, v))

    # ---- hand-written known-answer inputs
    hand = {
        "single_query": ([[[[1.0, 0.0]]]], [[[[1.0, 0.0], [0.0, 1.0]]]], [[[[1.0, 0.0], [0.0, 1.0]]]]),
        "pattern": ([[[[1.0, 0.0, 0.0, 0.0]]]],
                    [[[[1.0, 0.0, 0.0, 0.0], [0.0] * 4, [0.0] * 4]]],
                    [[[[10.0, 0.0, 0.0, 0.0], [0.0] * 4, [0.0] * 4]]]),
        "manual2x2": ([[[[1.0, 2.0], [3.0, 4.0]]]], [[[[5.0, 6.0], [7.0, 8.0]]]],
                      [[[[0.1, 0.2], [0.3, 0.4]]]]),
        "const100": (np.full((1, 1, 4, 4), 100.0), np.full((1, 1, 4, 4), 100.0),
                     np.full((1, 1, 4, 4), 100.0)),
    }
    for name, (q, k, v) in hand.items():
        q, k, v = (np.asarray(x, dtype=np.float32) for x in (q, k, v))
        g.update({f"hand_{name}_q": q, f"hand_{name}_k": k, f"hand_{name}_v": v,
                  f"hand_{name}_out": ref(q, k, v)})

    # ---- dense masks
    S = 12
    q, k, v = seeded(201, 2, 2, S, 8), seeded(202, 2, 2, S, 8), seeded(203, 2, 2, S, 8)
    tril = np.tril(np.ones((S, S), dtype=bool))
    m_1e9 = np.broadcast_to(np.where(tril, 0.0, -1e9).astype(np.float32), (2, 2, S, S)).copy()
    m_inf = np.broadcast_to(np.where(tril, 0.0, -np.inf).astype(np.float32), (2, 2, S, S)).copy()
    m_row = m_inf.copy()
    m_row[0, 1, 3, :] = -np.inf                      # a fully masked row -> NaN in the reference
    m_rand = seeded(204, 2, 2, S, S)
    g.update(mask_q=q, mask_k=k, mask_v=v, mask_m1e9=m_1e9, mask_minf=m_inf, mask_mrow=m_row,
             mask_mrand=m_rand, mask_out1e9=ref(q, k, v, m_1e9), mask_outinf=ref(q, k, v, m_inf),
             mask_outrow=ref(q, k, v, m_row), mask_outrand=ref(q, k, v, m_rand))

    # ---- ragged shapes
    for i, (B, H, Sq, Sk, dk, dv) in enumerate([(2, 2, 4, 6, 8, 8), (1, 2, 4, 8, 8, 8), (2, 3, 37, 75, 24, 40),
                                                (1, 1, 1, 130, 96, 520), (1, 2, 65, 33, 100, 7)]):
        q, k, v = seeded(300 + i, B, H, Sq, dk), seeded(310 + i, B, H, Sk, dk), seeded(320 + i, B, H, Sk, dv)
        g.update({f"ragged{i}_q": q, f"ragged{i}_k": k, f"ragged{i}_v": v, f"ragged{i}_out": ref(q, k, v)})

    # ---- fp16 accuracy shapes: inputs from seeds (checksummed), sampled output rows
    f16_shapes = [(1, 1, 64, 64, 64, 64), (1, 1, 80, 80, 64, 64), (1, 1, 128, 128, 64, 64),
                  (2, 4, 256, 256, 64, 64), (2, 4, 256, 256, 128, 128), (2, 4, 256, 256, 256, 256),
                  (2, 8, 256, 256, 512, 512)]
    g["f16_shapes"] = np.asarray(f16_shapes, dtype=np.int64)
    for i, (B, H, Sq, Sk, dk, dv) in enumerate(f16_shapes):
        q = seeded(400 + i, B, H, Sq, dk).astype(np.float16)
        k = seeded(420 + i, B, H, Sk, dk).astype(np.float16)
        v = seeded(440 + i, B, H, Sk, dv).astype(np.float16)
        out = ref(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32))
        rows = np.unique(np.concatenate([np.arange(0, Sq, max(Sq // 8, 1)), [Sq - 1]])).astype(np.int64)
        g.update({f"f16_{i}_digest": digest(q, k, v), f"f16_{i}_rows": rows,
                  f"f16_{i}_out": out[:, :, rows, :].astype(np.float32)})

    # ---- grouped heads + causal + key lengths through the reference's dense forms
    B, Hq, Hkv, S, d = 2, 4, 2, 96, 64
    q = seeded(501, B, Hq, S, d).astype(np.float16).astype(np.float32)
    k = (0.5 * seeded(502, B, Hkv, S, d)).astype(np.float16).astype(np.float32)
    v = (0.5 * seeded(503, B, Hkv, S, d)).astype(np.float16).astype(np.float32)
    lens = np.asarray([96, 61], dtype=np.int32)
    krep, vrep = np.repeat(k, Hq // Hkv, axis=1), np.repeat(v, Hq // Hkv, axis=1)
    vis = np.tril(np.ones((S, S), dtype=bool))[None, None] & (np.arange(S)[None, None, None, :] < lens[:, None, None, None])
    mask = np.broadcast_to(np.where(vis, 0.0, -np.inf).astype(np.float32), (B, Hq, S, S)).copy()
    g.update(gqa_q=q.astype(np.float16), gqa_k=k.astype(np.float16), gqa_v=v.astype(np.float16),
             gqa_lens=lens, gqa_out=ref(q, krep, vrep, mask))

    # ---- the linear layers either side of SDPA in MultiHeadAttention.forward, and the whole forward,
    #      composed from the reference's own matmul_cpu and sdpa_cpu exactly as layers.py:112-128 spells out
    x, w, b = seeded(601, 2, 9, 24), seeded(602, 10, 24), seeded(603, 10)
    g.update(lin_x=x, lin_w=w, lin_b=b, lin_out=oracle.ref_linear(x, w, b), lin_out_nobias=oracle.ref_linear(x, w))
    B, S, Sk, E, H = 2, 10, 13, 32, 4
    xq, xk, xv = seeded(611, B, S, E), seeded(612, B, Sk, E), seeded(613, B, Sk, E)
    std = np.float32(np.sqrt(2.0 / (E + E)))
    P = {n: seeded(620 + i, E, E) * std for i, n in enumerate(("q_weight", "k_weight", "v_weight", "out_weight"))}
    P.update({n: 0.1 * seeded(630 + i, E) for i, n in enumerate(("q_bias", "k_bias", "v_bias", "out_bias"))})

    def split(t, S_):
        return np.ascontiguousarray(t.reshape(B, S_, H, E // H).transpose(0, 2, 1, 3))

    q = split(oracle.ref_linear(xq, P["q_weight"], P["q_bias"]), S)
    k = split(oracle.ref_linear(xk, P["k_weight"], P["k_bias"]), Sk)
    v = split(oracle.ref_linear(xv, P["v_weight"], P["v_bias"]), Sk)
    a = np.ascontiguousarray(ref(q, k, v).transpose(0, 2, 1, 3)).reshape(B, S, E)
    g.update(mha_xq=xq, mha_xk=xk, mha_xv=xv, mha_out=oracle.ref_linear(a, P["out_weight"], P["out_bias"]),
             **{f"mha_{n}": arr for n, arr in P.items()})

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sdpa_golden.npz")
    np.savez_compressed(path, **g)
    print(path, os.path.getsize(path), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
