"""Partition of one SDPA call over the GPUs of a box.

The path has no exchange step: one (batch, K/V-head) pair -- its K, its V and the
``q_heads // kv_heads`` query heads that read them -- is an independent unit.
Units are numbered b * kv_heads + kv_head, which is also their order in memory
for contiguous [B, H, S, d] tensors, so a contiguous range of units is a
contiguous slab of Q, of K, of V and of the output.  Each rank takes one such
range and runs the ordinary single-GPU kernel on it as a
[n_units, group, S, d] x [n_units, 1, S, d] problem.  No collective is involved.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    unit_begin: int      # first (batch, kv-head) unit of this rank
    unit_end: int        # one past the last
    group: int           # query heads per K/V head

    @property
    def n_units(self) -> int:
        return self.unit_end - self.unit_begin

    @property
    def q_head_begin(self) -> int:
        """First flattened query head (b * q_heads + h) of this rank."""
        return self.unit_begin * self.group

    @property
    def q_head_end(self) -> int:
        return self.unit_end * self.group


def partition(batch: int, kv_heads: int, q_heads: int, world: int, rank: int) -> Shard:
    """Contiguous, balanced split of the batch*kv_heads units: the first
    ``units % world`` ranks get one unit more."""
    if q_heads % kv_heads:
        raise ValueError("q_heads must be a multiple of kv_heads")
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    units = batch * kv_heads
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return Shard(rank, world, begin, end, q_heads // kv_heads)


def shard_arrays(shard: Shard, q, k, v, kv_lens: Optional[Sequence[int]] = None):
    """Views of this rank's slabs, reshaped to the local problem
    q [n, group, Sq, d_k], k [n, 1, Sk, d_k], v [n, 1, Sk, d_v], lens [n] or None."""
    B, Hq, Sq, dk = q.shape
    Hkv, Sk, dv = k.shape[1], k.shape[2], v.shape[3]
    n, g = shard.n_units, shard.group
    qf = q.reshape(B * Hkv, g, Sq, dk)[shard.unit_begin:shard.unit_end]
    kf = k.reshape(B * Hkv, 1, Sk, dk)[shard.unit_begin:shard.unit_end]
    vf = v.reshape(B * Hkv, 1, Sk, dv)[shard.unit_begin:shard.unit_end]
    lens = None
    if kv_lens is not None:
        per_unit = np.repeat(np.asarray(kv_lens, dtype=np.int32), Hkv)
        lens = np.ascontiguousarray(per_unit[shard.unit_begin:shard.unit_end])
    assert qf.shape[0] == n
    return qf, kf, vf, lens


def place_output(shard: Shard, full_out, local_out) -> None:
    """Write a rank's [n, group, Sq, d_v] result into the full [B, Hq, Sq, d_v] array."""
    B, Hq, Sq, dv = full_out.shape
    if not full_out.flags.c_contiguous:
        raise ValueError("place_output: the full array must be C-contiguous (a reshape of anything else is a copy, "
                         "and the rank's result would be written into that copy)")
    flat = full_out.reshape(B * Hq, Sq, dv)
    flat[shard.q_head_begin:shard.q_head_end] = local_out.reshape(-1, Sq, dv)


def shard_grad(shard: Shard, grad):
    """View of this rank's slab of the upstream gradient [B, Hq, Sq, d_v] as [n, group, Sq, d_v]
    (the backward pass shards exactly like the forward: a unit's dK / dV sum only over its own query heads)."""
    B, Hq, Sq, dv = grad.shape
    return grad.reshape(-1, shard.group, Sq, dv)[shard.unit_begin:shard.unit_end]


def place_kv_grad(shard: Shard, full_grad, local_grad) -> None:
    """Write a rank's [n, 1, Sk, d] dK or dV into the full [B, Hkv, Sk, d] array."""
    B, Hkv, Sk, d = full_grad.shape
    if not full_grad.flags.c_contiguous:
        raise ValueError("place_kv_grad: the full array must be C-contiguous")
    full_grad.reshape(B * Hkv, Sk, d)[shard.unit_begin:shard.unit_end] = local_grad.reshape(-1, Sk, d)
