"""CPU suite for the multi-GPU partition: units are split contiguously, every
rank works on views only, and two gloo ranks reassemble the exact full result
(each rank evaluating its shard with the CPU oracle -- the partition logic, not
the kernel, is what runs here)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import oracle
from conftest import seeded
from tensorax_b200 import sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("B,Hkv,Hq", [(4, 8, 8), (8, 8, 32), (4, 16, 16), (3, 5, 10)])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_partition_is_contiguous_balanced_and_complete(B, Hkv, Hq, world):
    shards = [sharding.partition(B, Hkv, Hq, world, r) for r in range(world)]
    assert shards[0].unit_begin == 0 and shards[-1].unit_end == B * Hkv
    for a, b in zip(shards, shards[1:]):
        assert a.unit_end == b.unit_begin
    sizes = [s.n_units for s in shards]
    assert max(sizes) - min(sizes) <= 1
    assert sum(s.q_head_end - s.q_head_begin for s in shards) == B * Hq


def test_sharded_evaluation_equals_unsharded():
    B, Hq, Hkv, S, d = 3, 4, 2, 40, 16
    q, k, v = seeded(1, B, Hq, S, d), seeded(2, B, Hkv, S, d), seeded(3, B, Hkv, S, d)
    lens = [40, 17, 29]
    full = oracle.sdpa_structured(q, k, v, causal=True, kv_lens=lens)
    for world in (2, 4):
        out = np.full_like(full, np.nan)
        for r in range(world):
            sh = sharding.partition(B, Hkv, Hq, world, r)
            qs, ks, vs, ls = sharding.shard_arrays(sh, q, k, v, lens)
            assert qs.base is not None                     # views, not copies
            sharding.place_output(sh, out, oracle.sdpa_structured(qs, ks, vs, causal=True, kv_lens=ls))
        assert np.array_equal(out.view(np.uint32), full.view(np.uint32))


def test_sharded_backward_equals_unsharded():
    B, Hq, Hkv, S, d = 3, 4, 2, 24, 8
    q, k, v, g = seeded(1, B, Hq, S, d), seeded(2, B, Hkv, S, d), seeded(3, B, Hkv, S, d), seeded(4, B, Hq, S, d)
    lens = [24, 11, 17]
    fq, fk, fv, _ = oracle.sdpa_backward(q, k, v, g, causal=True, kv_lens=lens)
    for world in (2, 3):
        dq, dk, dv = (np.full(x.shape, np.nan) for x in (fq, fk, fv))
        for r in range(world):
            sh = sharding.partition(B, Hkv, Hq, world, r)
            qs, ks, vs, ls = sharding.shard_arrays(sh, q, k, v, lens)
            lq, lk, lv, _ = oracle.sdpa_backward(qs, ks, vs, sharding.shard_grad(sh, g), causal=True, kv_lens=ls)
            sharding.place_output(sh, dq, lq)
            sharding.place_kv_grad(sh, dk, lk)
            sharding.place_kv_grad(sh, dv, lv)
        assert np.array_equal(dq, fq) and np.array_equal(dk, fk) and np.array_equal(dv, fv)


_WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["TX_ROOT"]); sys.path.insert(0, os.path.join(os.environ["TX_ROOT"], "tests"))
import numpy as np, torch, torch.distributed as dist
import oracle
from conftest import seeded
from tensorax_b200 import sharding
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
B, Hq, Hkv, S, d = 2, 4, 2, 24, 8
q, k, v = seeded(11, B, Hq, S, d), seeded(12, B, Hkv, S, d), seeded(13, B, Hkv, S, d)
sh = sharding.partition(B, Hkv, Hq, world, rank)
qs, ks, vs, _ = sharding.shard_arrays(sh, q, k, v)
local = oracle.sdpa_structured(qs, ks, vs, causal=True)
dist.barrier()
# no data-path collective exists in the product; the gather below is only this test's check
parts = [None] * world
dist.all_gather_object(parts, (sh.unit_begin, sh.unit_end, local))
if rank == 0:
    out = np.full((B, Hq, S, d), np.nan, np.float32)
    for r, (b, e, loc) in enumerate(parts):
        sharding.place_output(sharding.partition(B, Hkv, Hq, world, r), out, loc)
    full = oracle.sdpa_structured(q, k, v, causal=True)
    assert np.array_equal(out.view(np.uint32), full.view(np.uint32))
    print("SHARD_OK")
dist.destroy_process_group()
"""


def test_two_gloo_ranks_reassemble_the_full_result(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, TX_ROOT=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "SHARD_OK" in proc.stdout


def test_placing_into_a_non_contiguous_array_is_refused():
    """A transposed view reshapes into a copy: the rank's result would vanish, so the helpers raise."""
    sh = sharding.partition(2, 2, 4, 2, 0)
    full = np.zeros((8, 4, 2, 4), dtype=np.float32).transpose(1, 2, 0, 3)      # [4, 2, 8, 4], not C-contiguous
    assert full.shape == (4, 2, 8, 4) and not full.flags.c_contiguous
    with pytest.raises(ValueError):
        sharding.place_output(sh, np.zeros((2, 4, 8, 4), np.float32).transpose(0, 1, 3, 2).transpose(0, 1, 3, 2)[:, :, ::-1],
                              np.zeros((sh.n_units, sh.group, 8, 4), np.float32))
    with pytest.raises(ValueError):
        sharding.place_kv_grad(sh, full[:2], np.zeros((sh.n_units, 1, 8, 4), np.float32))
