"""Multi-GPU partitioning: pure host logic, plus a world_size-2 gloo run of the sharded path on CPU tensors."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tinyfa_b200 import sharding as sh

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_fixed_config3_shapes():
    """batch 4 x 8 KV heads = 32 units over 1/2/4/8 GPUs (the GQA config of the benchmark plan)."""
    for world, (nb, nh) in {1: (4, 8), 2: (2, 8), 4: (1, 8), 8: (1, 4)}.items():
        plan = sh.plan_fixed(4, 8, world)
        assert len(plan) == world
        covered = []
        for s in plan:
            assert s.batch_end - s.batch_begin == nb and s.kv_head_end - s.kv_head_begin == nh
            covered += list(range(s.unit_begin, s.unit_end))
        assert covered == list(range(32))
    with pytest.raises(ValueError):
        sh.plan_fixed(3, 8, 5)


def test_slice_and_place_fixed_roundtrip():
    g = torch.Generator().manual_seed(0)
    Q = torch.randn(2, 5, 8, 16, generator=g)
    K = torch.randn(2, 7, 2, 16, generator=g)
    V = torch.randn(2, 7, 2, 16, generator=g)
    out = torch.zeros_like(Q)
    for s in sh.plan_fixed(2, 2, 4):
        q, k, v = sh.slice_fixed(Q, K, V, s)
        assert q.shape == (1, 5, 4, 16) and k.shape == (1, 7, 1, 16) and q.is_contiguous()
        sh.place_fixed(out, q, s, 4)
    assert torch.equal(out, Q)


def test_plan_varlen_balances_and_covers():
    rng = np.random.default_rng(0)
    lens = [int(x) for x in rng.integers(128, 8193, 16)]
    for world in (1, 2, 4, 8):
        plan = sh.plan_varlen(lens, lens, world, True)
        assert sorted(i for p in plan for i in p) == list(range(16))
        loads = [sum(sh.causal_cost(lens[i], lens[i], True) for i in p) for p in plan]
        assert max(loads) <= sum(loads) / world + max(sh.causal_cost(l, l, True) for l in lens)


def test_causal_cost_matches_mask_count():
    for lq, lkv in [(5, 9), (9, 5), (7, 7), (1, 1), (128, 32)]:
        brute = sum(1 for i in range(lq) for j in range(lkv) if j <= i)
        assert sh.causal_cost(lq, lkv, True) == brute
        assert sh.causal_cost(lq, lkv, False) == lq * lkv


def _naive(q, k, v, causal):
    """float64 attention on torch CPU tensors [B,S,H,D] (test-local helper)."""
    B, Sq, Hq, D = q.shape
    group = Hq // k.shape[2]
    out = torch.zeros(q.shape, dtype=torch.float64)
    for h in range(Hq):
        s = torch.einsum("bqd,bkd->bqk", q[:, :, h].double(), k[:, :, h // group].double()) / D ** 0.5
        if causal:
            i = torch.arange(Sq)[:, None]
            j = torch.arange(k.shape[1])[None, :]
            s = s.masked_fill(j > i, float("-inf"))
        out[:, :, h] = torch.einsum("bqk,bkd->bqd", torch.softmax(s, -1), v[:, :, h // group].double())
    return out


def _worker(rank, world, port, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(123)  # same inputs on every rank, sliced locally
    Q = torch.randn(2, 12, 4, 16, generator=g)
    K = torch.randn(2, 12, 2, 16, generator=g)
    V = torch.randn(2, 12, 2, 16, generator=g)
    shard = sh.plan_fixed(2, 2, world)[rank]
    q, k, v = sh.slice_fixed(Q, K, V, shard)
    o = _naive(q, k, v, True).float()
    # the single collective of the design: an all-gather of the outputs for the validation copy
    parts = [torch.zeros_like(o) for _ in range(world)]
    dist.all_gather(parts, o)
    if rank == 0:
        full = torch.zeros_like(Q)
        for s, part in zip(sh.plan_fixed(2, 2, world), parts):
            sh.place_fixed(full, part, s, 2)
        torch.save(full, tmp)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_shards_reassemble(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    out = str(tmp_path / "full.pt")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    full = torch.load(out)
    g = torch.Generator().manual_seed(123)
    Q = torch.randn(2, 12, 4, 16, generator=g)
    K = torch.randn(2, 12, 2, 16, generator=g)
    V = torch.randn(2, 12, 2, 16, generator=g)
    assert torch.allclose(full.double(), _naive(Q, K, V, True), atol=1e-6)


def test_slice_varlen_roundtrip():
    cu = [0, 3, 8, 10, 16]
    Q = torch.arange(16 * 2 * 4, dtype=torch.float32).reshape(16, 2, 4)
    plan = sh.plan_varlen([3, 5, 2, 6], [3, 5, 2, 6], 2, True)
    out = torch.zeros_like(Q)
    for ids in plan:
        q, k, v, lq, lkv = sh.slice_varlen(Q, Q, Q, cu, cu, ids)
        assert lq[-1] == q.shape[0] and lq == lkv
        sh.place_varlen(out, q, cu, ids)
    assert torch.equal(out, Q)
