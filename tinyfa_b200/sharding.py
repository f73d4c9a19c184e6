"""Host-side partitioning of one attention problem over the GPUs of a node.

The reference is a single-GPU library (its grid is (query tiles, batch, Q heads), reference
csrc/flash_attn/launcher.cuh:32) and has no multi-GPU code.  Attention forward has no exchange step:
every (batch, KV head) pair with the Q heads of its group, and every packed sequence, is independent
(reference csrc/flash_attn/params.cuh:138-141).  So the work is split into independent shards, each
shard is an ordinary API call on its own device, and outputs stay sharded; nothing here communicates.

Pure Python / torch indexing, no device code: usable (and tested) on CPU tensors.
"""
from dataclasses import dataclass
from typing import List, Sequence, Tuple


@dataclass(frozen=True)
class FixedShard:
    """A contiguous range of (batch, KV head) units: units [unit_begin, unit_end) of batch*heads_kv."""
    rank: int
    unit_begin: int
    unit_end: int
    batch_begin: int
    batch_end: int
    kv_head_begin: int  # within a batch entry; full range unless a batch entry is split across ranks
    kv_head_end: int


def plan_fixed(batch: int, heads_kv: int, world: int) -> List[FixedShard]:
    """Split batch*heads_kv units into `world` equal contiguous ranges.

    Requires that every rank's range is either whole batch entries or a head range inside one batch
    entry, so that its tensors stay dense [B', S, H', D]: world must divide batch*heads_kv, and either
    world divides batch or batch divides world.
    """
    units = batch * heads_kv
    if world <= 0 or units % world != 0:
        raise ValueError(f"world size {world} must divide batch*heads_kv = {units}")
    per = units // world
    if not (per % heads_kv == 0 or heads_kv % per == 0):
        raise ValueError("a shard must be whole batch entries or a head range inside one batch entry")
    shards = []
    for r in range(world):
        u0, u1 = r * per, (r + 1) * per
        if per % heads_kv == 0:
            shards.append(FixedShard(r, u0, u1, u0 // heads_kv, u1 // heads_kv, 0, heads_kv))
        else:
            b = u0 // heads_kv
            shards.append(FixedShard(r, u0, u1, b, b + 1, u0 % heads_kv, u0 % heads_kv + per))
    return shards


def slice_fixed(Q, K, V, shard: FixedShard):
    """Dense per-rank tensors for a FixedShard.  Q [B,Sq,Hq,D]; K,V [B,Skv,Hkv,D]."""
    heads_q, heads_kv = Q.shape[2], K.shape[2]
    group = heads_q // heads_kv
    b0, b1, h0, h1 = shard.batch_begin, shard.batch_end, shard.kv_head_begin, shard.kv_head_end
    q = Q[b0:b1, :, h0 * group:h1 * group, :].contiguous()
    k = K[b0:b1, :, h0:h1, :].contiguous()
    v = V[b0:b1, :, h0:h1, :].contiguous()
    return q, k, v


def place_fixed(O_full, o_shard, shard: FixedShard, group: int):
    """Write a rank's output back into the full [B,Sq,Hq,D] tensor (validation copy only)."""
    O_full[shard.batch_begin:shard.batch_end, :, shard.kv_head_begin * group:shard.kv_head_end * group, :] = o_shard


def causal_cost(len_q: int, len_kv: int, causal: bool) -> int:
    """Number of (query, key) pairs a sequence costs: top-left causal keeps key j <= query i."""
    if not causal:
        return len_q * len_kv
    full_rows = max(0, len_q - len_kv)       # rows i >= len_kv see every key
    tri = min(len_q, len_kv)
    return full_rows * len_kv + tri * (tri + 1) // 2


def plan_varlen(lens_q: Sequence[int], lens_kv: Sequence[int], world: int, causal: bool) -> List[List[int]]:
    """Assign sequences to ranks: longest-first greedy on the pair count.  Returns sequence indices per rank
    (each list sorted ascending, so a rank's packed tensors keep the original order)."""
    if len(lens_q) != len(lens_kv):
        raise ValueError("lens_q and lens_kv differ in length")
    if world <= 0:
        raise ValueError("world must be positive")
    order = sorted(range(len(lens_q)), key=lambda i: -causal_cost(lens_q[i], lens_kv[i], causal))
    load = [0] * world
    assign: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda x: (load[x], x))
        assign[r].append(i)
        load[r] += causal_cost(lens_q[i], lens_kv[i], causal)
    return [sorted(a) for a in assign]


def slice_varlen(Q, K, V, cu_q: Sequence[int], cu_kv: Sequence[int], seq_ids: Sequence[int]):
    """Packed per-rank tensors for the given sequences.  Returns q, k, v, cu_q_local, cu_kv_local (python lists)."""
    import torch

    q_parts, k_parts, v_parts = [], [], []
    lq, lkv = [0], [0]
    for i in seq_ids:
        q_parts.append(Q[cu_q[i]:cu_q[i + 1]])
        k_parts.append(K[cu_kv[i]:cu_kv[i + 1]])
        v_parts.append(V[cu_kv[i]:cu_kv[i + 1]])
        lq.append(lq[-1] + (cu_q[i + 1] - cu_q[i]))
        lkv.append(lkv[-1] + (cu_kv[i + 1] - cu_kv[i]))
    if not q_parts:
        empty_q, empty_k = Q[:0].contiguous(), K[:0].contiguous()
        return empty_q, empty_k, V[:0].contiguous(), lq, lkv
    return (torch.cat(q_parts).contiguous(), torch.cat(k_parts).contiguous(), torch.cat(v_parts).contiguous(), lq, lkv)


def place_varlen(O_full, o_shard, cu_q: Sequence[int], seq_ids: Sequence[int]):
    """Scatter a rank's packed output back into the full packed tensor (validation copy only)."""
    off = 0
    for i in seq_ids:
        n = cu_q[i + 1] - cu_q[i]
        O_full[cu_q[i]:cu_q[i + 1]] = o_shard[off:off + n]
        off += n


def attention_flops(batch: int, heads_q: int, seq_q: int, seq_kv: int, head_dim: int, causal: bool) -> float:
    """FLOP count used for every throughput figure (reference benchmarks/benchmark.py:31-33)."""
    f = 4.0 * batch * heads_q * seq_q * seq_kv * head_dim
    return f / 2 if causal else f


def varlen_flops(lens_q: Sequence[int], lens_kv: Sequence[int], heads_q: int, head_dim: int, causal: bool) -> float:
    return sum(attention_flops(1, heads_q, a, b, head_dim, causal) for a, b in zip(lens_q, lens_kv))
