"""Seeded random shapes through every kernel family, against the fp64 oracle (run with -m gpu).

The reference's suite fixes 180 shapes (reference tests/cpp/test_flash_attn.cu:350-655); this adds shapes it does not
have: sequence lengths around the 128-row tile and 128-key block edges, query and key lengths that differ, GQA
ratios up to 8, single-token queries, and packed batches with empty and one-row sequences.
"""
import numpy as np
import pytest
import torch

import cases
import tinyfa_b200 as tf
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu

DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
HEAD_DIMS = (32, 64, 96, 128, 192, 256)
EDGE_LENGTHS = (1, 2, 15, 17, 63, 64, 65, 127, 128, 129, 191, 255, 256, 257, 383, 385, 511, 513, 640, 769, 1025)


def _draw(rng):
    dtype = ("bf16", "fp16", "fp32")[int(rng.integers(0, 3))]
    D = HEAD_DIMS[int(rng.integers(0, 6))]
    hkv = int(rng.integers(1, 4))
    group = (1, 1, 2, 4, 8)[int(rng.integers(0, 5))]
    B = int(rng.integers(1, 4))
    sq = EDGE_LENGTHS[int(rng.integers(0, len(EDGE_LENGTHS)))]
    skv = EDGE_LENGTHS[int(rng.integers(0, len(EDGE_LENGTHS)))]
    causal = bool(rng.integers(0, 2))
    return dtype, B, sq, skv, hkv * group, hkv, D, causal


@pytest.mark.parametrize("seed", range(48))
def test_random_fixed_length_shapes(seed):
    rng = np.random.default_rng(1000 + seed)
    dtype, B, Sq, Skv, Hq, Hkv, D, causal = _draw(rng)
    Q = rng.normal(0, 1, (B, Sq, Hq, D)).astype(np.float32)
    K = rng.normal(0, 1, (B, Skv, Hkv, D)).astype(np.float32)
    V = rng.normal(0, 1, (B, Skv, Hkv, D)).astype(np.float32)
    Qd, Kd, Vd = (torch.from_numpy(x).to(DT[dtype]).cuda() for x in (Q, K, V))
    O = tf.flash_attn_forward(Qd, Kd, Vd, is_causal=causal)
    out = O.float().cpu().numpy()
    ref = ao.fixed(Qd.float().cpu().numpy(), Kd.float().cpu().numpy(), Vd.float().cpu().numpy(), causal, "f64")
    assert np.isfinite(out).all()
    err = np.abs(out - ref).max()
    assert err <= cases.MAXABS_TOL[dtype], (dtype, B, Sq, Skv, Hq, Hkv, D, causal, err)


@pytest.mark.parametrize("seed", range(24))
def test_random_packed_batches(seed):
    rng = np.random.default_rng(2000 + seed)
    dtype, _, _, _, Hq, Hkv, D, causal = _draw(rng)
    nseq = int(rng.integers(1, 6))
    pool = (0, 1, 3, 64, 127, 128, 129, 200, 256, 300, 513)
    sq = [pool[int(rng.integers(0, len(pool)))] for _ in range(nseq)]
    skv = [pool[int(rng.integers(0, len(pool)))] for _ in range(nseq)]
    if sum(sq) == 0:
        sq[0] = 5
    if sum(skv) == 0:
        skv[0] = 7
    cu_q = np.concatenate([[0], np.cumsum(sq)]).astype(np.int32)
    cu_kv = np.concatenate([[0], np.cumsum(skv)]).astype(np.int32)
    Q = rng.normal(0, 1, (int(cu_q[-1]), Hq, D)).astype(np.float32)
    K = rng.normal(0, 1, (int(cu_kv[-1]), Hkv, D)).astype(np.float32)
    V = rng.normal(0, 1, (int(cu_kv[-1]), Hkv, D)).astype(np.float32)
    Qd, Kd, Vd = (torch.from_numpy(x).to(DT[dtype]).cuda() for x in (Q, K, V))
    O = tf.flash_attn_varlen_forward(Qd, Kd, Vd, torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_kv).cuda(),
                                     max(sq), max(skv), is_causal=causal)
    out = O.float().cpu().numpy()
    ref = ao.varlen(Qd.float().cpu().numpy(), Kd.float().cpu().numpy(), Vd.float().cpu().numpy(), cu_q, cu_kv, causal,
                    "f64")
    assert np.isfinite(out).all()
    err = np.abs(out - ref).max()
    assert err <= cases.MAXABS_TOL[dtype], (dtype, sq, skv, Hq, Hkv, D, causal, err)


@pytest.mark.parametrize("seed", range(24))
def test_random_long_causal_gqa_and_small_head_dims(seed):
    """Shapes that reach the forms picked by the dispatcher for them: causal GQA with the group's heads interleaved
    into one tile (group sizes with and without a power-of-two part, lengths of several tiles), head dims 32 / 64 in
    one-tile CTAs, head dims 32 / 96 with MMAs of their own shape, the heaviest-first work order with more items than
    CTAs; packed batches through the C ABI with the totals left to the device (-1)."""
    from tinyfa_b200 import _lib

    rng = np.random.default_rng(3000 + seed)
    dtype = ("bf16", "fp16")[seed % 2]
    D = (32, 64, 96, 128, 192, 256)[seed % 6]
    group = (1, 2, 3, 4, 6, 8)[int(rng.integers(0, 6))]
    Hkv = int(rng.integers(1, 3))
    Hq = Hkv * group
    causal = bool(seed % 3)
    if seed % 4 != 3:
        B = int(rng.integers(1, 3))
        Sq = int(rng.integers(300, 1400))
        Skv = Sq if rng.integers(0, 2) else int(rng.integers(300, 1400))
        Q = rng.normal(0, 1, (B, Sq, Hq, D)).astype(np.float32)
        K = rng.normal(0, 1, (B, Skv, Hkv, D)).astype(np.float32)
        V = rng.normal(0, 1, (B, Skv, Hkv, D)).astype(np.float32)
        Qd, Kd, Vd = (torch.from_numpy(x).to(DT[dtype]).cuda() for x in (Q, K, V))
        O = tf.flash_attn_forward(Qd, Kd, Vd, is_causal=causal)
        ref = ao.fixed(Qd.float().cpu().numpy(), Kd.float().cpu().numpy(), Vd.float().cpu().numpy(), causal, "f64")
        what = (dtype, B, Sq, Skv, Hq, Hkv, D, causal)
    else:
        nseq = int(rng.integers(2, 5))
        sq = [int(rng.integers(1, 900)) for _ in range(nseq)]
        skv = [int(rng.integers(1, 900)) for _ in range(nseq)]
        cu_q = np.concatenate([[0], np.cumsum(sq)]).astype(np.int32)
        cu_kv = np.concatenate([[0], np.cumsum(skv)]).astype(np.int32)
        Q = rng.normal(0, 1, (int(cu_q[-1]), Hq, D)).astype(np.float32)
        K = rng.normal(0, 1, (int(cu_kv[-1]), Hkv, D)).astype(np.float32)
        V = rng.normal(0, 1, (int(cu_kv[-1]), Hkv, D)).astype(np.float32)
        Qd, Kd, Vd = (torch.from_numpy(x).to(DT[dtype]).cuda() for x in (Q, K, V))
        cq, ck = torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_kv).cuda()
        O = torch.zeros_like(Qd)
        code = {"fp16": 1, "bf16": 2}[dtype]
        rc = _lib.load().tfa_b200_fwd_varlen(Qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), O.data_ptr(), cq.data_ptr(),
                                             ck.data_ptr(), code, nseq, max(sq), max(skv), -1, -1, Hq, Hkv, D, int(causal),
                                             torch.cuda.current_stream().cuda_stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        ref = ao.varlen(Qd.float().cpu().numpy(), Kd.float().cpu().numpy(), Vd.float().cpu().numpy(), cu_q, cu_kv, causal,
                        "f64")
        what = (dtype, sq, skv, Hq, Hkv, D, causal)
    out = O.float().cpu().numpy()
    assert np.isfinite(out).all(), what
    err = np.abs(out - ref).max()
    assert err <= cases.MAXABS_TOL[dtype], (what, err)


def test_no_bounded_wait_gave_up_during_fuzzing():
    tf.device_status()
