"""The CPU oracle against the reference's golden vectors (no GPU needed)."""
import json
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

from make_golden import inputs_fixed, inputs_varlen  # noqa: E402
from oracle import attention_oracle as ao  # noqa: E402

GOLD = np.load(os.path.join(HERE, "golden", "ref_cpu_golden.npz"))
META = json.load(open(os.path.join(HERE, "golden", "ref_cpu_golden.json")))


def _run(case, precision):
    if case["kind"] == "fixed":
        Q, K, V = inputs_fixed(case["seed"], tuple(case["dims"]))
        return ao.fixed(Q, K, V, case["causal"], precision)
    Q, K, V, cu_q, cu_kv = inputs_varlen(case["seed"], case["sq"], case["skv"], case["Hq"], case["Hkv"], case["D"])
    return ao.varlen(Q, K, V, cu_q, cu_kv, case["causal"], precision)


@pytest.mark.parametrize("case", META, ids=[c["name"] for c in META])
def test_port_f32_bit_exact_against_reference_golden(case):
    """The float variant follows the reference CPU code operation for operation: identical bits."""
    out = _run(case, "f32")
    gold = GOLD[case["name"]]
    assert out.dtype == np.float32 and out.shape == gold.shape
    assert np.array_equal(out, gold)


@pytest.mark.parametrize("case", META, ids=[c["name"] for c in META])
def test_port_f64_matches_reference_golden(case):
    """The double variant is the same mathematics: within fp32 rounding of the reference output."""
    out = _run(case, "f64")
    assert np.abs(out - GOLD[case["name"]].astype(np.float64)).max() <= 2e-6


@pytest.mark.skipif(not ao.ref_cpu_available(), reason="reference CPU library not built in this checkout")
@pytest.mark.parametrize("causal", [False, True])
def test_port_against_live_reference_cpu(causal):
    rng = np.random.default_rng(7)
    Q = rng.uniform(-1, 1, (2, 45, 6, 64)).astype(np.float32)
    K = rng.uniform(-1, 1, (2, 71, 2, 64)).astype(np.float32)
    V = rng.uniform(-1, 1, (2, 71, 2, 64)).astype(np.float32)
    assert np.array_equal(ao.fixed(Q, K, V, causal, "f32"), ao.ref_cpu_fixed(Q, K, V, causal))
    assert np.array_equal(ao.ref_cpu_fixed(Q, K, V, causal, threads=True), ao.ref_cpu_fixed(Q, K, V, causal))


def test_causal_is_top_left_aligned():
    """Key j is visible to query i iff j <= i, whatever Sq and Skv are (reference cpu_reference.h:29)."""
    rng = np.random.default_rng(1)
    Q = rng.standard_normal((1, 5, 1, 32)).astype(np.float32)
    K = rng.standard_normal((1, 9, 1, 32)).astype(np.float32)
    V = rng.standard_normal((1, 9, 1, 32)).astype(np.float32)
    O = ao.fixed(Q, K, V, True)
    # row 0 sees only key 0 -> output is V[0]
    assert np.allclose(O[0, 0, 0], V[0, 0, 0], atol=1e-6)
    # keys >= Sq never matter when Sq < Skv
    K2, V2 = K.copy(), V.copy()
    K2[:, 5:] = 99.0
    V2[:, 5:] = -99.0
    assert np.array_equal(ao.fixed(Q, K2, V2, True), O)
    # Sq > Skv: rows i >= Skv see every key, i.e. equal the non-causal result
    Ql = rng.standard_normal((1, 12, 1, 32)).astype(np.float32)
    assert np.allclose(ao.fixed(Ql, K, V, True)[:, 9:], ao.fixed(Ql, K, V, False)[:, 9:], atol=1e-12)


def test_gqa_head_map_and_varlen_equivalence():
    rng = np.random.default_rng(2)
    Q = rng.standard_normal((1, 20, 6, 32)).astype(np.float32)
    K = rng.standard_normal((1, 20, 2, 32)).astype(np.float32)
    V = rng.standard_normal((1, 20, 2, 32)).astype(np.float32)
    O = ao.fixed(Q, K, V, False)
    # consecutive Q heads share a KV head: hq // 3
    for hq in range(6):
        single = ao.fixed(Q[:, :, hq:hq + 1], K[:, :, hq // 3:hq // 3 + 1], V[:, :, hq // 3:hq // 3 + 1], False)
        assert np.allclose(O[:, :, hq:hq + 1], single, atol=1e-12)
    # packed varlen equals per-sequence fixed
    cu = np.array([0, 7, 20], dtype=np.int32)
    Ov = ao.varlen(Q[0], K[0], V[0], cu, cu, True)
    for s in range(2):
        a, b = cu[s], cu[s + 1]
        assert np.allclose(Ov[a:b], ao.fixed(Q[:, a:b], K[:, a:b], V[:, a:b], True)[0], atol=1e-12)


def test_empty_key_sequence_gives_zero():
    Q = np.ones((3, 2, 32), dtype=np.float32)
    K = np.ones((4, 2, 32), dtype=np.float32)
    cu_q = np.array([0, 1, 3], dtype=np.int32)
    cu_kv = np.array([0, 0, 4], dtype=np.int32)
    O = ao.varlen(Q, K, K, cu_q, cu_kv, False)
    assert np.all(O[0] == 0) and np.allclose(O[1:], 1.0)
