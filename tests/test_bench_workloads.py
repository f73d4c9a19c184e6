"""bench.py's workload table covers every benchmark configuration, with the FLOP counts of the measurement plan."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_every_benchmark_configuration_is_a_workload():
    w = bench.WORKLOADS
    assert bench.DEFAULT_WORKLOAD == "bf16_noncausal_b2_s4096_h32_d128"
    for dt in ("bf16", "fp16"):
        for causal in ("causal", "noncausal"):
            assert f"{dt}_{causal}_b2_s4096_h32_d128" in w
    assert "fp32_noncausal_b1_s128_h4_d64" in w
    assert "bf16_causal_gqa_b4_s8192_h32_8_d128" in w
    assert "bf16_causal_varlen_gqa_16seq_h32_8_d128" in w
    for hd in (32, 64, 96, 192, 256):
        assert f"fp16_causal_b8_s2048_h16_d{hd}" in w
    assert "bf16_decode_b64_skv32768_h32_8_d128" in w
    for name in bench.STRONG_WORKLOADS:
        assert name in w


def test_flop_counts_follow_the_reference_formula():
    """4*B*H*Sq*Skv*D, halved when causal (reference benchmarks/benchmark.py:31-33)."""
    w = bench.WORKLOADS
    assert bench.flops_of(w["bf16_noncausal_b2_s4096_h32_d128"]) == 4 * 2 * 32 * 4096 * 4096 * 128  # 549.76 GFLOP
    assert bench.flops_of(w["bf16_causal_b2_s4096_h32_d128"]) == 4 * 2 * 32 * 4096 * 4096 * 128 / 2
    assert bench.flops_of(w["bf16_causal_gqa_b4_s8192_h32_8_d128"]) == 4 * 4 * 32 * 8192 * 8192 * 128 / 2
    assert bench.flops_of(w["fp32_noncausal_b1_s128_h4_d64"]) == 4 * 1 * 4 * 128 * 128 * 64
    assert abs(bench.flops_of(w["fp16_causal_b8_s2048_h16_d32"]) - 1.0737e9 * 32) / (1.0737e9 * 32) < 1e-3


def test_packed_workload_lengths_are_the_seeded_ones():
    """16 lengths uniform in [128, 8192] from seed 0: the same draw as the full-size parity test uses."""
    w = bench.WORKLOADS["bf16_causal_varlen_gqa_16seq_h32_8_d128"]
    lens = bench.varlen_lengths(w)
    expect = [int(x) for x in np.random.default_rng(0).integers(128, 8193, 16)]
    assert lens == expect and len(lens) == 16 and min(lens) >= 128 and max(lens) <= 8192
    assert bench.flops_of(w, lens) == sum(4.0 * 32 * L * L * 128 for L in lens) / 2
    dead = bench.WORKLOADS["bf16_causal_varlen_gqa_1long_15short_h32_8_d128"]
    assert bench.varlen_lengths(dead) == [8192] + [128] * 15
