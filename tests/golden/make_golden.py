"""Generates tests/golden/ref_cpu_golden.npz from the REFERENCE's own CPU attention.

Run in a container where the reference checkout is mounted:
    make -C oracle ref_cpu && python tests/golden/make_golden.py
It feeds seeded inputs (numpy PCG64, uniform(-1, 1) like the reference tests' value range,
reference tests/cpp/test_flash_attn.cu:29-35) to tfa::test::cpuAttentionFixedLen / cpuAttentionVarLen
(reference tests/cpp/cpu_reference.h:14-66, 68-129, compiled unchanged behind oracle/ref_cpu_shim.cpp) and
stores only the outputs; the tests regenerate the inputs from the recorded seeds.  The case list restates
shapes of the reference's own suite (tests/cpp/test_flash_attn.cu:350-571), scaled down (fewer heads / batches) so that the
fixture stays a few hundred KB.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import attention_oracle as ao  # noqa: E402

# name, kind, dims, causal
FIXED = [
    ("basic_small", (1, 16, 16, 1, 1, 32), False),
    ("hd64_medium", (2, 32, 32, 2, 2, 64), False),
    ("hd96_causal", (1, 40, 40, 1, 1, 96), True),
    ("hd128_gqa_causal", (1, 24, 24, 4, 2, 128), True),
    ("hd192", (1, 20, 20, 1, 1, 192), False),
    ("hd256_causal_gqa", (1, 16, 16, 2, 1, 256), True),
    ("not_multiple_of_tile", (1, 67, 83, 1, 1, 64), False),
    ("primes", (1, 97, 101, 1, 1, 32), False),
    ("causal_q_longer_unaligned", (1, 97, 53, 1, 1, 64), True),
    ("causal_q_shorter", (1, 32, 128, 1, 1, 64), True),
    ("single_query", (2, 1, 16, 4, 4, 64), False),
    ("single_kv_token_causal", (2, 16, 1, 2, 2, 32), True),
    ("minimal", (1, 1, 1, 1, 1, 32), False),
    ("mqa_causal", (1, 24, 24, 8, 1, 32), True),
]
VARLEN = [
    ("varlen_basic", [32, 64, 48], [32, 64, 48], 1, 1, 32, False),
    ("varlen_unequal_causal_gqa", [16, 48, 24], [64, 96, 128], 4, 2, 32, True),
    ("varlen_not_aligned", [17, 53, 89], [23, 67, 101], 1, 1, 64, False),
    ("varlen_single_tokens", [1, 64, 1, 32], [1, 64, 1, 32], 1, 1, 64, False),
    ("varlen_q_longer_causal", [64, 128, 96], [32, 64, 48], 1, 1, 32, True),
    ("varlen_all_features_hd128", [33, 67, 51], [45, 89, 73], 2, 1, 64, True),
]


def inputs_fixed(seed, dims):
    B, Sq, Skv, Hq, Hkv, D = dims
    rng = np.random.default_rng(seed)
    Q = rng.uniform(-1, 1, (B, Sq, Hq, D)).astype(np.float32)
    K = rng.uniform(-1, 1, (B, Skv, Hkv, D)).astype(np.float32)
    V = rng.uniform(-1, 1, (B, Skv, Hkv, D)).astype(np.float32)
    return Q, K, V


def inputs_varlen(seed, sq, skv, Hq, Hkv, D):
    rng = np.random.default_rng(seed)
    cu_q = np.concatenate([[0], np.cumsum(sq)]).astype(np.int32)
    cu_kv = np.concatenate([[0], np.cumsum(skv)]).astype(np.int32)
    Q = rng.uniform(-1, 1, (int(cu_q[-1]), Hq, D)).astype(np.float32)
    K = rng.uniform(-1, 1, (int(cu_kv[-1]), Hkv, D)).astype(np.float32)
    V = rng.uniform(-1, 1, (int(cu_kv[-1]), Hkv, D)).astype(np.float32)
    return Q, K, V, cu_q, cu_kv


def main():
    assert ao.ref_cpu_available(), "build oracle/_ref/libtinyfa_refcpu.so first (make -C oracle ref_cpu)"
    arrays, meta = {}, []
    for i, (name, dims, causal) in enumerate(FIXED):
        seed = 1000 + i
        Q, K, V = inputs_fixed(seed, dims)
        arrays[name] = ao.ref_cpu_fixed(Q, K, V, causal)
        meta.append(dict(name=name, kind="fixed", dims=list(dims), causal=causal, seed=seed))
    for i, (name, sq, skv, Hq, Hkv, D, causal) in enumerate(VARLEN):
        seed = 2000 + i
        Q, K, V, cu_q, cu_kv = inputs_varlen(seed, sq, skv, Hq, Hkv, D)
        arrays[name] = ao.ref_cpu_varlen(Q, K, V, cu_q, cu_kv, causal)
        meta.append(dict(name=name, kind="varlen", sq=sq, skv=skv, Hq=Hq, Hkv=Hkv, D=D, causal=causal, seed=seed))
    np.savez_compressed(os.path.join(HERE, "ref_cpu_golden.npz"), **arrays)
    with open(os.path.join(HERE, "ref_cpu_golden.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print("wrote", len(meta), "cases,", os.path.getsize(os.path.join(HERE, "ref_cpu_golden.npz")), "bytes")


if __name__ == "__main__":
    main()
