"""fp32, head dim 128: the 8 x 8 thread-tile kernel (the form large problems get) against the 4 x 8 kernel and the fp64
oracle, on shapes small enough to check every element (run with -m gpu)."""
import numpy as np
import pytest
import torch

import tinyfa_b200 as tf
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu

SHAPES = [  # batch, seqQ, seqKV, headsQ, headsKV
    (1, 128, 128, 1, 1),
    (1, 129, 257, 2, 1),
    (2, 300, 500, 4, 2),
    (1, 1000, 777, 3, 3),
    (1, 64, 1300, 2, 2),
    (1, 1, 130, 2, 1),
]


def _with_form(form, fn):
    tf.set_option("fp32_t8", form)
    try:
        out = fn()
        torch.cuda.synchronize()
        return out
    finally:
        tf.set_option("fp32_t8", 1)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_tile8_form_against_the_oracle_and_the_other_form(shape, causal):
    B, Sq, Skv, Hq, Hkv = shape
    rng = np.random.default_rng(31 + Sq + Skv)
    Q = rng.normal(0, 1, (B, Sq, Hq, 128)).astype(np.float32)
    K = rng.normal(0, 1, (B, Skv, Hkv, 128)).astype(np.float32)
    V = rng.normal(0, 1, (B, Skv, Hkv, 128)).astype(np.float32)
    Qd, Kd, Vd = (torch.from_numpy(x).cuda() for x in (Q, K, V))
    small = _with_form(0, lambda: tf.flash_attn_forward(Qd, Kd, Vd, is_causal=causal)).cpu().numpy()
    big = _with_form(2, lambda: tf.flash_attn_forward(Qd, Kd, Vd, is_causal=causal)).cpu().numpy()
    ref = ao.fixed(Q, K, V, causal, "f64")
    assert np.isfinite(big).all()
    assert np.abs(big - ref).max() <= 1e-4, (shape, causal)
    assert np.abs(big - small).max() <= 5e-6, (shape, causal)


def test_tile8_form_packed_input_with_poisoned_neighbours():
    lens_q, lens_kv = [17, 200, 64, 300], [40, 200, 150, 511]
    cu_q = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
    cu_kv = np.concatenate([[0], np.cumsum(lens_kv)]).astype(np.int32)
    rng = np.random.default_rng(9)
    Q = rng.normal(0, 1, (int(cu_q[-1]), 4, 128)).astype(np.float32)
    K = rng.normal(0, 1, (int(cu_kv[-1]), 2, 128)).astype(np.float32)
    V = rng.normal(0, 1, (int(cu_kv[-1]), 2, 128)).astype(np.float32)
    Kp, Vp = K.copy(), V.copy()
    for b in (1, 3):  # sequences 1 and 3 are poison; 0 and 2 must come out as if they held zeros
        Kp[cu_kv[b]:cu_kv[b + 1]] = np.nan
        Vp[cu_kv[b]:cu_kv[b + 1]] = np.inf
        K[cu_kv[b]:cu_kv[b + 1]] = 0
        V[cu_kv[b]:cu_kv[b + 1]] = 0
    cq, ck = torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_kv).cuda()
    out = _with_form(2, lambda: tf.flash_attn_varlen_forward(torch.from_numpy(Q).cuda(), torch.from_numpy(Kp).cuda(),
                                                             torch.from_numpy(Vp).cuda(), cq, ck, max(lens_q),
                                                             max(lens_kv), is_causal=True)).cpu().numpy()
    ref = ao.varlen(Q, K, V, cu_q, cu_kv, True, "f64")
    for b in (0, 2):
        rows = slice(int(cu_q[b]), int(cu_q[b + 1]))
        assert np.isfinite(out[rows]).all()
        assert np.abs(out[rows] - ref[rows]).max() <= 1e-4
    tf.device_status()
