"""Head dims 192 / 256, CTA-pair form (clusters of two CTAs that share every K/V block through one MMA over both SMs)
against the one-tile form and the fp64 oracle (run with -m gpu).

The two forms do the same arithmetic in the same order, so their outputs must agree bit for bit; the one-tile form is
the one the reference's 180 restated cases and the fuzz families have pinned against the oracle.
"""
import numpy as np
import pytest
import torch

import cases
import tinyfa_b200 as tf
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu

DT = {"fp16": torch.float16, "bf16": torch.bfloat16}

# (batch, seqQ, seqKV, headsQ, headsKV): ragged lengths, a second tile that is partly or wholly past the end of the
# sequence, GQA groups (whose heads are interleaved into the tiles when causal), more items than there are CTA pairs
SHAPES = [
    (1, 129, 129, 1, 1),
    (1, 256, 256, 2, 2),
    (2, 300, 500, 2, 1),
    (1, 640, 1025, 6, 2),
    (3, 777, 1300, 4, 4),
    (4, 1024, 1024, 8, 8),
    (1, 2304, 2304, 4, 1),
]


def _both_forms(Q, K, V, causal):
    out = []
    try:
        for pair in (0, 1):
            tf.set_option("pair_cta", pair)
            out.append(tf.flash_attn_forward(Q, K, V, is_causal=causal))
        torch.cuda.synchronize()
    finally:
        tf.set_option("pair_cta", -1)
    return out


@pytest.mark.parametrize("D", [192, 256])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_pair_form_is_bit_identical_to_the_one_tile_form(shape, causal, dtype, D):
    B, Sq, Skv, Hq, Hkv = shape
    g = torch.Generator(device="cuda").manual_seed(7 + D + Sq)
    Q = torch.randn(B, Sq, Hq, D, generator=g, device="cuda").to(DT[dtype])
    K = torch.randn(B, Skv, Hkv, D, generator=g, device="cuda").to(DT[dtype])
    V = torch.randn(B, Skv, Hkv, D, generator=g, device="cuda").to(DT[dtype])
    single, pair = _both_forms(Q, K, V, causal)
    tf.device_status()
    assert torch.equal(single, pair), (shape, causal, dtype, D, (single.float() - pair.float()).abs().max().item())


@pytest.mark.parametrize("D", [192, 256])
@pytest.mark.parametrize("causal", [False, True])
def test_pair_form_against_the_fp64_oracle(causal, D):
    rng = np.random.default_rng(11 + D)
    B, Sq, Skv, Hq, Hkv = 2, 391, 700, 4, 2
    Q = rng.normal(0, 1, (B, Sq, Hq, D)).astype(np.float32)
    K = rng.normal(0, 1, (B, Skv, Hkv, D)).astype(np.float32)
    V = rng.normal(0, 1, (B, Skv, Hkv, D)).astype(np.float32)
    for dtype in ("fp16", "bf16"):
        Qd, Kd, Vd = (torch.from_numpy(x).to(DT[dtype]).cuda() for x in (Q, K, V))
        _, pair = _both_forms(Qd, Kd, Vd, causal)
        ref = ao.fixed(Qd.float().cpu().numpy(), Kd.float().cpu().numpy(), Vd.float().cpu().numpy(), causal, "f64")
        out = pair.float().cpu().numpy()
        assert np.isfinite(out).all()
        assert np.abs(out - ref).max() <= cases.MAXABS_TOL[dtype], (dtype, D, causal)


def test_pair_form_leaves_rows_past_the_output_alone_and_reports_no_timeout():
    """Guard band: the second CTA of the last pair owns rows past the end of a 129-row sequence and must store nothing."""
    D, Sq = 256, 129
    g = torch.Generator(device="cuda").manual_seed(3)
    Q = torch.randn(1, Sq, 2, D, generator=g, device="cuda").half()
    K = torch.randn(1, Sq, 2, D, generator=g, device="cuda").half()
    V = torch.randn(1, Sq, 2, D, generator=g, device="cuda").half()
    lib = tf._lib.load()
    buf = torch.full((Sq * 2 * D + 4096,), 7.0, device="cuda", dtype=torch.float16)
    O = buf[: Sq * 2 * D].view(1, Sq, 2, D)
    try:
        tf.set_option("pair_cta", 1)
        rc = lib.tfa_b200_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), 1, 1, Sq, Sq, 2, 2, D, 1,
                              torch.cuda.current_stream().cuda_stream)
        assert rc == 0, tf._lib.last_error()
        torch.cuda.synchronize()
    finally:
        tf.set_option("pair_cta", -1)
    assert (buf[Sq * 2 * D:] == 7.0).all()
    tf.device_status()


def test_pair_form_on_many_streams_and_in_a_replayed_graph():
    """Cluster launches take their work counters like every other launch: per stream, or per captured launch.  Forty
    streams with pair-form launches in flight and a captured pair-form launch replayed in between all give the bits
    of a launch that ran alone."""
    lib = tf._lib.load()
    B, Sq, Skv, Hq, Hkv, D = 1, 640, 640, 6, 6, 256
    g = torch.Generator(device="cuda").manual_seed(5)
    Q = torch.randn(B, Sq, Hq, D, generator=g, device="cuda").to(torch.bfloat16)
    K = torch.randn(B, Skv, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
    V = torch.randn(B, Skv, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)

    def launch(O, stream):
        return lib.tfa_b200_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), 2, B, Sq, Skv, Hq, Hkv, D, 1, stream)

    try:
        tf.set_option("pair_cta", 1)
        alone = torch.zeros_like(Q)
        assert launch(alone, torch.cuda.current_stream().cuda_stream) == 0, tf._lib.last_error()
        torch.cuda.synchronize()
        Og = torch.zeros_like(Q)
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                rc = launch(Og, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, tf._lib.last_error()
        streams = [torch.cuda.Stream() for _ in range(40)]
        outs = [torch.zeros_like(Q) for _ in range(80)]
        torch.cuda.synchronize()
        replay_stream = torch.cuda.Stream()
        for rep in range(2):
            for i, st in enumerate(streams):
                assert launch(outs[rep * 40 + i], st.cuda_stream) == 0, tf._lib.last_error()
                if i % 10 == 0:
                    with torch.cuda.stream(replay_stream):
                        graph.replay()
        torch.cuda.synchronize()
    finally:
        tf.set_option("pair_cta", -1)
    assert torch.equal(Og, alone)
    for O in outs:
        assert torch.equal(O, alone)
    tf.device_status()
