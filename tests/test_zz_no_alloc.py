"""The allocation-free decode entry point against the regular one, through the C ABI.

Collected last on purpose (file name), so that a run stopping at the first failure has already run every other
test.  The entry point serves callers that may not let a library allocate device memory (engines that plan all of
it themselves, decode loops that cannot risk a stalling allocation); its split partials live in a fixed array of
the library instead of a stream-ordered allocation, so two calls in a row reuse - and overwrite - the same memory.
"""
import numpy as np
import pytest
import torch

import tinyfa_b200 as tf
from tinyfa_b200 import _lib

pytestmark = pytest.mark.gpu


def _inputs(B, Skv, Hq, Hkv, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn(B, 1, Hq, D, generator=g).to(dtype).cuda()
    K = torch.randn(B, Skv, Hkv, D, generator=g).to(dtype).cuda()
    V = torch.randn(B, Skv, Hkv, D, generator=g).to(dtype).cuda()
    return Q, K, V


def _noalloc(Q, K, V, causal, splits):
    lib = _lib.load()
    O = torch.full_like(Q, 3.0)
    B, Sq, Hq, D = Q.shape
    code = {torch.float16: 1, torch.bfloat16: 2}[Q.dtype]
    rc = lib.tfa_b200_fwd_decode_noalloc(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), code, B, Sq, K.shape[1],
                                         Hq, K.shape[2], D, int(causal), splits, torch.cuda.current_stream().cuda_stream)
    return rc, O


def test_two_calls_in_a_row_match_the_regular_entry_point():
    # second call has a different shape and split count: it must not see anything of the first call's partials
    for (B, Skv, Hq, Hkv, D, dtype, splits) in [(4, 3000, 32, 8, 128, torch.bfloat16, 5), (2, 1111, 8, 2, 64, torch.float16, 3)]:
        Q, K, V = _inputs(B, Skv, Hq, Hkv, D, dtype, seed=B)
        tf.set_option("split_kv", splits)
        try:
            expect = tf.flash_attn_forward(Q, K, V)
        finally:
            tf.set_option("split_kv", -1)
        rc, O = _noalloc(Q, K, V, False, splits)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert (O.float() - expect.float()).abs().max().item() <= 2e-2
        # and against fp64 directly
        ref = torch.softmax((Q[:, 0].double().view(B, Hkv, Hq // Hkv, D) @ K.double().permute(0, 2, 3, 1)) / D ** 0.5, -1) \
            @ V.double().permute(0, 2, 1, 3)
        assert (O[:, 0].double() - ref.reshape(B, Hq, D)).abs().max().item() <= 2e-2


def test_rejects_what_does_not_fit_or_does_not_apply():
    Q, K, V = _inputs(64, 512, 32, 8, 128, torch.bfloat16, seed=1)
    # 128 splits would need 128 * 64 * 32 * 129 floats = 33.8 M > 4 Mi: refused, nothing launched, O untouched
    rc, O = _noalloc(Q, K, V, False, 128)
    assert rc == 0, _lib.last_error()  # the split count is first clamped to seqLenKV / 64 = 8: 2.1 M floats, fits
    Q, K, V = _inputs(64, 8192, 64, 8, 128, torch.bfloat16, seed=2)
    rc, O = _noalloc(Q, K, V, False, 128)  # 128 * 64 * 64 * 129 floats: far beyond the array
    assert rc == 6 and "scratch" in _lib.last_error()
    torch.cuda.synchronize()
    assert torch.all(O == 3.0)
    # a long query block is not a decode shape
    g = torch.Generator().manual_seed(0)
    Ql = torch.randn(1, 64, 8, 128, generator=g).to(torch.bfloat16).cuda()
    Kl = torch.randn(1, 512, 8, 128, generator=g).to(torch.bfloat16).cuda()
    lib = _lib.load()
    Ol = torch.empty_like(Ql)
    rc = lib.tfa_b200_fwd_decode_noalloc(Ql.data_ptr(), Kl.data_ptr(), Kl.data_ptr(), Ol.data_ptr(), 2, 1, 64, 512, 8, 8,
                                         128, 0, 0, None)
    assert rc == 3


@pytest.mark.parametrize("case", [
    # (B, Sq, Skv, Hq, Hkv, D, dtype, causal, splits)
    (3, 1, 2000, 8, 2, 32, torch.float16, False, 0),     # the library picks the split count
    (2, 1, 900, 8, 2, 96, torch.bfloat16, False, 1),     # one split: no partials, the array is not touched
    (2, 3, 1500, 10, 2, 192, torch.bfloat16, True, 4),   # several query positions, causal
    (1, 2, 1024, 16, 2, 256, torch.float16, True, 3),
])
def test_other_shapes_and_no_device_memory_taken(case):
    """More of the shapes the entry point accepts, each against fp64, and the property it exists for: free device
    memory is the same before and after the call (first a warm-up call, so that one-time set-up is not counted)."""
    B, Sq, Skv, Hq, Hkv, D, dtype, causal, splits = case
    g = torch.Generator().manual_seed(B + D)
    Q = torch.randn(B, Sq, Hq, D, generator=g).to(dtype).cuda()
    K = torch.randn(B, Skv, Hkv, D, generator=g).to(dtype).cuda()
    V = torch.randn(B, Skv, Hkv, D, generator=g).to(dtype).cuda()
    rc, _ = _noalloc(Q, K, V, causal, splits)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    lib = _lib.load()
    O = torch.full_like(Q, 3.0)  # allocated before the measured call (torch's allocator may grow for it)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    code = {torch.float16: 1, torch.bfloat16: 2}[dtype]
    rc = lib.tfa_b200_fwd_decode_noalloc(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), code, B, Sq, Skv, Hq, Hkv,
                                         D, int(causal), splits, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    group = Hq // Hkv
    s = torch.einsum("bqhd,bkhd->bhqk", Q.double(), K.double().repeat_interleave(group, dim=2)) / D ** 0.5
    if causal:
        mask = torch.arange(Skv, device="cuda")[None, :] > torch.arange(Sq, device="cuda")[:, None]
        s.masked_fill_(mask, float("-inf"))
    ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), V.double().repeat_interleave(group, dim=2))
    assert (O.double() - ref).abs().max().item() <= 2e-2


def test_exact_fit_and_one_over_the_limit():
    """The partials of a call may fill the built-in array exactly; one row more is refused before anything launches."""
    limit = 4 * 1024 * 1024
    # the partials take splits * rows * (D + 1) floats; with D = 128 and 4 splits, 8128 rows (508 batch entries of 16
    # heads) need 4 194 048 floats, which fits, and 509 batch entries need 4 202 304, which does not
    D, splits = 128, 4
    rows_fit = limit // (splits * (D + 1))  # 8128
    assert splits * rows_fit * (D + 1) <= limit < splits * (rows_fit + 1) * (D + 1)
    Hq, Hkv = 16, 16
    for B, expect in ((rows_fit // Hq, 0), (rows_fit // Hq + 1, 6)):
        g = torch.Generator().manual_seed(3)
        Q = torch.randn(B, 1, Hq, D, generator=g).to(torch.bfloat16).cuda()
        K = torch.randn(B, 256, Hkv, D, generator=g).to(torch.bfloat16).cuda()
        rc, O = _noalloc(Q, K, K, False, splits)
        torch.cuda.synchronize()
        assert rc == expect, (B, rc, _lib.last_error())
        if expect == 6:
            assert torch.all(O == 3.0)
