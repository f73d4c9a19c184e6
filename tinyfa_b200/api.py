"""Python mirror of the reference's torch binding, on top of the C ABI.

Same function names, positional order, keyword names, defaults, checks and return contract as
`flash_attn_forward` / `flash_attn_varlen_forward` in the reference binding
(reference csrc/binding/flash_attn_binding.cu:80-117, 119-161, 163-172): every violated precondition
raises RuntimeError, the result is a new contiguous tensor shaped like Q, and the launch goes to
torch's current stream.  One addition: the call runs under a device guard for Q's device (the
reference launches on whichever device is current).
"""
import torch

from . import _lib

_DTYPE_CODE = {torch.float16: 1, torch.bfloat16: 2, torch.float32: 3}


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _check_input(x, name):
    _check(isinstance(x, torch.Tensor), f"{name} must be a torch.Tensor")
    _check(x.device.type == "cuda", f"{name} must be a CUDA tensor")
    _check(x.is_contiguous(), f"{name} must be contiguous")


def _dtype_code(t, fn):
    code = _DTYPE_CODE.get(t.dtype)
    _check(code is not None, f"{fn} only supports fp16, bf16 and fp32, got {t.dtype}")
    return code


def flash_attn_forward(Q, K, V, is_causal=False):
    """Fixed-length attention forward.  Q [B,Sq,Hq,D]; K,V [B,Skv,Hkv,D]; returns O like Q."""
    _check_input(Q, "Q")
    _check_input(K, "K")
    _check_input(V, "V")
    _check(Q.dim() == 4, "Q must be 4D [batch, seqQ, numHeadsQ, headDim]")
    _check(K.dim() == 4, "K must be 4D [batch, seqKV, numHeadsKV, headDim]")
    _check(V.dim() == 4, "V must be 4D [batch, seqKV, numHeadsKV, headDim]")
    _check(Q.dtype == K.dtype and Q.dtype == V.dtype, "Q, K, V must have the same dtype")
    batch, seq_q, heads_q, head_dim = Q.shape
    seq_kv, heads_kv = K.shape[1], K.shape[2]
    _check(K.shape[0] == batch and V.shape[0] == batch, "Batch sizes must match")
    _check(V.shape[1] == seq_kv, "K and V must have the same seqlen")
    _check(K.shape[3] == head_dim and V.shape[3] == head_dim, "Head dims must match")
    _check(V.shape[2] == heads_kv, "K and V must have the same number of heads")
    _check(heads_kv > 0 and heads_q % heads_kv == 0, "numHeadsQ must be divisible by numHeadsKV (GQA)")
    code = _dtype_code(Q, "flash_attn_forward")
    _check(K.device == Q.device and V.device == Q.device, "Q, K, V must be on the same device")

    lib = _lib.load()
    with torch.cuda.device(Q.device):
        # Every query row is written when there is at least one key, so the reference's zero fill
        # (binding:106) only matters for the degenerate shapes.
        O = torch.empty_like(Q) if (seq_kv > 0 and Q.numel() > 0) else torch.zeros_like(Q)
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.tfa_b200_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), code, batch, seq_q, seq_kv,
                              heads_q, heads_kv, head_dim, 1 if is_causal else 0, stream)
    _lib.check(rc, "flash_attn_forward")
    return O


def flash_attn_varlen_forward(Q, K, V, cu_seqlens_q, cu_seqlens_kv, max_seqlen_q, max_seqlen_kv, is_causal=False):
    """Packed variable-length forward.  Q [totalQ,Hq,D]; K,V [totalKV,Hkv,D]; cu_seqlens int32 [B+1] on the device."""
    _check_input(Q, "Q")
    _check_input(K, "K")
    _check_input(V, "V")
    _check_input(cu_seqlens_q, "cu_seqlens_q")
    _check_input(cu_seqlens_kv, "cu_seqlens_kv")
    _check(Q.dim() == 3, "Q must be 3D [totalQ, numHeadsQ, headDim]")
    _check(K.dim() == 3, "K must be 3D [totalKV, numHeadsKV, headDim]")
    _check(V.dim() == 3, "V must be 3D [totalKV, numHeadsKV, headDim]")
    _check(cu_seqlens_q.dim() == 1 and cu_seqlens_kv.dim() == 1, "cu_seqlens must be 1D")
    _check(cu_seqlens_q.dtype == torch.int32 and cu_seqlens_kv.dtype == torch.int32, "cu_seqlens must be int32")
    _check(Q.dtype == K.dtype and Q.dtype == V.dtype, "Q, K, V must have the same dtype")
    batch = cu_seqlens_q.shape[0] - 1
    heads_q, head_dim = Q.shape[1], Q.shape[2]
    heads_kv = K.shape[1]
    _check(K.shape[2] == head_dim and V.shape[2] == head_dim, "Head dims must match")
    _check(V.shape[1] == heads_kv, "K and V must have the same number of heads")
    _check(heads_kv > 0 and heads_q % heads_kv == 0, "numHeadsQ must be divisible by numHeadsKV (GQA)")
    _check(cu_seqlens_kv.shape[0] == batch + 1, "cu_seqlens_q and cu_seqlens_kv must have the same length")
    _check(V.shape[0] == K.shape[0], "K and V must have the same seqlen")
    code = _dtype_code(Q, "flash_attn_varlen_forward")
    _check(all(t.device == Q.device for t in (K, V, cu_seqlens_q, cu_seqlens_kv)),
           "Q, K, V and cu_seqlens must be on the same device")

    lib = _lib.load()
    with torch.cuda.device(Q.device):
        O = torch.zeros_like(Q)  # sequences without keys keep zeros (binding:148)
        if batch > 0:
            stream = torch.cuda.current_stream().cuda_stream
            rc = lib.tfa_b200_fwd_varlen(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(),
                                         cu_seqlens_q.data_ptr(), cu_seqlens_kv.data_ptr(), code, batch,
                                         int(max_seqlen_q), int(max_seqlen_kv), Q.shape[0], K.shape[0], heads_q,
                                         heads_kv, head_dim, 1 if is_causal else 0, stream)
            _lib.check(rc, "flash_attn_varlen_forward")
    return O


def is_head_dim_compiled(head_dim):
    """Mirror of tfa::isHeadDimCompiled (reference csrc/flash_attn/config.cuh:102-131)."""
    return bool(_lib.load().tfa_b200_head_dim_supported(int(head_dim)))


def device_status():
    """Synchronise the current device; raise RuntimeError if a kernel gave up on a bounded wait."""
    import ctypes

    site = ctypes.c_int(0)
    rc = _lib.load().tfa_b200_device_status(ctypes.byref(site))
    _lib.check(rc, "device_status")


def set_option(name, value):
    _lib.check(_lib.load().tfa_b200_set_option(name.encode(), int(value)), f"set_option({name})")
