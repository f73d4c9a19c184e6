"""Attention forward for tensors that live in (pinned) HOST memory.

The reference API only takes device tensors (reference csrc/binding/flash_attn_binding.cu:12,84-86); a caller whose
Q/K/V sit in host memory would copy three tensors in, call it, and copy the result out, with the GPU idle during the
copies and the PCIe link idle during the kernel.  This helper does the same work as that sequence but overlaps it:
the problem is cut into independent pieces (batch entries; for non-causal attention also blocks of query rows, whose
outputs depend on all keys but on no other query), each piece's host->device copies, kernel and device->host copy
run on three streams, so that copies of piece i+1 and the output copy of piece i-1 proceed while piece i computes.
Only contiguous slices are copied.  The result equals flash_attn_forward on the same values.
"""
import torch

from .api import flash_attn_forward

_streams = {}


def _get_streams(device):
    key = torch.device(device).index
    if key not in _streams:
        _streams[key] = (torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device))
    return _streams[key]


def flash_attn_forward_host(Q, K, V, is_causal=False, out=None, device=None, q_chunks=4):
    """Q [B,Sq,Hq,D], K/V [B,Skv,Hkv,D]: CPU tensors (pin them for asynchronous copies).  Returns `out`, a pinned
    CPU tensor shaped like Q (allocated if None).  The caller's current stream waits for the last output copy;
    synchronise that stream (or the device) before reading `out` on the host."""
    if Q.device.type != "cpu" or K.device.type != "cpu" or V.device.type != "cpu":
        raise RuntimeError("flash_attn_forward_host takes CPU tensors; use flash_attn_forward for device tensors")
    if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()):
        raise RuntimeError("Q, K, V must be contiguous")
    if Q.dim() != 4 or K.dim() != 4 or V.dim() != 4:
        raise RuntimeError("Q, K, V must be 4D [batch, seq, heads, headDim]")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if out is None:
        out = torch.empty(Q.shape, dtype=Q.dtype).pin_memory()
    B, Sq = Q.shape[0], Q.shape[1]
    n_q = 1 if (is_causal or Sq < 256 * q_chunks) else q_chunks  # a query-row block with top-left causal masking
    rows = (Sq + n_q - 1) // n_q                                   # would need a row offset the API does not have
    if B * n_q < 4:
        # too few independent pieces for the overlap to pay for its stream hand-offs (measured: 2 pieces are slower
        # than the plain sequence): copy in, run, copy out on the caller's stream
        with torch.cuda.device(dev):
            o = flash_attn_forward(Q.to(dev, non_blocking=True), K.to(dev, non_blocking=True),
                                   V.to(dev, non_blocking=True), is_causal=is_causal)
            out.copy_(o, non_blocking=True)
        return out
    s_in, s_run, s_out = _get_streams(dev)
    with torch.cuda.device(dev):
        cur = torch.cuda.current_stream()
        for s in (s_in, s_run, s_out):
            s.wait_stream(cur)
        keep = []
        for b in range(B):
            with torch.cuda.stream(s_in):
                k = K[b:b + 1].to(dev, non_blocking=True)
                v = V[b:b + 1].to(dev, non_blocking=True)
            for c in range(n_q):
                r0, r1 = c * rows, min(Sq, (c + 1) * rows)
                if r0 >= r1:
                    continue
                with torch.cuda.stream(s_in):
                    q = Q[b:b + 1, r0:r1].to(dev, non_blocking=True)
                    e_in = torch.cuda.Event()
                    e_in.record(s_in)
                with torch.cuda.stream(s_run):
                    s_run.wait_event(e_in)
                    o = flash_attn_forward(q, k, v, is_causal=is_causal)
                    e_run = torch.cuda.Event()
                    e_run.record(s_run)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(e_run)
                    out[b:b + 1, r0:r1].copy_(o, non_blocking=True)
                keep.append((q, k, v, o))
        # device buffers were allocated on side streams: make every stream that used them finish before the
        # caller's stream continues (and before the allocator may hand the memory out again)
        for s in (s_in, s_run, s_out):
            cur.wait_stream(s)
        for q, k, v, o in keep:
            for t in (q, k, v, o):
                t.record_stream(cur)
    return out
