#!/usr/bin/env python3
"""Forward-attention benchmark with the reference's command line and protocol.

Same flags, defaults and table as the reference's benchmarks/benchmark.py (reference :21-28, :182-213, :245-292):

    python -m tinyfa_b200.benchmark
    python -m tinyfa_b200.benchmark --causal
    python -m tinyfa_b200.benchmark --head-dim 64 --dtype bf16
    python -m tinyfa_b200.benchmark --sweep          # all dtype x causal x head-dim

Protocol as in the reference (:27-51): batch 2, 32 heads, sequence lengths 512..8192, 20 warm-up and 40 timed
calls with CUDA events, median; FLOPs = 4*B*H*S^2*D, halved when causal (:31-33); timed through the Python API,
i.e. including the output allocation.  Baselines, when importable: Dao-AILab flash_attn (valid here because seqQ ==
seqKV, where its bottom-right causal convention coincides with the top-left one) and torch SDPA - the same two the
reference compares with (:59-67).
"""
import argparse
import itertools

import torch
import torch.nn.functional as F

import tinyfa_b200

BATCH = 2
SEQLENS = [512, 1024, 2048, 4096, 8192]
NHEADS = 32
WARMUP = 20
REPEATS = 40
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def flops_fwd(batch, seqlen, nheads, headdim, causal=False):
    f = 4 * batch * nheads * seqlen * seqlen * headdim
    return f // 2 if causal else f


def benchmark_fn(fn, warmup=WARMUP, repeats=REPEATS):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def run_tinyfa(Q, K, V, causal):
    return tinyfa_b200.flash_attn_forward(Q, K, V, is_causal=causal)


def run_flash_attn_official(Q, K, V, causal):
    from flash_attn import flash_attn_func

    return flash_attn_func(Q, K, V, causal=causal)


def run_torch_sdpa(Q, K, V, causal):
    q, k, v = Q.transpose(1, 2), K.transpose(1, 2), V.transpose(1, 2)
    return F.scaled_dot_product_attention(q, k, v, is_causal=causal).transpose(1, 2)


def pick_baseline(dtype):
    if dtype != torch.float32:
        try:
            import flash_attn  # noqa: F401

            return "flash_attn", run_flash_attn_official
        except Exception:
            pass
    return "torch_sdpa", run_torch_sdpa


def bench_config(dtype_name, head_dim, causal):
    dtype = DTYPES[dtype_name]
    base_name, base_fn = pick_baseline(dtype)
    print(f"\n== dtype={dtype_name} head_dim={head_dim} causal={causal} batch={BATCH} heads={NHEADS} "
          f"(baseline: {base_name}) ==")
    print(f"{'seqlen':>8} {'ours ms':>10} {'ours TFLOPS':>12} {base_name + ' ms':>16} {base_name + ' TFLOPS':>18} "
          f"{'speed-up':>9} {'max err':>10}")
    for seqlen in SEQLENS:
        g = torch.Generator(device="cuda").manual_seed(seqlen)
        Q, K, V = (torch.randn(BATCH, seqlen, NHEADS, head_dim, device="cuda", dtype=torch.float32,
                               generator=g).to(dtype) for _ in range(3))
        fl = flops_fwd(BATCH, seqlen, NHEADS, head_dim, causal)
        ms = benchmark_fn(lambda: run_tinyfa(Q, K, V, causal))
        try:
            ms_b = benchmark_fn(lambda: base_fn(Q, K, V, causal))
            err = (run_tinyfa(Q, K, V, causal).float() - base_fn(Q, K, V, causal).float()).abs().max().item()
            print(f"{seqlen:>8} {ms:>10.3f} {fl / ms / 1e9:>12.2f} {ms_b:>16.3f} {fl / ms_b / 1e9:>18.2f} "
                  f"{ms_b / ms:>8.2f}x {err:>10.2e}")
        except Exception as ex:  # baseline does not support this configuration
            print(f"{seqlen:>8} {ms:>10.3f} {fl / ms / 1e9:>12.2f} {'n/a':>16} {'n/a':>18} {'':>9} ({type(ex).__name__})")


def main():
    ap = argparse.ArgumentParser(description="attention forward benchmark (reference-compatible command line)")
    ap.add_argument("--dtype", default="fp16", choices=sorted(DTYPES))
    ap.add_argument("--head-dim", type=int, default=128, choices=[32, 64, 96, 128, 192, 256])
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--sweep", action="store_true", help="all dtype x causal x head-dim combinations")
    args = ap.parse_args()
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    print(f"device: {torch.cuda.get_device_name(0)}")
    if args.sweep:
        for dt, causal, hd in itertools.product(["fp16", "bf16"], [False, True], [32, 64, 96, 128, 192, 256]):
            bench_config(dt, hd, causal)
    else:
        bench_config(args.dtype, args.head_dim, args.causal)


if __name__ == "__main__":
    main()
