#!/usr/bin/env python3
"""Forward-attention benchmark with the reference's command line and protocol.

Same flags and defaults as the reference's benchmarks/benchmark.py (reference :182-213), and one more, --seqlens:

    python -m tinyfa_b200.benchmark
    python -m tinyfa_b200.benchmark --causal
    python -m tinyfa_b200.benchmark --head-dim 64 --dtype bf16
    python -m tinyfa_b200.benchmark --sweep          # all dtype x causal x head-dim
    python -m tinyfa_b200.benchmark --seqlens 4096   # a subset of the sequence lengths

Protocol as in the reference (:21-51): batch 2, 32 heads, sequence lengths 512..8192, 20 untimed and 40 timed
calls bracketed by CUDA events, the median reported; FLOPs = 4*B*H*S^2*D, halved when causal; timed through the
Python API, i.e. including the output allocation.  Before the table, one correctness line per configuration as in the
reference (:70-85): PASS / WARN on max-abs error < 0.05 against the baseline, with mean error and cosine similarity.
Baselines, when importable: Dao-AILab flash_attn (valid here because seqQ == seqKV, where its bottom-right causal
convention coincides with the top-left one) and torch SDPA - the same two the reference compares with (:59-67).
"""
import argparse
import statistics

import torch

import tinyfa_b200
from tinyfa_b200.sharding import attention_flops

PROTOCOL = {"batch": 2, "heads": 32, "seqlens": (512, 1024, 2048, 4096, 8192), "untimed": 20, "timed": 40}
TORCH_DTYPE = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
HEAD_DIMS = (32, 64, 96, 128, 192, 256)


class EventTimer:
    """Median device time of a callable: `untimed` calls first, then `timed` calls each between two CUDA events."""

    def __init__(self, untimed=PROTOCOL["untimed"], timed=PROTOCOL["timed"]):
        self.untimed, self.timed = untimed, timed

    def median_ms(self, call):
        for _ in range(self.untimed):
            call()
        torch.cuda.synchronize()
        samples = []
        for _ in range(self.timed):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            call()
            end.record()
            end.synchronize()
            samples.append(begin.elapsed_time(end))
        return statistics.median(samples)


def ours(Q, K, V, causal):
    return tinyfa_b200.flash_attn_forward(Q, K, V, is_causal=causal)


def _baseline(dtype):
    """(name, callable) of the comparison kernel: flash_attn for 16-bit types when installed, else torch SDPA."""
    if dtype != torch.float32:
        try:
            from flash_attn import flash_attn_func

            return "flash_attn", lambda Q, K, V, causal: flash_attn_func(Q, K, V, causal=causal)
        except Exception:
            pass

    def sdpa(Q, K, V, causal):  # SDPA wants [batch, heads, seq, dim]
        out = torch.nn.functional.scaled_dot_product_attention(Q.permute(0, 2, 1, 3), K.permute(0, 2, 1, 3),
                                                               V.permute(0, 2, 1, 3), is_causal=causal)
        return out.permute(0, 2, 1, 3)

    return "torch_sdpa", sdpa


def correctness_line(Q, K, V, causal, base_name, base_fn):
    """One line per configuration, like the reference prints before its table (reference :70-85)."""
    want = base_fn(Q, K, V, causal).float().flatten()
    got = ours(Q, K, V, causal).float().flatten()
    gap = (got - want).abs()
    worst, mean = gap.max().item(), gap.mean().item()
    cosine = (torch.dot(got, want) / (got.norm() * want.norm()).clamp_min(1e-30)).item()
    verdict = "PASS" if worst < 0.05 else "WARN"
    line = f"  [{verdict}] tinyfa vs {base_name}: max_err={worst:.6f}, mean_err={mean:.6f}, cos_sim={cosine:.6f}"
    print(line)
    return verdict, worst


def bench_config(dtype_name, head_dim, causal, seqlens=PROTOCOL["seqlens"], timer=None):
    timer = timer or EventTimer()
    dtype = TORCH_DTYPE[dtype_name]
    B, H = PROTOCOL["batch"], PROTOCOL["heads"]
    base_name, base_fn = _baseline(dtype)
    print(f"\n== dtype={dtype_name} head_dim={head_dim} causal={causal} batch={B} heads={H} (baseline: {base_name}) ==")
    rows = []
    for n, seqlen in enumerate(seqlens):
        gen = torch.Generator(device="cuda").manual_seed(seqlen)
        Q, K, V = (torch.randn(B, seqlen, H, head_dim, device="cuda", generator=gen).to(dtype) for _ in range(3))
        if n == 0:
            try:
                correctness_line(Q, K, V, causal, base_name, base_fn)
            except Exception as ex:  # the baseline does not take this configuration
                print(f"  [SKIP] no correctness line: {base_name} raised {type(ex).__name__}")
            print(f"{'seqlen':>8} {'ours ms':>10} {'ours TFLOPS':>12} {base_name + ' ms':>16} {base_name + ' TFLOPS':>18} "
                  f"{'speed-up':>9}")
        work = attention_flops(B, H, seqlen, seqlen, head_dim, causal)
        ms = timer.median_ms(lambda: ours(Q, K, V, causal))
        try:
            ms_base = timer.median_ms(lambda: base_fn(Q, K, V, causal))
            print(f"{seqlen:>8} {ms:>10.3f} {work / ms / 1e9:>12.2f} {ms_base:>16.3f} {work / ms_base / 1e9:>18.2f} "
                  f"{ms_base / ms:>8.2f}x")
        except Exception as ex:
            ms_base = None
            print(f"{seqlen:>8} {ms:>10.3f} {work / ms / 1e9:>12.2f} {'n/a':>16} {'n/a':>18} {'':>9} ({type(ex).__name__})")
        rows.append((seqlen, ms, work / ms / 1e9, ms_base))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description="attention forward benchmark (reference-compatible command line)")
    ap.add_argument("--dtype", default="fp16", choices=sorted(TORCH_DTYPE))
    ap.add_argument("--head-dim", type=int, default=128, choices=list(HEAD_DIMS))
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--sweep", action="store_true", help="all dtype x causal x head-dim combinations")
    ap.add_argument("--seqlens", type=int, nargs="+", default=list(PROTOCOL["seqlens"]))
    args = ap.parse_args(argv)
    torch.backends.cuda.matmul.allow_tf32 = False  # the comparison kernels stay in full fp32 where they compute in it
    torch.backends.cudnn.allow_tf32 = False
    print(f"device: {torch.cuda.get_device_name(0)}")
    if args.sweep:
        for dt in ("fp16", "bf16"):
            for causal in (False, True):
                for hd in HEAD_DIMS:
                    bench_config(dt, hd, causal, args.seqlens)
    else:
        bench_config(args.dtype, args.head_dim, args.causal, args.seqlens)


if __name__ == "__main__":
    main()
