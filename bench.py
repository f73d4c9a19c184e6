#!/usr/bin/env python3
"""Benchmark of the attention-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one attention forward over one batch of synthetic input (seeded N(0,1), generated in fp32 and cast).
Default workload: bf16, non-causal, batch 2, seq 4096, 32 heads, head dim 128, layout [B,S,H,D] - the shape
the reference quotes its throughput on (reference README.md:56-64, benchmarks/benchmark.py:21-28).  FLOPs are
4*B*H*Sq*Skv*D, halved when causal (reference benchmarks/benchmark.py:31-33); packed variable-length input: the
sum of that over the sequences.  `--workload list` prints the names.

With N > 1 the script runs under torchrun, one rank per GPU; each rank processes its own independently seeded
batch of the same shape (weak scaling, no collective on the data path); time is the max over ranks.  The line then
also carries a `strong` block: the batch-4 GQA problem split by (batch x KV head) and the 16-sequence packed
problem split by sequence over the N ranks, each with its throughput, its speed-up over the unsplit problem on one
GPU, and the max-abs difference of the all-gathered shard outputs against the unsplit result (the one collective
of the design, outside the timed regions).

Prints ONE JSON line.  `value` is throughput with inputs resident in HBM, over the K bracketed steps; `e2e` is
the same metric through the public Python API with pinned HOST buffers (host->device copies of Q, K, V and
device->host copy of O inside the timed region; median of per-step times).  `roofline` holds the kernel alone
through the C ABI (median of per-launch CUDA-event times) against the measured burst peak, and in
`roofline.sustained` a back-to-back loop of at least 400 launches and 0.6 s against the measured sustained peak with the SM clock sampled
during that loop.  `--impl reference` runs the reference's own CUDA kernels (built for sm_100a from the
reference sources by oracle/Makefile) through the reference's tfa::flashAttn API on the same shape; if that
library was not built it times the reference's CPU attention instead and says so.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _fixed(dtype, causal, B, Sq, Skv, Hq, Hkv, D):
    return {"kind": "decode" if Sq == 1 else "fixed", "dtype": dtype, "causal": causal, "B": B, "Sq": Sq, "Skv": Skv,
            "Hq": Hq, "Hkv": Hkv, "D": D}


WORKLOADS = {
    "bf16_noncausal_b2_s4096_h32_d128": _fixed("bf16", False, 2, 4096, 4096, 32, 32, 128),
    "bf16_causal_b2_s4096_h32_d128": _fixed("bf16", True, 2, 4096, 4096, 32, 32, 128),
    "fp16_noncausal_b2_s4096_h32_d128": _fixed("fp16", False, 2, 4096, 4096, 32, 32, 128),
    "fp16_causal_b2_s4096_h32_d128": _fixed("fp16", True, 2, 4096, 4096, 32, 32, 128),
    "bf16_causal_gqa_b4_s8192_h32_8_d128": _fixed("bf16", True, 4, 8192, 8192, 32, 8, 128),
    # 16 packed sequences, lengths uniform in [128, 8192] from the seed, same length for Q and K/V
    "bf16_causal_varlen_gqa_16seq_h32_8_d128": {"kind": "varlen", "dtype": "bf16", "causal": True, "nseq": 16,
                                                "lo": 128, "hi": 8192, "seed": 0, "Hq": 32, "Hkv": 8, "D": 128},
    # one long sequence and fifteen short ones: a grid sized by the longest sequence is almost all dead tiles
    # (the reference launches them, reference csrc/flash_attn/launcher.cuh:98)
    "bf16_causal_varlen_gqa_1long_15short_h32_8_d128": {"kind": "varlen", "dtype": "bf16", "causal": True,
                                                        "lens": [8192] + [128] * 15, "Hq": 32, "Hkv": 8, "D": 128},
    # small shapes of the reference's own test and benchmark lists (reference tests/cpp/test_flash_attn.cu:388-420,
    # benchmarks/benchmark.py:23): launch- and latency-bound
    "bf16_causal_b2_s512_h32_d128": _fixed("bf16", True, 2, 512, 512, 32, 32, 128),
    "fp16_noncausal_b2_s128_h4_d64": _fixed("fp16", False, 2, 128, 128, 4, 4, 64),
    "fp16_causal_b8_s2048_h16_d32": _fixed("fp16", True, 8, 2048, 2048, 16, 16, 32),
    "fp16_causal_b8_s2048_h16_d64": _fixed("fp16", True, 8, 2048, 2048, 16, 16, 64),
    "fp16_causal_b8_s2048_h16_d96": _fixed("fp16", True, 8, 2048, 2048, 16, 16, 96),
    "fp16_causal_b8_s2048_h16_d192": _fixed("fp16", True, 8, 2048, 2048, 16, 16, 192),
    "fp16_causal_b8_s2048_h16_d256": _fixed("fp16", True, 8, 2048, 2048, 16, 16, 256),
    # the same sizes without the mask: the CTA-pair form of head dim 256 with every key block a full one
    "fp16_noncausal_b8_s2048_h16_d256": _fixed("fp16", False, 8, 2048, 2048, 16, 16, 256),
    # fp32 runs on the CUDA cores (no TF32): the small known-answer shape and a throughput shape
    "fp32_noncausal_b1_s128_h4_d64": _fixed("fp32", False, 1, 128, 128, 4, 4, 64),
    "fp32_noncausal_b2_s4096_h32_d128": _fixed("fp32", False, 2, 4096, 4096, 32, 32, 128),
    # decode shapes are HBM-bound: reported in GB/s of K+V read once
    "bf16_decode_b64_skv32768_h32_8_d128": _fixed("bf16", False, 64, 1, 32768, 32, 8, 128),
    "bf16_decode_b8_skv32768_h32_8_d128": _fixed("bf16", False, 8, 1, 32768, 32, 8, 128),
    "bf16_decode_b1_skv32768_h32_8_d128": _fixed("bf16", False, 1, 1, 32768, 32, 8, 128),
}
DEFAULT_WORKLOAD = "bf16_noncausal_b2_s4096_h32_d128"
STRONG_WORKLOADS = ("bf16_causal_gqa_b4_s8192_h32_8_d128", "bf16_causal_varlen_gqa_16seq_h32_8_d128")
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
# (decode batch 64: the batch-8 capture scaled by units processed; traffic grows in proportion to batch).
NCU_TRAFFIC_BYTES = {
    "bf16_noncausal_b2_s4096_h32_d128": 247334144,
    "bf16_causal_b2_s4096_h32_d128": 266387456,
    "bf16_causal_varlen_gqa_16seq_h32_8_d128": 1342815744,
    "bf16_causal_gqa_b4_s8192_h32_8_d128": 644488192,
    "fp16_causal_b8_s2048_h16_d64": 114779392,
    "fp16_causal_b8_s2048_h16_d32": 52913664,
    "fp16_causal_b8_s2048_h16_d96": 184531200,
    "fp16_causal_b8_s2048_h16_d192": 386672128,
    "fp16_causal_b8_s2048_h16_d256": 524141824,
    "fp32_noncausal_b2_s4096_h32_d128": 519461120,
    "bf16_decode_b8_skv32768_h32_8_d128": 1078060032,
    "bf16_decode_b64_skv32768_h32_8_d128": 8624480256,
}
FALLBACK_PEAK_TFLOPS = 1590.0  # earlier measurement on this pool, used only when MEASURED_PEAKS.json is absent
ESIZE = {"bf16": 2, "fp16": 2, "fp32": 4}


def varlen_lengths(w):
    import numpy as np

    if "lens" in w:
        return list(w["lens"])
    rng = np.random.default_rng(w["seed"])
    return [int(x) for x in rng.integers(w["lo"], w["hi"] + 1, w["nseq"])]


def flops_of(w, lens=None):
    if w["kind"] == "varlen":
        f = sum(4.0 * w["Hq"] * L * L * w["D"] for L in lens)
    else:
        f = 4.0 * w["B"] * w["Hq"] * w["Sq"] * w["Skv"] * w["D"]
    return f / 2 if w["causal"] else f


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs (read-only query)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, since=None):
        """Summary of the samples (taken after `since`, a time.perf_counter() value, when given)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        return self.summary(since)

    def summary(self, since=None, until=None):
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in list(self.lines):
            if (since is not None and ts < since) or (until is not None and ts > until):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return None


def measured_peak():
    p = _peaks()
    if p and "bf16_tflops" in p:
        return float(p["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return FALLBACK_PEAK_TFLOPS, "fallback"


def measured_sustained_peak():
    p = _peaks()
    if p and "bf16_tflops_sustained" in p:
        return float(p["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return 1400.0, "fallback"


def measured_hbm():
    p = _peaks()
    if p and "hbm_gbs" in p:
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, copy)"
    return 6650.0, "fallback"


def fp32_fma_peak():
    """fp32 FMA peak of the CUDA cores: SMs x 128 lanes x 2 FLOP x max SM clock (nominal; no measured figure)."""
    p = _peaks()
    mhz = float(p["sm_max_mhz"]) if p and "sm_max_mhz" in p else 1965.0
    return 148 * 128 * 2 * mhz * 1e6 / 1e12, "nominal: 148 SMs x 128 fp32 lanes x 2 x %.0f MHz" % mhz


def cpu_baseline(w, target_seconds=12.0):
    """Naive fp32 attention on the host cores on a bounded sample of the workload: the first q_rows query rows of
    every (batch, head).  Uses the reference's own cpu_reference.h when it was compiled here, else the port.
    Packed variable-length workloads are sampled as one fixed-length problem of their longest sequence."""
    import numpy as np

    from oracle import attention_oracle as ao

    if w["kind"] == "varlen":
        L = max(varlen_lengths(w))
        w = _fixed(w["dtype"], w["causal"], 1, L, L, w["Hq"], w["Hkv"], w["D"])
    causal, B, Sq, Skv, Hq, Hkv, D = w["causal"], w["B"], w["Sq"], w["Skv"], w["Hq"], w["Hkv"], w["D"]
    if w["kind"] == "decode":  # bound the memory: a slice of the batch and of the keys
        B, Skv = min(B, 4), min(Skv, 8192)
    rng = np.random.default_rng(0)
    Q = rng.standard_normal((B, Sq, Hq, D), dtype=np.float32)
    K = rng.standard_normal((B, Skv, Hkv, D), dtype=np.float32)
    V = rng.standard_normal((B, Skv, Hkv, D), dtype=np.float32)
    use_ref = ao.ref_cpu_available()

    # Sample = the first `rows` query rows of every (batch, head).  Non-causal: against all keys.  Causal: against the
    # first `rows` keys, i.e. the same workload at sequence length `rows` (rows beyond the diagonal are masked anyway);
    # FLOPs are counted like the metric does (halved), although the reference CPU code still evaluates exp and P.V
    # over every key of a row.
    def run(rows):
        Kc, Vc = (np.ascontiguousarray(K[:, :rows]), np.ascontiguousarray(V[:, :rows])) if causal else (K, V)
        t0 = time.perf_counter()
        if use_ref:
            ao.ref_cpu_fixed(Q, Kc, Vc, causal, threads=True, q_rows=rows)
        else:
            ao.fixed(Q, Kc, Vc, causal, "f32", q_rows=rows)
        return time.perf_counter() - t0

    def sample_flops(rows):
        if not causal:
            return 4.0 * B * Hq * rows * Skv * D
        pairs = sum(min(i + 1, min(rows, Skv)) for i in range(rows))
        return 4.0 * B * Hq * pairs * D

    # Grow the sample geometrically, re-measuring every time: a causal sample of the FIRST rows has so little work per
    # row at the start that a rate taken from a small probe would badly under-estimate what the cores can do.
    rows = min(32, Sq)
    t = run(rows)
    while rows < Sq:
        nxt = min(rows * 2, Sq)
        predicted = t * sample_flops(nxt) / max(sample_flops(rows), 1.0)
        if t >= target_seconds / 3 or predicted > 1.5 * target_seconds:
            break
        rows = nxt
        t = run(rows)
    cores = ao.ref_cpu().tfa_refcpu_num_threads() if use_ref else ao.num_threads()
    return {"value": sample_flops(rows) / t / 1e12, "unit": "TFLOP/s", "cores": int(cores),
            "kind": "reference" if use_ref else "port",
            "sample": (f"B{B} Hq{Hq} Hkv{Hkv} D{D}: first {rows} of {Sq} query rows of every (batch, head), "
                       + (f"first {min(rows, Skv)} keys (causal sub-problem)" if causal else f"all {Skv} keys")
                       + f"; {t:.1f} s; fp32 naive")}


class Problem:
    """One attention problem on one device: tensors, the three ways of running a step, and its FLOP count."""

    def __init__(self, w, dev, impl, seed, torch, shard=None, world=1, rank=0, host_inputs=True):
        self.w, self.dev, self.impl, self.torch = w, dev, impl, torch
        self.dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[w["dtype"]]
        self.code = {"fp16": 1, "bf16": 2, "fp32": 3}[w["dtype"]]
        self.causal = w["causal"]
        self.kind = w["kind"]
        self.host = None
        self.shard = shard
        from oracle import attention_oracle as ao  # only the reference legs execute anything in it

        self.ao = ao
        if impl == "ours":
            import tinyfa_b200 as tf
            from tinyfa_b200 import _lib

            self.tf, self._lib, self.lib = tf, _lib, _lib.load()
        g = torch.Generator(device=dev).manual_seed(seed)
        H, Hkv, D = w["Hq"], w["Hkv"], w["D"]
        if self.kind == "varlen":
            from tinyfa_b200 import sharding

            self.all_lens = varlen_lengths(w)
            total = sum(self.all_lens)
            Q = torch.randn(total, H, D, generator=g, device=dev).to(self.dt)
            K = torch.randn(total, Hkv, D, generator=g, device=dev).to(self.dt)
            V = torch.randn(total, Hkv, D, generator=g, device=dev).to(self.dt)
            cu = [0]
            for L in self.all_lens:
                cu.append(cu[-1] + L)
            self.full_cu = cu
            if shard is not None:  # shard = list of sequence indices
                Q, K, V, cu, _ = sharding.slice_varlen(Q, K, V, cu, cu, shard)
                self.lens = [self.all_lens[i] for i in shard]
            else:
                self.lens = list(self.all_lens)
            self.Q, self.K, self.V = Q, K, V
            self.cu = torch.tensor(cu, dtype=torch.int32, device=dev)
            self.max_len = max(self.lens) if self.lens else 0
            self.flops = flops_of(w, self.lens)
            self.flops_full = flops_of(w, self.all_lens)
        else:
            B, Sq, Skv = w["B"], w["Sq"], w["Skv"]
            Q = torch.randn(B, Sq, H, D, generator=g, device=dev).to(self.dt)
            # decode shapes hold GBs of K/V: generated in the 16-bit type directly
            gen_dt = self.dt if self.kind == "decode" else torch.float32
            K = torch.randn(B, Skv, Hkv, D, generator=g, device=dev, dtype=gen_dt).to(self.dt)
            V = torch.randn(B, Skv, Hkv, D, generator=g, device=dev, dtype=gen_dt).to(self.dt)
            if shard is not None:  # shard = sharding.FixedShard
                from tinyfa_b200 import sharding

                Q, K, V = sharding.slice_fixed(Q, K, V, shard)
            self.Q, self.K, self.V = Q, K, V
            self.flops_full = flops_of(w)
            self.flops = self.flops_full * (Q.shape[0] * Q.shape[2]) / (B * H)
        self.O_pre = torch.empty_like(self.Q) if impl == "ours" else torch.zeros_like(self.Q)
        es = ESIZE[w["dtype"]]
        if host_inputs:
            if self.kind == "decode":  # K/V are a resident cache: the end-to-end leg moves Q and O only
                self.host = [self.Q.cpu().pin_memory()]
            else:
                self.host = [t.cpu().pin_memory() for t in (self.Q, self.K, self.V)]
            self.host_out = torch.empty(self.Q.shape, dtype=self.dt).pin_memory()
            self.h2d = sum(t.numel() for t in self.host) * es  # cu_seqlens stay on the device (4 * (B + 1) bytes)
            self.d2h = self.Q.numel() * es
        self.bytes_qkvo = (2 * self.Q.numel() + self.K.numel() + self.V.numel()) * es
        self.kv_bytes = (self.K.numel() + self.V.numel()) * es

    # ---- the public Python API (allocates O like the reference binding)
    def step_api(self):
        if self.impl == "ours":
            if self.kind == "varlen":
                return self.tf.flash_attn_varlen_forward(self.Q, self.K, self.V, self.cu, self.cu, self.max_len,
                                                         self.max_len, is_causal=self.causal)
            return self.tf.flash_attn_forward(self.Q, self.K, self.V, is_causal=self.causal)
        if self.kind == "varlen":
            return self.ao.ref_gpu_varlen(self.Q, self.K, self.V, self.cu, self.cu, self.max_len, self.max_len, self.causal)
        return self.ao.ref_gpu_fixed(self.Q, self.K, self.V, self.causal)

    # ---- the kernel alone through the C ABI, output pre-allocated
    def step_kernel(self):
        torch = self.torch
        if self.impl != "ours":
            if self.kind == "varlen":
                self.ao.ref_gpu_varlen(self.Q, self.K, self.V, self.cu, self.cu, self.max_len, self.max_len, self.causal)
            else:
                self.ao.ref_gpu_fixed(self.Q, self.K, self.V, self.causal, out=self.O_pre)
            return
        Q, K, V, O = self.Q, self.K, self.V, self.O_pre
        stream = torch.cuda.current_stream().cuda_stream
        if self.kind == "varlen":
            rc = self.lib.tfa_b200_fwd_varlen(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), self.cu.data_ptr(),
                                              self.cu.data_ptr(), self.code, len(self.lens), self.max_len, self.max_len,
                                              Q.shape[0], K.shape[0], Q.shape[1], K.shape[1], Q.shape[2],
                                              int(self.causal), stream)
        else:
            rc = self.lib.tfa_b200_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), self.code, Q.shape[0],
                                       Q.shape[1], K.shape[1], Q.shape[2], K.shape[2], Q.shape[3], int(self.causal),
                                       stream)
        if rc != 0:
            raise RuntimeError(self._lib.last_error())

    # ---- host buffers in, host buffer out
    def step_e2e(self):
        dev = self.dev
        if self.impl == "ours" and self.kind == "fixed":
            # this library's entry point for host-resident tensors: same copies, overlapped with the kernel
            self.tf.flash_attn_forward_host(self.host[0], self.host[1], self.host[2], is_causal=self.causal,
                                            out=self.host_out, device=dev)
            return
        if self.kind == "decode":
            q, k, v = self.host[0].to(dev, non_blocking=True), self.K, self.V
        else:
            q, k, v = (t.to(dev, non_blocking=True) for t in self.host)
        if self.kind == "varlen":
            if self.impl == "ours":
                o = self.tf.flash_attn_varlen_forward(q, k, v, self.cu, self.cu, self.max_len, self.max_len,
                                                      is_causal=self.causal)
            else:
                o = self.ao.ref_gpu_varlen(q, k, v, self.cu, self.cu, self.max_len, self.max_len, self.causal)
        elif self.impl == "ours":
            o = self.tf.flash_attn_forward(q, k, v, is_causal=self.causal)
        else:
            o = self.ao.ref_gpu_fixed(q, k, v, self.causal)  # the reference API takes device tensors only
        self.host_out.copy_(o, non_blocking=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + ["list"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: leave the strong-scaling block out")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 400-launch sustained loop")
    ap.add_argument("--kernel-only", action="store_true",
                    help="W + K launches of the kernel through the C ABI and a short line, nothing else: the command "
                         "the ncu captures under profiles/ wrap")
    args = ap.parse_args()
    if args.workload == "list":
        print("\n".join(sorted(WORKLOADS)))
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = WORKLOADS[args.workload]

    from oracle import attention_oracle as ao  # only the reference / cpu_baseline legs execute anything in it

    metric = "attention fwd TFLOPS (bf16/fp16 hd128 seq4096)"
    if args.impl == "reference" and not ao.ref_gpu_available():
        # the reference's kernels were not built: time the reference's CPU attention on rank 0 alone
        if rank != 0:
            return
        cb = cpu_baseline(w)
        line = {"impl": "reference", "metric": metric, "value": cb["value"],
                "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": {"workload": args.workload},
                "runs_on": "host cpu (the reference's CUDA kernels were not built)", "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    def bracket(fn, steps, warmup):
        """`steps` calls between two events, barrier + synchronize on both sides; total ms, max over ranks."""
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    def per_step(fn, steps, warmup):
        """Median of per-step CUDA-event times (ms), max over ranks."""
        for _ in range(warmup):
            fn()
        barrier()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in evs:
            a.record()
            fn()
            b.record()
        barrier()
        return max_over_ranks(statistics.median(a.elapsed_time(b) for a, b in evs))

    prob = Problem(w, dev, args.impl, 1234 + rank, torch, host_inputs=not args.kernel_only)
    decode = prob.kind == "decode"
    if args.kernel_only:
        ms = per_step(prob.step_kernel, args.steps, args.warmup)
        if rank == 0:
            print(json.dumps({"workload": args.workload, "kernel_ms": ms, "launches": args.steps + args.warmup,
                              "tflops": prob.flops / (ms * 1e-3) / 1e12, "kv_gbs": prob.kv_bytes / (ms * 1e-3) / 1e9}))
        if world > 1:
            dist.destroy_process_group()
        return

    # The clock sampler (50 ms period) runs over all timed regions: one region is only tens of ms long.
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    ms_total = bracket(prob.step_api, args.steps, args.warmup)
    ms_step = ms_total / args.steps
    ms_step_median = per_step(prob.step_api, args.steps, 0)
    ms_kernel = per_step(prob.step_kernel, args.steps, args.warmup)
    e2e_steps, e2e_warm = max(20, args.steps), 5
    ms_e2e = per_step(prob.step_e2e, e2e_steps, e2e_warm)
    sustained = None
    if not args.no_sustained:
        # a longer back-to-back burst of the same kernel: throughput once the power cap has pulled the clock down
        # at least 400 launches (100 for kernels of several ms) and at least ~0.6 s, so that the 50 ms clock sampler
        # sees the loop
        n_sus = 400 if ms_kernel < 5 else 100
        n_sus = min(20000, max(n_sus, int(600.0 / max(ms_kernel, 1e-3))))
        bracket(prob.step_kernel, 20, 0)
        t_sus0 = time.perf_counter()
        ms_sus = bracket(prob.step_kernel, n_sus, 0) / n_sus
        t_sus1 = time.perf_counter()
        sustained = (ms_sus, n_sus, t_sus0, t_sus1)
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary()
    if args.impl == "ours":
        import ctypes

        site = ctypes.c_int(0)
        st = prob.lib.tfa_b200_device_status(ctypes.byref(site))
        if st != 0:
            raise RuntimeError(f"device status {st} site {site.value}")

    strong = None
    if world > 1 and not args.no_strong and args.impl == "ours":
        strong = strong_block(torch, dist, dev, rank, world, barrier, max_over_ranks, per_step)

    if rank == 0:
        fl = prob.flops
        es = ESIZE[w["dtype"]]
        cfg = {"workload": args.workload, "layout": "[total,H,D] + cu_seqlens" if prob.kind == "varlen" else "[B,S,H,D]",
               "causal": w["causal"], "heads_q": w["Hq"], "heads_kv": w["Hkv"], "head_dim": w["D"],
               "sharding": "replicas",
               "l2": "Q,K,V,O = %d MiB per rank and step > 126 MB L2; no flush" % (prob.bytes_qkvo >> 20)}
        if prob.kind == "varlen":
            cfg.update({"sequences": len(prob.lens), "total_tokens": sum(prob.lens), "max_len": prob.max_len,
                        "lengths": prob.lens})
        else:
            cfg.update({"batch_per_gpu": w["B"], "seq_q": w["Sq"], "seq_kv": w["Skv"]})
        if prob.bytes_qkvo < 126e6:
            cfg["l2"] = "working set %d MiB fits the 126 MB L2 (reported as is; the shape is the workload)" % (prob.bytes_qkvo >> 20)
        if decode:
            hbm, hbm_src = measured_hbm()
            kvb = prob.kv_bytes
            val = lambda ms: kvb / (ms * 1e-3) / 1e9
            unit, metric_name = "GB/s", "attention fwd decode GB/s (K and V read once)"
            roof = {"bound": "hbm", "achieved": val(ms_kernel), "peak": hbm, "unit": "GB/s", "frac": val(ms_kernel) / hbm,
                    "peak_source": hbm_src}
            sus_peak, sus_src = hbm, hbm_src
        else:
            val = lambda ms: fl / (ms * 1e-3) / 1e12
            unit, metric_name = "TFLOP/s", metric
            if w["dtype"] == "fp32":
                peak, peak_src = fp32_fma_peak()
                roof = {"bound": "fma", "achieved": val(ms_kernel), "peak": peak, "unit": "TFLOP/s",
                        "frac": val(ms_kernel) / peak, "peak_source": peak_src}
                sus_peak, sus_src = peak, peak_src
            else:
                peak, peak_src = measured_peak()
                roof = {"bound": "tensor", "achieved": val(ms_kernel), "peak": peak, "unit": "TFLOP/s",
                        "frac": val(ms_kernel) / peak, "peak_source": peak_src}
                sus_peak, sus_src = measured_sustained_peak()
            cfg["per_gpu_tflops"] = val(ms_step)
            cfg["pct_of_nominal_2250"] = 100.0 * val(ms_step) / 2250.0
        roof["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload) if args.impl == "ours" else None
        roof["kernel_ms"] = ms_kernel
        if sustained is not None:
            ms_sus, n_sus, t0, t1 = sustained
            sc = sampler.summary(since=t0, until=t1)
            roof["sustained"] = {"achieved": val(ms_sus), "peak": sus_peak, "frac": val(ms_sus) / sus_peak,
                                 "peak_source": sus_src, "launches": n_sus, "kernel_ms": ms_sus,
                                 "sm_mhz": sc["sm_mhz"], "reasons": sc["reasons"]}
        line = {
            "metric": metric_name, "value": world * val(ms_step), "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "ms_per_step_median": ms_step_median,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": cfg, "roofline": roof,
            "e2e": {"value": world * val(ms_e2e), "unit": unit, "h2d_bytes_per_step": prob.h2d,
                    "d2h_bytes_per_step": prob.d2h, "ms_per_step": ms_e2e, "steps": e2e_steps, "warmup": e2e_warm,
                    "statistic": "median of per-step CUDA-event times, max over ranks"},
            # kernels of this library inside the K bracketed steps: one per step, two (split + combine) on the split-KV path
            "gpu_launches": args.steps * (2 if decode and w["B"] * w["Hkv"] < 148 else 1), "clocks": clocks,
        }
        if strong is not None:
            line["strong"] = strong
        if args.impl == "reference":
            line["impl"] = "reference"
            line["runs_on"] = "reference CUDA kernels (SM8x tile table) compiled for sm_100a"
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def strong_block(torch, dist, dev, rank, world, barrier, max_over_ranks, per_step, steps=15, warmup=5):
    """Strong scaling of the two multi-GPU problems: ONE global problem (every rank generates the same tensors from
    the same seed) split over the ranks, outputs left sharded; the unsplit problem timed on every rank (max) gives
    the 1-GPU figure of the same run.  One all-gather per problem builds the validation copy."""
    from tinyfa_b200 import sharding

    out = {}
    for name in STRONG_WORKLOADS:
        w = WORKLOADS[name]
        whole = Problem(w, dev, "ours", 4321, torch, host_inputs=False)
        ms1 = per_step(whole.step_kernel, steps, warmup)
        o_full = whole.step_api()
        if w["kind"] == "varlen":
            plan = sharding.plan_varlen(whole.all_lens, whole.all_lens, world, w["causal"])
            shard = plan[rank]
            how = "by sequence (longest-first greedy on the causal pair count)"
        else:
            plan = sharding.plan_fixed(w["B"], w["Hkv"], world)
            shard = plan[rank]
            how = "by (batch x KV head), %d units per rank" % (shard.unit_end - shard.unit_begin)
        part = Problem(w, dev, "ours", 4321, torch, shard=shard, host_inputs=False)
        has_work = part.Q.numel() > 0
        msN = per_step(part.step_kernel if has_work else (lambda: None), steps, warmup)
        # validation copy: gather every rank's shard output (padded to the largest shard) and compare on rank 0
        o_local = part.step_api() if has_work else part.Q
        flat = o_local.reshape(-1)
        n_local = torch.tensor([flat.numel()], device=dev, dtype=torch.int64)
        sizes = [torch.zeros_like(n_local) for _ in range(world)]
        dist.all_gather(sizes, n_local)
        n_max = int(max(int(s.item()) for s in sizes))
        padded = torch.zeros(n_max, dtype=flat.dtype, device=dev)
        padded[:flat.numel()] = flat
        parts = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded)
        diff = None
        if rank == 0:
            glued = torch.zeros_like(o_full)
            for r in range(world):
                n = int(sizes[r].item())
                if n == 0:
                    continue
                if w["kind"] == "varlen":
                    sharding.place_varlen(glued, parts[r][:n].reshape(-1, w["Hq"], w["D"]), whole.full_cu, plan[r])
                else:
                    s = plan[r]
                    shp = (s.batch_end - s.batch_begin, w["Sq"], (s.kv_head_end - s.kv_head_begin) * (w["Hq"] // w["Hkv"]), w["D"])
                    sharding.place_fixed(glued, parts[r][:n].reshape(shp), s, w["Hq"] // w["Hkv"])
            diff = float((glued.float() - o_full.float()).abs().max().item())
        fl = whole.flops_full
        out[name] = {"split": how, "tflops_1gpu": fl / (ms1 * 1e-3) / 1e12, "ms_1gpu": ms1,
                     "tflops": fl / (msN * 1e-3) / 1e12, "ms": msN, "speedup": ms1 / msN, "n_gpus": world,
                     "validation_max_abs_diff": diff,
                     "statistic": "median of %d per-step CUDA-event times after %d warm-ups, max over ranks" % (steps, warmup)}
        del whole, part, o_full, parts, padded
        torch.cuda.empty_cache()
        barrier()
    return out


if __name__ == "__main__":
    main()
