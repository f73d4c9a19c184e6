#!/usr/bin/env python3
"""Benchmark of the attention-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one attention forward over one batch of synthetic input (seeded N(0,1), generated in fp32 and cast).
Default workload: bf16, non-causal, batch 2, seq 4096, 32 heads, head dim 128, layout [B,S,H,D] - the shape
the reference quotes its throughput on (reference README.md:56-64, benchmarks/benchmark.py:21-28).  FLOPs are
4*B*H*Sq*Skv*D, halved when causal (reference benchmarks/benchmark.py:31-33).

With N > 1 the script runs under torchrun, one rank per GPU; each rank processes its own independently seeded
batch of the same shape (weak scaling, no collective on the data path); time is the max over ranks.

Prints ONE JSON line.  `value` is throughput with inputs resident in HBM; `e2e` is the same metric through the
public Python API with pinned HOST buffers (host->device copies of Q, K, V and device->host copy of O inside the
timed region).  `--impl reference` runs the reference's own CUDA kernels (built for sm_100a from the reference
sources by oracle/Makefile) through the reference's tfa::flashAttn API on the same shape; if that library was
not built it times the reference's CPU attention instead and says so.
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

WORKLOADS = {
    # name: (dtype, causal, B, Sq, Skv, Hq, Hkv, D)
    "bf16_noncausal_b2_s4096_h32_d128": ("bf16", False, 2, 4096, 4096, 32, 32, 128),
    "bf16_causal_b2_s4096_h32_d128": ("bf16", True, 2, 4096, 4096, 32, 32, 128),
    "fp16_noncausal_b2_s4096_h32_d128": ("fp16", False, 2, 4096, 4096, 32, 32, 128),
    "fp16_causal_b2_s4096_h32_d128": ("fp16", True, 2, 4096, 4096, 32, 32, 128),
    "bf16_causal_gqa_b4_s8192_h32_8_d128": ("bf16", True, 4, 8192, 8192, 32, 8, 128),
    # decode shapes are HBM-bound: reported in GB/s of K+V read once
    "bf16_decode_b64_skv32768_h32_8_d128": ("bf16", False, 64, 1, 32768, 32, 8, 128),
    "bf16_decode_b8_skv32768_h32_8_d128": ("bf16", False, 8, 1, 32768, 32, 8, 128),
}
DEFAULT_WORKLOAD = "bf16_noncausal_b2_s4096_h32_d128"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
# (decode: batch-8 capture scaled by units processed; traffic grows in proportion to batch).
NCU_TRAFFIC_BYTES = {
    "bf16_noncausal_b2_s4096_h32_d128": 201475328 + 46450432,
    "bf16_decode_b64_skv32768_h32_8_d128": int((1074021000 + 4879104) * 8),
    "bf16_decode_b8_skv32768_h32_8_d128": 1074021000 + 4879104,
}
FALLBACK_PEAK_TFLOPS = 1590.0  # earlier measurement on this pool, used only when MEASURED_PEAKS.json is absent


def flops_of(w):
    _, causal, B, Sq, Skv, Hq, _, D = w
    f = 4.0 * B * Hq * Sq * Skv * D
    return f / 2 if causal else f


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs (read-only query)."""

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

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
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


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        return FALLBACK_PEAK_TFLOPS, "fallback"


def measured_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, copy)"
    except Exception:
        return 6650.0, "fallback"


def cpu_baseline(w, target_seconds=12.0):
    """Naive fp32 attention on the host cores on a bounded sample of the workload: the first q_rows query rows of
    every (batch, head).  Uses the reference's own cpu_reference.h when it was compiled here, else the port."""
    import numpy as np

    from oracle import attention_oracle as ao

    _, causal, B, Sq, Skv, Hq, Hkv, D = w
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
            "sample": (f"first {rows} of {Sq} query rows of every (batch, head), "
                       + (f"first {min(rows, Skv)} keys (causal sub-problem)" if causal else "all keys")
                       + f"; {t:.1f} s; fp32 naive")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank runs its own copy of the workload; strong: the ONE workload is split over the "
                         "ranks by (batch x KV head) with tinyfa_b200.sharding.plan_fixed, outputs stay sharded")
    ap.add_argument("--validate", action="store_true",
                    help="strong scaling only: all-gather the sharded outputs once and compare with the unsharded result")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = WORKLOADS[args.workload]
    dtype_name, causal, B, Sq, Skv, Hq, Hkv, D = w

    from oracle import attention_oracle as ao  # only the reference / cpu_baseline legs execute anything in it

    if args.impl == "reference" and not ao.ref_gpu_available():
        # the reference's kernels were not built: time the reference's CPU attention on rank 0 alone
        if rank != 0:
            return
        cb = cpu_baseline(w)
        line = {"impl": "reference", "metric": "attention fwd TFLOPS (bf16/fp16 hd128 seq4096)", "value": cb["value"],
                "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": {"workload": args.workload, "runs_on": "host cpu"},
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16}[dtype_name]

    decode = Sq == 1
    strong = args.scaling == "strong" and world > 1 and not decode
    shard = None
    if strong:
        from tinyfa_b200 import sharding

        shard = sharding.plan_fixed(B, Hkv, world)[rank]  # contiguous (batch, KV head) units of the ONE global problem
    g = torch.Generator().manual_seed(1234 + (0 if strong else rank))
    if decode:
        # GBs of K/V: generated on the device; the end-to-end leg moves Q and O only (K/V are a resident cache)
        gd = torch.Generator(device=dev).manual_seed(1234 + rank)
        Q = torch.randn(B, Sq, Hq, D, generator=gd, device=dev).to(dt)
        K = torch.randn(B, Skv, Hkv, D, generator=gd, device=dev, dtype=dt)
        V = torch.randn(B, Skv, Hkv, D, generator=gd, device=dev, dtype=dt)
        host = [Q.cpu().pin_memory()]
    else:
        full = [torch.randn(B, S, H, D, generator=g).to(dt) for S, H in ((Sq, Hq), (Skv, Hkv), (Skv, Hkv))]
        if strong:
            host = [t.pin_memory() for t in sharding.slice_fixed(full[0], full[1], full[2], shard)]
        else:
            host = [t.pin_memory() for t in full]
        Q, K, V = (t.to(dev) for t in host)
        B, Hq, Hkv = Q.shape[0], Q.shape[2], K.shape[2]  # per-rank shapes from here on
    globalB, globalHq, globalHkv = w[2], w[5], w[6]

    host_out = torch.empty(B, Sq, Hq, D, dtype=dt).pin_memory()
    if args.impl == "ours":
        import tinyfa_b200 as tf
        from tinyfa_b200 import _lib

        lib = _lib.load()
        code = {"fp16": 1, "bf16": 2}[dtype_name]
        O_pre = torch.empty_like(Q)

        def step_api():
            return tf.flash_attn_forward(Q, K, V, is_causal=causal)

        def step_kernel():
            rc = lib.tfa_b200_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O_pre.data_ptr(), code, B, Sq, Skv, Hq, Hkv,
                                  D, int(causal), torch.cuda.current_stream().cuda_stream)
            if rc != 0:
                raise RuntimeError(_lib.last_error())
    else:
        O_pre = torch.zeros_like(Q)

        def step_api():  # the reference binding zero-fills a fresh output every call (binding:106)
            return ao.ref_gpu_fixed(Q, K, V, causal)

        def step_kernel():
            ao.ref_gpu_fixed(Q, K, V, causal, out=O_pre)

    def step_e2e():
        if args.impl == "ours" and not decode:
            # this library's entry point for host-resident tensors: same copies, overlapped with the kernel
            tf.flash_attn_forward_host(host[0], host[1], host[2], is_causal=causal, out=host_out, device=dev)
            return
        if decode:
            q, k, v = host[0].to(dev, non_blocking=True), K, V
        else:
            q, k, v = (t.to(dev, non_blocking=True) for t in host)
        if args.impl == "ours":
            o = tf.flash_attn_forward(q, k, v, is_causal=causal)
        else:
            o = ao.ref_gpu_fixed(q, k, v, causal)  # the reference API takes device tensors only
        host_out.copy_(o, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    # The clock sampler (50 ms period) runs over all three timed regions: one region is only tens of ms long.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total = timed(step_api, args.steps, args.warmup)
    ms_kernel = timed(step_kernel, args.steps, args.warmup) / args.steps
    ms_e2e = timed(step_e2e, max(3, args.steps // 3), 3) / max(3, args.steps // 3)
    # a longer back-to-back burst of the same step, only to give the sampler a region under sustained load
    timed(step_kernel, 400, 0)
    clocks = sampler.stop() if rank == 0 else None

    if args.impl == "ours":
        import ctypes

        site = ctypes.c_int(0)
        st = lib.tfa_b200_device_status(ctypes.byref(site))
        if st != 0:
            raise RuntimeError(f"device status {st} site {site.value}")

    validation = None
    if strong and args.validate and args.impl == "ours":
        # the one collective of the design: gather the sharded outputs for a validation copy
        o_local = step_api()
        parts = [torch.empty_like(o_local) for _ in range(world)]
        dist.all_gather(parts, o_local)
        if rank == 0:
            Qf, Kf, Vf = (t.to(dev) for t in full)
            o_full = tf.flash_attn_forward(Qf, Kf, Vf, is_causal=causal)
            glued = torch.empty_like(o_full)
            for sh, part in zip(sharding.plan_fixed(globalB, globalHkv, world), parts):
                sharding.place_fixed(glued, part, sh, globalHq // globalHkv)
            validation = float((glued.float() - o_full.float()).abs().max().item())

    fl = flops_of(w)  # the whole workload
    ms_step = ms_total / args.steps
    if strong:
        value = fl / (ms_step * 1e-3) / 1e12          # total work fixed, split over the ranks
        fl_kernel = fl / world                        # one rank's share
    else:
        value = world * fl / (ms_step * 1e-3) / 1e12  # every rank processed the whole workload
        fl_kernel = fl
    peak, peak_src = measured_peak()
    achieved = fl_kernel / (ms_kernel * 1e-3) / 1e12
    esize = 2
    bytes_in = (B * Sq * Hq * D + 2 * B * Skv * Hkv * D) * esize
    bytes_out = B * Sq * Hq * D * esize

    if decode and rank == 0:
        kv_bytes = 2.0 * B * Skv * Hkv * D * esize
        hbm, hbm_src = measured_hbm()
        line = {
            "metric": "attention fwd decode GB/s (K and V read once)", "value": world * kv_bytes / (ms_step * 1e-3) / 1e9,
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
            "config": {"workload": args.workload, "layout": "[B,S,H,D]", "causal": causal, "batch_per_gpu": B,
                       "seq_q": Sq, "seq_kv": Skv, "heads_q": Hq, "heads_kv": Hkv, "head_dim": D,
                       "l2": "K,V = %.2f GB per step > 126 MB L2; no flush" % (kv_bytes / 1e9)},
            "roofline": {"bound": "hbm", "achieved": kv_bytes / (ms_kernel * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                         "frac": kv_bytes / (ms_kernel * 1e-3) / 1e9 / hbm,
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload) if args.impl == "ours" else None, "peak_source": hbm_src,
                         "kernel_ms": ms_kernel},
            "e2e": {"value": world * kv_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": B * Sq * Hq * D * esize, "d2h_bytes_per_step": bytes_out, "ms_per_step": ms_e2e},
            "gpu_launches": args.steps, "clocks": clocks,
        }
        if args.impl == "reference":
            line["impl"] = "reference"
        print(json.dumps(line))
    elif rank == 0:
        line = {
            "metric": "attention fwd TFLOPS (bf16/fp16 hd128 seq4096)", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": dtype_name, "data": "synthetic",
            "config": {"workload": args.workload, "layout": "[B,S,H,D]", "causal": causal, "batch_per_gpu": B,
                       "seq_q": Sq, "seq_kv": Skv, "heads_q": Hq, "heads_kv": Hkv, "head_dim": D,
                       "sharding": ("batch x KV head, %d units per rank, outputs sharded" % (shard.unit_end - shard.unit_begin))
                       if strong else "replicas",
                       "validation_max_abs_diff": validation,
                       "l2": "Q,K,V,O = %d MiB per rank and step > 126 MB L2; no flush" % ((bytes_in + bytes_out) >> 20),
                       "per_gpu_tflops": value / world,
                       "pct_of_nominal_2250": 100.0 * value / world / 2250.0},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload) if args.impl == "ours" else None,
                         "peak_source": peak_src,
                         "kernel_ms": ms_kernel},
            "e2e": {"value": (fl if strong else world * fl) / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": bytes_in,
                    "d2h_bytes_per_step": bytes_out, "ms_per_step": ms_e2e},
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        if args.impl == "reference":
            line["impl"] = "reference"
            line["config"]["runs_on"] = "reference CUDA kernels (SM8x tile table) compiled for sm_100a"
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
