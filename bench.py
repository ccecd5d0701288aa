"""Throughput benchmark for the GEMM / attention / decode kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload: non-causal attention f16, batch 8, 32 heads, Sq = Skv = 1024, head dim 128.
Other workloads (same JSON line): gemm_f16, attn_causal, attn_bwd_causal, paged_decode, gemm_fp8.

A step is one pass of the kernel over one batch of synthetic inputs.  Each step is timed with
CUDA events on the launching stream; between steps either the inputs are larger than L2 or L2 is
flushed by writing a 256 MB buffer (stated in ``config.l2``).  With N > 1 every rank runs the
same workload on its own GPU (independent units: batch x head shards; no data-path collective),
the timed region is bracketed by barrier + synchronize and the maximum over ranks is used.

``--impl reference`` times the CPU restatement of the reference path (the oracle) on the host
cores on a bounded sample of the same workload; rank 0 only.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

SCALE = 128 ** -0.5


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
class Workload:
    # dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel, one launch, from the ncu
    # capture summarised under profiles/ (None = no capture for this workload yet)
    traffic_bytes = None
    name = ""
    metric = ""
    unit = "TFLOP/s"
    dtype = "f16"
    bound = "tensor"
    launches_per_step = 1
    needs_flush = False

    scaling = "weak"  # per-GPU work fixed as N grows, unless a workload says otherwise

    def config(self) -> dict: ...
    def setup(self, dev): ...
    def shard(self, world: int, rank: int):
        """Called before setup() when N > 1; default: every rank runs the whole workload (independent units)."""
    def step(self): ...
    def units_per_step(self) -> float:
        """flops (tensor-bound) or bytes (hbm-bound) per step."""
    def setup_e2e(self, dev): ...
    def step_e2e(self): ...
    def e2e_bytes(self) -> tuple: ...
    def cpu_sample(self) -> tuple:
        """Runs the oracle on a bounded sample; returns (units processed, seconds, description)."""


class AttentionWL(Workload):
    def __init__(self, name, batch, heads, seq, dtype, causal, std, traffic=None):
        self.name = name
        self.traffic_bytes = traffic
        self.b, self.h, self.s = batch, heads, seq
        self.tdtype = dtype
        self.dtype = "f16" if dtype == torch.float16 else "bf16"
        self.causal = causal
        self.std = std
        kind = "causal" if causal else "non-causal"
        self.metric = f"attention fwd TFLOP/s ({kind} {self.dtype} B{batch} H{heads} S{seq} D128)"

    def config(self):
        nbytes = 4 * self.b * self.h * self.s * 128 * 2
        return {"workload": self.name, "batch": self.b, "heads": self.h, "seq_q": self.s, "seq_kv": self.s,
                "head_dim": 128, "causal": self.causal, "scale": SCALE,
                "l2": f"inputs larger than L2 ({nbytes / 1e6:.0f} MB touched per step)"}

    def _make(self, dev, seed=10):
        g = torch.Generator(device=dev).manual_seed(seed)
        return [(torch.randn(self.b, self.h, self.s, 128, generator=g, device=dev) * self.std).to(self.tdtype)
                for _ in range(3)]

    def setup(self, dev):
        self.q, self.k, self.v = self._make(dev)

    def step(self):
        self.o = torch.ops.b200k.attention(self.q, self.k, self.v, SCALE, self.causal)

    def units_per_step(self):
        f = 4.0 * self.b * self.h * self.s * self.s * 128
        return f / 2 if self.causal else f

    def setup_e2e(self, dev):
        from iree_turbine_b200 import host_api

        q, k, v = self._make(dev)
        self.hq, self.hk, self.hv = (t.cpu().pin_memory() for t in (q, k, v))
        self.ho = torch.empty_like(self.hq).pin_memory()
        self.e2e = host_api.AttentionHost(self.b, self.h, self.h, self.s, self.s, self.tdtype, dev)

    def step_e2e(self):
        self.e2e(self.hq, self.hk, self.hv, self.ho, SCALE, self.causal)

    def e2e_bytes(self):
        n = self.b * self.h * self.s * 128 * 2
        return 3 * n, n

    def cpu_sample(self):
        from oracle import oracle

        bs, hs = 1, min(self.h, 8 if self.s > 2048 else 32)
        q, k, v = oracle.make_attention_inputs(bs, hs, hs, self.s, self.s, 128, self.tdtype, seed=10, std=self.std)
        best = None
        for _ in range(2):
            t0 = time.perf_counter()
            oracle.attention(q, k, v, SCALE, self.causal)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        f = 4.0 * bs * hs * self.s * self.s * 128
        f = f / 2 if self.causal else f
        return f, best, f"oracle.attention on batch {bs} x {hs} heads of the same shape, best of 2"


class AttentionBwdWL(AttentionWL):
    """Attention backward (dQ, dK, dV from q, k, v, o, dO).  Work is counted as five 128-deep
    products per score element (2.5 x the forward count), the usual convention; the kernels
    execute seven (the scores and dP are recomputed in both passes).  The forward's row statistic
    (lse) is an input, as in a training step."""

    launches_per_step = 3  # delta, dQ (+ statistics), dK/dV

    def __init__(self, name, batch, heads, seq, dtype, causal, std):
        super().__init__(name, batch, heads, seq, dtype, causal, std)
        kind = "causal" if causal else "non-causal"
        self.metric = f"attention bwd TFLOP/s ({kind} {self.dtype} B{batch} H{heads} S{seq} D128)"

    def _make_do(self, dev, seed=11):
        g = torch.Generator(device=dev).manual_seed(seed)
        return torch.randn(self.b, self.h, self.s, 128, generator=g, device=dev).to(self.tdtype)

    def setup(self, dev):
        self.q, self.k, self.v = self._make(dev)
        self.d_o = self._make_do(dev)
        self.o, self.lse = torch.ops.b200k.attention_lse(self.q, self.k, self.v, SCALE, self.causal)

    def step(self):
        self.grads = torch.ops.b200k.attention_bwd(self.q, self.k, self.v, self.o, self.d_o, SCALE, self.causal,
                                                   self.lse)

    def units_per_step(self):
        return 2.5 * super().units_per_step()

    def setup_e2e(self, dev):
        self.host_in = [t.cpu().pin_memory() for t in (self.q, self.k, self.v, self.o, self.d_o)]
        self.host_lse = self.lse.cpu().pin_memory()
        self.host_out = [torch.empty_like(self.host_in[0]).pin_memory() for _ in range(3)]

    def step_e2e(self):
        dev_in = [t.to(self.q.device, non_blocking=True) for t in self.host_in]
        grads = torch.ops.b200k.attention_bwd(*dev_in, SCALE, self.causal,
                                              self.host_lse.to(self.q.device, non_blocking=True))
        for h, g in zip(self.host_out, grads):
            h.copy_(g, non_blocking=True)

    def e2e_bytes(self):
        n = self.b * self.h * self.s * 128 * 2
        return 5 * n + self.b * self.h * self.s * 4, 3 * n

    def cpu_sample(self):
        from oracle import oracle

        bs, hs = 1, min(self.h, 4 if self.s > 2048 else 16)
        q, k, v = oracle.make_attention_inputs(bs, hs, hs, self.s, self.s, 128, self.tdtype, seed=10, std=self.std)
        d_o = torch.randn(q.shape, generator=torch.Generator().manual_seed(11)).to(self.tdtype)
        best = None
        for _ in range(2):
            t0 = time.perf_counter()
            oracle.attention_bwd(q, k, v, d_o, SCALE, self.causal)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        f = 2.5 * 4.0 * bs * hs * self.s * self.s * 128
        f = f / 2 if self.causal else f
        return f, best, f"oracle.attention_bwd on batch {bs} x {hs} heads of the same shape, best of 2"


class GemmWL(Workload):
    needs_flush = True

    def __init__(self, name, n, fp8):
        self.name, self.n, self.fp8 = name, n, fp8
        self.traffic_bytes = 417.1e6 if (fp8 and n == 8192) else (16.9e6 if (not fp8 and n == 2048) else None)
        # the measured peak is a bf16 GEMM; e4m3 runs the tensor pipe at twice that rate
        self.peak_scale = 2.0 if fp8 else 1.0
        self.dtype = "e4m3" if fp8 else "f16"
        out = "bf16" if fp8 else "f32"
        self.metric = f"GEMM TFLOP/s ({self.dtype} NT M=N=K={n}, fp32 accumulate, {out} out)"
        self.needs_flush = (2 * n * n * (1 if fp8 else 2) + n * n * (2 if fp8 else 4)) < 200e6

    def config(self):
        cfg = {"workload": self.name, "m": self.n, "n": self.n, "k": self.n,
               "l2": "L2 flushed between steps (256 MB write)" if self.needs_flush else "operands larger than L2"}
        if self.world > 1:
            cfg["parallelism"] = (f"column-parallel over N on {self.world} GPUs, all-gather of C fused into the "
                                  "GEMM epilogue (peer stores) + cross-rank barrier inside the timed step")
        return cfg

    world, rank = 1, 0

    def shard(self, world, rank):
        # fp8 GEMM: column-parallel over N, all-gather of C fused into the epilogue (strong scaling).
        # f16 2048^3 is too small to shard: independent replicas.
        if self.fp8:
            self.world, self.rank = world, rank
            self.scaling = "strong"

    def setup(self, dev):
        g = torch.Generator(device=dev).manual_seed(10)
        a = torch.randn(self.n, self.n, generator=g, device=dev)
        b = torch.randn(self.n, self.n, generator=g, device=dev)
        if self.fp8:
            self.a, self.sa = torch.ops.b200k.quantize_e4m3(a)
            self.b, self.sb = torch.ops.b200k.quantize_e4m3(b)
        else:
            self.a, self.b = a.half(), b.half()
        if self.world > 1:
            from iree_turbine_b200 import dist as tdist

            lo, hi = tdist.shard_range(self.n, self.world, self.rank)
            self.b = self.b[lo:hi].contiguous()
            self.fused = tdist.FusedColumnParallelGemm(self.n, self.n, torch.bfloat16)

    def step(self):
        if self.world > 1:
            self.fused(self.a, self.b, self.sa, self.sb)
            self.c = self.fused.finish()
        elif self.fp8:
            self.c = torch.ops.b200k.gemm_fp8_nt(self.a, self.b, self.sa, self.sb)
        else:
            self.c = torch.ops.b200k.gemm_nt(self.a, self.b)

    def units_per_step(self):
        return 2.0 * self.n ** 3 / self.world

    def setup_e2e(self, dev):
        from iree_turbine_b200 import host_api

        if self.world > 1:
            # sharded run: the rank's operands come from pinned host memory each step, the full C
            # is read back by every rank
            self.ha, self.hb = self.a.cpu().pin_memory(), self.b.cpu().pin_memory()
            self.hc = torch.empty(self.n, self.n, dtype=torch.bfloat16).pin_memory()
            return
        self.setup(dev)
        self.ha, self.hb = self.a.cpu().pin_memory(), self.b.cpu().pin_memory()
        out_dtype = torch.bfloat16 if self.fp8 else torch.float32
        self.hc = torch.empty(self.n, self.n, dtype=out_dtype).pin_memory()
        self.e2e = host_api.GemmHost(self.n, self.n, self.n, self.a.dtype, out_dtype, dev)

    def step_e2e(self):
        if self.world > 1:
            self.a.copy_(self.ha, non_blocking=True)
            self.b.copy_(self.hb, non_blocking=True)
            self.fused(self.a, self.b, self.sa, self.sb)
            self.hc.copy_(self.fused.finish(), non_blocking=True)
        elif self.fp8:
            self.e2e(self.ha, self.hb, self.hc, self.sa, self.sb)
        else:
            self.e2e(self.ha, self.hb, self.hc)

    def e2e_bytes(self):
        es = 1 if self.fp8 else 2
        if self.world > 1:
            return self.n * self.n * es + self.b.numel() * es, self.n * self.n * 2
        return 2 * self.n * self.n * es, self.n * self.n * (2 if self.fp8 else 4)

    def cpu_sample(self):
        from oracle import oracle

        rows = self.n if self.n <= 2048 else 512
        if self.fp8:
            a8, b8, sa, sb = oracle.make_fp8_gemm_inputs(rows, self.n, self.n, seed=10)
            fn = lambda: oracle.gemm_fp8_nt(a8, b8, sa, sb)  # noqa: E731
        else:
            a, b = oracle.make_gemm_inputs(rows, self.n, self.n, torch.float16, seed=10)
            fn = lambda: oracle.gemm_nt(a, b)  # noqa: E731
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            fn()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return 2.0 * rows * self.n * self.n, best, f"oracle GEMM on {rows} rows of A against all of B, best of 3"


class PagedDecodeWL(Workload):
    unit = "GB/s"
    bound = "hbm"
    launches_per_step = 2
    metric = "paged-decode HBM GB/s (f16, 64 seqs, 32 q-heads / 8 kv-heads, D128, len U[512,8192], page 16)"

    traffic_bytes = 1179.2e6

    def __init__(self, name):
        self.name = name

    def config(self):
        return {"workload": self.name, "num_seqs": 64, "q_heads": 32, "kv_heads": 8, "head_dim": 128, "page_size": 16,
                "len_range": [512, 8192], "sum_len": int(self.sum_len) if hasattr(self, "sum_len") else None,
                "l2": "KV pool larger than L2 (about 1.1 GB read per step)"}

    def _host_inputs(self):
        from oracle import oracle

        return oracle.make_paged_decode_inputs(seed=10)

    def setup(self, dev):
        q, kc, vc, bt, sl = self._host_inputs()
        self.sum_len = int(sl.sum())
        self.pages = int(((sl + 15) // 16).sum())
        self.host = (q, kc, vc, bt, sl)
        self.q, self.kc, self.vc, self.bt, self.sl = (t.to(dev) for t in (q, kc, vc, bt, sl))

    def step(self):
        self.o = torch.ops.b200k.paged_decode_attention(self.q, self.kc, self.vc, self.bt, self.sl, SCALE)

    def units_per_step(self):
        # K and V rows actually read + Q and O + block-table entries + seq_lens
        return self.sum_len * 8 * 128 * 2 * 2 + 2 * 64 * 32 * 128 * 2 + 4 * self.pages + 4 * 64

    def setup_e2e(self, dev):
        # The KV pool is state that lives on the device across decode steps; per step the host
        # provides the query, the block table and the lengths and reads the output back.
        self.setup(dev)
        q, kc, vc, bt, sl = self.host
        self.hq, self.hbt, self.hsl = q.pin_memory(), bt.pin_memory(), sl.pin_memory()
        self.ho = torch.empty_like(q).pin_memory()

    def step_e2e(self):
        q = self.hq.to(self.q.device, non_blocking=True)
        bt = self.hbt.to(self.q.device, non_blocking=True)
        sl = self.hsl.to(self.q.device, non_blocking=True)
        o = torch.ops.b200k.paged_decode_attention(q, self.kc, self.vc, bt, sl, SCALE)
        self.ho.copy_(o, non_blocking=True)

    def e2e_bytes(self):
        return self.hq.numel() * 2 + self.hbt.numel() * 4 + self.hsl.numel() * 4, self.ho.numel() * 2

    def cpu_sample(self):
        from oracle import oracle

        q, kc, vc, bt, sl = self._host_inputs()
        sub = torch.arange(8)
        t0 = time.perf_counter()
        oracle.paged_decode_attention(q[sub], kc, vc, bt[sub], sl[sub], SCALE)
        dt = time.perf_counter() - t0
        nbytes = int(sl[sub].sum()) * 8 * 128 * 2 * 2
        return float(nbytes), dt, "oracle.paged_decode_attention on the first 8 of the 64 sequences, one run"


WORKLOADS = {
    "attn_noncausal": lambda: AttentionWL("attn_noncausal", 8, 32, 1024, torch.float16, False, 1.0, 249.1e6),
    "attn_causal": lambda: AttentionWL("attn_causal", 4, 32, 4096, torch.bfloat16, True, 0.5),
    "attn_bwd_causal": lambda: AttentionBwdWL("attn_bwd_causal", 4, 32, 4096, torch.bfloat16, True, 0.5),
    "gemm_f16": lambda: GemmWL("gemm_f16", 2048, False),
    "gemm_fp8": lambda: GemmWL("gemm_fp8", 8192, True),
    "paged_decode": lambda: PagedDecodeWL("paged_decode"),
}


# ---------------------------------------------------------------------------------------------
# clocks sampler
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# arms
# ---------------------------------------------------------------------------------------------
def run_reference(wl: Workload, args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        sys.exit(0)
    torch.set_num_threads(os.cpu_count() or 1)
    times, units = [], 0.0
    desc = ""
    for i in range(args.warmup + args.steps):
        u, dt, desc = wl.cpu_sample()
        if i >= args.warmup:
            times.append(dt)
            units = u
    per_step = sum(times) / len(times)
    scale = 1e12 if wl.unit == "TFLOP/s" else 1e9
    value = units / per_step / scale
    cfg = wl.config()
    return {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def timed_steps(step_fn, steps, warmup, flush_buf, stream):
    """Runs warmup + steps; returns per-step milliseconds measured with CUDA events on `stream`."""
    for _ in range(warmup):
        if flush_buf is not None:
            flush_buf.fill_(1)
        step_fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(steps):
        if flush_buf is not None:
            flush_buf.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        step_fn()
        e1.record(stream)
        evs.append((e0, e1))
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


def run_ours(wl: Workload, args) -> dict:
    import torch.distributed as dist

    import iree_turbine_b200 as tb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peaks = load_peaks()
    stream = torch.cuda.current_stream()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if wl.needs_flush else None
    if world > 1:
        wl.shard(world, rank)
    wl.setup(dev)
    units = wl.units_per_step()
    scale = 1e12 if wl.unit == "TFLOP/s" else 1e9

    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    if sampler:
        sampler.start()
    ms = timed_steps(wl.step, args.steps, max(args.warmup, 3), flush, stream)
    barrier()
    total_ms = sum(ms)
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    status = tb.device_status()

    # end-to-end through the host-buffer API (copies inside the timed region)
    wl.setup_e2e(dev)
    barrier()
    e2e_ms = timed_steps(wl.step_e2e, args.steps, max(args.warmup, 3), None, stream)
    barrier()
    e2e_total = sum(e2e_ms)
    if world > 1:
        t = torch.tensor([e2e_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_total = float(t.item())
    clocks = sampler.stop() if sampler else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return {}

    per_step_ms = total_ms / args.steps
    value = world * units / (per_step_ms * 1e-3) / scale
    kernel_ms = statistics.mean(ms)
    achieved = units / (kernel_ms * 1e-3) / scale
    peak = peaks["hbm_gbs"] if wl.bound == "hbm" else peaks["tflops"] * getattr(wl, "peak_scale", 1.0)
    h2d, d2h = wl.e2e_bytes()
    e2e_value = world * units / (e2e_total / args.steps * 1e-3) / scale

    cu, cdt, cdesc = wl.cpu_sample() if world == 1 else (None, None, None)
    cpu_baseline = None
    if cu is not None:
        cpu_baseline = {"value": cu / cdt / scale, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
                        "sample": cdesc}
    out = {
        "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": per_step_ms, "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(),
        "roofline": {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": wl.unit,
                     "frac": achieved / peak, "traffic": wl.traffic_bytes, "peak_source": peaks["source"] + (" (burst)" if getattr(wl, "peak_scale", 1.0) == 1.0 else " (burst) bf16 GEMM x 2 for e4m3"),
                     "min_ms": min(ms), "median_ms": statistics.median(ms)},
        "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "clocks": clocks,
        "gpu_launches": wl.launches_per_step * args.steps,
        "device_status": status,
    }
    if world > 1:
        dist.destroy_process_group()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="attn_noncausal", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200k", choices=["b200k", "reference"])
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]()
    if args.impl == "reference":
        out = run_reference(wl, args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the kernels have no CPU path (use --impl reference for the CPU arm)")
        out = run_ours(wl, args)
    if out:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
