"""Throughput benchmark for the GEMM / attention / decode kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--no-extras] [--impl reference]

The headline workload (``--workload``, default ``attn_causal``) is causal prefill attention bf16,
batch 4, 32 heads, S = 4096, head dim 128.  With N > 1 it is ONE problem sharded by heads (32 / N
heads of every batch element per GPU, no data-path collective): strong scaling.  The other
workloads of the metric -- ``gemm_f16`` (2048^3, fp32 out), ``attn_noncausal`` (f16 B8 H32 S1024),
``paged_decode`` (64 sequences, GQA 32/8, page 16) and ``gemm_fp8`` (8192^3 e4m3, bf16 out;
column-parallel over N with N > 1) -- and the backward of the headline problem
(``attn_bwd_causal``, a next-row of the path) are measured in the same run and reported under
``"workloads"`` in the same JSON line, each with its own roofline, end-to-end figure, CPU baseline
(N = 1) and a parity figure against the CPU oracle on a sampled slice (computed after the timed
region).  ``--no-extras`` measures the headline workload only.

A step is one pass of the kernel over one batch of synthetic inputs.  Each step is timed with
CUDA events on the launching stream; the inputs are larger than L2 (``config.l2`` says how; the
small GEMM walks through operand sets and replays its steps from a CUDA graph).  Timed regions are bracketed by
barrier + synchronize and the maximum over ranks is used.  Besides the per-step (burst) figure
a sustained leg runs the headline kernel back to back for at least a second, with the SM clock
sampled meanwhile, and is compared with the sustained cuBLAS figure of MEASURED_PEAKS.json.

``--impl reference`` times the CPU statement of the reference path on the host cores on a bounded
sample of the same workload (the faster of the oracle and torch's own CPU operator); rank 0 only.
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


def best_of(fn, n):
    best = None
    for _ in range(n):
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


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
    peak_scale = 1.0
    scaling = "strong"
    world, rank = 1, 0

    def shard(self, world: int, rank: int):
        self.world, self.rank = world, rank

    def config(self) -> dict: ...
    def setup(self, dev): ...
    def step(self): ...
    def units_per_step(self) -> float:
        """flops (tensor-bound) or bytes (hbm-bound) THIS RANK processes per step."""
    def setup_e2e(self, dev): ...
    def step_e2e(self): ...
    def e2e_bytes(self) -> tuple: ...
    def cpu_sample(self) -> tuple:
        """Runs the CPU statement on a bounded sample; returns (units processed, seconds, description)."""
    def parity(self) -> dict:
        """Compares the last step's result with the CPU oracle on a sampled slice (untimed)."""

    def release(self):
        for k in list(self.__dict__):
            if isinstance(self.__dict__[k], torch.Tensor) or k in ("e2e", "fused", "host", "grads", "sets", "used"):
                del self.__dict__[k]


def _close(got: torch.Tensor, ref: torch.Tensor, rtol=1e-2, atol=1e-2) -> dict:
    """max |got - ref| and the worst ratio to the allclose bound atol + rtol |ref| (<= 1 passes)."""
    d = (got.float().cpu() - ref.float()).abs()
    bound = atol + rtol * ref.float().abs()
    return {"max_abs_err": float(d.max()), "worst_over_bound": float((d / bound).max()), "rtol": rtol, "atol": atol,
            "ok": bool((d <= bound).all())}


class AttentionWL(Workload):
    def __init__(self, name, batch, heads, seq, dtype, causal, std, traffic=None):
        self.name = name
        self.traffic_bytes = traffic
        self.b, self.h, self.s = batch, heads, seq
        self.h_local, self.h0 = heads, 0
        self.tdtype = dtype
        self.dtype = "f16" if dtype == torch.float16 else "bf16"
        self.causal = causal
        self.std = std
        kind = "causal" if causal else "non-causal"
        self.metric = f"attention fwd TFLOP/s ({kind} {self.dtype} B{batch} H{heads} S{seq} D128)"

    def shard(self, world, rank):
        from iree_turbine_b200 import dist as tdist

        super().shard(world, rank)
        if self.h % world:
            raise SystemExit(f"bench.py: {self.h} heads cannot be split evenly over {world} GPUs")
        self.h0, h1 = tdist.shard_range(self.h, world, rank)
        self.h_local = h1 - self.h0

    def config(self):
        nbytes = 4 * self.b * self.h_local * self.s * 128 * 2
        cfg = {"workload": self.name, "batch": self.b, "heads": self.h, "seq_q": self.s, "seq_kv": self.s,
               "head_dim": 128, "causal": self.causal, "scale": SCALE,
               "l2": f"inputs larger than L2 ({nbytes / 1e6:.0f} MB touched per step and GPU)"}
        if self.world > 1:
            cfg["parallelism"] = (f"one problem, heads sharded over {self.world} GPUs ({self.h_local} heads of every "
                                  "batch element per GPU), no collective")
            if nbytes < 200e6:
                cfg["l2"] = f"L2 flushed between steps (256 MB write); {nbytes / 1e6:.0f} MB touched per step and GPU"
        return cfg

    @property
    def needs_flush(self):
        return 4 * self.b * self.h_local * self.s * 128 * 2 < 200e6

    def _make(self, dev, seed=10):
        """The whole problem from one seed (identical on every rank), then this rank's heads."""
        g = torch.Generator(device=dev).manual_seed(seed)
        out = []
        for _ in range(3):
            t = (torch.randn(self.b, self.h, self.s, 128, generator=g, device=dev) * self.std).to(self.tdtype)
            out.append(t[:, self.h0:self.h0 + self.h_local].contiguous())
        return out

    def setup(self, dev):
        self.q, self.k, self.v = self._make(dev)

    def step(self):
        self.o = torch.ops.b200k.attention(self.q, self.k, self.v, SCALE, self.causal)

    def units_per_step(self):
        f = 4.0 * self.b * self.h_local * self.s * self.s * 128
        return f / 2 if self.causal else f

    def setup_e2e(self, dev):
        from iree_turbine_b200 import host_api

        self.hq, self.hk, self.hv = (t.cpu().pin_memory() for t in (self.q, self.k, self.v))
        self.ho = torch.empty_like(self.hq).pin_memory()
        self.e2e = host_api.AttentionHost(self.b, self.h_local, self.h_local, self.s, self.s, self.tdtype, dev)

    def step_e2e(self):
        self.e2e(self.hq, self.hk, self.hv, self.ho, SCALE, self.causal)

    def e2e_bytes(self):
        n = self.b * self.h_local * self.s * 128 * 2
        return 3 * n, n

    def cpu_sample(self, heads=None):
        """The faster of the two CPU statements of the same math: the oracle (scores materialised)
        and torch's fused CPU operator on fp32 upcasts."""
        from oracle import oracle

        bs = 1
        hs = heads if heads is not None else min(self.h, 16 if self.s > 2048 else 32)
        q, k, v = oracle.make_attention_inputs(bs, hs, hs, self.s, self.s, 128, self.tdtype, seed=10, std=self.std)
        qf, kf, vf = q.float(), k.float(), v.float()
        t_sdpa = best_of(lambda: torch.nn.functional.scaled_dot_product_attention(
            qf, kf, vf, is_causal=self.causal, scale=SCALE), 2)
        t_oracle = best_of(lambda: oracle.attention(q, k, v, SCALE, self.causal), 1)
        f = 4.0 * bs * hs * self.s * self.s * 128
        f = f / 2 if self.causal else f
        which = "torch CPU scaled_dot_product_attention on fp32 upcasts" if t_sdpa <= t_oracle else "oracle.attention"
        return f, min(t_sdpa, t_oracle), (f"{which} (the faster of the two; the other took "
                                          f"{max(t_sdpa, t_oracle):.2f} s) on batch {bs} x {hs} heads of the same shape")

    def parity(self):
        from oracle import oracle

        picks = [(0, 0), (self.b - 1, self.h_local - 1)]
        worst = None
        for b, h in picks:
            ref = oracle.attention(self.q[b:b + 1, h:h + 1].cpu(), self.k[b:b + 1, h:h + 1].cpu(),
                                   self.v[b:b + 1, h:h + 1].cpu(), SCALE, self.causal)
            r = _close(self.o[b:b + 1, h:h + 1], ref)
            if worst is None or r["worst_over_bound"] > worst["worst_over_bound"]:
                worst = r
        worst["sample"] = f"(batch, local head) {picks} of this rank's output against oracle.attention"
        return worst


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
        t = torch.randn(self.b, self.h, self.s, 128, generator=g, device=dev).to(self.tdtype)
        return t[:, self.h0:self.h0 + self.h_local].contiguous()

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
        n = self.b * self.h_local * self.s * 128 * 2
        return 5 * n + self.b * self.h_local * self.s * 4, 3 * n

    def cpu_sample(self):
        from oracle import oracle

        bs, hs = 1, min(self.h, 4 if self.s > 2048 else 16)
        q, k, v = oracle.make_attention_inputs(bs, hs, hs, self.s, self.s, 128, self.tdtype, seed=10, std=self.std)
        d_o = torch.randn(q.shape, generator=torch.Generator().manual_seed(11)).to(self.tdtype)
        best = best_of(lambda: oracle.attention_bwd(q, k, v, d_o, SCALE, self.causal), 2)
        f = 2.5 * 4.0 * bs * hs * self.s * self.s * 128
        f = f / 2 if self.causal else f
        return f, best, f"oracle.attention_bwd on batch {bs} x {hs} heads of the same shape, best of 2"

    def parity(self):
        from oracle import oracle

        b, h = self.b - 1, self.h_local - 1
        sl = (slice(b, b + 1), slice(h, h + 1))
        refs = oracle.attention_bwd(self.q[sl].cpu(), self.k[sl].cpu(), self.v[sl].cpu(), self.d_o[sl].cpu(), SCALE,
                                    self.causal)
        worst = 0.0
        for got, ref in zip(self.grads, refs):
            worst = max(worst, float((got[sl].float().cpu() - ref).abs().max() / max(float(ref.abs().max()), 1.0)))
        return {"max_err_over_max_ref": worst, "tol": 1e-2, "ok": worst <= 1e-2,
                "sample": f"(batch, local head) ({b}, {h}): dQ, dK, dV against oracle.attention_bwd"}


class GemmWL(Workload):
    def __init__(self, name, n, fp8, mode="fused_gather"):
        self.name, self.n, self.fp8 = name, n, fp8
        self.mode = mode  # N > 1, fp8 only: "shard_only" | "fused_gather" | "fused_gather_multimem" | "nccl_gather"
        self.traffic_bytes = 417.1e6 if (fp8 and n == 8192) else (16.9e6 if (not fp8 and n == 2048) else None)
        # the measured peak is a bf16 GEMM; e4m3 runs the tensor pipe at twice that rate
        self.peak_scale = 2.0 if fp8 else 1.0
        self.dtype = "e4m3" if fp8 else "f16"
        out = "bf16" if fp8 else "f32"
        self.metric = f"GEMM TFLOP/s ({self.dtype} NT M=N=K={n}, fp32 accumulate, {out} out)"
        # Operands smaller than L2 (the 2048^3 problem: 16.8 MB): the steps walk through enough
        # operand sets that a set has left L2 before it is used again, and are launched back to back
        # (no flush kernel in between, one CUDA-event pair around the K steps), which is how a chain
        # of GEMMs runs; the kernel's programmatic dependent launch needs consecutive launches.
        operand_bytes = 2 * n * n * (1 if fp8 else 2)
        self.num_sets = 1 if fp8 or operand_bytes >= 200e6 else -(-320_000_000 // operand_bytes)
        self.back_to_back = self.num_sets > 1
        self.needs_flush = False
        self.turn = 0

    def shard(self, world, rank):
        # fp8 GEMM: column-parallel over N (strong scaling).  f16 2048^3 is too small to shard:
        # independent replicas (weak scaling), every rank the whole problem.
        super().shard(world, rank)
        if not self.fp8:
            self.scaling = "weak"

    @property
    def sharded(self):
        return self.fp8 and self.world > 1

    def config(self):
        cfg = {"workload": self.name, "m": self.n, "n": self.n, "k": self.n,
               "l2": (f"{self.num_sets} operand sets used in turn ({self.num_sets * 2 * self.n * self.n * 2 / 1e6:.0f} MB "
                      "between two uses of a set), launches back to back" if self.num_sets > 1
                      else "operands larger than L2")}
        if self.sharded:
            how = {"shard_only": "column shards of C left in place (no exchange)",
                   "fused_gather": "all-gather of C fused into the GEMM epilogue (peer stores) + cross-rank barrier "
                                   "inside the timed step",
                   "fused_gather_multimem": "all-gather of C fused into the GEMM epilogue (one multimem.st per piece "
                                            "through the NVSwitch multicast address) + cross-rank barrier inside "
                                            "the timed step",
                   "nccl_gather": "local GEMM, then NCCL all-gather of C + de-interleaving copy inside the timed step"}
            cfg["parallelism"] = f"column-parallel over N on {self.world} GPUs, {how[self.mode]}"
        elif self.world > 1:
            cfg["parallelism"] = f"{self.world} independent replicas of the whole problem"
        return cfg

    def setup(self, dev):
        g = torch.Generator(device=dev).manual_seed(10)
        a = torch.randn(self.n, self.n, generator=g, device=dev)
        b = torch.randn(self.n, self.n, generator=g, device=dev)
        if self.fp8:
            self.a, self.sa = torch.ops.b200k.quantize_e4m3(a)
            self.b, self.sb = torch.ops.b200k.quantize_e4m3(b)
        else:
            self.a, self.b = a.half(), b.half()
            self.sets = [(self.a, self.b)]
            for _ in range(self.num_sets - 1):
                self.sets.append((torch.randn(self.n, self.n, generator=g, device=dev).half(),
                                  torch.randn(self.n, self.n, generator=g, device=dev).half()))
        del a, b
        self.col0 = 0
        if self.sharded:
            from iree_turbine_b200 import dist as tdist

            lo, hi = tdist.shard_range(self.n, self.world, self.rank)
            self.col0 = lo
            self.b = self.b[lo:hi].contiguous()
            if self.mode.startswith("fused_gather"):
                self.fused = tdist.FusedColumnParallelGemm(self.n, self.n, torch.bfloat16,
                                                           multicast=self.mode.endswith("multimem"))

    def step(self):
        if self.sharded and self.mode.startswith("fused_gather"):
            self.fused(self.a, self.b, self.sa, self.sb)
            self.c = self.fused.finish()
        elif self.sharded and self.mode == "nccl_gather":
            from iree_turbine_b200 import dist as tdist

            self.c = tdist.gather_columns(torch.ops.b200k.gemm_fp8_nt(self.a, self.b, self.sa, self.sb))
        elif self.fp8:
            self.c = torch.ops.b200k.gemm_fp8_nt(self.a, self.b, self.sa, self.sb)
        else:
            self.used = self.sets[self.turn % self.num_sets]
            self.turn += 1
            self.c = torch.ops.b200k.gemm_nt(*self.used)

    def units_per_step(self):
        return 2.0 * self.n ** 3 / (self.world if self.sharded else 1)

    def setup_e2e(self, dev):
        from iree_turbine_b200 import host_api

        self.ha, self.hb = self.a.cpu().pin_memory(), self.b.cpu().pin_memory()
        if self.sharded:
            # sharded run: the rank's operands come from pinned host memory each step, the full C
            # (or the rank's shard, when it stays in place) is read back by every rank
            cols = self.b.size(0) if self.mode == "shard_only" else self.n
            self.hc = torch.empty(self.n, cols, dtype=torch.bfloat16).pin_memory()
            return
        out_dtype = torch.bfloat16 if self.fp8 else torch.float32
        self.hc = torch.empty(self.n, self.n, dtype=out_dtype).pin_memory()
        self.e2e = host_api.GemmHost(self.n, self.n, self.n, self.a.dtype, out_dtype, dev)

    def step_e2e(self):
        if self.sharded:
            self.a.copy_(self.ha, non_blocking=True)
            self.b.copy_(self.hb, non_blocking=True)
            self.step()
            self.hc.copy_(self.c, non_blocking=True)
        elif self.fp8:
            self.e2e(self.ha, self.hb, self.hc, self.sa, self.sb)
        else:
            self.e2e(self.ha, self.hb, self.hc)

    def e2e_bytes(self):
        es = 1 if self.fp8 else 2
        if self.sharded:
            return self.n * self.n * es + self.b.numel() * es, self.hc.numel() * 2
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
        best = best_of(fn, 3)
        return 2.0 * rows * self.n * self.n, best, f"oracle GEMM on {rows} rows of A against all of B, best of 3"

    def parity(self):
        from oracle import oracle

        rows = 128
        r0 = self.n - rows
        if not self.fp8:
            a, b = self.used[0][r0:].cpu(), self.used[1].cpu()  # the operand set of the last step
        else:
            a, b = self.a[r0:].cpu(), self.b.cpu()
        if not self.fp8:
            r = _close(self.c[r0:], oracle.gemm_nt(a, b))
            r["sample"] = f"last {rows} rows of C against oracle.gemm_nt"
            return r
        ref = oracle.gemm_fp8_nt(a, b, self.sa.cpu(), self.sb.cpu())  # this rank's columns
        got = self.c[r0:]
        what = "this rank's column shard"
        if self.sharded and self.mode != "shard_only":
            # the gathered matrix: this rank's own columns against the oracle, and every column
            # against the rank that computed it (all ranks must hold identical bits)
            import torch.distributed as dist

            mine = got[:, self.col0:self.col0 + self.b.size(0)]
            digest = got.view(torch.int16).to(torch.int64).sum().reshape(1)
            lo, hi = digest.clone(), digest.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            same = bool((lo == hi).item())
            got = mine
            what = "this rank's columns of the GATHERED matrix"
        else:
            same = None
        fro, mx = oracle.fp8_errors(got, ref)
        out = {"rel_frobenius": fro, "max_abs_over_rms": mx, "tol": 3e-2, "ok": fro <= 3e-2 and mx <= 3e-2,
               "sample": f"last {rows} rows, {what}, against oracle.gemm_fp8_nt"}
        if same is not None:
            out["gathered_rows_identical_on_all_ranks"] = same
            out["ok"] = out["ok"] and same
        return out


class PagedDecodeWL(Workload):
    unit = "GB/s"
    bound = "hbm"
    launches_per_step = 2
    metric = "paged-decode HBM GB/s (f16, 64 seqs, 32 q-heads / 8 kv-heads, D128, len U[512,8192], page 16)"

    traffic_bytes = 1179.2e6

    def __init__(self, name):
        self.name = name

    def config(self):
        cfg = {"workload": self.name, "num_seqs": 64, "q_heads": 32, "kv_heads": 8, "head_dim": 128, "page_size": 16,
               "len_range": [512, 8192], "sum_len": int(self.sum_len) if hasattr(self, "sum_len") else None,
               "l2": "KV pool larger than L2 (about 1.1 GB read per step)"}
        if self.world > 1:
            cfg["parallelism"] = (f"one problem, KV heads sharded over {self.world} GPUs ({8 // self.world} KV heads and "
                                  "their query heads per GPU, the rank's slice of the page pool resident), "
                                  "no collective")
            cfg["l2"] = "L2 flushed between steps (256 MB write)"
        return cfg

    @property
    def needs_flush(self):
        return self.world > 1

    def _host_inputs(self):
        from oracle import oracle

        return oracle.make_paged_decode_inputs(seed=10)

    def setup(self, dev):
        """N > 1: one problem sharded by KV head (8 KV heads, so N <= 8): a rank holds its heads' slice
        of the page pool and the matching query heads of every sequence -- equal bytes on every rank
        whatever the sequence lengths are."""
        from iree_turbine_b200 import dist as tdist

        q, kc, vc, bt, sl = self._host_inputs()
        lo, hi = tdist.shard_range(8, self.world, self.rank)
        q = q[:, lo * 4:hi * 4].contiguous()
        kc, vc = kc[:, lo:hi].contiguous(), vc[:, lo:hi].contiguous()
        self.kv_heads = hi - lo
        self.sum_len = int(sl.sum())
        self.pages = int(((sl + 15) // 16).sum())
        self.host = (q, kc, vc, bt, sl)
        self.q, self.kc, self.vc, self.bt, self.sl = (t.to(dev) for t in (q, kc, vc, bt, sl))

    def step(self):
        self.o = torch.ops.b200k.paged_decode_attention(self.q, self.kc, self.vc, self.bt, self.sl, SCALE)

    def units_per_step(self):
        # K and V rows actually read + Q and O + block-table entries + seq_lens
        return self.sum_len * self.kv_heads * 128 * 2 * 2 + 2 * self.q.numel() * 2 + 4 * self.pages + 4 * self.sl.numel()

    def setup_e2e(self, dev):
        # The KV pool is state that lives on the device across decode steps; per step the host
        # provides the query, the block table and the lengths and reads the output back.
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

    def parity(self):
        from oracle import oracle

        q, kc, vc, bt, sl = self.host
        n = q.size(0)
        picks = sorted({0, n - 1, int(sl.argmax()), int(sl.argmin())})
        sub = torch.tensor(picks)
        ref = oracle.paged_decode_attention(q[sub], kc, vc, bt[sub], sl[sub], SCALE)
        r = _close(self.o[sub.to(self.o.device)], ref)
        r["sample"] = f"sequences {picks} of this rank (first, last, longest, shortest) against the oracle"
        return r


WORKLOADS = {
    "attn_causal": lambda: AttentionWL("attn_causal", 4, 32, 4096, torch.bfloat16, True, 0.5, 528.2e6),
    "attn_noncausal": lambda: AttentionWL("attn_noncausal", 8, 32, 1024, torch.float16, False, 1.0, 249.1e6),
    "attn_bwd_causal": lambda: AttentionBwdWL("attn_bwd_causal", 4, 32, 4096, torch.bfloat16, True, 0.5),
    "gemm_f16": lambda: GemmWL("gemm_f16", 2048, False),
    "gemm_fp8": lambda: GemmWL("gemm_fp8", 8192, True),
    "gemm_fp8_shard_only": lambda: GemmWL("gemm_fp8_shard_only", 8192, True, "shard_only"),
    "gemm_fp8_nccl_gather": lambda: GemmWL("gemm_fp8_nccl_gather", 8192, True, "nccl_gather"),
    "gemm_fp8_multimem": lambda: GemmWL("gemm_fp8_multimem", 8192, True, "fused_gather_multimem"),
    "paged_decode": lambda: PagedDecodeWL("paged_decode"),
}
DEFAULT = "attn_causal"
# the other configurations of the metric, measured in the same run
EXTRAS = ["gemm_f16", "attn_noncausal", "paged_decode", "gemm_fp8", "attn_bwd_causal"]


# ---------------------------------------------------------------------------------------------
# clocks sampler
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU every `period_ms` through NVML (read-only
    queries) on a background thread, from start() to close(); window(t0, t1) summarises the samples
    taken between two time.monotonic() stamps.  "Under load" = samples while the GPU-idle reason
    was not set.  Falls back to an nvidia-smi query loop if NVML cannot be loaded."""

    REASONS = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}
    IDLE = 0x1

    def __init__(self, index: int, period_ms: float = 2.0):
        self.index, self.period = index, period_ms * 1e-3
        self.samples = []  # (monotonic time, sm MHz, reason bits)
        self.max_mhz = None
        self.how = None
        self._stop = threading.Event()
        self.thread = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)

            def loop():
                while not self._stop.is_set():
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                        bits = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                        self.samples.append((time.monotonic(), mhz, bits))
                    except Exception:  # noqa: BLE001 - a failed read is a missing sample
                        pass
                    time.sleep(self.period)

            self.how = "nvml"
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self._start_smi()
        return self

    def _start_smi(self):
        fields = ("clocks.sm,clocks.max.sm,clocks_event_reasons.gpu_idle,clocks_event_reasons.sw_power_cap,"
                  "clocks_event_reasons.hw_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                  "clocks_event_reasons.hw_thermal_slowdown")
        try:
            proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={fields}",
                                     "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                    stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.how = "nvidia-smi"

        def loop():
            bit = [self.IDLE, 0x4, 0x8, 0x20, 0x40]
            for line in proc.stdout:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) == 7 and parts[0].isdigit():
                    self.max_mhz = int(parts[1]) if parts[1].isdigit() else self.max_mhz
                    bits = sum(b for b, v in zip(bit, parts[2:]) if v == "Active")
                    self.samples.append((time.monotonic(), int(parts[0]), bits))
                if self._stop.is_set():
                    break
            proc.terminate()

        self.thread = threading.Thread(target=loop, daemon=True)
        self.thread.start()

    def window(self, t0: float, t1: float) -> dict:
        if self.how is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}
        rows = [s for s in self.samples if t0 <= s[0] <= t1]
        busy = [s for s in rows if not (s[2] & self.IDLE)]
        use = busy if busy else rows
        reasons = [n for n, b in self.REASONS.items() if any(s[2] & b for s in rows)]
        return {"sm_mhz": statistics.median(s[1] for s in use) if use else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(rows), "samples_under_load": len(busy), "how": self.how}

    def close(self):
        self._stop.set()


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
        "scaling": wl.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def queued_launches(step_fn, steps):
    """A callable that runs `steps` steps at the GPU's pace rather than the host's (a step of 17 us is
    shorter than a Python call through the operator): the steps captured once in a CUDA graph and
    replayed; if capture is refused, a plain loop queued behind a spin kernel.  Returns (run, how)."""
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(steps):
                step_fn()
        torch.cuda.synchronize()
        return graph.replay, f"{steps} steps captured in one CUDA graph, replayed once"
    except Exception as e:  # noqa: BLE001 - any capture failure falls back to the plain loop
        torch.cuda.synchronize()
        why = str(e).splitlines()[0][:80]

        def run():
            torch.cuda._sleep(int(4e6))  # ~2 ms: the launches below are all queued before it ends
            for _ in range(steps):
                step_fn()

        return run, f"plain loop queued behind a spin kernel (graph capture refused: {why})"


def timed_steps(step_fn, steps, warmup, flush_buf, stream, back_to_back=False):
    """Runs warmup + steps; returns per-step milliseconds measured with CUDA events on `stream`.
    back_to_back: nothing is put between the launches, one event pair brackets the K steps and every
    step is given the mean."""
    for _ in range(warmup):
        if flush_buf is not None:
            flush_buf.fill_(1)
        step_fn()
    torch.cuda.synchronize()
    if back_to_back and flush_buf is None:
        run, how = queued_launches(step_fn, steps)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        run()
        e1.record(stream)
        torch.cuda.synchronize()
        timed_steps.how = how
        return [e0.elapsed_time(e1) / steps] * steps
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


class Ctx:
    """Process-wide state of one bench run: ranks, device, peaks, the L2-flush buffer."""

    def __init__(self):
        import torch.distributed as dist

        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = torch.device("cuda", self.local)
        torch.cuda.set_device(self.dev)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = load_peaks()
        self.stream = torch.cuda.current_stream()
        self.flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=self.dev)
        self.sampler = ClockSampler(self.local).start() if self.rank == 0 else None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(self, ok: bool) -> bool:
        if self.world == 1:
            return ok
        t = torch.tensor([1 if ok else 0], device=self.dev, dtype=torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())


def measure(wl: Workload, ctx: Ctx, steps: int, warmup: int, with_cpu: bool, sustained_s: float = 0.0) -> dict:
    """One workload: device-timed steps, parity against the oracle, the end-to-end leg, the CPU
    baseline (N = 1 only) and, for the headline workload, the sustained leg.  Rank 0's dictionary is
    complete; timings are the maximum over ranks."""
    import iree_turbine_b200 as tb

    world = ctx.world
    if world > 1:
        wl.shard(world, ctx.rank)
    wl.setup(ctx.dev)
    units = wl.units_per_step()
    all_units = units * world  # whole-job units per step: every rank does `units`
    scale = 1e12 if wl.unit == "TFLOP/s" else 1e9
    flush = ctx.flush if wl.needs_flush else None

    ctx.barrier()
    t_begin = time.monotonic()
    ms = timed_steps(wl.step, steps, warmup, flush, ctx.stream, getattr(wl, "back_to_back", False))
    ctx.barrier()
    clocks = ctx.sampler.window(t_begin, time.monotonic()) if ctx.sampler else None
    total_ms = ctx.max_over_ranks(sum(ms))
    status = tb.device_status()

    par = wl.parity()
    par["ok_on_all_ranks"] = ctx.all_ok(bool(par.get("ok")))

    sustained = None
    if sustained_s > 0:
        # back-to-back launches for >= sustained_s seconds, one event pair around the whole loop
        n = max(steps, int(sustained_s * 1e3 / max(statistics.median(ms), 1e-3)) + 1)
        ctx.barrier()
        t_begin = time.monotonic()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if getattr(wl, "back_to_back", False):
            chunk = 100
            run, _ = queued_launches(wl.step, chunk)
            n = -(-n // chunk) * chunk
            e0.record(ctx.stream)
            for _ in range(n // chunk):
                run()
            e1.record(ctx.stream)
        else:
            e0.record(ctx.stream)
            for _ in range(n):
                wl.step()
            e1.record(ctx.stream)
        ctx.barrier()
        loop_ms = ctx.max_over_ranks(e0.elapsed_time(e1))
        c2 = ctx.sampler.window(t_begin, time.monotonic()) if ctx.sampler else None
        val = all_units * n / (loop_ms * 1e-3) / scale
        peak_s = ctx.peaks["tflops_sustained"] * wl.peak_scale if wl.bound == "tensor" else ctx.peaks["hbm_gbs"]
        sustained = {"value": val, "unit": wl.unit, "launches": n, "seconds": loop_ms * 1e-3,
                     "ms_per_step": loop_ms / n, "clocks": c2,
                     "frac_of_sustained_peak": val / world / peak_s,
                     "sustained_peak": peak_s, "peak_source": ctx.peaks["source"] + " (sustained)",
                     "note": "back-to-back launches, no L2 flush in between; one CUDA-event pair around the loop"}

    # end-to-end through the host-buffer API (copies inside the timed region)
    wl.setup_e2e(ctx.dev)
    ctx.barrier()
    e2e_ms = timed_steps(wl.step_e2e, steps, warmup, None, ctx.stream)
    ctx.barrier()
    e2e_total = ctx.max_over_ranks(sum(e2e_ms))
    h2d, d2h = wl.e2e_bytes()

    cpu_baseline = None
    if with_cpu and world == 1:
        cu, cdt, cdesc = wl.cpu_sample()
        cpu_baseline = {"value": cu / cdt / scale, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
                        "sample": cdesc}

    per_step_ms = total_ms / steps
    kernel_ms = statistics.mean(ms)
    achieved = units / (kernel_ms * 1e-3) / scale
    peak = ctx.peaks["hbm_gbs"] if wl.bound == "hbm" else ctx.peaks["tflops"] * wl.peak_scale
    out = {
        "metric": wl.metric, "value": all_units / (per_step_ms * 1e-3) / scale, "unit": wl.unit, "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": per_step_ms, "higher_is_better": True,
        "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(),
        "roofline": {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": wl.unit,
                     "frac": achieved / peak, "traffic": wl.traffic_bytes,
                     "peak_source": ctx.peaks["source"] + (" (burst)" if wl.peak_scale == 1.0 else
                                                            " (burst) bf16 GEMM x 2 for e4m3"),
                     "min_ms": min(ms), "median_ms": statistics.median(ms),
                     "note": "per rank: this rank's units / its mean step time"},
        "parity": par,
        "cpu_baseline": cpu_baseline,
        "e2e": {"value": all_units / (e2e_total / steps * 1e-3) / scale, "unit": wl.unit,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "clocks": clocks,
        "gpu_launches": wl.launches_per_step * steps,
        "device_status": status,
    }
    if getattr(wl, "back_to_back", False):
        out["config"]["timed_region"] = getattr(timed_steps, "how", "") + "; one CUDA-event pair around the K steps"
    if wl.scaling == "weak" and world > 1:
        out["note"] = "independent replicas: value = N x one rank's units / max time"
    if sustained:
        out["sustained"] = sustained
    wl.release()
    torch.cuda.empty_cache()
    return out


def run_ours(args) -> dict:
    ctx = Ctx()
    torch.set_num_threads(os.cpu_count() or 1)
    steps, warmup = args.steps, max(args.warmup, 3)
    main = measure(WORKLOADS[args.workload](), ctx, steps, warmup, with_cpu=True, sustained_s=args.sustained)
    if not args.no_extras:
        extras = {}
        names = [n for n in EXTRAS if n != args.workload]
        if args.workload != DEFAULT:
            names.insert(0, DEFAULT)
        for name in names:
            if name == "gemm_fp8" and ctx.world > 1:
                # the one workload with an exchange step: three legs
                legs = {}
                for leg in ("gemm_fp8_shard_only", "gemm_fp8", "gemm_fp8_multimem", "gemm_fp8_nccl_gather"):
                    try:
                        legs[WORKLOADS[leg]().mode] = measure(WORKLOADS[leg](), ctx, steps, warmup, with_cpu=False)
                    except RuntimeError as e:  # no multicast address on this box: every rank raises alike
                        legs[WORKLOADS[leg]().mode] = {"unavailable": str(e)}
                extras[name] = {"legs": legs}
            else:
                extras[name] = measure(WORKLOADS[name](), ctx, steps, warmup, with_cpu=True)
        main["workloads"] = extras
    if ctx.sampler:
        ctx.sampler.close()
    if ctx.world > 1:
        ctx.dist.destroy_process_group()
    return main if ctx.rank == 0 else {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="measure the headline workload only")
    ap.add_argument("--sustained", type=float, default=1.0,
                    help="seconds of back-to-back launches for the sustained leg (0 = skip)")
    ap.add_argument("--impl", default="b200k", choices=["b200k", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        out = run_reference(WORKLOADS[args.workload](), args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the kernels have no CPU path (use --impl reference for the CPU arm)")
        out = run_ours(args)
    if out:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
