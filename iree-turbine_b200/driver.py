"""Command-line bench driver that speaks the reference driver's language.

It accepts the MIOpen-style and aten-style command lines the reference's ``iree-boo-driver``
accepts for the ops this library covers, and writes the same CSV, so results line up column by
column with the reference's (iree/turbine/kernel/boo/driver/driver.py:213-244: a column
``arguments`` holding the command, then ``"<backend> {min,max,mean,stddev,num_dispatches}"`` per
backend; the header contract is checked in tests/kernel/boo/driver/csv_output_test.py:11-24).

Commands:

* ``gemmfp16 --a_w M --a_h K --b_w N [--transA 0|1] [--transB 0|1] [-F 1]`` (and ``gemm`` for
  float32).  The flag meanings are the reference parser's, not its help text's: it builds
  ``a_shape = [a_w, a_h]``, ``b_shape = [a_h, b_w]`` and reads ``m, k = a_shape``
  (kernel/boo/op_exports/gemm.py:104-107,150-214), so ``--a_w`` is M, ``--a_h`` is K and
  ``--b_w`` is N, whatever the short flags ``-k/-m/-n`` suggest.  With ``--transA 1`` A is stored
  [K, M] and transposed in the op; with ``--transB 1`` B is stored [N, K] (gemm.py:217-230).
* ``aten::mm "<dims>" "<types>" "<strides>" "<concrete>"`` and ``aten::scaled_dot_product_attention
  ...`` in the reference's profiler-style format (kernel/boo/op_exports/aten.py:176-198,
  driver/sample_commands.txt:22,26): operands are created with exactly the given strides.

Backends: ``b200k`` (default; this library's kernels) and ``torch`` (the ATen op on the same
device).  The GEMM kernel reads either storage order of each operand ([M, K] or [K, M]; [K, N] or
[N, K]), so the four transA / transB forms run as given; an operand with no contiguous dimension is
repacked once before timing, and the line printed for the command says so.
A command or backend that cannot run (float32 GEMM, head dim other than 128 / 64, a mask, ...) gets
``N.A.`` in its columns, as in the reference.  Times are microseconds per call, measured with CUDA
events on the current stream after 3 untimed calls.  There is no CPU path.
"""

from __future__ import annotations

import argparse
import ast
import csv
import math
import os
import shlex
import statistics
import sys
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

__all__ = ["ALL_STATS", "DEFAULT_BACKEND", "BACKENDS", "GemmCommand", "AtenCommand", "parse_command", "main"]

ALL_STATS = ["min", "max", "mean", "stddev", "num_dispatches"]
DEFAULT_BACKEND = "b200k"
BACKENDS = ("b200k", "torch")
_GEMM_DTYPES = {"gemm": torch.float32, "gemmfp16": torch.float16}
_ATEN_DTYPES = {
    "c10::BFloat16": torch.bfloat16,
    "c10::Half": torch.float16,
    "float": torch.float32,
    "double": torch.float64,
}
SEED = 10  # the reference driver's seed for sample arguments (driver/driver.py:612)


class Unsupported(Exception):
    """The command is well formed but this backend does not cover it."""


# ---------------------------------------------------------------------------------------------
# command parsing (no GPU needed)
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class GemmCommand:
    m: int
    k: int
    n: int
    transpose_a: bool
    transpose_b: bool
    dtype: torch.dtype
    mode: int  # 1 forward; 2 / 3 the reference's backward products (dA, dB)

    @property
    def func_name(self) -> str:
        """The reference's kernel name for this problem (gemm.py:104-117)."""
        items = ["gemm", str(self.dtype).removeprefix("torch."), {1: "forward", 2: "a_backward", 3: "b_backward"}[self.mode],
                 f"{self.m}x{self.k}x{self.n}"]
        if self.transpose_a:
            items.append("transA")
        if self.transpose_b:
            items.append("transB")
        return "_".join(items)


@dataclass(frozen=True)
class AtenCommand:
    name: str  # e.g. "aten::mm"
    input_dims: list
    input_type: list
    input_strides: list
    concrete_inputs: list


def _gemm_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="gemm", add_help=False)
    p.add_argument("command", choices=list(_GEMM_DTYPES))
    p.add_argument("--a_w", "-k", type=int, default=256)
    p.add_argument("--a_h", "-m", type=int, default=256)
    p.add_argument("--b_w", "-n", type=int, default=256)
    p.add_argument("--transA", "-u", type=int, default=0)
    p.add_argument("--transB", "-v", type=int, default=0)
    p.add_argument("--forw", "-F", type=int, default=1)
    return p


def _aten_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="aten", add_help=False)
    for name in ("name", "input_dims", "input_type", "input_strides", "concrete_inputs"):
        p.add_argument(name)
    return p


def timing_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(add_help=False)
    p.add_argument("--time", "-t", type=int, default=1)
    p.add_argument("--iter", type=int, default=100)
    return p


def parse_command(argv: Sequence[str]):
    """One command (timing flags already removed) -> GemmCommand or AtenCommand."""
    if not argv:
        raise ValueError("empty command")
    head = argv[0]
    if head in _GEMM_DTYPES:
        a = _gemm_parser().parse_args(list(argv))
        if min(a.a_w, a.a_h, a.b_w) <= 0:
            raise ValueError(f"matrix sizes must be positive: {shlex.join(argv)}")
        if a.forw not in (1, 2, 3):
            raise ValueError(f"Unsupported mode {a.forw}.")
        return GemmCommand(m=a.a_w, k=a.a_h, n=a.b_w, transpose_a=bool(a.transA), transpose_b=bool(a.transB),
                           dtype=_GEMM_DTYPES[head], mode=a.forw)
    if head.startswith("aten::"):
        a = _aten_parser().parse_args(list(argv))
        return AtenCommand(a.name, ast.literal_eval(a.input_dims), ast.literal_eval(a.input_type),
                           ast.literal_eval(a.input_strides), ast.literal_eval(a.concrete_inputs))
    raise ValueError(f"unknown command {head!r}")


# ---------------------------------------------------------------------------------------------
# building the callables
# ---------------------------------------------------------------------------------------------
def _randn_strided(dims, strides, dtype, device, gen) -> torch.Tensor:
    size = 1 + sum((d - 1) * s for d, s in zip(dims, strides)) if dims else 1
    base = torch.randn(size, generator=gen, device=device, dtype=torch.float32).to(dtype)
    return torch.as_strided(base, dims, strides)


def _fp64_cpu(*tensors):
    return [t.detach().cpu().double() if isinstance(t, torch.Tensor) else t for t in tensors]


def _rows_contiguous(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.size(1)


def _mm_callable(backend: str, a: torch.Tensor, b: torch.Tensor, notes: List[str]) -> Callable[[], torch.Tensor]:
    """a [M, K], b [K, N] as the op sees them (views with arbitrary strides)."""
    if backend == "torch":
        return lambda: torch.mm(a, b)
    if backend == "cpu_fp64":
        a64, b64 = _fp64_cpu(a, b)
        return lambda: torch.mm(a64, b64)
    if a.dtype not in (torch.float16, torch.bfloat16) or a.dtype != b.dtype:
        raise Unsupported(f"b200k GEMM takes float16 / bfloat16 operands, not {a.dtype}")
    # the kernel reads either storage order of each operand; only a layout with no contiguous
    # dimension (or rows that are not 16-byte multiples) is repacked, once, before timing
    def pick(t: torch.Tensor, what: str):
        if _rows_contiguous(t) and t.stride(0) % 8 == 0 and t.size(1) % 8 == 0:
            return t, False
        tt = t.t()
        if _rows_contiguous(tt) and tt.stride(0) % 8 == 0 and tt.size(1) % 8 == 0:
            return tt, True
        notes.append(f"{what} repacked to contiguous rows before timing")
        return t.contiguous(), False

    a_s, ta = pick(a, "A")
    b_s, tb_ = pick(b, "B")
    return lambda: torch.ops.b200k.gemm(a_s, b_s, ta, tb_, a.dtype)


def build_callable(cmd, backend: str, device, notes: List[str], fill: Optional[str] = None) -> Callable[[], torch.Tensor]:
    """``backend``: "b200k", "torch" (the vendor kernel on the same device) or "cpu_fp64" (the torch
    operator on CPU in float64: the reference value of the numerics report).  ``fill``: None = seeded
    normal operands; "structured" = zeros with one block of ones per operand (numerics.apply_block_of_ones)."""
    from .numerics import apply_block_of_ones

    gen = torch.Generator(device=device).manual_seed(SEED)
    made = [0]

    def shaped(t: torch.Tensor) -> torch.Tensor:
        if fill == "structured" and t.is_floating_point():
            apply_block_of_ones(t, seed=made[0])
        made[0] += 1
        return t

    if isinstance(cmd, GemmCommand):
        def stored(rows, cols):
            return shaped(torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32).to(cmd.dtype))

        if cmd.mode == 1:
            a_store = stored(*((cmd.k, cmd.m) if cmd.transpose_a else (cmd.m, cmd.k)))
            b_store = stored(*((cmd.n, cmd.k) if cmd.transpose_b else (cmd.k, cmd.n)))
            a = a_store.t() if cmd.transpose_a else a_store
            b = b_store.t() if cmd.transpose_b else b_store
            return _mm_callable(backend, a, b, notes)
        # The reference's backward modes (kernel/boo/op_exports/gemm.py:233-270) take the output
        # gradient and the OTHER operand as stored; a final transpose for a transposed operand is a
        # view there and costs nothing, so only the product is timed.
        d_c = stored(cmd.m, cmd.n)
        if cmd.mode == 2:  # dA = dC @ B^T
            b_store = stored(*((cmd.n, cmd.k) if cmd.transpose_b else (cmd.k, cmd.n)))
            return _mm_callable(backend, d_c, b_store if cmd.transpose_b else b_store.t(), notes)
        a_store = stored(*((cmd.k, cmd.m) if cmd.transpose_a else (cmd.m, cmd.k)))  # dB = A^T @ dC
        return _mm_callable(backend, a_store if cmd.transpose_a else a_store.t(), d_c, notes)
    name = cmd.name.removeprefix("aten::")
    tensors = []
    for dims, ty, strides, concrete in zip(cmd.input_dims, cmd.input_type, cmd.input_strides, cmd.concrete_inputs):
        if concrete == "" and ty in _ATEN_DTYPES:
            tensors.append(shaped(_randn_strided(dims, strides, _ATEN_DTYPES[ty], device, gen)))
        else:
            tensors.append(None if concrete in ("", "None") else ast.literal_eval(concrete))
    if name == "mm":
        return _mm_callable(backend, tensors[0], tensors[1], notes)
    if name == "bmm":
        a, b = tensors[:2]
        if backend == "torch":
            return lambda: torch.bmm(a, b)
        if backend == "cpu_fp64":
            a64, b64 = _fp64_cpu(a, b)
            return lambda: torch.bmm(a64, b64)
        if a.dtype not in (torch.float16, torch.bfloat16) or a.dtype != b.dtype:
            raise Unsupported("b200k bmm covers float16 / bfloat16 operands of one dtype")
        return lambda: torch.ops.b200k.bmm(a, b, a.dtype)
    if name == "scaled_dot_product_attention":
        q, k, v = tensors[:3]
        rest = tensors[3:] + [None] * 5
        mask, dropout_p, is_causal, scale, enable_gqa = rest[:5]
        dropout_p = 0.0 if dropout_p is None else float(dropout_p)
        is_causal = bool(is_causal)
        if backend in ("torch", "cpu_fp64"):
            kwargs = {} if scale is None else {"scale": float(scale)}
            if enable_gqa:
                kwargs["enable_gqa"] = True
            if backend == "cpu_fp64":
                q64, k64, v64, m64 = _fp64_cpu(q, k, v, mask)
                return lambda: torch.nn.functional.scaled_dot_product_attention(q64, k64, v64, m64, dropout_p, is_causal,
                                                                                **kwargs)
            return lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, mask, dropout_p, is_causal, **kwargs)
        if mask is not None or dropout_p != 0.0:
            raise Unsupported("b200k attention takes no mask and no dropout")
        if q.size(-1) not in (64, 128) or q.dtype not in (torch.float16, torch.bfloat16):
            raise Unsupported("b200k attention covers head dims 128 and 64 in float16 / bfloat16")
        if is_causal and q.size(2) != k.size(2):
            raise Unsupported("causal with different query / key lengths is aligned differently by the two ops")
        s = float(scale) if scale is not None else 1.0 / math.sqrt(q.size(-1))
        return lambda: torch.ops.b200k.attention(q, k, v, s, is_causal)
    raise Unsupported(f"aten::{name} is not covered")


# ---------------------------------------------------------------------------------------------
# timing
# ---------------------------------------------------------------------------------------------
def time_callable(fn: Callable[[], torch.Tensor], iters: int, device) -> dict:
    """Per-call device time in microseconds over `iters` calls after 3 untimed ones."""
    with torch.cuda.device(device):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
        for i in range(iters):
            starts[i].record()
            fn()
            ends[i].record()
        torch.cuda.synchronize()
    us = [s.elapsed_time(e) * 1e3 for s, e in zip(starts, ends)]
    return {"min": min(us), "max": max(us), "mean": statistics.fmean(us),
            "stddev": statistics.pstdev(us) if len(us) > 1 else 0.0, "num_dispatches": iters}


# ---------------------------------------------------------------------------------------------
# main
# ---------------------------------------------------------------------------------------------
def _meta_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(
        prog="b200k-driver",
        usage="%(prog)s [-h] [... MIOpenDriver / aten command ...] [--commands-file COMMANDS_FILE]",
        description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--commands-file", type=str, help="read commands from a file, one per line ('#' starts a comment)")
    p.add_argument("--backends", action="append", choices=list(BACKENDS),
                   help=f"backend to run; may be given several times (default '{DEFAULT_BACKEND}')")
    p.add_argument("--csv", type=str, default=None, help="file to write the timing table to")
    p.add_argument("--gpu-id", type=int, default=0)
    p.add_argument("--verify-numerics", action="store_true",
                   help="per command, also print the numerics report (error statistics of b200k and of torch on the "
                        "same device against a float64 CPU result, and the block-of-ones indexing test); a failed "
                        "report makes the exit code non-zero")
    p.add_argument("--verbose", action="store_true", default=None)
    return p


def csv_headers(backends: Sequence[str]) -> List[str]:
    return ["arguments"] + [f"{b} {s}" for b in backends for s in ALL_STATS]


def main(args: Optional[List[str]] = None) -> int:
    args = list(sys.argv[1:] if args is None else args)
    meta, extra = _meta_parser().parse_known_args(args)
    verbose = meta.csv is None if meta.verbose is None else meta.verbose
    extra = [a for arg in extra for a in arg.split("\t")]
    if meta.commands_file:
        tsv = meta.commands_file.endswith(".tsv")
        with open(meta.commands_file) as f:
            commands = [(line.strip().split("\t") if tsv else shlex.split(line)) + extra
                        for line in f if line.strip() and not line.startswith("#")]
    else:
        commands = [extra]
    backends = meta.backends or [DEFAULT_BACKEND]
    with open(meta.csv if meta.csv is not None else os.devnull, "w", newline="") as csv_file:
        out = csv.writer(csv_file)
        out.writerow(csv_headers(backends))
        if not torch.cuda.is_available():
            raise RuntimeError("b200k-driver needs a CUDA device: the kernels have no CPU path")
        return _run_commands(commands, backends, out, torch.device("cuda", meta.gpu_id), verbose,
                             verify_numerics=meta.verify_numerics)


def _run_commands(commands, backends, out, device, verbose: bool, verify_numerics: bool = False) -> int:
    import iree_turbine_b200  # noqa: F401  (registers torch.ops.b200k.*)

    errors = 0
    for n, argv in enumerate(commands, 1):
        print(f"\n>>> {shlex.join(argv)}\n" if verbose else f"Running test : {n}")
        t_args, cmd_args = timing_parser().parse_known_args(argv)
        row: List[str] = [shlex.join(argv)]
        try:
            cmd = parse_command(cmd_args)
        except (ValueError, SystemExit, SyntaxError) as e:
            print(f"  cannot parse: {e}")
            errors += 1
            row += ["N.A."] * (len(ALL_STATS) * len(backends))
            out.writerow(row)
            continue
        for b in backends:
            notes: List[str] = []
            try:
                with torch.no_grad():
                    fn = build_callable(cmd, b, device, notes)
                    stats = time_callable(fn, max(t_args.iter, 1), device)
                row += [f"{stats[s]:.3f}" if s != "num_dispatches" else str(stats[s]) for s in ALL_STATS]
                if verbose:
                    extra_note = f" ({'; '.join(notes)})" if notes else ""
                    print(f"  {b}: min {stats['min']:.2f} us, mean {stats['mean']:.2f} us over {stats['num_dispatches']} calls{extra_note}")
            except Unsupported as e:
                row += ["N.A."] * len(ALL_STATS)
                if verbose:
                    print(f"  {b}: N.A. ({e})")
            except Exception as e:  # a failing backend does not stop the run, as in the reference
                errors += 1
                row += ["N.A."] * len(ALL_STATS)
                print(f"  {b}: failed: {e!r}")
        out.writerow(row)
        if verify_numerics:
            from . import numerics

            try:
                verdict = numerics.verify_command(cmd, device, command_text=shlex.join(argv))
                print(numerics.format_verdict(verdict))
                errors += 0 if verdict.passed else 1
            except Unsupported as e:
                print(f"numerics: N.A. ({e})")
    return 0 if errors == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
