"""rocmlir-tuning-driver for this library: measures the tuning space of each problem on the GPU and writes the
winners as a tuning database in the reference's text form.

The reference splits this job between a C++ tool that times the configurations of one kernel
(mlir/tools/rocmlir-tuning-driver/rocmlir-tuning-driver.cpp:131-185, 234-400) and a script that walks a list of
problems and appends `arch <tab> numCUs <tab> problem <tab> perfConfig [<tab> TFlops]` lines
(mlir/utils/performance/tuningRunner.py:393-404). Here one command does both:

    python -m rocmlir_b200.tuning_driver --configs problems.txt --tuning-space full --tflops -o tuned/sm_100a.tsv
    python -m rocmlir_b200.tuning_driver -c "--operation gemm --arch sm_100a --t f16 --out_datatype f16 --g 1 --m 4096 --n 4096 --k 4096"

A problem is one line of `--key value` options as miirCreateHandle takes them ('#' starts a comment). Every
configuration is timed with CUDA events over `--iters` launches after two warm-up launches, rotating over enough
operand sets that no launch finds its inputs in L2 (a ranking taken on L2-resident operands picked tiles that lose on
cold ones); operands hold random values of the element type, because all-zero data draws less power and runs at
clocks real data never sees. The library loads the written file as its
default database when it lies at tuned/sm_100a.tsv beside the shared library, or is named by RB_TUNING_DB.
"""
from __future__ import annotations

import argparse
import re
import sys
from typing import List, Optional, Tuple

from . import _lib as L
from . import miir, tuning

L2_FLUSH_BYTES = 300 << 20
SPACES = {"quick": tuning.QUICK, "full": tuning.FULL, "exhaustive": tuning.EXHAUSTIVE}


def _opt(options: str, key: str, default: Optional[str] = None) -> Optional[str]:
    m = re.search(r"--" + re.escape(key) + r"\s+(\S+)", options)
    return m.group(1) if m else default


def flops_of(options: str) -> float:
    """Floating-point (or integer) operations of the problem, as perfRunner.py counts them (:627-630 and :403-412)."""
    op = _opt(options, "operation", "conv")
    geti = lambda k, d=1: int(_opt(options, k, str(d)))
    if op == "gemm":
        return 2.0 * geti("g") * geti("m") * geti("n") * geti("k")
    if op == "attention":
        return 2.0 * geti("g") * geti("seq_len_q") * geti("seq_len_k") * (geti("head_dim_qk") + geti("head_dim_v"))
    return (2.0 * geti("batchsize") * geti("in_channels") * geti("out_channels") * geti("out_h") * geti("out_w") *
            geti("fil_h") * geti("fil_w") / geti("groupsize"))


def _random_operand(nbytes: int, options: str):
    """Seeded random values of the problem's element type as a byte buffer: all-zero operands draw far less power
    than real data, the clocks rise, and the ranking (and the TFlops column) would describe a different machine."""
    import torch
    t = _opt(options, "t") or _opt(options, "in_type") or "f16"
    gen = torch.Generator(device="cuda").manual_seed(nbytes & 0xFFFF)
    if t in ("f16", "fp16"):
        x = torch.randn(max(8, nbytes // 2), device="cuda", generator=gen).half()
    elif t in ("bf16",):
        x = torch.randn(max(8, nbytes // 2), device="cuda", generator=gen).bfloat16()
    elif t in ("f32", "fp32"):
        x = torch.randn(max(4, nbytes // 4), device="cuda", generator=gen)
    else:                                   # 8-bit types: every code (two of the 256 fp8 codes are NaN: harmless here)
        x = torch.randint(0, 256, (max(16, nbytes),), device="cuda", generator=gen, dtype=torch.uint8)
    return x.view(torch.uint8)


def tune_one(options: str, space: int, iters: int) -> Tuple[Optional[str], List[Tuple[str, float]], Optional[float]]:
    """Returns (problem key, [(perf_config, milliseconds)] fastest first, milliseconds of the library's own rule)."""
    import torch
    prob = tuning.Problem(options)
    key = prob.key
    configs = prob.quick_space() if space == tuning.QUICK else prob.space(space)
    base = re.sub(r"--perf_config\s+\S+", "", options)
    results = []
    bufs = None
    for perf in [None] + list(configs):  # None: the library's own rule (what a launch does without a database)
        try:
            h = miir.Handle(base if perf is None else base + " --perf_config " + perf)
        except ValueError:
            continue                     # not applicable to this problem
        with h:
            h.lower_tuning_params()
            if bufs is None:
                # enough independent operand sets that consecutive launches never find their inputs in the 126 MB L2
                sizes = h.arg_sizes()
                nsets = max(1, min(16, -(-L2_FLUSH_BYTES // max(1, sum(sizes)))))
                bufs = [[_random_operand(s, options) if s else None for s in sizes] for _ in range(nsets)]
            ws = torch.empty(max(16, h.workspace_size), dtype=torch.uint8, device="cuda")
            run = lambda b: h.launch(b[0], b[1], b[2], extra=b[3], workspace=ws)
            try:
                for b in bufs[:2]:
                    run(b)
            except miir.MiirError as e:
                print(f"    {perf or 'rule-based choice'}: not runnable ({e})", file=sys.stderr)
                continue
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for i in range(iters):
                run(bufs[i % len(bufs)])
            e1.record()
            torch.cuda.synchronize()
            if L.kernel_status() != 0:
                raise RuntimeError(f"kernel status {L.kernel_status():#x} under {perf}")
            results.append((perf, e0.elapsed_time(e1) / iters))
    default_ms = next((ms for perf, ms in results if perf is None), None)
    results = sorted((r for r in results if r[0] is not None), key=lambda r: r[1])
    return key, results, default_ms


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="rocmlir-tuning-driver", description=__doc__.split("\n\n")[0])
    ap.add_argument("-c", "--config", action="append", default=[], help="one problem as an option string")
    ap.add_argument("--configs", help="file with one problem per line")
    ap.add_argument("--tuning-space", default="full", choices=sorted(SPACES))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tflops", action="store_true", help="fifth column: TFlops of the winner")
    ap.add_argument("--min-gain", type=float, default=0.0,
                    help="write a row only when the winner beats the library's own rule by this fraction (0: always, as tuningRunner.py does)")
    ap.add_argument("-o", "--output", default="-", help="database file to APPEND to ('-': stdout), like tuningRunner.py")
    args = ap.parse_args(argv)
    problems = list(args.config)
    if args.configs:
        with open(args.configs) as f:
            problems += [l.strip() for l in f if l.strip() and not l.lstrip().startswith("#")]
    if not problems:
        ap.error("no problems given")
    out = sys.stdout if args.output == "-" else open(args.output, "a")
    with out:
        cols = "# arch\tnumCUs\ttestVector\tperfConfig" + ("\tTFlops" if args.tflops else "")
        print(f"{cols} ({args.tuning_space})", file=out)
        for options in problems:
            key, results, default_ms = tune_one(options, SPACES[args.tuning_space], args.iters)
            if not key or not results:
                print(f"rocmlir-tuning-driver: nothing to tune for: {options}", file=sys.stderr)
                continue
            perf, ms = results[0]
            tf = flops_of(options) / (ms * 1e-3) / 1e12
            print(f"{key.replace(chr(9), ' | ')}: {perf} {ms * 1e3:.1f} us {tf:.1f} TFlops "
                  f"(of {len(results)} configurations; slowest {results[-1][1] * 1e3:.1f} us)", file=sys.stderr)
            gain = (default_ms / ms - 1.0) if default_ms else float("inf")
            if gain < args.min_gain:
                print(f"    rule-based choice {default_ms * 1e3:.1f} us: winner gains {gain * 100:.1f} % < {args.min_gain * 100:.0f} %, no row written",
                      file=sys.stderr)
                continue
            print(f"{key}\t{perf}" + (f"\t{tf:.2f}" if args.tflops else ""), file=out, flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
