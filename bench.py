#!/usr/bin/env python
"""Benchmark of the contraction hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1 and per rank for N > 1): the fp16 GEMM of the headline configuration,
C = A.B with M = N = K = 4096, A and B row-major, f32 accumulate, f16 output, A,B ~ 0.1 * N(0,1) from
a seed. One step = one pass over a batch of `--sets` independent operand sets (distinct A, B, C buffers,
8 by default = 805 MB, larger than the 126 MB L2, so every GEMM of a step reads cold operands).
Ranks hold independent batches (no data-path collective): weak scaling.

Prints ONE JSON line (rank 0): device-resident throughput (`value`), the same metric through the
host-buffer entry point with the copies timed (`e2e`), the roofline of the GEMM kernel, the clocks seen
under load, and a CPU baseline (the reference's validation loop nest restated in oracle/, timed on a
bounded sample of the same workload).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 4096
FLOPS_PER_GEMM = 2.0 * M * N * K                      # perfRunner.py:627-630 convention: 2*g*m*k*n
BYTES_PER_GEMM = 3 * M * N * 2                        # each operand read once, C written once, f16
METRIC = "TFLOP/s, fp16 GEMM M=N=K=4096 (rock.gemm, f32 accumulate, f16 out)"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of gemm_tcgen05_kernel on this workload, from the
# ncu capture summarised in profiles/gemm_f16_4096_ncu.md (89.3 MB read + 15.6 MB written).
NCU_DRAM_BYTES_PER_LAUNCH = 104.32e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return {"burst": float(d["bf16_tflops"]), "sustained": float(d["bf16_tflops_sustained"]),
                    "hbm": float(d["hbm_gbs"]), "source": "measured"}
        except Exception:
            pass
    return {"burst": 1590.0, "sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_operands(sets: int, seed: int, device):
    """A, B ~ 0.1 * N(0,1) rounded to f16; generated on the host from a seeded stream, then copied."""
    import numpy as np
    import torch
    out = []
    rng = np.random.Generator(np.random.PCG64(seed))
    for _ in range(sets):
        a = (rng.standard_normal((M, K), dtype=np.float32) * np.float32(0.1)).astype(np.float16)
        b = (rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.1)).astype(np.float16)
        out.append((torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory()))
    return out


def cpu_reference_sample(seconds_target: float, threads: int):
    """Times the oracle's rock.gemm loop nest (the reference's CPU validation path) on a row sample of the
    4096^3 problem and returns (TFLOP/s, description)."""
    import numpy as np
    import oracle
    rng = np.random.Generator(np.random.PCG64(1))
    b = oracle.round_to((rng.standard_normal((1, K, N), dtype=np.float32) * np.float32(0.1)), oracle.F16)
    rows = max(threads, 8)
    a = oracle.round_to((rng.standard_normal((1, rows, K), dtype=np.float32) * np.float32(0.1)), oracle.F16)
    t0 = time.perf_counter()
    oracle.gemm_f32(a, b, 1, rows, N, K, threads=threads)
    dt = time.perf_counter() - t0
    # scale the sample so that it takes about seconds_target, then time that
    rows2 = int(min(M, max(rows, rows * seconds_target / max(dt, 1e-6))))
    rows2 = max(threads, rows2 // threads * threads)
    a = oracle.round_to((rng.standard_normal((1, rows2, K), dtype=np.float32) * np.float32(0.1)), oracle.F16)
    t0 = time.perf_counter()
    oracle.gemm_f32(a, b, 1, rows2, N, K, threads=threads)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows2 * N * K / dt / 1e12
    return tflops, dt, f"{rows2} of {M} rows of one 4096^3 GEMM (f32-widened operands, k innermost), {dt:.1f} s"


def run_reference(args, rank: int, world: int):
    """--impl reference: the reference's own CPU implementation of the path. Its validator is generated MLIR
    that needs mlir-cpu-runner (not buildable here), so the timed code is the oracle port of that loop nest."""
    if rank != 0:
        return
    import oracle
    threads = oracle.max_threads()
    vals = []
    per_step = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        tf, dt, desc = cpu_reference_sample(per_step, threads)
        if i >= args.warmup:
            vals.append((tf, dt))
    tflops = sum(v[0] for v in vals) / len(vals)
    ms = 1e3 * sum(v[1] for v in vals) / len(vals)
    line = {"impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "fp16 GEMM 4096x4096x4096, A,B ~ 0.1*N(0,1)", "sample_per_step": desc},
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": desc},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# Secondary workloads (--workload NAME): the other configurations of the baseline, one JSON line each with the
# same keys (device-resident throughput + roofline; no end-to-end or CPU leg). The headline stays gemm_f16.
# ---------------------------------------------------------------------------------------------------------
RESNET = {"a": dict(c=64, k=64, h=56, w=56, y=3, x=3, pad_h=1, pad_w=1),
          "b": dict(c=256, k=64, h=56, w=56, y=1, x=1),
          "c": dict(c=128, k=128, h=28, w=28, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1),
          "d": dict(c=512, k=2048, h=7, w=7, y=1, x=1)}


def build_workload(name, dev, sets, rank=0, world=1):
    """Returns (step_fn, work_per_step, unit, algorithmic_bytes_per_step, bound, dtype, description, kernel) for this
    rank's shard of the configuration (rocmlir_b200.sharding: GEMM by columns of B and C, GEMM+GEMM by rows,
    convolution by batch - backward weight with an all-reduce of the partial gradients -, attention by group)."""
    import math
    import torch
    import torch.distributed as dist
    from rocmlir_b200 import sharding
    from rocmlir_b200.gemm import Epilogue, gemm, gemm_gemm, problem, workspace_size
    from rocmlir_b200 import _lib as L
    g = torch.Generator(device="cpu").manual_seed(1 + rank)

    def randn(shape, scale, dtype):
        return (torch.randn(shape, generator=g) * scale).to(dtype).to(dev)

    if name.startswith("gemm_"):
        kind = name[5:]
        if kind in ("f16", "bf16", "f16_bias_relu"):
            dt = torch.bfloat16 if kind == "bf16" else torch.float16
            m = k = 4096
            n = sharding.gemm_column_shard(4096, rank, world).size
            ops = [(randn((m, k), 0.1, dt), randn((k, n), 0.1, dt), torch.empty((m, n), dtype=dt, device=dev)) for _ in range(sets)]
            epi = None
            if kind == "f16_bias_relu":
                epi = Epilogue(bias=randn((n,), 0.1, dt), relu=True, mid_type=L.F16)
            ws = torch.empty(max(16, workspace_size(problem(ops[0][0], ops[0][1], False, False, False, dt))), dtype=torch.uint8, device=dev)
            step = lambda: [gemm(a, b, out=c, epilogue=epi, workspace=ws) for a, b, c in ops]
            return step, 2.0 * m * n * k * sets, "TFLOP/s", (m * k + k * n + m * n) * 2.0 * sets, "tensor", kind.split("_")[0], \
                f"{kind} GEMM 4096^3, A,B row-major, f32 accumulate" + (", C' = relu(C + bias[N])" if epi else ""), "gemm_tcgen05_kernel"
        m, k = 2048, 4096
        n = sharding.gemm_column_shard(11008, rank, world).size
        if kind.startswith("i8"):
            ops = [(torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).to(dev),
                    torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).to(dev)) for _ in range(sets)]
            requant = kind == "i8_requant"
            odt = torch.int8 if requant else torch.int32
            outs = [torch.empty((m, n), dtype=odt, device=dev) for _ in range(sets)]
            epi = Epilogue(col_scale=(torch.rand(n, generator=g) * 0.009 + 0.001).to(dev), requant_scale=12.0) if requant else None
            step = lambda: [gemm(a, b, trans_b=True, out=c, out_dtype=odt, epilogue=epi) for (a, b), c in zip(ops, outs)]
            obytes = 1 if requant else 4
            return step, 2.0 * m * n * k * sets, "TOP/s", (m * k + n * k + m * n * obytes) * sets, "tensor", "i8", \
                f"int8 GEMM 2048x11008x4096 (B stored N x K), i32 accumulate" + (", dequant x s_col[n], requant to i8 (RNE, saturate)" if requant else ", i32 out"), "gemm_tcgen05_kernel"
        if kind == "fp8":
            ops = [(randn((m, k), 1.0, torch.float8_e4m3fn), randn((n, k), 1.0, torch.float8_e4m3fn)) for _ in range(sets)]
            outs = [torch.empty((m, n), dtype=torch.bfloat16, device=dev) for _ in range(sets)]
            epi = Epilogue(alpha=0.25 * 0.5)
            step = lambda: [gemm(a, b, trans_b=True, out=c, out_dtype=torch.bfloat16, epilogue=epi) for (a, b), c in zip(ops, outs)]
            return step, 2.0 * m * n * k * sets, "TFLOP/s", (m * k + n * k + m * n * 2) * sets, "tensor", "fp8", \
                "fp8-e4m3 GEMM 2048x11008x4096 (B stored N x K), f32 accumulate, x sA*sB, bf16 out", "gemm_tcgen05_kernel"
    if name == "gemm_gemm_f16":
        k1, n1, n2 = 1024, 1024, 1024
        m = sharding.shard_range(4096, rank, world, granule=128).size
        ops = [(randn((m, k1), 0.1, torch.float16), randn((k1, n1), 0.1, torch.float16), randn((n1, n2), 0.1, torch.float16),
                torch.empty((m, n2), dtype=torch.float16, device=dev)) for _ in range(sets)]
        ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
        step = lambda: [gemm_gemm(a, b1, b2, out=o, workspace=ws) for a, b1, b2, o in ops]
        return step, (2.0 * m * k1 * n1 + 2.0 * m * n1 * n2) * sets, "TFLOP/s", 2.0 * (m * k1 + k1 * n1 + n1 * n2 + m * n2) * sets, \
            "tensor", "f16", "fp16 GEMM+GEMM M4096 K1 1024 N1 1024 N2 1024 (two launches, intermediate in L2)", "gemm_tcgen05_kernel x2"
    if name.startswith("conv_"):
        from rocmlir_b200.conv import ConvConfig, conv, workspace_size as conv_ws
        if name == "conv_f32_nchw":
            cfg = ConvConfig(n=sharding.conv_batch_shard(16, rank, world).size, c=64, k=64, h=56, w=56, y=3, x=3, pad_h=1, pad_w=1,
                             fil_layout="kcyx", in_layout="nchw", out_layout="nkhw")
            dt, direction, scale, lo = torch.float32, 0, None, True
            desc = "fp32 conv2d forward NCHW/KCYX N16 C64 56x56 K64 3x3 s1 p1, uniform[-1,1)"
        else:
            _, _, _, shape, dirname = name.split("_", 4)  # conv_f16_nhwc_<a-d>_<fwd|bwd_data|bwd_weight>
            direction = {"fwd": 0, "bwd_data": 1, "bwd_weight": 2}[dirname]
            cfg = ConvConfig(n=sharding.conv_batch_shard(256, rank, world).size, **RESNET[shape])
            dt = torch.float16
            desc = f"fp16 NHWC conv N256 {RESNET[shape]} {dirname}, tensors ~ 0.05*N(0,1)"
        nsets = max(1, min(sets, 2))
        ts = []
        if dt == torch.float32:
            mk = lambda nel: (torch.rand(nel, generator=g) * 2 - 1).to(dev)
        else:
            mk = lambda nel: (torch.randn(nel, generator=g) * 0.05).to(dt).to(dev)
        # the filter (gradient) tensors of all sets live in one flat bucket, so that a batch-sharded backward-weight
        # step needs one all-reduce (gradient bucketing), not one per convolution
        bucket = mk(cfg.numel("fil") * nsets)
        for i_set in range(nsets):
            ts.append((bucket[i_set * cfg.numel("fil"):(i_set + 1) * cfg.numel("fil")], mk(cfg.numel("in")), mk(cfg.numel("out"))))
        ws = torch.empty(max(16, conv_ws(cfg, dt, direction)), dtype=torch.uint8, device=dev)

        def step():
            for f, i, o in ts:
                conv(cfg, direction, f, i, o, workspace=ws)
            if direction == 2 and world > 1:
                sharding.allreduce_weight_gradient(bucket)   # the one exchange of the path
        es = 4 if dt == torch.float32 else 2
        abytes = (cfg.numel("fil") + cfg.numel("in") + cfg.numel("out")) * es * nsets
        ai = cfg.flops() / (abytes / nsets)
        return step, cfg.flops() * nsets, "TFLOP/s", abytes, ("tensor" if ai > 281 else "hbm"), ("f32" if es == 4 else "f16"), desc, \
            "conv_gather / permute5 + gemm_tcgen05_kernel"
    if name.startswith("attention_f16"):
        from rocmlir_b200.attention import attention, flops
        causal = name.endswith("causal")
        S, D = 2048, 128
        G = sharding.attention_group_shard(512, rank, world).size
        q = randn((G, S, D), 1.0, torch.float16); kk = randn((G, D, S), 1.0, torch.float16); v = randn((G, S, D), 1.0, torch.float16)
        o = torch.empty_like(q)
        step = lambda: attention(q, kk, v, scale=1.0 / math.sqrt(D), causal=causal, out=o)
        return step, flops(G, S, S, D, D, causal), "TFLOP/s", 4.0 * G * S * D * 2, "tensor", "f16", \
            f"fp16 attention batch 16 x 32 heads, S 2048, D 128, {'causal' if causal else 'non-causal'}, Q/K/V ~ N(0,1)", "attention_fwd_kernel"
    raise SystemExit(f"unknown workload {name}")


WORKLOADS = (["gemm_f16", "gemm_bf16", "gemm_f16_bias_relu", "gemm_i8", "gemm_i8_requant", "gemm_fp8", "gemm_gemm_f16",
              "conv_f32_nchw", "attention_f16", "attention_f16_causal"] +
             [f"conv_f16_nhwc_{s}_{d}" for s in "abcd" for d in ("fwd", "bwd_data", "bwd_weight")])


def run_secondary(args, name, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from rocmlir_b200 import _lib as L
    from rocmlir_b200 import sharding
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    step, work, unit, abytes, bound, dtype, desc, kernel = build_workload(name, dev, args.sets, rank, world)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    # A step of small kernels is bound by the host's launch path (about 11 us per library call, 18 us through the
    # Python mirror), so the step is captured once into a CUDA graph and replayed: the library allocates nothing and
    # its launches are capturable. Not under torchrun (the NCCL all-reduce of a step stays outside graphs here).
    run, per_step_launches, graphed = step, None, False
    if not args.no_graph and world == 1:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                l0 = L.launch_count()
                with torch.cuda.graph(graph, stream=side):
                    step()
                per_step_launches = L.launch_count() - l0
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
            run, graphed = graph.replay, True
        except Exception as e:   # capture refused: time the plain step
            print(f"[bench] graph capture failed ({e}); timing direct launches", file=sys.stderr)
            torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = L.launch_count()
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    barrier()
    ms = sharding.job_time_ms(e0.elapsed_time(e1), device=dev)     # slowest rank
    launches = per_step_launches * args.steps if graphed else L.launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:   # whole-job work: the shards need not be equal
        t = torch.tensor([float(work), float(abytes)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        work, abytes = t.tolist()
    if rank != 0:
        return
    peaks = measured_peaks()
    value = work * args.steps / (ms * 1e-3) / 1e12
    capped = bool(clocks) and "sw_power_cap" in (clocks.get("reasons") or [])
    kind = "sustained" if (ms >= 1000.0 or capped) else "burst"
    if bound == "tensor":
        # the measured tensor peak is a bf16 figure; 8-bit kinds are held against twice it, f32 (3xTF32) against a sixth
        mult = {"i8": 2.0, "fp8": 2.0, "f32": 1.0 / 6.0}.get(dtype, 1.0)
        peak, achieved, runit = peaks[kind] * mult * world, value, unit
    else:
        peak, achieved, runit = peaks["hbm"] * world, abytes * args.steps / (ms * 1e-3) / 1e9, "GB/s"
    line = {"metric": f"{unit}, {desc}", "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak" if world == 1 else "strong",
            "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": desc, "kernel_status": L.kernel_status(),
                       "launch": "CUDA graph replay of one captured step" if graphed else "direct launches",
                       "parallelism": "one GPU" if world == 1 else f"the configuration sharded over {world} GPUs "
                                      "(GEMM: columns; convolution: batch; attention: groups)",
                       "l2": "operand sets rotate / tensors exceed L2" if abytes > 126e6 * world else "working set fits L2 (stated)"},
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": runit, "frac": achieved / peak,
                         "peak_source": f"{peaks['source']} ({kind}; {'HBM copy' if bound == 'hbm' else 'cuBLAS bf16 x type factor'}"
                                        + (f" x {world} GPUs)" if world > 1 else ")"),
                         "traffic": None, "algorithmic_bytes": abytes, "kernel": kernel,
                         "avg_launch_ms": ms / max(1, launches)},
            "e2e": None, "gpu_launches": int(launches), "clocks": clocks}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gemm_f16", help="gemm_f16 (headline) or one of bench.WORKLOADS / 'all'")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sets", type=int, default=8, help="independent operand sets per step")
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (used for ncu captures)")
    ap.add_argument("--no-graph", action="store_true", help="secondary workloads: direct launches instead of a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload != "gemm_f16":
        if world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        for name in (WORKLOADS[1:] if args.workload == "all" else [args.workload]):
            run_secondary(args, name, rank, world, local_rank)
        if world > 1:
            dist.destroy_process_group()
        return

    import torch
    import torch.distributed as dist
    from rocmlir_b200 import _lib as L
    from rocmlir_b200 import sharding
    from rocmlir_b200.gemm import gemm, gemm_host

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=dev)

    host_sets = make_operands(args.sets, seed=1 + rank, device=dev)
    dev_sets = [(a.to(dev), b.to(dev), torch.empty((M, N), dtype=torch.float16, device=dev)) for a, b in host_sets]
    variant = args.variant if args.variant else None
    from rocmlir_b200.gemm import problem, workspace_size
    if variant is not None:
        L.lib().rbSetGemmVariant(int(variant))
    ws_bytes = workspace_size(problem(dev_sets[0][0], dev_sets[0][1], False, False, False, torch.float16))
    workspace = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

    def step_device():
        for a, b, c in dev_sets:
            gemm(a, b, out=c, variant=variant, workspace=workspace)

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = L.launch_count()
    barrier()
    e0.record()
    for _ in range(args.steps):
        step_device()
    e1.record()
    barrier()
    launches = L.launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    status = L.kernel_status()
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: host buffers in, host result out, through rbGemmHost (copies inside the timed region) ----
    host_out = torch.empty((M, N), dtype=torch.float16).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))
    e2e_ms_total = float("nan")
    if not args.no_e2e:
        for a, b in host_sets[:2]:
            gemm_host(a, b, host_out, variant=variant)
        barrier()
        e0.record()
        for _ in range(e2e_steps):
            for a, b in host_sets:
                gemm_host(a, b, host_out, variant=variant)
        e1.record()
        barrier()
        e2e_ms_total = e0.elapsed_time(e1)

    # a multi-rank job takes as long as its slowest rank
    ms_total = sharding.job_time_ms(ms_total, device=dev)
    e2e_ms_total = sharding.job_time_ms(e2e_ms_total, device=dev)

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms_total / args.steps
        total_flops = FLOPS_PER_GEMM * args.sets * args.steps * world
        value = total_flops / (ms_total * 1e-3) / 1e12
        e2e_value = FLOPS_PER_GEMM * args.sets * e2e_steps * world / (e2e_ms_total * 1e-3) / 1e12
        per_launch_ms = ms_total / max(1, launches)
        achieved = FLOPS_PER_GEMM / (per_launch_ms * 1e-3) / 1e12
        # the sustained cuBLAS figure is the denominator once the run is long enough to sit at the power cap
        # (the clock record says so), the burst figure for a short timed region at full clocks
        capped = bool(clocks) and "sw_power_cap" in (clocks.get("reasons") or [])
        peak_kind = "sustained" if (ms_total >= 1000.0 or capped) else "burst"
        peak = peaks[peak_kind]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "fp16 GEMM 4096x4096x4096, A,B row-major, f32 accumulate, f16 out, A,B ~ 0.1*N(0,1)",
                       "gemms_per_step": args.sets,
                       "l2": f"inputs larger than L2: {args.sets} operand sets = {args.sets * BYTES_PER_GEMM / 1e6:.0f} MB per step",
                       "parallelism": f"{world} independent replicas of the batch (weak scaling, no collective)",
                       "kernel_variant": args.variant, "kernel_status": status},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "peak_source": f"{peaks['source']} cuBLAS bf16 {peak_kind} (timed region {ms_total:.0f} ms)",
                         "frac_of_nominal_2250": achieved / 2250.0,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "algorithmic_bytes": BYTES_PER_GEMM,
                         "kernel": "gemm_tcgen05_kernel", "avg_launch_ms": per_launch_ms},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": args.sets * 2 * M * K * 2,
                    "d2h_bytes_per_step": args.sets * M * N * 2, "steps": e2e_steps,
                    "api": "rbGemmHost (pinned host A, B -> device, GEMM, C -> host, stream sync)"},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            import oracle
            threads = oracle.max_threads()
            tf, dt, desc = cpu_reference_sample(12.0, threads)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
