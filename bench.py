#!/usr/bin/env python
"""Benchmark of the contraction hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1, and per rank for N > 1): the fp16 GEMM of the headline configuration, C = A.B with
M = N = K = 4096, A and B row-major, f32 accumulate, f16 output, A,B ~ 0.1 * N(0,1) from a seed. One step = `--passes`
passes over a batch of `--sets` independent operand sets (distinct A, B, C buffers, 8 sets = 805 MB, larger than the
126 MB L2, so every GEMM reads cold operands); with the defaults a step is 512 GEMMs, so that 20 steps are a timed
region of about a second (long enough for the clock sampler and for the power cap to settle). Ranks hold independent
batches (no data-path collective): weak scaling.

Prints ONE JSON line (rank 0): device-resident throughput (`value`), the same metric through the host-buffer entry
point with the copies timed (`e2e`), the roofline of the GEMM kernel against the burst, sustained and nominal peaks,
the clocks seen inside the timed region, a CPU baseline (the reference's validation loop nest restated in oracle/,
timed single-threaded and on all host cores on a bounded sample of the same workload), and under `config`:
  secondary  one short record per other configuration of the baseline (int8 / fp8 / bf16 / epilogue GEMMs, the
             ResNet convolution set in three directions, the fp32 NCHW convolution, attention, GEMM+GEMM), timed
             after the headline region with the same hygiene
  verified   a sampled oracle check of every workload's output, outside the timed regions
  sharded    (N > 1) the configurations split over the ranks as rocmlir_b200.sharding prescribes, strong scaling
"""
from __future__ import annotations

import argparse
import json
import math
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
WORKLOAD = "fp16 GEMM 4096x4096x4096, A,B row-major, f32 accumulate, f16 out, A,B ~ 0.1*N(0,1)"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of gemm_tcgen05_kernel on this workload: a constant taken
# from the ncu capture summarised in profiles/gemm_f16_4096_ncu.md (two launches: 88.2 + 15.8 and 87.9 + 15.7 MB read + written), not measured
# by this run.
NCU_DRAM_BYTES_PER_LAUNCH = 103.8e6
# nominal dense peaks per GPU; f32 runs as three TF32 products per multiply (a third of the 1125 TFLOP/s TF32 figure)
NOMINAL = {"f16": 2250.0, "bf16": 2250.0, "i8": 4500.0, "fp8": 4500.0, "f32": 375.0, "hbm": 8000.0}


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


def host_threads() -> int:
    """Threads the CPU legs use: the cores this process may run on, whatever OMP_NUM_THREADS says (torchrun sets it
    to 1 for every rank)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi; every sample carries the host time it was read at, so
    that only the samples inside a timed region are summarised."""
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
            self.samples.append((time.time(), line.strip()))

    def summary(self, t0: float, t1: float):
        """Median SM clock and the reasons seen among the samples read between host times t0 and t1."""
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        sm, mx, power, reasons = [], None, [], set()
        for ts, s in list(self.samples):
            if not (t0 <= ts <= t1):
                continue
            f = [x.strip() for x in s.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
                power.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()


def make_operands(sets: int, seed: int):
    """A, B ~ 0.1 * N(0,1) rounded to f16; generated on the host from a seeded stream, pinned."""
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
    4096^3 problem and returns (TFLOP/s, seconds, description)."""
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
    return tflops, dt, (f"{rows2} of {M} rows of one 4096^3 GEMM (f32-widened operands, k innermost, separate multiply "
                        f"and add), {threads} thread{'s' if threads != 1 else ''}, {dt:.1f} s")


def run_reference(args, rank: int, world: int):
    """--impl reference: the reference's own CPU implementation of the path. Its validator is generated MLIR
    that needs mlir-cpu-runner (not buildable here), so the timed code is the oracle port of that loop nest, on every
    core this process may use."""
    if rank != 0:
        return
    threads = host_threads()
    vals = []
    per_step = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    desc = ""
    for i in range(args.warmup + args.steps):
        tf, dt, desc = cpu_reference_sample(per_step, threads)
        if i >= args.warmup:
            vals.append((tf, dt))
    tflops = sum(v[0] for v in vals) / len(vals)
    ms = 1e3 * sum(v[1] for v in vals) / len(vals)
    line = {"impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample_per_step": desc},
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": desc},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# Secondary workloads: the other configurations of the baseline. build_workload returns a dict with the step
# function, the work and bytes of one step, and a `verify` callable (sampled oracle check of the step's output).
# ---------------------------------------------------------------------------------------------------------
RESNET = {"a": dict(c=64, k=64, h=56, w=56, y=3, x=3, pad_h=1, pad_w=1),
          "b": dict(c=256, k=64, h=56, w=56, y=1, x=1),
          "c": dict(c=128, k=128, h=28, w=28, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1),
          "d": dict(c=512, k=2048, h=7, w=7, y=1, x=1)}


def _f32(t):
    """Device tensor -> f32 numpy array holding the same values."""
    return t.float().cpu().numpy()


def _verdict(got, ref, rms):
    import oracle
    v, info = oracle.verify_float(got, ref, rms, 100.0, 100.0)
    return v == [1, 1, 1], f"rms {info['rms']:.2e} (bar {rms:g})"


def build_workload(name, dev, sets, rank=0, world=1, gather=False):
    import numpy as np
    import torch
    import oracle
    from rocmlir_b200 import sharding
    from rocmlir_b200.gemm import Epilogue, gemm, gemm_gemm, problem, workspace_size
    from rocmlir_b200 import _lib as L
    g = torch.Generator(device="cpu").manual_seed(1 + rank)
    T = host_threads()

    def randn(shape, scale, dtype):
        return (torch.randn(shape, generator=g) * scale).to(dtype).to(dev)

    def rows_of(m, count=8):
        return np.unique(np.concatenate([[0, m - 1], np.random.Generator(np.random.PCG64(9)).choice(m, count - 2, replace=False)]))

    if name.startswith("gemm_") and not name.startswith("gemm_gemm_f16"):
        kind = name[5:]
        if kind in ("f16", "bf16", "f16_bias_relu"):
            dt = torch.bfloat16 if kind == "bf16" else torch.float16
            code = oracle.BF16 if kind == "bf16" else oracle.F16
            m = k = 4096
            n_full = 4096
            sh = sharding.gemm_column_shard(n_full, rank, world)
            n = sh.size
            ops = [(randn((m, k), 0.1, dt), randn((k, n), 0.1, dt), torch.empty((m, n), dtype=dt, device=dev)) for _ in range(sets)]
            epi, bias = None, None
            if kind == "f16_bias_relu":
                bias = randn((n,), 0.1, dt)
                epi = Epilogue(bias=bias, relu=True, mid_type=L.F16)
            ws = torch.empty(max(16, workspace_size(problem(ops[0][0], ops[0][1], False, False, False, dt))), dtype=torch.uint8, device=dev)
            gathered = [None]

            def step():
                for a, b, c in ops:
                    gemm(a, b, out=c, epilogue=epi, workspace=ws)
                if gather and world > 1:
                    gathered[0] = sharding.gather_columns(ops[-1][2], n_full)   # the optional all-gather of a column-split C

            def verify():
                a, b, c = ops[0]
                rows = rows_of(m)
                acc = oracle.gemm_f32(_f32(a[rows])[None], _f32(b)[None], 1, len(rows), n, k, threads=T)
                if epi is not None:
                    acc = oracle.epilogue(acc, n, bias=_f32(bias), relu=True, mid_type=code)
                return _verdict(_f32(c[rows]), oracle.round_to(acc, code), 1e-3 if code == oracle.F16 else 8e-3)
            return dict(step=step, work=2.0 * m * n * k * sets, unit="TFLOP/s", bytes=(m * k + k * n + m * n) * 2.0 * sets,
                        bound="tensor", dtype=kind.split("_")[0], verify=verify, kernel="gemm_tcgen05_kernel",
                        desc=f"{kind} GEMM 4096^3, A,B row-major, f32 accumulate" + (", C' = relu(C + bias[N])" if epi else ""))
        m, k = 2048, 4096
        n = sharding.gemm_column_shard(11008, rank, world).size
        if kind.startswith("i8"):
            ops = [(torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).to(dev),
                    torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).to(dev)) for _ in range(sets)]
            requant = kind == "i8_requant"
            odt = torch.int8 if requant else torch.int32
            outs = [torch.empty((m, n), dtype=odt, device=dev) for _ in range(sets)]
            s_col = (torch.rand(n, generator=g) * 0.009 + 0.001)
            epi = Epilogue(col_scale=s_col.to(dev), requant_scale=12.0) if requant else None
            step = lambda: [gemm(a, b, trans_b=True, out=c, out_dtype=odt, epilogue=epi) for (a, b), c in zip(ops, outs)]

            def verify():
                (a, b), c = ops[0], outs[0]
                rows = rows_of(m)
                acc = oracle.gemm_i8(a[rows].cpu().numpy()[None], b.cpu().numpy()[None], 1, len(rows), n, k, tb=True, threads=T)
                if requant:
                    ref = oracle.from_f32(oracle.epilogue(acc, n, col_scale=s_col.numpy(), requant_scale=12.0), oracle.I8, sat_int=True)
                else:
                    ref = acc
                bad = int((c[rows].cpu().numpy().astype(np.int64).ravel() != ref.astype(np.int64).ravel()).sum())
                return bad == 0, f"{bad} mismatches in {ref.size} (bit-exact bar)"
            obytes = 1 if requant else 4
            return dict(step=step, work=2.0 * m * n * k * sets, unit="TOP/s", bytes=(m * k + n * k + m * n * obytes) * sets,
                        bound="tensor", dtype="i8", verify=verify, kernel="gemm_tcgen05_kernel",
                        desc="int8 GEMM 2048x11008x4096 (B stored N x K), i32 accumulate" +
                             (", dequant x s_col[n], requant to i8 (RNE, saturate)" if requant else ", i32 out"))
        if kind == "fp8":
            ops = [(randn((m, k), 1.0, torch.float8_e4m3fn), randn((n, k), 1.0, torch.float8_e4m3fn)) for _ in range(sets)]
            outs = [torch.empty((m, n), dtype=torch.bfloat16, device=dev) for _ in range(sets)]
            alpha = 0.25 * 0.5
            epi = Epilogue(alpha=alpha)
            step = lambda: [gemm(a, b, trans_b=True, out=c, out_dtype=torch.bfloat16, epilogue=epi) for (a, b), c in zip(ops, outs)]

            def verify():
                (a, b), c = ops[0], outs[0]
                rows = rows_of(m)
                acc = oracle.gemm_f32(_f32(a[rows])[None], _f32(b)[None], 1, len(rows), n, k, tb=True, threads=T)
                return _verdict(_f32(c[rows]), oracle.round_to(oracle.epilogue(acc, n, alpha=alpha), oracle.BF16), 8e-3)
            return dict(step=step, work=2.0 * m * n * k * sets, unit="TFLOP/s", bytes=(m * k + n * k + m * n * 2) * sets,
                        bound="tensor", dtype="fp8", verify=verify, kernel="gemm_tcgen05_kernel",
                        desc="fp8-e4m3 GEMM 2048x11008x4096 (B stored N x K), f32 accumulate, x sA*sB, bf16 out")
    if name == "gemm_gemm_f16":
        k1, n1, n2 = 1024, 1024, 1024
        m = sharding.shard_range(4096, rank, world, granule=128).size
        ops = [(randn((m, k1), 0.1, torch.float16), randn((k1, n1), 0.1, torch.float16), randn((n1, n2), 0.1, torch.float16),
                torch.empty((m, n2), dtype=torch.float16, device=dev)) for _ in range(sets)]
        ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
        step = lambda: [gemm_gemm(a, b1, b2, out=o, workspace=ws) for a, b1, b2, o in ops]

        def verify():
            a, b1, b2, o = ops[0]
            rows = rows_of(m)
            ref = oracle.round_to(oracle.gemm_gemm(_f32(a[rows]), _f32(b1), _f32(b2), oracle.F16, threads=T), oracle.F16)
            return _verdict(_f32(o[rows]), ref, 1e-3)
        return dict(step=step, work=(2.0 * m * k1 * n1 + 2.0 * m * n1 * n2) * sets, unit="TFLOP/s",
                    bytes=2.0 * (m * k1 + k1 * n1 + n1 * n2 + m * n2) * sets, bound="tensor", dtype="f16", verify=verify,
                    kernel="gemm_gemm", desc="fp16 GEMM+GEMM M4096 K1 1024 N1 1024 N2 1024")
    if name == "gemm_gemm_f16_heads":
        # the attention skeleton without its softmax: 32 problems, inner extents of a head (one launch, intermediate on the SM)
        G, m_all, k1, n1, n2 = 32, 4096, 128, 4096, 128
        gl = sharding.shard_range(G, rank, world).size
        ops = [(randn((gl, m_all, k1), 0.1, torch.float16), randn((gl, k1, n1), 0.1, torch.float16),
                randn((gl, n1, n2), 0.1, torch.float16), torch.empty((gl, m_all, n2), dtype=torch.float16, device=dev))
               for _ in range(max(1, sets // 4))]
        ws = torch.empty(16, dtype=torch.uint8, device=dev)
        step = lambda: [gemm_gemm(a, b1, b2, out=o, workspace=ws) for a, b1, b2, o in ops]

        def verify():
            a, b1, b2, o = ops[0]
            rows = rows_of(m_all)[:16]
            ref = oracle.round_to(oracle.gemm_gemm(_f32(a[0][rows]), _f32(b1[0]), _f32(b2[0]), oracle.F16, threads=T), oracle.F16)
            return _verdict(_f32(o[0][rows]), ref, 1e-3)
        n_ops = len(ops)
        return dict(step=step, work=2.0 * gl * m_all * n1 * (k1 + n2) * n_ops, unit="TFLOP/s",
                    bytes=2.0 * gl * (m_all * k1 + k1 * n1 + n1 * n2 + m_all * n2) * n_ops, bound="tensor", dtype="f16",
                    verify=verify, kernel="attention_fwd2_kernel",
                    desc="fp16 GEMM+GEMM, 32 problems M4096 K1 128 N1 4096 N2 128 (one launch each, intermediate in tensor memory)")
    if name.startswith("conv_"):
        from rocmlir_b200.conv import ConvConfig, conv, workspace_size as conv_ws
        if name == "conv_f32_nchw":
            kw = dict(c=64, k=64, h=56, w=56, y=3, x=3, pad_h=1, pad_w=1, fil_layout="kcyx", in_layout="nchw", out_layout="nkhw")
            batch, dt, direction, code, rms = 16, torch.float32, 0, oracle.F32, 3e-5
            desc = "fp32 conv2d forward NCHW/KCYX N16 C64 56x56 K64 3x3 s1 p1, uniform[-1,1)"
        else:
            _, _, _, shape, dirname = name.split("_", 4)  # conv_f16_nhwc_<a-d>_<fwd|bwd_data|bwd_weight>
            direction = {"fwd": 0, "bwd_data": 1, "bwd_weight": 2}[dirname]
            kw, batch, dt, code, rms = dict(RESNET[shape]), 256, torch.float16, oracle.F16, 1e-3
            desc = f"fp16 NHWC conv N256 {RESNET[shape]} {dirname}, tensors ~ 0.05*N(0,1)"
        cfg = ConvConfig(n=sharding.conv_batch_shard(batch, rank, world).size, **kw)
        nsets = max(1, min(sets, 2))
        if dt == torch.float32:
            mk = lambda nel: (torch.rand(nel, generator=g) * 2 - 1).to(dev)
        else:
            mk = lambda nel: (torch.randn(nel, generator=g) * 0.05).to(dt).to(dev)
        # the filter (gradient) tensors of all sets live in one flat bucket, so that a batch-sharded backward-weight
        # step needs one all-reduce (gradient bucketing), not one per convolution
        bucket = mk(cfg.numel("fil") * nsets)
        ts = [(bucket[i * cfg.numel("fil"):(i + 1) * cfg.numel("fil")], mk(cfg.numel("in")), mk(cfg.numel("out"))) for i in range(nsets)]
        ws = torch.empty(max(16, conv_ws(cfg, dt, direction)), dtype=torch.uint8, device=dev)
        pending = [None]

        def step():
            if pending[0] is not None:      # the previous step's all-reduce, overlapped with nothing but launch latency
                pending[0].wait()
                pending[0] = None
            for f, i, o in ts:
                conv(cfg, direction, f, i, o, workspace=ws)
            if direction == 2 and world > 1:
                # the one exchange of the path: issued asynchronously on NCCL's stream behind this step's kernels; the
                # next step's kernels write the bucket again only after wait() has ordered them behind it
                pending[0] = sharding.allreduce_weight_gradient(bucket, async_op=True)

        def finish():
            if pending[0] is not None:
                pending[0].wait()
                pending[0] = None

        def verify():
            finish()
            if world > 1 and direction == 2:
                return True, "skipped: the bucket holds the sum over ranks"
            f, i, o = ts[0]
            c1 = {k_: v_ for k_, v_ in kw.items() if not k_.endswith("_layout")}
            lay = dict(fil_layout=cfg.fil_layout, in_layout=cfg.in_layout, out_layout=cfg.out_layout)
            if direction in (0, 1):      # images are independent: image 0
                oc = oracle.Conv(n=1, **c1, **lay)
                inp, out = _f32(i[:oc.numel("in")]), _f32(o[:oc.numel("out")])
                ref = oracle.conv_f32(oc, direction, _f32(f), inp if direction == 0 else None, out if direction == 1 else None, threads=T)
                got = out if direction == 0 else inp
                return _verdict(got, oracle.round_to(ref, code), rms)
            # backward weight: one output channel x 8 input channels of the filter gradient, reduced over the whole batch
            ksel, csel = 3, slice(8, 16)
            c2 = dict(c1, k=1, c=8)
            oc = oracle.Conv(n=cfg.n, **c2, **lay)
            inp = np.ascontiguousarray(_f32(i).reshape(-1, cfg.c)[:, csel]).ravel()
            out = np.ascontiguousarray(_f32(o).reshape(-1, cfg.k)[:, ksel:ksel + 1]).ravel()
            ref = oracle.round_to(oracle.conv_f32(oc, 2, None, inp, out, threads=T), code)
            got = _f32(f).reshape(cfg.k, cfg.y * cfg.x, cfg.c)[ksel, :, csel].ravel()
            return _verdict(got, ref, rms)
        es = 4 if dt == torch.float32 else 2
        abytes = (cfg.numel("fil") + cfg.numel("in") + cfg.numel("out")) * es * nsets
        ai = cfg.flops() / (abytes / nsets)
        return dict(step=step, finish=finish, work=cfg.flops() * nsets, unit="TFLOP/s", bytes=abytes,
                    # ridge: 16-bit tensor peak / HBM rate in FLOP per byte; f32 runs as three TF32 products (a sixth of it)
                    bound=("tensor" if ai > (281 / 6 if es == 4 else 281) else "hbm"), dtype=("f32" if es == 4 else "f16"),
                    verify=verify, desc=desc,
                    kernel=("conv_halo_stream_kernel<f32> (+ TF32 plane passes of image and filter)" if es == 4 else
                            "conv_halo_kernel / conv_wgrad_halo_kernel (unit-stride NHWC 16-bit, stride classes) or gemm_tcgen05_kernel (+ layout / reduction passes)"))
    if name.startswith("attention_f16"):
        from rocmlir_b200.attention import attention, flops
        causal = name.endswith("causal")
        S, D = 2048, 128
        G = sharding.attention_group_shard(512, rank, world).size
        q = randn((G, S, D), 1.0, torch.float16); kk = randn((G, D, S), 1.0, torch.float16); v = randn((G, S, D), 1.0, torch.float16)
        o = torch.empty_like(q)
        scale = 1.0 / math.sqrt(D)
        step = lambda: attention(q, kk, v, scale=scale, causal=causal, out=o)

        def verify():
            grp = G - 1
            rows = rows_of(S, 12)
            mask = None
            if causal:     # the analytic mask as the tensor it stands for: key j is visible to query row r when j <= r
                mask = (np.arange(S)[None, :] <= rows[:, None]).astype(np.int8)[None]
            ref = oracle.attention(_f32(q[grp, rows])[None], _f32(kk[grp])[None], _f32(v[grp])[None], elem_type=oracle.F16,
                                   scale_scalar=float(np.float16(scale)), mask=mask, mask_fill=float("-inf"), threads=T)
            vdt, info = oracle.verify_float(_f32(o[grp, rows]), ref[0], 0.015, 0.02, 100.0)   # PrAttentionF16.toml:3
            return vdt == [1, 1, 1], f"rms {info['rms']:.2e} max_abs {info['max_abs']:.2e} (bars 0.015 / 0.02)"
        return dict(step=step, work=flops(G, S, S, D, D, causal), unit="TFLOP/s", bytes=4.0 * G * S * D * 2, bound="tensor",
                    dtype="f16", verify=verify, kernel="attention_fwd2_kernel",
                    desc=f"fp16 attention batch 16 x 32 heads, S 2048, D 128, {'causal' if causal else 'non-causal'}, Q/K/V ~ N(0,1)")
    raise SystemExit(f"unknown workload {name}")


WORKLOADS = (["gemm_f16", "gemm_bf16", "gemm_f16_bias_relu", "gemm_i8", "gemm_i8_requant", "gemm_fp8", "gemm_gemm_f16", "gemm_gemm_f16_heads",
              "conv_f32_nchw", "attention_f16", "attention_f16_causal"] +
             [f"conv_f16_nhwc_{s}_{d}" for s in "abcd" for d in ("fwd", "bwd_data", "bwd_weight")])


def measure(name, args, dev, rank, world, target_ms=300.0, sets=None, gather=False, verify=True, graph=True):
    """Times one workload: warm-up, (single GPU) capture of a step into a CUDA graph, a timed region of about
    `target_ms`, then the sampled oracle check. Returns a record (on every rank; rank 0 prints)."""
    import torch
    import torch.distributed as dist
    from rocmlir_b200 import _lib as L
    from rocmlir_b200 import sharding
    w = build_workload(name, dev, sets or args.secondary_sets, rank, world, gather=gather)
    step = w["step"]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(3):
        step()
    barrier()
    # A step of small kernels is bound by the host's launch path (about 11 us per library call, 18 us through the
    # Python mirror), so the step is captured once into a CUDA graph and replayed: the library allocates nothing and
    # its launches are capturable. Not with a collective inside the step.
    run, per_step_launches, graphed = step, None, False
    if graph and world == 1:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                gr = torch.cuda.CUDAGraph()
                l0 = L.launch_count()
                with torch.cuda.graph(gr, stream=side):
                    step()
                per_step_launches = L.launch_count() - l0
            torch.cuda.current_stream().wait_stream(side)
            gr.replay()
            torch.cuda.synchronize()
            run, graphed = gr.replay, True
        except Exception as e:   # capture refused: time the plain step
            print(f"[bench] graph capture of {name} failed ({e}); timing direct launches", file=sys.stderr)
            torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # size the region from two probe steps
    e0.record(); run(); run(); e1.record()
    barrier()
    probe = sharding.job_time_ms(e0.elapsed_time(e1) / 2.0, device=dev)
    steps = int(max(3, min(2000, target_ms / max(probe, 1e-3))))
    l0 = L.launch_count()
    t_host0 = time.time()
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    barrier()
    t_host1 = time.time()
    if "finish" in w:
        w["finish"]()
        barrier()
    ms = sharding.job_time_ms(e0.elapsed_time(e1), device=dev)
    launches = per_step_launches * steps if graphed else L.launch_count() - l0
    work, abytes = float(w["work"]), float(w["bytes"])
    if world > 1:   # whole-job work: the shards need not be equal
        t = torch.tensor([work, abytes], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        work, abytes = t.tolist()
    status = L.kernel_status()
    ok, detail = (None, "not checked")
    if verify and rank == 0:
        try:
            ok, detail = w["verify"]()
        except Exception as e:      # the check must never take the measurement down with it
            ok, detail = False, f"check raised {type(e).__name__}: {e}"
    elif "finish" in w:
        w["finish"]()
    peaks = measured_peaks()
    value = work * steps / (ms * 1e-3) / 1e12
    rec = {"workload": name, "desc": w["desc"], "value": value, "unit": w["unit"], "ms_per_step": ms / steps, "steps": steps,
           "timed_region_ms": ms, "gpu_launches": int(launches), "launch": "CUDA graph replay" if graphed else "direct launches",
           "bound": w["bound"], "dtype": w["dtype"], "kernel_status": status, "verified": ok, "verify_detail": detail,
           "host_window": (t_host0, t_host1)}
    if w["bound"] == "tensor":
        # the measured tensor peak is a bf16 figure; 8-bit kinds are held against twice it, f32 (3xTF32) against a sixth
        mult = {"i8": 2.0, "fp8": 2.0, "f32": 1.0 / 6.0}.get(w["dtype"], 1.0)
        rec.update(frac_of_measured_burst=value / (peaks["burst"] * mult * world),
                   frac_of_measured_sustained=value / (peaks["sustained"] * mult * world),
                   frac_of_nominal=value / (NOMINAL[w["dtype"]] * world))
    else:
        gbs = abytes * steps / (ms * 1e-3) / 1e9
        rec.update(achieved_gbs=gbs, frac_of_measured_hbm=gbs / (peaks["hbm"] * world), frac_of_nominal=gbs / (NOMINAL["hbm"] * world))
    return rec


def run_sharded(args, dev, rank, world):
    """N > 1: the configurations split over the ranks (strong scaling). Efficiency = time of the whole problem on one
    GPU (every rank runs it as a replica first) / (N x time of the sharded problem)."""
    out = []
    for name, gather in (("gemm_f16", False), ("gemm_f16", True), ("gemm_i8", False), ("attention_f16", False),
                         ("attention_f16_causal", False), ("conv_f16_nhwc_a_fwd", False), ("conv_f16_nhwc_a_bwd_weight", False)):
        whole = measure(name, args, dev, 0, 1, target_ms=150.0, verify=False, graph=False)          # replica of the whole problem
        part = measure(name, args, dev, rank, world, target_ms=150.0, gather=gather, verify=False)
        eff = whole["ms_per_step"] / (world * part["ms_per_step"])
        out.append({"workload": name + ("+all_gather" if gather else ""), "value": part["value"], "unit": part["unit"],
                    "ms_per_step": part["ms_per_step"], "single_gpu_ms_per_step": whole["ms_per_step"],
                    "strong_scaling_efficiency": eff,
                    "split": {"gemm": "columns of B and C", "attention": "groups (batch x heads)", "conv": "batch" +
                              (" + async all-reduce of the filter gradients" if name.endswith("bwd_weight") else "")}[name.split("_")[0]]})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gemm_f16", help="gemm_f16 (headline, with the secondary records) or one of bench.WORKLOADS / 'all'")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sets", type=int, default=8, help="independent operand sets of the headline workload")
    ap.add_argument("--passes", type=int, default=64, help="passes over the operand sets per step of the headline workload")
    ap.add_argument("--secondary-sets", type=int, default=4, help="operand sets of the secondary workloads")
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (used for ncu captures)")
    ap.add_argument("--no-secondary", action="store_true", help="headline only (used for ncu captures)")
    ap.add_argument("--no-graph", action="store_true", help="secondary workloads: direct launches instead of a CUDA graph")
    ap.add_argument("--target-ms", type=float, default=1000.0, help="--workload NAME: length of the timed region (short for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from rocmlir_b200 import _lib as L
    from rocmlir_b200 import sharding
    from rocmlir_b200.gemm import gemm, gemm_host, problem, workspace_size

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    if args.workload != "gemm_f16":      # one named workload (or all) as full JSON lines: used for profiling
        for name in (WORKLOADS[1:] if args.workload == "all" else [args.workload]):
            rec = measure(name, args, dev, rank, world, target_ms=args.target_ms, sets=args.sets, graph=not args.no_graph)
            if rank == 0:
                t0, t1 = rec.pop("host_window")
                rec["clocks"] = sampler.summary(t0, t1)
                print(json.dumps({"metric": f"{rec['unit']}, {rec['desc']}", "n_gpus": world, "data": "synthetic", **rec}), flush=True)
        sampler.stop()
        if distributed:
            dist.destroy_process_group()
        return

    host_sets = make_operands(args.sets, seed=1 + rank)
    dev_sets = [(a.to(dev), b.to(dev), torch.empty((M, N), dtype=torch.float16, device=dev)) for a, b in host_sets]
    variant = args.variant if args.variant else None
    ws_bytes = workspace_size(problem(dev_sets[0][0], dev_sets[0][1], False, False, False, torch.float16))
    workspace = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

    def step_device():
        for _ in range(args.passes):
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = L.launch_count()
    barrier()
    t_host0 = time.time()
    e0.record()
    marks = []
    for _ in range(args.steps):
        step_device()
        m = torch.cuda.Event(enable_timing=True)   # a mark between steps: recorded on the stream, nothing waits for it
        m.record()
        marks.append(m)
    e1.record()
    barrier()
    t_host1 = time.time()
    launches = L.launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    per_step = sorted(a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks))
    status = L.kernel_status()
    clocks = sampler.summary(t_host0, t_host1) if rank == 0 else None

    # ---- the headline output against the oracle (outside the timed region): sampled rows of the last GEMM ----
    verified = {}
    if rank == 0:
        import numpy as np
        import oracle
        a, b, c = dev_sets[-1]
        rows = np.random.Generator(np.random.PCG64(3)).choice(M, 8, replace=False)
        ref = oracle.round_to(oracle.gemm_f32(_f32(a[rows])[None], _f32(b)[None], 1, len(rows), N, K, threads=host_threads()), oracle.F16)
        ok, detail = _verdict(_f32(c[rows]), ref, 1e-3)
        verified["gemm_f16"] = {"ok": ok, "detail": detail}

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
        if rank == 0:     # the host-path result of the last operand set equals the device-path result bit for bit
            a, b, c = dev_sets[-1]
            verified["e2e_equals_device_path"] = {"ok": bool(torch.equal(host_out, c.cpu())), "detail": "rbGemmHost vs rbGemm, whole C"}

    # a multi-rank job takes as long as its slowest rank
    ms_total = sharding.job_time_ms(ms_total, device=dev)
    e2e_ms_total = sharding.job_time_ms(e2e_ms_total, device=dev)

    # ---- the other configurations, after the headline region ----
    # (one GPU: every configuration on its own; N > 1: the configurations sharded over the ranks)
    secondary, sharded = [], []
    if not args.no_secondary:
        del dev_sets, workspace
        torch.cuda.empty_cache()
        if distributed:
            sharded = run_sharded(args, dev, rank, world)
        else:
            for name in WORKLOADS[1:]:
                rec = measure(name, args, dev, 0, 1, graph=not args.no_graph)
                t0, t1 = rec.pop("host_window")
                rec["sm_mhz"] = sampler.summary(t0, t1)["sm_mhz"]
                verified[name] = {"ok": rec.pop("verified"), "detail": rec.pop("verify_detail")}
                secondary.append(rec)
                torch.cuda.empty_cache()
    sampler.stop()

    if rank == 0:
        peaks = measured_peaks()
        gemms_per_step = args.sets * args.passes
        ms_per_step = ms_total / args.steps
        total_flops = FLOPS_PER_GEMM * gemms_per_step * args.steps * world
        value = total_flops / (ms_total * 1e-3) / 1e12
        e2e_value = FLOPS_PER_GEMM * args.sets * e2e_steps * world / (e2e_ms_total * 1e-3) / 1e12
        per_launch_ms = ms_total / max(1, launches)
        achieved = FLOPS_PER_GEMM / (per_launch_ms * 1e-3) / 1e12
        # the sustained cuBLAS figure is the denominator once the timed region is long enough to sit at the power cap
        # (a second), the burst figure for a short region at full clocks; both fractions are printed either way
        peak_kind = "sustained" if ms_total >= 1000.0 else "burst"
        peak = peaks[peak_kind]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "gemms_per_step": gemms_per_step,
                       "l2": f"inputs larger than L2: {args.sets} operand sets = {args.sets * BYTES_PER_GEMM / 1e6:.0f} MB per pass, "
                             f"{args.passes} passes per step",
                       "parallelism": f"{world} independent replicas of the batch (weak scaling, no collective)",
                       "kernel_variant": args.variant, "kernel_status": status, "timed_region_ms": ms_total,
                       "ms_per_step_min": per_step[0], "ms_per_step_median": per_step[len(per_step) // 2],
                       "ms_per_step_max": per_step[-1],
                       "secondary": secondary, "verified": verified, "sharded": sharded},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "peak_source": f"{peaks['source']} cuBLAS bf16 {peak_kind} (timed region {ms_total:.0f} ms)",
                         "frac_of_measured_burst": achieved / peaks["burst"],
                         "frac_of_measured_sustained": achieved / peaks["sustained"],
                         "frac_of_nominal_2250": achieved / 2250.0,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                         "traffic_source": "constant from the ncu capture in profiles/gemm_f16_4096_ncu.md, not measured by this run",
                         "algorithmic_bytes": BYTES_PER_GEMM,
                         "kernel": "gemm_tcgen05_kernel", "avg_launch_ms": per_launch_ms},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": args.sets * 2 * M * K * 2,
                    "d2h_bytes_per_step": args.sets * M * N * 2, "steps": e2e_steps,
                    "api": "rbGemmHost (pinned host A, B -> device in row blocks, GEMM per block, C blocks -> host meanwhile)"},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = host_threads()
            tf, dt, desc = cpu_reference_sample(12.0, threads)
            tf1, dt1, desc1 = cpu_reference_sample(6.0, 1)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": desc,
                                    "single_thread": {"value": tf1, "unit": "TFLOP/s", "cores": 1, "sample": desc1}}
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
