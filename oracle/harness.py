"""The validation harness behind the `rocmlir-gen` / `rocmlir-driver` tools of this repository (oracle/bin/): takes
rocmlir-gen's command line, generates the inputs the way `rocmlir-gen -ph -pv -rand N` does, runs the operation on
the GPU through the library, runs the CPU restatement of the reference's validator, compares with the reference's
verifier and thresholds, and gives the verdict line `[1 1 1]`
(mlir/tools/rocmlir-gen/rocmlir-gen.cpp:73-785 flags, :996-1092 defaults, :837-972 layout and padding fix-ups,
:1325-1486 data fill, :2696-2886 verification). It stands in for the reference's pipeline
`rocmlir-gen ... -pv | rocmlir-driver -c | mlir-cpu-runner`:

    oracle/bin/rocmlir-gen --operation gemm -t f16 -g 3 -m 1024 -k 769 -n 1024 --arch sm_100a -pv -rand 1 | oracle/bin/rocmlir-driver -c

CHECKER-SIDE infrastructure like the rest of oracle/: the one place where the library and the oracle meet. The product
package never imports it.
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import oracle  # noqa: E402


def _torch_dtype(code):
    import torch
    return {oracle.F32: torch.float32, oracle.F16: torch.float16, oracle.BF16: torch.bfloat16, oracle.I8: torch.int8,
            oracle.I32: torch.int32, oracle.F8E4M3: torch.float8_e4m3fn, oracle.F8E5M2: torch.float8_e5m2}[code]


def to_device(raw: np.ndarray, code: int, device="cuda"):
    """Raw storage bits (as produced by oracle.from_f32) -> torch tensor of the matching dtype."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(raw).view(np.int16) if raw.dtype == np.uint16 else np.ascontiguousarray(raw))
    return t.to(device).view(_torch_dtype(code))


def from_device(t, code: int) -> np.ndarray:
    """Torch tensor -> raw storage bits as numpy."""
    import torch
    if code in (oracle.F16, oracle.BF16):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    if code in (oracle.F8E4M3, oracle.F8E5M2):
        return t.contiguous().view(torch.uint8).cpu().numpy()
    return t.contiguous().cpu().numpy()


class Unsupported(Exception):
    """The flags describe something this library has no kernel for (the reason says what)."""


# flags that take no value (cl::opt<bool> given bare); `-flag=true|false` also works for them
BOOL_FLAGS = {"p", "pv", "ph", "pr", "pi", "pv_with_gpu", "pv_with_mlir", "prc", "reverse_grid", "with-attn-scale",
              "with-attn-bias", "transA", "transB", "transC", "transQ", "transK", "transV", "transO", "emit-tuning-key",
              "host-harness", "verifier-keep-perf-config", "disable-split-k-for-tuning", "print-results"}


def parse_flags(text: str) -> Dict[str, str]:
    """-k v | -k=v | --k v | --k=v | bare boolean flags. Later occurrences overwrite earlier ones."""
    toks = text.split()
    out: Dict[str, str] = {}
    i = 0
    while i < len(toks):
        t = toks[i]
        if not t.startswith("-") or t.lstrip("-") == "" or t.lstrip("-")[0].isdigit():
            raise ValueError(f"unexpected token {t!r}")
        key = t.lstrip("-")
        if "=" in key:
            key, val = key.split("=", 1)
            out[key] = val
            i += 1
        elif key in BOOL_FLAGS:
            out[key] = "true"
            i += 1
        else:
            if i + 1 >= len(toks):
                raise ValueError(f"flag {t!r} needs a value")
            out[key] = toks[i + 1]
            i += 2
    return out


TYPE_CODES = {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16, "i8": oracle.I8, "i32": oracle.I32,
              "fp8": oracle.F8E4M3, "f8E4M3FN": oracle.F8E4M3, "bf8": oracle.F8E5M2, "f8E5M2": oracle.F8E5M2}


@dataclass
class Types:
    a: int
    b: int
    out: int


def resolve_types(f: Dict[str, str]) -> Types:
    """The -t callback and its defaults (rocmlir-gen.cpp:430-455, 1000-1008)."""
    fil = f.get("fil_dtype", "f32")
    inp = f.get("in_dtype", "f32")
    out = f.get("out_dtype", f.get("out_datatype", ""))
    t = f.get("t", f.get("dtype"))
    if t is not None:
        if "_" in t:
            fil, inp = t.split("_", 1)
        else:
            fil = inp = t
        if out == "":
            if t == "i8":
                out = "i32"
            elif t.startswith(("f8", "fp8", "bf8")):
                out = "f32"
            elif fil == inp:
                out = t
    if out == "":
        out = "f32"
    for name in (fil, inp, out):
        if name not in TYPE_CODES:
            raise Unsupported(f"element type {name}")
    if fil != inp and not {fil, inp} <= {"fp8", "bf8", "f8E4M3FN", "f8E5M2"}:
        raise Unsupported("mixed input types other than the two 8-bit float formats")
    return Types(TYPE_CODES[fil], TYPE_CODES[inp], TYPE_CODES[out])


class Planned(Exception):
    """Raised by plan() once a command line has been parsed, typed and sized, before any tensor is filled."""


_PLAN_ONLY = False


class Filler:
    """Tensors filled in kernel-argument order (rocmlir-gen.cpp:3157-3218): one libc rand() per element with
    `-rand N`, the fixed pattern or all-ones otherwise."""

    def __init__(self, f: Dict[str, str]):
        if _PLAN_ONLY:
            raise Planned()
        self.mode = f.get("rand", "fixed")
        self.rand_float = f.get("rand_type", "int") == "float"
        self.mn = int(f.get("rand_min", 0))
        self.mx = int(f.get("rand_max", 1))
        self.random = self.mode not in ("fixed", "none")
        if self.random:
            seed = int(self.mode)
            if seed == 0:
                raise Unsupported("-rand 0 seeds from the clock: not reproducible")
            oracle.seed(seed)
        # -rand_side: only that tensor (argument index 0 filter, 1 input, 2 output) is random; the others get the
        # degenerate range [1, 1] (rocmlir-gen.cpp:1325-1357), i.e. the constant 1 (0.1 in float mode)
        side = f.get("rand_side", "both")[0]
        self.only = {"f": 0, "i": 1, "o": 2}.get(side, -1)
        self.index = 0

    def tensor(self, n: int, code: int):
        """-> (values as f32 after rounding to the element type, raw storage bits)"""
        is_int = code in (oracle.I8, oracle.I32)
        idx = self.index
        self.index += 1
        if self.random:
            if self.only >= 0 and self.only != idx:
                vals = oracle.fill_random(n, self.rand_float, 1, 1)
            elif self.rand_float:
                vals = oracle.fill_random(n, True, self.mn, self.mx)
            else:
                vals = oracle.fill_random(n, False, -5, 5)
        elif self.mode == "none":
            vals = np.full(n, 0.1 if self.rand_float else 1.0, np.float32)
        else:
            vals = oracle.fill_pattern(n, [1.0, -1.0, 2.0] if is_int else [0.5, -1.0, 0.75])
        if code == oracle.I32:
            raw = vals.astype(np.int32)
            return raw.astype(np.float32), raw
        raw = oracle.from_f32(vals, code)
        return oracle.to_f32(raw, code), raw


def thresholds(f: Dict[str, str], test_code: int):
    """rocmlir-gen.cpp:2850-2861"""
    rms = 0.001 if test_code == oracle.F16 else 0.00003
    if "RMS_threshold" in f:
        rms = float(f["RMS_threshold"])
    abs_thr = float(f.get("absDiff_threshold", 100.0))
    rel_thr = float(f.get("relDiff_threshold", 0.000001))
    if test_code == oracle.F16:
        rel_thr = 100.0
    return rms, abs_thr, rel_thr


def verdict_for(got_raw: np.ndarray, want: np.ndarray, code: int, f: Dict[str, str]) -> List[int]:
    if code in (oracle.I8, oracle.I32):
        v, _ = oracle.verify_int(got_raw, want.astype(np.int64))
        return v
    got = oracle.to_f32(got_raw, code) if code != oracle.F32 else got_raw
    want = oracle.round_to(want, code)       # the validation result is truncated to the kernel's type (:2822-2839)
    rms, a, r = thresholds(f, code)
    v, _ = oracle.verify_float(got, want, rms, a, r)
    return v


def as_bool(f: Dict[str, str], key: str) -> bool:
    return f.get(key, "false").lower() in ("true", "1")


def translate_perf_config(f: Dict[str, str]) -> Optional[int]:
    """The reference's perf strings name AMD tile parameters; the only field with a meaning here is the split-K
    factor of a `v2:` GEMM string (7th field), which selects the same number of K ranges."""
    pc = f.get("perf_config", "")
    if pc.startswith("v2:"):
        parts = pc[3:].split(",")
        if len(parts) >= 7 and int(parts[6]) > 1:
            return int(parts[6]) << 16
    return None


# ---------------------------------------------------------------------------------------------------------------------
def run_gemm(f: Dict[str, str]) -> List[int]:
    from rocmlir_b200.gemm import gemm
    ty = resolve_types(f)
    if as_bool(f, "p"):
        g, m, k, n = 1, 1024, 769, 512
    else:
        g, m, k, n = int(f.get("g", 1)), int(f["m"]), int(f["k"]), int(f["n"])
    ta, tb, tc = as_bool(f, "transA"), as_bool(f, "transB"), as_bool(f, "transC")
    if (g * m * n) > (1 << 29):
        raise Unsupported("result larger than 2 GiB elements: the CPU validator alone would take the test budget")
    fill = Filler(f)
    a_shape = (g, k, m) if ta else (g, m, k)
    b_shape = (g, n, k) if tb else (g, k, n)
    c_shape = (g, n, m) if tc else (g, m, n)
    a_f, a_r = fill.tensor(int(np.prod(a_shape)), ty.a)
    b_f, b_r = fill.tensor(int(np.prod(b_shape)), ty.b)
    fill.tensor(int(np.prod(c_shape)), ty.out)        # the output buffer is an argument too: it consumes rand() calls
    is_int = ty.a == oracle.I8
    if is_int and ty.out not in (oracle.I32,):
        raise Unsupported("i8 GEMM with a non-i32 result needs an epilogue")
    threads = oracle.max_threads()
    if is_int:
        want = oracle.gemm_i8(a_r.reshape(a_shape), b_r.reshape(b_shape), g, m, n, k, ta, tb, tc, threads=threads)
    else:
        want = oracle.gemm_f32(a_f.reshape(a_shape), b_f.reshape(b_shape), g, m, n, k, ta, tb, tc, threads=threads)
    a_d = to_device(a_r.reshape(a_shape), ty.a)
    b_d = to_device(b_r.reshape(b_shape), ty.b)
    store = f.get("store-method", "set")
    if store not in ("set", "atomic_add"):
        raise ValueError(f"unknown store method {store}")
    if store == "atomic_add":
        # C += A.B on an output the host harness has pre-filled with zero, as the reference's harness does for kernels
        # that accumulate (insertPrefills, rocmlir-gen.cpp:2890-2920): the verdict is against the plain product
        import torch
        if is_int:
            raise Unsupported("store method atomic_add exists for float results")
        out = torch.zeros(c_shape, dtype=_torch_dtype(ty.out), device="cuda")
        gemm(a_d, b_d, trans_a=ta, trans_b=tb, trans_c=tc, out_dtype=_torch_dtype(ty.out), out=out, accumulate=True,
             variant=translate_perf_config(f) or 0)
    else:
        out = gemm(a_d, b_d, trans_a=ta, trans_b=tb, trans_c=tc, out_dtype=_torch_dtype(ty.out),
                   variant=translate_perf_config(f) or 0)
    got = from_device(out, ty.out)
    return verdict_for(got.reshape(c_shape), want, ty.out, f)


def conv_config(f: Dict[str, str]):
    from rocmlir_b200.conv import ConvConfig
    if as_bool(f, "p"):
        d = dict(g=1, n=128, c=8, k=128, h=32, w=32, y=3, x=3)   # rocmlir-gen.cpp:1023-1046 (no mfma forced)
        f = {**{"dilation_h": "1", "dilation_w": "1", "conv_stride_h": "1", "conv_stride_w": "1"}, **f}
    else:
        g = int(f.get("groupsize", 1))
        ci, co = int(f["in_channels"]), int(f["out_channels"])
        if ci % g or co % g:
            raise ValueError("channels must be divisible by the group count")
        d = dict(g=g, n=int(f["batchsize"]), c=ci // g, k=co // g, h=int(f["in_h"]), w=int(f["in_w"]),
                 y=int(f["fil_h"]), x=int(f["fil_w"]))
    pad = {}
    for ax in ("h", "w"):
        combined = int(f.get(f"padding_{ax}", 0))
        left, right = int(f.get(f"padding_{ax}_l", 0)), int(f.get(f"padding_{ax}_r", 0))
        if combined > 0 and left == 0 and right == 0:      # rocmlir-gen.cpp:880-897
            left = right = combined
        pad[ax] = (left, right)
    sh, sw = int(f.get("conv_stride_h", 1)), int(f.get("conv_stride_w", 1))
    dh, dw = int(f.get("dilation_h", 1)), int(f.get("dilation_w", 1))

    def fix_right(inp, fil, pl, pr, stride, dil):              # rocmlir-gen.cpp:905-971
        out = (inp + pl + pr - (fil - 1) * dil - 1) // stride + 1
        need = 1 + (fil - 1) * dil + (out - 1) * stride
        return pr + max(0, need - (inp + pl + pr))
    pr_h = fix_right(d["h"], d["y"], pad["h"][0], pad["h"][1], sh, dh)
    pr_w = fix_right(d["w"], d["x"], pad["w"][0], pad["w"][1], sw, dw)
    fl, il, ol = f.get("fil_layout", "gkcyx"), f.get("in_layout", "ngchw"), f.get("out_layout", "ngkhw")
    for name, lay in (("filter", fl), ("input", il)):          # verifyConvLayout, rocmlir-gen.cpp:974-994
        pair = [c for c in lay if c in ("yx01" if name == "filter" else "hw01")]
        pos = [lay.index(c) for c in pair]
        if len(pos) != 2 or abs(pos[0] - pos[1]) != 1:
            raise ValueError(f"unsupported {name} layout: disjointed image dimensions")
    if len(fl.replace("g", "")) == 5:
        # three image letters: nDims = 3, depth sizes default to 1 (rocmlir-gen.cpp:3545-3581)
        from rocmlir_b200.conv import Conv3dConfig
        dd, zz = max(1, int(f.get("in_d", 1))), max(1, int(f.get("fil_d", 1)))
        combined = int(f.get("padding_d", 0))
        pd_l, pd_r = int(f.get("padding_d_l", 0)), int(f.get("padding_d_r", 0))
        if combined > 0 and pd_l == 0 and pd_r == 0:
            pd_l = pd_r = combined
        sd, dld = int(f.get("conv_stride_d", 1)), int(f.get("dilation_d", 1))
        pd_r = fix_right(dd, zz, pd_l, pd_r, sd, dld)
        cfg3 = Conv3dConfig(d=dd, z=zz, stride_d=sd, stride_h=sh, stride_w=sw, dil_d=dld, dil_h=dh, dil_w=dw,
                            pad_d=pd_l, pad_h=pad["h"][0], pad_w=pad["w"][0], pad_d_r=pd_r, pad_h_r=pr_h, pad_w_r=pr_w,
                            fil_layout=fl, in_layout=il, out_layout=ol, **d)
        if "out_d" in f and int(f["out_d"]) != cfg3.dout:
            raise ValueError("out_d does not follow from the other sizes")
        return cfg3
    cfg = ConvConfig(stride_h=sh, stride_w=sw, dil_h=dh, dil_w=dw, pad_h=pad["h"][0], pad_w=pad["w"][0], pad_h_r=pr_h,
                     pad_w_r=pr_w, fil_layout=fl, in_layout=il, out_layout=ol, **d)
    if "out_h" in f and int(f["out_h"]) != cfg.ho or "out_w" in f and int(f["out_w"]) != cfg.wo:
        raise ValueError("out_h / out_w do not follow from the other sizes")
    return cfg


def run_conv(f: Dict[str, str], direction: int) -> List[int]:
    from rocmlir_b200.conv import conv
    ty = resolve_types(f)
    cfg = conv_config(f)
    code = ty.a
    f8 = code in (oracle.F8E4M3, oracle.F8E5M2)
    if ty.b != ty.a:
        raise Unsupported("convolution with two different 8-bit float formats")
    if (code == oracle.I8 or f8) and direction != 0:
        raise ValueError("8-bit convolutions are forward only")
    out_code = oracle.I32 if code == oracle.I8 else oracle.F32 if f8 else code
    if ty.out != out_code:
        raise Unsupported("convolution output type differs from the input type")
    three = hasattr(cfg, "dout")
    if three:
        from rocmlir_b200.conv import conv3d as conv
        ocfg = oracle.Conv3d(n=cfg.n, c=cfg.c, k=cfg.k, d=cfg.d, h=cfg.h, w=cfg.w, z=cfg.z, y=cfg.y, x=cfg.x, g=cfg.g,
                             stride_d=cfg.stride_d, stride_h=cfg.stride_h, stride_w=cfg.stride_w, dil_d=cfg.dil_d,
                             dil_h=cfg.dil_h, dil_w=cfg.dil_w, pad_d=cfg.pad_d, pad_h=cfg.pad_h, pad_w=cfg.pad_w,
                             pad_d_r=cfg.pad_d_r, pad_h_r=cfg.pad_h_r, pad_w_r=cfg.pad_w_r, fil_layout=cfg.fil_layout,
                             in_layout=cfg.in_layout, out_layout=cfg.out_layout)
    else:
        ocfg = oracle.Conv(n=cfg.n, c=cfg.c, k=cfg.k, h=cfg.h, w=cfg.w, y=cfg.y, x=cfg.x, g=cfg.g,
                           stride_h=cfg.stride_h, stride_w=cfg.stride_w, dil_h=cfg.dil_h, dil_w=cfg.dil_w,
                           pad_h=cfg.pad_h, pad_w=cfg.pad_w, pad_h_r=cfg.pad_h_r, pad_w_r=cfg.pad_w_r,
                           fil_layout=cfg.fil_layout, in_layout=cfg.in_layout, out_layout=cfg.out_layout)
    fill = Filler(f)
    fil_f, fil_r = fill.tensor(ocfg.numel("fil"), code)
    in_f, in_r = fill.tensor(ocfg.numel("in"), code)
    out_f, out_r = fill.tensor(ocfg.numel("out"), out_code)
    threads = oracle.max_threads()
    if three:
        want = oracle.conv3d_i8(ocfg, fil_r, in_r, threads=threads) if code == oracle.I8 else \
            oracle.conv3d_f32(ocfg, direction, fil_f, in_f, out_f, threads=threads)
    elif code == oracle.I8:
        want = oracle.conv_i8(ocfg, fil_r, in_r, threads=threads)
    else:
        want = oracle.conv_f32(ocfg, direction, fil_f, in_f, out_f, threads=threads)
    t = {"fil": to_device(fil_r, code), "in": to_device(in_r, code), "out": to_device(out_r, out_code)}
    res = conv(cfg, direction, t["fil"], t["in"], t["out"])
    res_code = out_code if direction == 0 else code
    return verdict_for(from_device(res, res_code).ravel(), want.ravel(), res_code, f)


def run_attention(f: Dict[str, str]) -> List[int]:
    from rocmlir_b200.attention import attention
    ty = resolve_types(f)
    code = ty.a
    quantized = code == oracle.I8       # first GEMM i8 x i8, everything else f16 (rocmlir-gen.cpp:3497-3515)
    if code not in (oracle.F32, oracle.F16, oracle.BF16, oracle.I8):
        raise Unsupported("attention exists for f32, f16, bf16 and the first-GEMM-quantised i8 form")
    if as_bool(f, "p"):
        g, sq, sk, d, dv = 1, 1024, 1024, 32, 32
    else:
        g = int(f.get("g", 1))
        sq, sk, d, dv = int(f["seq_len_q"]), int(f["seq_len_k"]), int(f["head_dim_qk"]), int(f["head_dim_v"])
    if code != oracle.F32 and (d % 8 or dv % 8 or d > 128 or dv > 128):
        raise Unsupported("head dimensions that are not multiples of 8 up to 128")
    tq, tv, to = as_bool(f, "transQ"), as_bool(f, "transV"), as_bool(f, "transO")
    tk = as_bool(f, "transK")
    fill = Filler(f)
    q_f, q_r = fill.tensor(g * sq * d, code)
    k_f, k_r = fill.tensor(g * sk * d, code)
    if quantized:
        code = oracle.F16
    v_f, v_r = fill.tensor(g * sk * dv, code)
    if quantized:
        qb_f, qb_r = fill.tensor(1, oracle.I8)          # kernel-argument order: q, k, v, quantBias, quantScale, ...
        qs_f, qs_r = fill.tensor(1, oracle.F16)
    sc = bi = None
    if as_bool(f, "with-attn-scale"):
        sc = fill.tensor(g * sq * sk, code)
    if as_bool(f, "with-attn-bias"):
        bi = fill.tensor(g * sq * sk, code)
    fill.tensor(g * sq * dv, code)
    # stored shapes follow the trans flags (rocmlir-gen.cpp:2149-2200); the oracle takes Q [G,Sq,D], K [G,D,Sk],
    # V [G,Sk,Dv] and returns O [G,Sq,Dv]
    q_shape = (g, d, sq) if tq else (g, sq, d)
    k_shape = (g, sk, d) if tk else (g, d, sk)
    v_shape = (g, dv, sk) if tv else (g, sk, dv)
    logical = lambda a, shape, t: np.ascontiguousarray(a.reshape(shape).transpose(0, 2, 1) if t else a.reshape(shape))
    sc_f = None if sc is None else sc[0].reshape(g, sq, sk)
    bi_f = None if bi is None else bi[0].reshape(g, sq, sk)
    kw = dict(trans_q=tq, trans_k=tk, trans_v=tv, trans_o=to,
              scale_tensor=None if sc is None else to_device(sc[1].reshape(g, sq, sk), code),
              bias=None if bi is None else to_device(bi[1].reshape(g, sq, sk), code))
    if quantized:
        want = oracle.attention_i8(logical(q_r, q_shape, tq), logical(k_r, k_shape, tk), logical(v_f, v_shape, tv),
                                   int(qb_f[0]), float(qs_f[0]), scale=sc_f, bias=bi_f, threads=oracle.max_threads())
        o = attention(to_device(q_r.reshape(q_shape), oracle.I8), to_device(k_r.reshape(k_shape), oracle.I8),
                      to_device(v_r.reshape(v_shape), code), quant_bias=to_device(qb_r, oracle.I8),
                      quant_scale=to_device(qs_r, oracle.F16), **kw)
    else:
        want = oracle.attention(logical(q_f, q_shape, tq), logical(k_f, k_shape, tk), logical(v_f, v_shape, tv),
                                elem_type=code, scale=sc_f, bias=bi_f, threads=oracle.max_threads())
        o = attention(to_device(q_r.reshape(q_shape), code), to_device(k_r.reshape(k_shape), code),
                      to_device(v_r.reshape(v_shape), code), **kw)
    if to:
        want = np.ascontiguousarray(want.transpose(0, 2, 1))
    return verdict_for(from_device(o, code).ravel(), want.ravel(), code, f)


def run(flags: str) -> List[int]:
    """Runs one rocmlir-gen command line; returns the verdict triple. Raises Unsupported / ValueError."""
    import torch
    from rocmlir_b200 import _lib as L
    f = parse_flags(flags.replace("%arch", "sm_100a"))
    arch = f.get("arch", "sm_100a")
    if arch not in ("sm_100a", "sm_100"):
        raise ValueError(f"architecture {arch} is not this hardware")
    if "pv_with_gpu" in f or "pv_with_mlir" in f:
        raise Unsupported("validation against a second GPU kernel: the CPU validator is the oracle here")
    op = f.get("operation", "conv")
    if op == "gemm":
        v = run_gemm(f)
    elif op in ("conv", "conv_bwd_data", "conv_bwd_weight"):
        v = run_conv(f, {"conv": 0, "conv_bwd_data": 1, "conv_bwd_weight": 2}[op])
    elif op == "attention":
        v = run_attention(f)
    else:
        raise ValueError(f"unknown operation {op}")
    torch.cuda.synchronize()
    if L.kernel_status() != 0:
        raise RuntimeError("a kernel reported a bounded-wait timeout")
    return v


def plan(flags: str) -> None:
    """Parses, types and sizes one command line exactly as run() does and stops before touching data or the GPU:
    raises Unsupported / ValueError like run(), returns None for a line run() would execute."""
    global _PLAN_ONLY
    f = parse_flags(flags.replace("%arch", "sm_100a"))
    if f.get("arch", "sm_100a") not in ("sm_100a", "sm_100"):
        raise ValueError("architecture is not this hardware")
    if "pv_with_gpu" in f or "pv_with_mlir" in f:
        raise Unsupported("validation against a second GPU kernel: the CPU validator is the oracle here")
    op = f.get("operation", "conv")
    _PLAN_ONLY = True
    try:
        if op == "gemm":
            run_gemm(f)
        elif op in ("conv", "conv_bwd_data", "conv_bwd_weight"):
            run_conv(f, {"conv": 0, "conv_bwd_data": 1, "conv_bwd_weight": 2}[op])
        elif op == "attention":
            run_attention(f)
        else:
            raise ValueError(f"unknown operation {op}")
    except Planned:
        return None
    finally:
        _PLAN_ONLY = False
    raise AssertionError("the operation ran without building a Filler")


def main(argv: List[str]) -> int:
    try:
        v = run(" ".join(argv))
    except Unsupported as e:
        print(f"unsupported: {e}", file=sys.stderr)
        return 2
    print("[" + " ".join(str(x) for x in v) + "]")
    return 0 if v == [1, 1, 1] else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
