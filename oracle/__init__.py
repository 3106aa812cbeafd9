"""numpy/ctypes front end of the CPU oracle (oracle/oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by bench.py's CPU-baseline leg;
never by the product package. Every function cites, in oracle.cpp, the reference code it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "liboracle.so")
REF_LIB_PATH = os.path.join(HERE, "_ref", "libconv-validation-wrappers.so")

F32, F16, BF16, I8, I32, F8E4M3, I64, F64, F8E5M2 = range(9)
_STORAGE = {F32: np.float32, F16: np.uint16, BF16: np.uint16, I8: np.int8, I32: np.int32, F8E4M3: np.uint8, F8E5M2: np.uint8,
            I64: np.int64}

_lib = None


def build() -> None:
    subprocess.run(["make", "-C", HERE], check=True, capture_output=True)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = C.CDLL(LIB_PATH)
        _lib.orc_random_integer_value.restype = C.c_float
        _lib.orc_random_integer_value.argtypes = [C.c_int16, C.c_int16]
        _lib.orc_random_float_value.restype = C.c_float
        _lib.orc_random_float_value.argtypes = [C.c_int16, C.c_int16]
        _lib.orc_verify_float.restype = C.c_int
        _lib.orc_verify_int.restype = C.c_int
        _lib.orc_max_threads.restype = C.c_int
    return _lib


def ref_lib() -> Optional[C.CDLL]:
    """The reference's own conv-validation-wrappers.cpp, compiled unmodified (None if not built)."""
    if not os.path.exists(REF_LIB_PATH):
        return None
    r = C.CDLL(REF_LIB_PATH)
    r.randomIntegerValue.restype = C.c_float
    r.randomIntegerValue.argtypes = [C.c_int16, C.c_int16]
    r.randomFloatValue.restype = C.c_float
    r.randomFloatValue.argtypes = [C.c_int16, C.c_int16]
    r.seedRandomValues.argtypes = [C.c_uint32]
    return r


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---- conversions -------------------------------------------------------------------------------------
def to_f32(raw: np.ndarray, dtype: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw)
    out = np.empty(raw.shape, np.float32)
    lib().orc_convert_to_f32(_p(raw), C.c_int(dtype), _p(out), C.c_int64(raw.size))
    return out


def from_f32(x: np.ndarray, dtype: int, sat_int: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, _STORAGE[dtype])
    lib().orc_convert_from_f32(_p(x), _p(out), C.c_int(dtype), C.c_int64(x.size), C.c_int(int(sat_int)))
    return out


def round_to(x: np.ndarray, dtype: int) -> np.ndarray:
    return to_f32(from_f32(x, dtype), dtype)


# ---- data fill -----------------------------------------------------------------------------------------
def seed(s: int) -> None:
    lib().orc_seed(C.c_uint32(s))


def fill_random(n: int, rand_float: bool, mn: int, mx: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_fill_random(_p(out), C.c_int64(n), C.c_int(int(rand_float)), C.c_int16(mn), C.c_int16(mx))
    return out


def fill_pattern(n: int, pattern: Sequence[float]) -> np.ndarray:
    out = np.empty(n, np.float32)
    pat = np.asarray(pattern, np.float32)
    lib().orc_fill_pattern(_p(out), C.c_int64(n), _p(pat), C.c_int(len(pat)))
    return out


# ---- gemm ---------------------------------------------------------------------------------------------------
def gemm_f32(a: np.ndarray, b: np.ndarray, G: int, M: int, N: int, K: int, ta=False, tb=False, tc=False,
             threads: int = 1) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    c = np.empty((G, N, M) if tc else (G, M, N), np.float32)
    lib().orc_gemm_f32(_p(a), _p(b), _p(c), C.c_int64(G), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int(int(ta)),
                       C.c_int(int(tb)), C.c_int(int(tc)), C.c_int(threads))
    return c


def gemm_f64(a, b, G, M, N, K, ta=False, tb=False, tc=False, threads: int = 1) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    c = np.empty((G, N, M) if tc else (G, M, N), np.float64)
    lib().orc_gemm_f64(_p(a), _p(b), _p(c), C.c_int64(G), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int(int(ta)),
                       C.c_int(int(tb)), C.c_int(int(tc)), C.c_int(threads))
    return c


def gemm_i8(a: np.ndarray, b: np.ndarray, G: int, M: int, N: int, K: int, ta=False, tb=False, tc=False,
            threads: int = 1) -> np.ndarray:
    a = np.ascontiguousarray(a, np.int8)
    b = np.ascontiguousarray(b, np.int8)
    c = np.empty((G, N, M) if tc else (G, M, N), np.int64)
    lib().orc_gemm_i8(_p(a), _p(b), _p(c), C.c_int64(G), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int(int(ta)),
                      C.c_int(int(tb)), C.c_int(int(tc)), C.c_int(threads))
    return c


# ---- convolution ----------------------------------------------------------------------------------------------
class _OrcConv(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("n", "g", "c", "k", "h", "w", "y", "x", "ho", "wo", "stride_h", "stride_w",
                                         "dil_h", "dil_w", "pad_h", "pad_w")] + \
               [("fs", C.c_int64 * 5), ("is_", C.c_int64 * 5), ("os", C.c_int64 * 5)]


def out_dim(inp: int, fil: int, pad_l: int, pad_r: int, stride: int, dil: int) -> int:
    """Output size rule of the reference (mlir/include/mlir/Dialect/Rock/Generator/ConvGenerator.h:98-104)."""
    return (inp + pad_l + pad_r - (fil - 1) * dil - 1) // stride + 1


def layout_strides(layout: str, sizes: dict) -> dict:
    """Element strides of each named dimension for a tensor stored in `layout` order (e.g. 'ngchw')."""
    strides, acc = {}, 1
    for d in reversed(layout):
        strides[d] = acc
        acc *= sizes[d]
    return strides


@dataclass
class Conv:
    n: int
    c: int          # channels per group
    k: int          # output channels per group
    h: int
    w: int
    y: int
    x: int
    g: int = 1
    stride_h: int = 1
    stride_w: int = 1
    dil_h: int = 1
    dil_w: int = 1
    pad_h: int = 0  # left padding
    pad_w: int = 0
    pad_h_r: Optional[int] = None
    pad_w_r: Optional[int] = None
    fil_layout: str = "gkcyx"
    in_layout: str = "ngchw"
    out_layout: str = "ngkhw"
    ho: int = field(init=False)
    wo: int = field(init=False)

    def __post_init__(self):
        pr_h = self.pad_h if self.pad_h_r is None else self.pad_h_r
        pr_w = self.pad_w if self.pad_w_r is None else self.pad_w_r
        self.ho = out_dim(self.h, self.y, self.pad_h, pr_h, self.stride_h, self.dil_h)
        self.wo = out_dim(self.w, self.x, self.pad_w, pr_w, self.stride_w, self.dil_w)

    def sizes(self):
        return {"fil": {"g": self.g, "k": self.k, "c": self.c, "y": self.y, "x": self.x},
                "in": {"n": self.n, "g": self.g, "c": self.c, "h": self.h, "w": self.w},
                "out": {"n": self.n, "g": self.g, "k": self.k, "h": self.ho, "w": self.wo}}

    def numel(self, which: str) -> int:
        return int(np.prod(list(self.sizes()[which].values())))

    def to_c(self) -> _OrcConv:
        s = self.sizes()
        fs = layout_strides(self.fil_layout, s["fil"])
        is_ = layout_strides(self.in_layout, s["in"])
        os_ = layout_strides(self.out_layout, s["out"])
        p = _OrcConv(self.n, self.g, self.c, self.k, self.h, self.w, self.y, self.x, self.ho, self.wo, self.stride_h,
                     self.stride_w, self.dil_h, self.dil_w, self.pad_h, self.pad_w)
        p.fs = (C.c_int64 * 5)(*[fs[d] for d in "gkcyx"])
        p.is_ = (C.c_int64 * 5)(*[is_[d] for d in "ngchw"])
        p.os = (C.c_int64 * 5)(*[os_[d] for d in "ngkhw"])
        return p


FWD, BWD_DATA, BWD_WEIGHT = 0, 1, 2


def conv_f32(p: Conv, direction: int, fil: Optional[np.ndarray], inp: Optional[np.ndarray],
             out: Optional[np.ndarray], threads: int = 1, f64: bool = False) -> np.ndarray:
    """Flat tensors in their storage layouts; returns the flat result tensor of the direction."""
    which = {FWD: "out", BWD_DATA: "in", BWD_WEIGHT: "fil"}[direction]
    res = np.zeros(p.numel(which), np.float64 if f64 else np.float32)
    fil = None if fil is None else np.ascontiguousarray(fil, np.float32)
    inp = None if inp is None else np.ascontiguousarray(inp, np.float32)
    out = None if out is None else np.ascontiguousarray(out, np.float32)
    cp = p.to_c()
    fn = lib().orc_conv_f64 if f64 else lib().orc_conv_f32
    fn(C.byref(cp), C.c_int(direction), _p(fil), _p(inp), _p(out), _p(res), C.c_int(threads))
    return res


def conv_i8(p: Conv, fil: np.ndarray, inp: np.ndarray, wrap_product: bool = True, threads: int = 1) -> np.ndarray:
    res = np.zeros(p.numel("out"), np.int64)
    fil = np.ascontiguousarray(fil, np.int8)
    inp = np.ascontiguousarray(inp, np.int8)
    cp = p.to_c()
    lib().orc_conv_i8(C.byref(cp), _p(fil), _p(inp), _p(res), C.c_int(int(wrap_product)), C.c_int(threads))
    return res


# ---- convolution with three image dimensions ----------------------------------------------------------------------
class _OrcConv3(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("n", "g", "c", "k", "d", "h", "w", "z", "y", "x", "dout", "ho", "wo",
                                         "stride_d", "stride_h", "stride_w", "dil_d", "dil_h", "dil_w",
                                         "pad_d", "pad_h", "pad_w")] + \
               [("fs", C.c_int64 * 6), ("is_", C.c_int64 * 6), ("os", C.c_int64 * 6)]


@dataclass
class Conv3d:
    """Sizes of a convolution over (d, h, w); c and k per group; pad_* are the left paddings, pad_*_r the right ones
    (default: equal). Layout letters: filter g k c z y x, input n g c d h w, output n g k d h w."""
    n: int
    c: int
    k: int
    d: int
    h: int
    w: int
    z: int
    y: int
    x: int
    g: int = 1
    stride_d: int = 1
    stride_h: int = 1
    stride_w: int = 1
    dil_d: int = 1
    dil_h: int = 1
    dil_w: int = 1
    pad_d: int = 0
    pad_h: int = 0
    pad_w: int = 0
    pad_d_r: Optional[int] = None
    pad_h_r: Optional[int] = None
    pad_w_r: Optional[int] = None
    fil_layout: str = "gkczyx"
    in_layout: str = "ngcdhw"
    out_layout: str = "ngkdhw"
    dout: int = field(init=False)
    ho: int = field(init=False)
    wo: int = field(init=False)

    def __post_init__(self):
        for ax in "dhw":
            if getattr(self, f"pad_{ax}_r") is None:
                setattr(self, f"pad_{ax}_r", getattr(self, f"pad_{ax}"))
        self.dout = out_dim(self.d, self.z, self.pad_d, self.pad_d_r, self.stride_d, self.dil_d)
        self.ho = out_dim(self.h, self.y, self.pad_h, self.pad_h_r, self.stride_h, self.dil_h)
        self.wo = out_dim(self.w, self.x, self.pad_w, self.pad_w_r, self.stride_w, self.dil_w)

    def sizes(self):
        return {"fil": {"g": self.g, "k": self.k, "c": self.c, "z": self.z, "y": self.y, "x": self.x},
                "in": {"n": self.n, "g": self.g, "c": self.c, "d": self.d, "h": self.h, "w": self.w},
                "out": {"n": self.n, "g": self.g, "k": self.k, "d": self.dout, "h": self.ho, "w": self.wo}}

    def numel(self, which: str) -> int:
        return int(np.prod(list(self.sizes()[which].values())))

    def shape(self, which: str):
        """Shape of the tensor as stored, i.e. in its layout's order."""
        s = self.sizes()[which]
        lay = {"fil": self.fil_layout, "in": self.in_layout, "out": self.out_layout}[which]
        return tuple(s[ch] for ch in lay)

    def to_c(self) -> _OrcConv3:
        s = self.sizes()
        fs = layout_strides(self.fil_layout, s["fil"])
        is_ = layout_strides(self.in_layout, s["in"])
        os_ = layout_strides(self.out_layout, s["out"])
        p = _OrcConv3(self.n, self.g, self.c, self.k, self.d, self.h, self.w, self.z, self.y, self.x, self.dout,
                      self.ho, self.wo, self.stride_d, self.stride_h, self.stride_w, self.dil_d, self.dil_h,
                      self.dil_w, self.pad_d, self.pad_h, self.pad_w)
        p.fs = (C.c_int64 * 6)(*[fs[ch] for ch in "gkczyx"])
        p.is_ = (C.c_int64 * 6)(*[is_[ch] for ch in "ngcdhw"])
        p.os = (C.c_int64 * 6)(*[os_[ch] for ch in "ngkdhw"])
        return p


def conv3d_f32(p: Conv3d, direction: int, fil: Optional[np.ndarray], inp: Optional[np.ndarray],
               out: Optional[np.ndarray], threads: int = 1, f64: bool = False) -> np.ndarray:
    """Flat tensors in their storage layouts; returns the flat result tensor of the direction."""
    which = {FWD: "out", BWD_DATA: "in", BWD_WEIGHT: "fil"}[direction]
    res = np.zeros(p.numel(which), np.float64 if f64 else np.float32)
    fil = None if fil is None else np.ascontiguousarray(fil, np.float32)
    inp = None if inp is None else np.ascontiguousarray(inp, np.float32)
    out = None if out is None else np.ascontiguousarray(out, np.float32)
    cp = p.to_c()
    fn = lib().orc_conv3d_f64 if f64 else lib().orc_conv3d_f32
    fn(C.byref(cp), C.c_int(direction), _p(fil), _p(inp), _p(out), _p(res), C.c_int(threads))
    return res


def conv3d_i8(p: Conv3d, fil: np.ndarray, inp: np.ndarray, threads: int = 1) -> np.ndarray:
    res = np.zeros(p.numel("out"), np.int64)
    fil = np.ascontiguousarray(fil, np.int8)
    inp = np.ascontiguousarray(inp, np.int8)
    cp = p.to_c()
    lib().orc_conv3d_i8(C.byref(cp), _p(fil), _p(inp), _p(res), C.c_int(threads))
    return res


# ---- attention / gemm+gemm ---------------------------------------------------------------------------------------
def attention(q, k, v, *, elem_type: int, scale=None, bias=None, mask=None, mask_fill: float = 0.0,
              scale_scalar: Optional[float] = None, causal: bool = False, g_range=None, threads: int = 1):
    """q [G,Sq,D], k [G,D,Sk], v [G,Sk,Dv] as f32 arrays holding elem_type-representable values."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    G, Sq, D = q.shape
    Sk, Dv = v.shape[1], v.shape[2]
    assert k.shape == (G, D, Sk)
    o = np.zeros((G, Sq, Dv), np.float32)
    scale = None if scale is None else np.ascontiguousarray(scale, np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    mask = None if mask is None else np.ascontiguousarray(mask, np.int8)
    g0, g1 = g_range if g_range is not None else (0, G)
    lib().orc_attention(_p(q), _p(k), _p(v), _p(scale), _p(bias), _p(mask), C.c_float(mask_fill),
                        C.c_int(int(scale_scalar is not None)), C.c_float(scale_scalar or 0.0), _p(o), C.c_int64(G),
                        C.c_int64(Sq), C.c_int64(Sk), C.c_int64(D), C.c_int64(Dv), C.c_int(elem_type),
                        C.c_int(int(causal)), C.c_int64(g0), C.c_int64(g1), C.c_int(threads))
    return o


def attention_i8(q, k, v, quant_bias: int, quant_scale: float, *, scale=None, bias=None, threads: int = 1):
    """First-GEMM-quantised attention: q [G,Sq,D] and k [G,D,Sk] int8, v [G,Sk,Dv] f32 holding f16 values,
    quant_bias the i8 zero point, quant_scale an f16 value; optional f16 scale / bias tensors [G,Sq,Sk]."""
    q = np.ascontiguousarray(q, np.int8)
    k = np.ascontiguousarray(k, np.int8)
    v = np.ascontiguousarray(v, np.float32)
    G, Sq, D = q.shape
    Sk, Dv = v.shape[1], v.shape[2]
    assert k.shape == (G, D, Sk)
    o = np.zeros((G, Sq, Dv), np.float32)
    scale = None if scale is None else np.ascontiguousarray(scale, np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().orc_attention_i8(_p(q), _p(k), _p(v), C.c_int(int(quant_bias)), C.c_float(float(quant_scale)), _p(scale),
                           _p(bias), _p(o), C.c_int64(G), C.c_int64(Sq), C.c_int64(Sk), C.c_int64(D), C.c_int64(Dv),
                           C.c_int(threads))
    return o


def gemm_gemm(a, b1, b2, mid_type: int, threads: int = 1) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    b1 = np.ascontiguousarray(b1, np.float32)
    b2 = np.ascontiguousarray(b2, np.float32)
    M, K1 = a.shape
    N1, N2 = b1.shape[1], b2.shape[1]
    o = np.empty((M, N2), np.float32)
    lib().orc_gemm_gemm(_p(a), _p(b1), _p(b2), _p(o), C.c_int64(M), C.c_int64(K1), C.c_int64(N1), C.c_int64(N2),
                        C.c_int(mid_type), C.c_int(threads))
    return o


# ---- epilogue -------------------------------------------------------------------------------------------------------
EPI_ALPHA, EPI_COL_SCALE, EPI_BIAS, EPI_RELU, EPI_REQUANT, EPI_ROUND_MID = 1, 2, 4, 8, 16, 32
EPI_CLIP, EPI_RESIDUAL, EPI_BIAS_ROW, EPI_BIAS_SCALAR, EPI_ZP_IN = 64, 128, 256, 512, 1024
EPI_UNARY = 4096
UNARY = {n: i + 1 for i, n in enumerate(("abs", "ceil", "erf", "exp", "floor", "log", "neg", "recip", "rsqrt", "sigmoid",
                                          "sqrt", "tanh"))}


def epilogue(acc: np.ndarray, N: int, *, alpha=None, col_scale=None, bias=None, relu=False, requant_scale=None,
             mid_type=None, bias_mode: str = "col", residual=None, clip=None, in_zero=None, unary=None) -> np.ndarray:
    """acc: f32 or i64 accumulators, last dimension N; `bias_mode` "col" (bias[n]), "row" (bias[row], rows counted
    over all leading dimensions) or "scalar"; `residual` an f32 array of acc's shape; `clip` = (lo, hi); `in_zero` the
    dequantisation zero point; `unary` one of UNARY (a name or its code). Returns f32 (convert with from_f32(..., sat_int=True) or quantize_i8)."""
    flags = 0
    if alpha is not None: flags |= EPI_ALPHA
    if col_scale is not None: flags |= EPI_COL_SCALE
    if bias is not None: flags |= EPI_BIAS | {"col": 0, "row": EPI_BIAS_ROW, "scalar": EPI_BIAS_SCALAR}[bias_mode]
    if relu: flags |= EPI_RELU
    if requant_scale is not None: flags |= EPI_REQUANT
    if mid_type is not None: flags |= EPI_ROUND_MID
    if residual is not None: flags |= EPI_RESIDUAL
    if clip is not None: flags |= EPI_CLIP
    if in_zero is not None: flags |= EPI_ZP_IN
    if unary is not None: flags |= EPI_UNARY
    ucode = UNARY[unary] if isinstance(unary, str) else int(unary or 0)
    rows = acc.size // N
    out = np.empty(acc.shape, np.float32)
    is_int = acc.dtype == np.int64
    accc = np.ascontiguousarray(acc)
    cs = None if col_scale is None else np.ascontiguousarray(col_scale, np.float32)
    bs = None if bias is None else np.ascontiguousarray(bias, np.float32).ravel()
    rs = None if residual is None else np.ascontiguousarray(residual, np.float32)
    assert rs is None or rs.size == acc.size
    recip = np.float32(1.0) / np.float32(requant_scale) if requant_scale is not None else np.float32(0)
    lo, hi = clip if clip is not None else (0.0, 0.0)
    lib().orc_epilogue(None if is_int else _p(accc), _p(accc) if is_int else None, _p(out), C.c_int64(rows),
                       C.c_int64(N), C.c_uint32(flags), C.c_float(np.float32(alpha or 0.0)), _p(cs), _p(bs),
                       C.c_float(recip), C.c_int(mid_type if mid_type is not None else F32), C.c_float(np.float32(lo)),
                       C.c_float(np.float32(hi)), C.c_float(np.float32(in_zero or 0.0)), _p(rs), C.c_int(ucode))
    return out


def quantize_i8(x: np.ndarray, zero_point: int = 0) -> np.ndarray:
    """The store of quantizelinear (MIGraphXToTosa.cpp:908-982): cast to i32 with round-half-even and saturation, add
    the zero point, clamp to [-128, 127]."""
    q = np.clip(np.rint(np.asarray(x, np.float64)), -2.0 ** 31, 2.0 ** 31 - 1).astype(np.int64) + int(zero_point)
    return np.clip(q, -128, 127).astype(np.int8)


# ---- verification ------------------------------------------------------------------------------------------------------
def verify_float(gpu: np.ndarray, val: np.ndarray, thr_rms: float, thr_abs: float, thr_rel: float):
    """Returns ([rms_ok, abs_ok, rel_ok], {'rms','max_abs','max_rel'}) like the reference's verdict line."""
    gpu = np.ascontiguousarray(gpu, np.float32).ravel()
    val = np.ascontiguousarray(val, np.float32).ravel()
    assert gpu.size == val.size
    m = (C.c_double * 3)()
    bits = lib().orc_verify_float(_p(gpu), _p(val), C.c_int64(gpu.size), C.c_float(thr_rms), C.c_float(thr_abs),
                                  C.c_float(thr_rel), m)
    return [bits & 1, (bits >> 1) & 1, (bits >> 2) & 1], {"rms": m[0], "max_abs": m[1], "max_rel": m[2]}


def verify_int(gpu: np.ndarray, val_i64: np.ndarray):
    gpu = np.ascontiguousarray(gpu).ravel()
    val = np.ascontiguousarray(val_i64, np.int64).ravel()
    t = I8 if gpu.dtype == np.int8 else I32
    cnt = (C.c_int64 * 2)()
    bits = lib().orc_verify_int(_p(gpu), C.c_int(t), _p(val), C.c_int64(gpu.size), cnt)
    return [bits & 1, (bits >> 1) & 1, (bits >> 2) & 1], {"mismatches": cnt[0], "overflows": cnt[1]}
