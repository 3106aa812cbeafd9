"""Host-side mirror of rock.gemm (mlir/include/mlir/Dialect/Rock/IR/RockOps.td:136-181) over the C ABI.

Operands are CUDA torch tensors used only as device buffers: A is G x M x K (trans_a: G x K x M),
B is G x K x N (trans_b: G x N x K), C is G x M x N (trans_c: G x N x M) — the flat row-major
buffers rocmlir-gen's kernels take. 2-D tensors are treated as G = 1.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib as L

_TORCH2RB = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16, torch.int8: L.I8,
             torch.int32: L.I32, torch.float8_e4m3fn: L.F8E4M3, torch.float8_e5m2: L.F8E5M2}
_RB2TORCH = {v: k for k, v in _TORCH2RB.items()}


def rb_dtype(t: torch.dtype) -> int:
    if t not in _TORCH2RB:
        raise L.RbError(L.INVALID_PARAM, f"unsupported element type {t}")
    return _TORCH2RB[t]


def torch_dtype(t: int) -> torch.dtype:
    return _RB2TORCH[t]


@dataclass
class Epilogue:
    """Fused elementwise tail of the GEMM; fields map one-to-one onto RbEpilogue."""
    alpha: Optional[float] = None               # per-tensor scale product (fp8 dequantisation)
    col_scale: Optional[torch.Tensor] = None    # f32 [N], dequantizelinear scale per output column
    bias: Optional[torch.Tensor] = None         # [N], f32 / f16 / bf16
    relu: bool = False
    requant_scale: Optional[float] = None       # quantizelinear scale; the kernel multiplies by fl32(1/scale)
    mid_type: Optional[int] = None              # declared GEMM result type: round to it before/after the bias add
    bias_mode: str = "col"                      # "col": bias[n]; "row": bias[m] (broadcast along N); "scalar": bias[0]
    residual: Optional[torch.Tensor] = None     # same shape and layout as C: the same-shape add of dot + add
    clip: Optional[tuple] = None                # (lo, hi): migraphx.clip after the rectifier
    in_zero: Optional[float] = None             # dequantizelinear zero point (subtracted from the accumulator)
    out_zero: Optional[int] = None              # quantizelinear zero point (added after the rounding cast, i8 results)
    unary: Optional[str] = None                 # one MIGraphX unary function ("sigmoid", "tanh", "erf", ...: _lib.UNARY) before the rectifier

    def to_c(self) -> L.RbEpilogue:
        e = L.RbEpilogue()
        flags = 0
        if self.alpha is not None:
            flags |= L.EPI_ALPHA
            e.alpha = float(np.float32(self.alpha))
        if self.col_scale is not None:
            assert self.col_scale.dtype == torch.float32 and self.col_scale.is_cuda and self.col_scale.is_contiguous()
            flags |= L.EPI_COL_SCALE
            e.col_scale = self.col_scale.data_ptr()
        if self.bias is not None:
            assert self.bias.is_cuda and self.bias.is_contiguous()
            flags |= L.EPI_BIAS
            e.bias = self.bias.data_ptr()
            e.bias_type = rb_dtype(self.bias.dtype)
            flags |= {"col": 0, "row": L.EPI_BIAS_ROW, "scalar": L.EPI_BIAS_SCALAR}[self.bias_mode]
        if self.residual is not None:
            assert self.residual.is_cuda and self.residual.is_contiguous()
            flags |= L.EPI_RESIDUAL
            e.residual = self.residual.data_ptr()
            e.res_type = rb_dtype(self.residual.dtype)
        if self.clip is not None:
            flags |= L.EPI_CLIP
            e.clip_lo, e.clip_hi = float(np.float32(self.clip[0])), float(np.float32(self.clip[1]))
        if self.in_zero is not None:
            flags |= L.EPI_ZP_IN
            e.in_zero = float(np.float32(self.in_zero))
        if self.out_zero is not None:
            flags |= L.EPI_ZP_OUT
            e.out_zero = int(self.out_zero)
        if self.unary is not None:
            flags |= L.EPI_UNARY
            e.unary = L.UNARY[self.unary]
        if self.relu:
            flags |= L.EPI_RELU
        if self.requant_scale is not None:
            flags |= L.EPI_REQUANT
            e.out_recip = float(np.float32(1.0) / np.float32(self.requant_scale))
        if self.mid_type is not None:
            flags |= L.EPI_ROUND_MID
            e.mid_type = int(self.mid_type)
        e.flags = flags
        return e


def _as3d(t: torch.Tensor) -> torch.Tensor:
    return t.unsqueeze(0) if t.dim() == 2 else t


def problem(a: torch.Tensor, b: torch.Tensor, trans_a: bool, trans_b: bool, trans_c: bool, out_dtype: torch.dtype,
            f32_mode: int = 0, accumulate: bool = False) -> L.RbGemmProblem:
    a3, b3 = _as3d(a), _as3d(b)
    g = a3.shape[0]
    m, k = (a3.shape[2], a3.shape[1]) if trans_a else (a3.shape[1], a3.shape[2])
    kb, n = (b3.shape[2], b3.shape[1]) if trans_b else (b3.shape[1], b3.shape[2])
    if kb != k or b3.shape[0] != g:
        raise L.RbError(L.INVALID_PARAM, f"shape mismatch: A {tuple(a.shape)} B {tuple(b.shape)}")
    if a.dtype == b.dtype:
        ab = rb_dtype(a.dtype)
    elif (a.dtype, b.dtype) == (torch.float8_e4m3fn, torch.float8_e5m2):
        ab = L.F8E4M3_E5M2      # rocmlir-gen's -t fp8_bf8
    elif (a.dtype, b.dtype) == (torch.float8_e5m2, torch.float8_e4m3fn):
        ab = L.F8E5M2_E4M3      # -t bf8_fp8
    else:
        raise L.RbError(L.UNSUPPORTED, "mixed A/B element types exist for the two 8-bit float formats only")
    return L.RbGemmProblem(g, m, n, k, int(trans_a), int(trans_b), int(trans_c), ab, rb_dtype(out_dtype), int(f32_mode),
                           int(accumulate))


def default_out_dtype(ab: torch.dtype) -> torch.dtype:
    # rocmlir-gen: -t i8 => i32 result, -t fp8 => f32 result (rocmlir-gen.cpp:432-458)
    if ab == torch.int8:
        return torch.int32
    if ab in (torch.float8_e4m3fn, torch.float8_e5m2):
        return torch.float32
    return ab


def workspace_size(p: L.RbGemmProblem) -> int:
    return int(L.lib().rbGemmWorkspaceSize(C.byref(p)))


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False, trans_c: bool = False,
         out_dtype: Optional[torch.dtype] = None, epilogue: Optional[Epilogue] = None,
         out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None, f32_mode: int = 0,
         variant: Optional[int] = None, accumulate: bool = False) -> torch.Tensor:
    """`accumulate`: C = C + A.B on the given `out` (rocmlir-gen's --store-method=atomic_add)."""
    if accumulate and out is None:
        raise L.RbError(L.INVALID_PARAM, "accumulate adds to `out`, which must be given")
    if not (a.is_cuda and b.is_cuda):
        raise L.RbError(L.CUDA_ERROR, "operands must be CUDA tensors (the library has no CPU path)")
    if not (a.is_contiguous() and b.is_contiguous()):
        raise L.RbError(L.INVALID_PARAM, "operands must be contiguous")
    out_dtype = out_dtype or default_out_dtype(a.dtype)
    p = problem(a, b, trans_a, trans_b, trans_c, out_dtype, f32_mode, accumulate)
    shape = (p.g, p.n, p.m) if trans_c else (p.g, p.m, p.n)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    else:
        assert out.is_contiguous() and out.dtype == out_dtype and out.numel() == p.g * p.m * p.n
    lib = L.lib()
    # The variant word is state of the calling thread inside the library: set it for this call only and put the
    # caller's value back, so that a tuned call does not change what later calls (of any operator) run.
    saved = lib.rbGetGemmVariant()
    try:
        if variant is not None:   # before the workspace query: a K split or a stream-K tail changes what is needed
            lib.rbSetGemmVariant(int(variant))
        ws_bytes = workspace_size(p)
        if ws_bytes and (workspace is None or workspace.numel() * workspace.element_size() < ws_bytes):
            workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
        e = epilogue.to_c() if epilogue is not None else None
        stream = torch.cuda.current_stream(a.device).cuda_stream
        st = lib.rbGemm(C.byref(p), C.byref(e) if e is not None else None, a.data_ptr(), b.data_ptr(), out.data_ptr(),
                        workspace.data_ptr() if workspace is not None else None,
                        workspace.numel() * workspace.element_size() if workspace is not None else 0, stream)
    finally:
        lib.rbSetGemmVariant(saved)
    L.check(st)
    if a.dim() == 2 and b.dim() == 2:
        out = out.view(shape[1], shape[2])
    return out


def gemm_host(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
              trans_c: bool = False, epilogue: Optional[Epilogue] = None, f32_mode: int = 0,
              variant: Optional[int] = None, device: Optional[torch.device] = None) -> torch.Tensor:
    """rbGemmHost: A, B and the result are HOST tensors (pinned memory makes the copies asynchronous); the
    call returns when the result is in `out`. Epilogue vectors, if any, are host tensors too."""
    if a.is_cuda or b.is_cuda or out.is_cuda:
        raise L.RbError(L.INVALID_PARAM, "gemm_host takes host tensors")
    p = problem(a, b, trans_a, trans_b, trans_c, out.dtype, f32_mode)
    assert out.is_contiguous() and out.numel() == p.g * p.m * p.n
    e = None
    if epilogue is not None:
        # build the struct from host pointers
        cs, bs = epilogue.col_scale, epilogue.bias
        e = L.RbEpilogue()
        tmp = Epilogue(alpha=epilogue.alpha, relu=epilogue.relu, requant_scale=epilogue.requant_scale,
                       mid_type=epilogue.mid_type).to_c()
        e.flags, e.alpha, e.out_recip, e.mid_type = tmp.flags, tmp.alpha, tmp.out_recip, tmp.mid_type
        if cs is not None:
            assert not cs.is_cuda and cs.dtype == torch.float32
            e.flags |= L.EPI_COL_SCALE
            e.col_scale = cs.data_ptr()
        if bs is not None:
            assert not bs.is_cuda
            e.flags |= L.EPI_BIAS
            e.bias = bs.data_ptr()
            e.bias_type = rb_dtype(bs.dtype)
    lib = L.lib()
    saved = lib.rbGetGemmVariant()
    try:
        if variant is not None:
            lib.rbSetGemmVariant(int(variant))
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            st = lib.rbGemmHost(C.byref(p), C.byref(e) if e is not None else None, a.data_ptr(), b.data_ptr(),
                                out.data_ptr(), stream)
    finally:
        lib.rbSetGemmVariant(saved)
    L.check(st)
    return out


def gemm_gemm(a: torch.Tensor, b1: torch.Tensor, b2: torch.Tensor, *, out: Optional[torch.Tensor] = None,
              workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """O = (A . B1) . B2 with the intermediate rounded to the element type (rbGemmGemm)."""
    a3, b13, b23 = _as3d(a), _as3d(b1), _as3d(b2)
    g, m, k1 = a3.shape
    n1, n2 = b13.shape[2], b23.shape[2]
    assert b13.shape == (g, k1, n1) and b23.shape == (g, n1, n2)
    for t in (a, b1, b2):
        if not t.is_cuda or not t.is_contiguous():
            raise L.RbError(L.INVALID_PARAM, "operands must be contiguous CUDA tensors")
    dt = rb_dtype(a.dtype)
    lib = L.lib()
    need = int(lib.rbGemmGemmWorkspaceSize(g, m, k1, n1, n2, dt))
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
    if out is None:
        out = torch.empty((g, m, n2), dtype=a.dtype, device=a.device)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    L.check(lib.rbGemmGemm(g, m, k1, n1, n2, dt, a.data_ptr(), b1.data_ptr(), b2.data_ptr(), out.data_ptr(),
                           workspace.data_ptr(), workspace.numel() * workspace.element_size(), stream))
    return out.view(m, n2) if a.dim() == 2 else out
