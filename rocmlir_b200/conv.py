"""Host-side mirror of rock.conv / conv_bwd_data / conv_bwd_weight over the C ABI.

Names and meanings follow rocmlir-gen's convolution flags (mlir/tools/rocmlir-gen/rocmlir-gen.cpp:73-785):
layouts are strings over g k c y x / n g c h w / n g k h w (a missing `g` is inserted where the reference
inserts it, rocmlir-gen.cpp:837-862), channels are per group, tensors are flat CUDA buffers in layout order.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib as L
from .gemm import rb_dtype

FWD, BWD_DATA, BWD_WEIGHT = 0, 1, 2
OPERATIONS = {"conv": FWD, "conv_bwd_data": BWD_DATA, "conv_bwd_weight": BWD_WEIGHT}


def out_dim(inp: int, fil: int, pad_l: int, pad_r: int, stride: int, dil: int) -> int:
    return (inp + pad_l + pad_r - (fil - 1) * dil - 1) // stride + 1


def add_group(layout: str, channel: str) -> str:
    """Inserts the group letter the way rocmlir-gen does for layouts given without it."""
    layout = layout.replace("0", "h" if channel != "f" else "y").replace("1", "w" if channel != "f" else "x")
    if "g" in layout:
        return layout
    if channel == "f":  # filter
        return "g" + layout
    ch = channel
    if layout[:2] == "n" + ch:
        return "ng" + ch + layout[2:]
    if layout[0] == "n" and layout[-1] == ch:
        return layout[:-1] + "g" + ch
    return "g" + layout


@dataclass
class ConvConfig:
    n: int
    c: int
    k: int
    h: int
    w: int
    y: int
    x: int
    g: int = 1
    stride_h: int = 1
    stride_w: int = 1
    dil_h: int = 1
    dil_w: int = 1
    pad_h: int = 0
    pad_w: int = 0
    pad_h_r: Optional[int] = None
    pad_w_r: Optional[int] = None
    fil_layout: str = "gkyxc"
    in_layout: str = "nhwgc"
    out_layout: str = "nhwgk"

    def __post_init__(self):
        # an unknown letter names the output-channel dimension (ConvGenerator.cpp:706-716): "nchw" for the output
        # tensor and "nchw" (GNCHW) for the filter are accepted spellings
        if "k" not in self.out_layout:
            self.out_layout = self.out_layout.replace("c", "k")
        if "k" not in self.fil_layout:
            self.fil_layout = self.fil_layout.replace("n", "k")
        self.fil_layout = add_group(self.fil_layout, "f")
        self.in_layout = add_group(self.in_layout, "c")
        self.out_layout = add_group(self.out_layout, "k")
        if self.pad_h_r is None:
            self.pad_h_r = self.pad_h
        if self.pad_w_r is None:
            self.pad_w_r = self.pad_w
        self.ho = out_dim(self.h, self.y, self.pad_h, self.pad_h_r, self.stride_h, self.dil_h)
        self.wo = out_dim(self.w, self.x, self.pad_w, self.pad_w_r, self.stride_w, self.dil_w)

    def numel(self, which: str) -> int:
        if which == "fil":
            return self.g * self.k * self.c * self.y * self.x
        if which == "in":
            return self.n * self.g * self.c * self.h * self.w
        return self.n * self.g * self.k * self.ho * self.wo

    def flops(self) -> float:
        # perfRunner.py:313-316: 2*n*c*k*ho*wo*y*x (per group, times groups)
        return 2.0 * self.n * self.g * self.c * self.k * self.ho * self.wo * self.y * self.x

    def to_c(self, dtype: torch.dtype, direction: int, f32_mode: int = 0) -> L.RbConvProblem:
        p = L.RbConvProblem(self.n, self.g, self.c, self.k, self.h, self.w, self.y, self.x, self.stride_h,
                            self.stride_w, self.dil_h, self.dil_w, self.pad_h, self.pad_w, self.pad_h_r, self.pad_w_r,
                            self.ho, self.wo, rb_dtype(dtype), direction, f32_mode)
        p.fil_layout = self.fil_layout.encode()
        p.in_layout = self.in_layout.encode()
        p.out_layout = self.out_layout.encode()
        return p


def workspace_size(cfg: ConvConfig, dtype: torch.dtype, direction: int, f32_mode: int = 0) -> int:
    p = cfg.to_c(dtype, direction, f32_mode)
    return int(L.lib().rbConvWorkspaceSize(C.byref(p)))


def conv(cfg: ConvConfig, direction: int, filter: torch.Tensor, input: torch.Tensor, output: torch.Tensor, *,
         workspace: Optional[torch.Tensor] = None, f32_mode: int = 0) -> torch.Tensor:
    """Runs the convolution; writes and returns the tensor the direction produces. All three tensors are flat
    (or any-shape contiguous) CUDA buffers in their layout order; the output of an i8 convolution is int32."""
    for t_, name in ((filter, "fil"), (input, "in"), (output, "out")):
        if not t_.is_cuda or not t_.is_contiguous():
            raise L.RbError(L.INVALID_PARAM, "tensors must be contiguous CUDA buffers (the library has no CPU path)")
        if t_.numel() != cfg.numel(name):
            raise L.RbError(L.INVALID_PARAM, f"{name} has {t_.numel()} elements, expected {cfg.numel(name)}")
    dtype = input.dtype
    p = cfg.to_c(dtype, direction, f32_mode)
    lib = L.lib()
    ws_bytes = int(lib.rbConvWorkspaceSize(C.byref(p)))
    if ws_bytes and (workspace is None or workspace.numel() * workspace.element_size() < ws_bytes):
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=input.device)
    stream = torch.cuda.current_stream(input.device).cuda_stream
    st = lib.rbConv(C.byref(p), filter.data_ptr(), input.data_ptr(), output.data_ptr(),
                    workspace.data_ptr() if workspace is not None else None,
                    workspace.numel() * workspace.element_size() if workspace is not None else 0, stream)
    L.check(st)
    return {FWD: output, BWD_DATA: input, BWD_WEIGHT: filter}[direction]


def conv_fused(cfg: ConvConfig, filter: torch.Tensor, input: torch.Tensor, output: torch.Tensor, epilogue,
               *, workspace: Optional[torch.Tensor] = None, f32_mode: int = 0) -> torch.Tensor:
    """Forward convolution with a fused elementwise tail (rbConvEpi): `epilogue` is a rocmlir_b200.gemm.Epilogue whose
    vectors are indexed by the output channel; the element type of `output` is the result type after the epilogue
    (e.g. int8 for a requantised i8 convolution)."""
    for t_, name in ((filter, "fil"), (input, "in"), (output, "out")):
        if not t_.is_cuda or not t_.is_contiguous():
            raise L.RbError(L.INVALID_PARAM, "tensors must be contiguous CUDA buffers (the library has no CPU path)")
        if t_.numel() != cfg.numel(name):
            raise L.RbError(L.INVALID_PARAM, f"{name} has {t_.numel()} elements, expected {cfg.numel(name)}")
    p = cfg.to_c(input.dtype, FWD, f32_mode)
    out_type = rb_dtype(output.dtype)
    lib = L.lib()
    ws_bytes = int(lib.rbConvEpiWorkspaceSize(C.byref(p), out_type))
    if ws_bytes and (workspace is None or workspace.numel() * workspace.element_size() < ws_bytes):
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=input.device)
    e = epilogue.to_c() if epilogue is not None else None
    stream = torch.cuda.current_stream(input.device).cuda_stream
    L.check(lib.rbConvEpi(C.byref(p), C.byref(e) if e is not None else None, out_type, filter.data_ptr(),
                          input.data_ptr(), output.data_ptr(),
                          workspace.data_ptr() if workspace is not None else None,
                          workspace.numel() * workspace.element_size() if workspace is not None else 0, stream))
    return output


# ---- three image dimensions ----------------------------------------------------------------------------------------
def _letters3(layout: str, kind: str) -> str:
    """Digit aliases 0 1 2 -> h w d (y x z for the filter), as ConvGenerator.cpp:622-627 translates them."""
    a, b, c = ("y", "x", "z") if kind == "f" else ("h", "w", "d")
    return layout.replace("0", a).replace("1", b).replace("2", c)


def _add_group3(layout: str, channel: str) -> str:
    if "g" in layout:
        return layout
    if channel == "f":
        return "g" + layout
    if layout[:2] == "n" + channel:
        return "ng" + channel + layout[2:]
    if layout[0] == "n" and layout[-1] == channel:
        return layout[:-1] + "g" + channel
    return "g" + layout


@dataclass
class Conv3dConfig:
    """rocmlir-gen's convolution flags with the depth ones (-in_d -fil_d -conv_stride_d -dilation_d -padding_d_l/_r,
    rocmlir-gen.cpp:171-260); layouts over g k c z y x / n g c d h w / n g k d h w or their digit spellings."""
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
    fil_layout: str = "gkzyxc"
    in_layout: str = "ndhwgc"
    out_layout: str = "ndhwgk"

    def __post_init__(self):
        self.fil_layout = _letters3(self.fil_layout, "f")
        self.in_layout = _letters3(self.in_layout, "c")
        self.out_layout = _letters3(self.out_layout, "k")
        if "k" not in self.out_layout:
            self.out_layout = self.out_layout.replace("c", "k")
        if "k" not in self.fil_layout:
            self.fil_layout = self.fil_layout.replace("n", "k")
        self.fil_layout = _add_group3(self.fil_layout, "f")
        self.in_layout = _add_group3(self.in_layout, "c")
        self.out_layout = _add_group3(self.out_layout, "k")
        for ax in "dhw":
            if getattr(self, f"pad_{ax}_r") is None:
                setattr(self, f"pad_{ax}_r", getattr(self, f"pad_{ax}"))
        self.dout = out_dim(self.d, self.z, self.pad_d, self.pad_d_r, self.stride_d, self.dil_d)
        self.ho = out_dim(self.h, self.y, self.pad_h, self.pad_h_r, self.stride_h, self.dil_h)
        self.wo = out_dim(self.w, self.x, self.pad_w, self.pad_w_r, self.stride_w, self.dil_w)

    def numel(self, which: str) -> int:
        if which == "fil":
            return self.g * self.k * self.c * self.z * self.y * self.x
        if which == "in":
            return self.n * self.g * self.c * self.d * self.h * self.w
        return self.n * self.g * self.k * self.dout * self.ho * self.wo

    def flops(self) -> float:
        return 2.0 * self.n * self.g * self.c * self.k * self.dout * self.ho * self.wo * self.z * self.y * self.x

    def to_c(self, dtype: torch.dtype, direction: int, f32_mode: int = 0) -> L.RbConv3dProblem:
        p = L.RbConv3dProblem(self.n, self.g, self.c, self.k, self.d, self.h, self.w, self.z, self.y, self.x,
                              self.stride_d, self.stride_h, self.stride_w, self.dil_d, self.dil_h, self.dil_w,
                              self.pad_d, self.pad_h, self.pad_w, self.pad_d_r, self.pad_h_r, self.pad_w_r,
                              self.dout, self.ho, self.wo, rb_dtype(dtype), direction, f32_mode)
        p.fil_layout = self.fil_layout.encode()
        p.in_layout = self.in_layout.encode()
        p.out_layout = self.out_layout.encode()
        return p


def conv3d(cfg: Conv3dConfig, direction: int, filter: torch.Tensor, input: torch.Tensor, output: torch.Tensor, *,
           workspace: Optional[torch.Tensor] = None, f32_mode: int = 0) -> torch.Tensor:
    """rbConv3d on flat contiguous CUDA buffers in layout order; returns the tensor the direction produces."""
    for t_, name in ((filter, "fil"), (input, "in"), (output, "out")):
        if not t_.is_cuda or not t_.is_contiguous():
            raise L.RbError(L.INVALID_PARAM, "tensors must be contiguous CUDA buffers (the library has no CPU path)")
        if t_.numel() != cfg.numel(name):
            raise L.RbError(L.INVALID_PARAM, f"{name} has {t_.numel()} elements, expected {cfg.numel(name)}")
    p = cfg.to_c(input.dtype, direction, f32_mode)
    lib = L.lib()
    ws_bytes = int(lib.rbConv3dWorkspaceSize(C.byref(p)))
    if ws_bytes and (workspace is None or workspace.numel() * workspace.element_size() < ws_bytes):
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=input.device)
    stream = torch.cuda.current_stream(input.device).cuda_stream
    st = lib.rbConv3d(C.byref(p), filter.data_ptr(), input.data_ptr(), output.data_ptr(),
                      workspace.data_ptr() if workspace is not None else None,
                      workspace.numel() * workspace.element_size() if workspace is not None else 0, stream)
    L.check(st)
    return {FWD: output, BWD_DATA: input, BWD_WEIGHT: filter}[direction]
