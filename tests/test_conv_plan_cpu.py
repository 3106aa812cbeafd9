"""Host-side planning of the convolution entry points (no GPU needed: workspace sizes and kernel counts only)."""
import ctypes as C

import torch

from rocmlir_b200 import _lib as L
from rocmlir_b200.conv import Conv3dConfig, ConvConfig


def ws2(cfg, direction, dtype=torch.float16):
    p = cfg.to_c(dtype, direction)
    return int(L.lib().rbConvWorkspaceSize(C.byref(p)))


def ws3(cfg, direction, dtype=torch.float16):
    p = cfg.to_c(dtype, direction)
    return int(L.lib().rbConv3dWorkspaceSize(C.byref(p)))


def kernels2(cfg, direction, dtype=torch.float16):
    p = cfg.to_c(dtype, direction)
    return int(L.lib().rbConvKernelCount(C.byref(p)))


def test_unit_depth_is_the_2d_problem():
    kw = dict(n=4, c=64, k=64, h=14, w=14, y=3, x=3, pad_h=1, pad_w=1)
    c2 = ConvConfig(fil_layout="kyxc", in_layout="nhwc", out_layout="nhwk", **kw)
    c3 = Conv3dConfig(d=1, z=1, fil_layout="kzyxc", in_layout="ndhwc", out_layout="ndhwk", **kw)
    for direction in (0, 1, 2):
        assert ws3(c3, direction) == ws2(c2, direction)
    # the digit spelling of the reference's regression suites names the same tensors
    c3d = Conv3dConfig(d=1, z=1, fil_layout="k012c", in_layout="n012c", out_layout="n012k", **kw)
    assert (c3d.fil_layout, c3d.in_layout, c3d.out_layout) == ("gkyxzc", "nhwdgc", "nhwdgk")
    assert ws3(c3d, 0) == ws2(c2, 0)


def test_folded_depth_needs_the_gathered_input():
    c3 = Conv3dConfig(n=2, c=16, k=32, d=6, h=8, w=8, z=3, y=3, x=3, pad_d=1, pad_h=1, pad_w=1)
    es = 2
    in2 = c3.n * c3.dout * c3.h * c3.w * c3.z * c3.c * es          # Z copies of every output depth slice
    fil2 = c3.k * c3.y * c3.x * c3.z * c3.c * es
    out2 = c3.n * c3.dout * c3.ho * c3.wo * c3.k * es
    assert ws3(c3, 0) >= in2 + fil2 + out2
    assert ws3(c3, 1) >= 2 * in2 + fil2 + out2                      # backward data keeps the folded gradient in f32
    # sizes that do not follow the output-size rule, or a filter deeper than the padded image, are refused (0)
    bad = c3.to_c(torch.float16, 0)
    bad.dout += 1
    assert L.lib().rbConv3dWorkspaceSize(C.byref(bad)) == 0
    deep = Conv3dConfig(n=1, c=8, k=8, d=2, h=4, w=4, z=5, y=1, x=1)
    assert deep.dout <= 0 and ws3(deep, 0) == 0
    # 8-bit types run forward only (ConvGenerator.cpp:631-638)
    assert ws3(c3, 0, torch.int8) > 0 and ws3(c3, 1, torch.int8) == 0


def test_strided_backward_data_runs_by_pixel_classes():
    # ResNet 3x3 stride-2 layer, NHWC f16: ONE launch of the halo kernel for the four classes, the mirrored taps read
    # straight from the KYXC filter (no filter pass)
    c = ConvConfig(n=8, c=128, k=128, h=28, w=28, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1,
                   fil_layout="kyxc", in_layout="nhwc", out_layout="nhwk")
    assert kernels2(c, 1) == 1
    # the same layer in f32 keeps the class GEMMs and the interleaving pass (the halo kernel is 16-bit)
    assert kernels2(c, 1, torch.float32) > 2
    # 1x1 stride 2: three of the four classes receive no tap: zero fill, one launch
    p1 = ConvConfig(n=8, c=64, k=128, h=28, w=28, y=1, x=1, stride_h=2, stride_w=2, fil_layout="kyxc",
                    in_layout="nhwc", out_layout="nhwk")
    assert kernels2(p1, 1) == 2
    # a 3 x 3 stride has nine classes: three launches of up to four
    s3 = ConvConfig(n=4, c=64, k=64, h=27, w=27, y=3, x=3, stride_h=3, stride_w=3, fil_layout="kyxc",
                    in_layout="nhwc", out_layout="nhwk")
    assert kernels2(s3, 1) == 3
    # a filter that is not channels-last (KCYX) needs the mirrored sub-filter pass
    kc = ConvConfig(n=8, c=128, k=128, h=28, w=28, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1,
                    fil_layout="kcyx", in_layout="nhwc", out_layout="nhwk")
    assert kernels2(kc, 1) == 2
    # unit stride: one launch of the halo kernel (mirrored taps read from the filter in place) when the filter fits into
    # shared memory; a 3x3 filter over 128 x 128 channels does not (288 KB) and keeps the implicit GEMM + filter pass
    u = ConvConfig(n=8, c=64, k=64, h=28, w=28, y=3, x=3, pad_h=1, pad_w=1, fil_layout="kyxc", in_layout="nhwc",
                   out_layout="nhwk")
    assert kernels2(u, 1) == 1 and kernels2(u, 0) == 1
    big = ConvConfig(n=8, c=128, k=128, h=28, w=28, y=3, x=3, pad_h=1, pad_w=1, fil_layout="kyxc", in_layout="nhwc",
                     out_layout="nhwk")
    assert kernels2(big, 1) == 2
    # unit-stride backward weight: the halo weight-gradient kernel and the sum of its slabs
    assert kernels2(u, 2) == 2
