"""Pins the oracle's three-dimensional convolution (oracle.conv3d_*), which restates the same generated loop nest
as the 2-D one with a third image dimension (rocmlir-gen.cpp:1745-1830):
  * with all depths 1 it must equal the 2-D oracle, which is pinned against the reference's known-answer tensors;
  * against torch's conv3d and its autograd (float64), an independent implementation, for depth > 1;
  * accumulation order: with -rand 1 integer data every partial sum is exact, so any order gives the same bits."""
import numpy as np
import pytest
import torch

import oracle
from helpers import reference_random

CASES = [
    dict(n=2, c=3, k=4, d=5, h=6, w=7, z=3, y=3, x=3, pad_d=1, pad_h=1, pad_w=1),
    dict(n=1, c=4, k=2, d=6, h=5, w=5, z=2, y=3, x=1, stride_d=2, stride_h=1, stride_w=2, pad_d=1, pad_h=0, pad_w=1),
    dict(n=2, c=2, k=4, g=2, d=7, h=4, w=4, z=3, y=1, x=1, dil_d=2, pad_d=2),
]


def torch_ref(p: oracle.Conv3d, direction, fil, inp, out):
    """float64 conv3d on canonical (n, g*c, d, h, w) tensors; inputs are flat arrays in the default layouts."""
    f = torch.tensor(fil.reshape(p.g, p.k, p.c, p.z, p.y, p.x), dtype=torch.float64)
    i = torch.tensor(inp.reshape(p.n, p.g, p.c, p.d, p.h, p.w), dtype=torch.float64)
    o = torch.tensor(out.reshape(p.n, p.g, p.k, p.dout, p.ho, p.wo), dtype=torch.float64)
    f5 = f.reshape(p.g * p.k, p.c, p.z, p.y, p.x).requires_grad_(True)
    i5 = i.reshape(p.n, p.g * p.c, p.d, p.h, p.w).requires_grad_(True)
    assert (p.pad_d, p.pad_h, p.pad_w) == (p.pad_d_r, p.pad_h_r, p.pad_w_r)
    y = torch.nn.functional.conv3d(i5, f5, stride=(p.stride_d, p.stride_h, p.stride_w),
                                   padding=(p.pad_d, p.pad_h, p.pad_w), dilation=(p.dil_d, p.dil_h, p.dil_w),
                                   groups=p.g)
    if direction == 0:
        return y.detach().numpy().ravel()
    y.backward(o.reshape(p.n, p.g * p.k, p.dout, p.ho, p.wo))
    return (i5.grad if direction == 1 else f5.grad).numpy().ravel()


@pytest.mark.parametrize("direction", [0, 1, 2])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(str(v) for v in c.values()))
def test_conv3d_oracle_matches_torch_float64(case, direction):
    p = oracle.Conv3d(**case)
    (ff, _), (inf, _), (of, _) = reference_random([(p.numel("fil"),), (p.numel("in"),), (p.numel("out"),)],
                                                  oracle.F32, seed=1)
    got = oracle.conv3d_f32(p, direction, ff, inf, of)
    ref = torch_ref(p, direction, ff, inf, of)
    np.testing.assert_array_equal(got.astype(np.float64), ref)     # integer data: exact in both


@pytest.mark.parametrize("direction", [0, 1, 2])
def test_conv3d_oracle_with_unit_depth_is_the_2d_oracle(direction):
    kw = dict(n=2, c=5, k=3, h=9, w=8, y=3, x=3, stride_h=2, pad_h=1, pad_w=1)
    p3 = oracle.Conv3d(d=1, z=1, fil_layout="gkcyxz", in_layout="ngchwd", out_layout="ngkhwd", **kw)
    p2 = oracle.Conv(fil_layout="gkcyx", in_layout="ngchw", out_layout="ngkhw", **kw)
    rng = np.random.default_rng(3)
    fil, inp, out = (rng.standard_normal(p2.numel(w)).astype(np.float32) for w in ("fil", "in", "out"))
    np.testing.assert_array_equal(oracle.conv3d_f32(p3, direction, fil, inp, out),
                                  oracle.conv_f32(p2, direction, fil, inp, out))


def test_conv3d_oracle_layout_permutation_and_i8():
    base = oracle.Conv3d(n=2, c=4, k=3, d=4, h=5, w=5, z=2, y=3, x=3, pad_h=1, pad_w=1)
    perm = oracle.Conv3d(n=2, c=4, k=3, d=4, h=5, w=5, z=2, y=3, x=3, pad_h=1, pad_w=1, fil_layout="gkzyxc",
                         in_layout="ndhwgc", out_layout="ndhwgk")
    (ff, fraw), (inf, iraw) = reference_random([(base.numel("fil"),), (base.numel("in"),)], oracle.I8, seed=1)
    f6 = ff.reshape(base.shape("fil"))
    i6 = inf.reshape(base.shape("in"))
    # same tensors stored channel-last
    fp = np.ascontiguousarray(np.transpose(f6, [0, 1, 3, 4, 5, 2])).ravel()
    ip = np.ascontiguousarray(np.transpose(i6, [0, 3, 4, 5, 1, 2])).ravel()
    a = oracle.conv3d_f32(base, 0, ff, inf, None).reshape(base.shape("out"))
    b = oracle.conv3d_f32(perm, 0, fp, ip, None).reshape(perm.shape("out"))
    np.testing.assert_array_equal(np.transpose(a, [0, 3, 4, 5, 1, 2]), b)
    i8 = oracle.conv3d_i8(base, fraw, iraw)
    np.testing.assert_array_equal(i8.astype(np.float64), a.ravel().astype(np.float64))
