"""GPU parity tests of rbConv (forward, backward data, backward weight) against the CPU oracle and against
the reference's own known-answer tensors (tests/golden/cpu_conv2d.json)."""
import json
import os

import numpy as np
import pytest

import oracle
from helpers import from_device, normal_data, reference_random, to_device, uniform_f32

pytestmark = pytest.mark.gpu

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "cpu_conv2d.json")))["cases"]
DIRS = {"conv": 0, "conv_bwd_data": 1, "conv_bwd_weight": 2}
RESULT = {0: "out", 1: "in", 2: "fil"}
RMS = {oracle.F32: 3e-5, oracle.F16: 1e-3, oracle.BF16: 8e-3}


def make_cfgs(**kw):
    """(library config, oracle config) for the same convolution."""
    from rocmlir_b200.conv import ConvConfig
    cfg = ConvConfig(**kw)
    ocfg = oracle.Conv(n=cfg.n, c=cfg.c, k=cfg.k, h=cfg.h, w=cfg.w, y=cfg.y, x=cfg.x, g=cfg.g, stride_h=cfg.stride_h,
                       stride_w=cfg.stride_w, dil_h=cfg.dil_h, dil_w=cfg.dil_w, pad_h=cfg.pad_h, pad_w=cfg.pad_w,
                       pad_h_r=cfg.pad_h_r, pad_w_r=cfg.pad_w_r, fil_layout=cfg.fil_layout, in_layout=cfg.in_layout,
                       out_layout=cfg.out_layout)
    assert (ocfg.ho, ocfg.wo) == (cfg.ho, cfg.wo)
    return cfg, ocfg


def run_conv(cfg, direction, code, raws, f32_mode=0):
    """raws: dict fil/in/out -> raw storage arrays (flat). Returns raw result tensor."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.conv import conv
    out_code = oracle.I32 if code == oracle.I8 else code
    t = {k: to_device(v, out_code if (k == "out" and code == oracle.I8) else code) for k, v in raws.items()}
    res = conv(cfg, direction, t["fil"], t["in"], t["out"], f32_mode=f32_mode)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return from_device(res, out_code if direction == 0 else code)


@pytest.mark.parametrize("case", GOLD, ids=lambda c: f"{c['file'][:-5]}-{c['prefix']}-{c['dtype']}")
def test_reference_known_answer_tensors(cuda_device, case):
    cfg, ocfg = make_cfgs(n=case["n"], c=case["c"], k=case["k"], h=case["h"], w=case["w"], y=case["y"], x=case["x"],
                          stride_h=case["stride_h"], stride_w=case["stride_w"], dil_h=case["dil_h"], dil_w=case["dil_w"],
                          pad_h=case["pad_h"], pad_w=case["pad_w"], fil_layout=case["fil_layout"],
                          in_layout=case["in_layout"], out_layout=case["out_layout"])
    d = DIRS[case["operation"]]
    code = oracle.I8 if case["dtype"] == "i8" else oracle.F32
    ones = {k: np.ones(ocfg.numel(k), np.float32) for k in ("fil", "in", "out")}
    raws = {k: oracle.from_f32(v, code) for k, v in ones.items()}
    if code == oracle.I8:
        raws["out"] = np.ones(ocfg.numel("out"), np.int32)
    got = run_conv(cfg, d, code, raws).astype(np.float64)
    np.testing.assert_array_equal(got.ravel(), np.asarray(case["expected"], np.float64))


# ResNet-50-shaped layers in miniature and the padding/odd-channel cases the reference's regression suites stress
# (mlir/test/e2e/PrResnet50.toml, conv_regression_fwd.toml, PaddedGemmConfig.toml): C = 3 / 7 / 13, 7x7 s2 p3 stem.
SHAPES = [
    dict(n=2, c=64, k=64, h=14, w=14, y=3, x=3, pad_h=1, pad_w=1),
    dict(n=2, c=256, k=64, h=14, w=14, y=1, x=1),
    dict(n=2, c=128, k=128, h=14, w=14, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1),
    dict(n=3, c=3, k=16, h=15, w=17, y=7, x=7, stride_h=2, stride_w=2, pad_h=3, pad_w=3),
    dict(n=1, c=13, k=7, h=9, w=9, y=3, x=3, dil_h=2, dil_w=2, pad_h=2, pad_w=2),
    dict(n=2, c=8, k=8, g=2, h=8, w=8, y=3, x=3, pad_h=1, pad_w=1),
]
LAYOUTS = {"nhwc": dict(fil_layout="kyxc", in_layout="nhwc", out_layout="nhwk"),
           "nchw": dict(fil_layout="kcyx", in_layout="nchw", out_layout="nkhw")}


@pytest.mark.parametrize("direction", [0, 1, 2])
@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
@pytest.mark.parametrize("code", [oracle.F16, oracle.F32, oracle.BF16])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(str(v) for v in s.values()))
def test_conv_exact_on_reference_integer_data(cuda_device, shape, code, layout, direction):
    cfg, ocfg = make_cfgs(**shape, **LAYOUTS[layout])
    # `-rand 1`: filter, input, output filled in kernel-argument order (rocmlir-gen.cpp:3193-3218)
    (ff, fraw), (inf, iraw), (of, oraw) = reference_random([(ocfg.numel("fil"),), (ocfg.numel("in"),),
                                                           (ocfg.numel("out"),)], code, seed=1)
    ref = oracle.conv_f32(ocfg, direction, ff, inf, of, threads=oracle.max_threads())
    ref_raw = oracle.from_f32(ref, code)
    got = run_conv(cfg, direction, code, {"fil": fraw, "in": iraw, "out": oraw})
    np.testing.assert_array_equal(got.ravel(), ref_raw.ravel())


# Shapes of the halo kernel with a streamed filter: 16-bit layers whose filter does not fit into shared memory beside the
# windows (forward and unit-stride backward data, up to 128 output channels), and f32 forward with reductions of up to
# 1024 elements (two TF32 planes of window and filter, NHWK or NKHW stored by the kernel): ragged last tiles, one and
# two sub-tiles per stage, dilation, asymmetric extents, images lower than a tile.
STREAMED = [
    (dict(n=3, c=128, k=128, h=13, w=11, y=3, x=3, pad_h=1, pad_w=1), (oracle.F16, oracle.BF16)),
    (dict(n=2, c=192, k=96, h=9, w=20, y=3, x=3, pad_h=1, pad_w=1), (oracle.F16,)),
    (dict(n=2, c=256, k=64, h=30, w=30, y=3, x=3, dil_h=2, dil_w=2, pad_h=2, pad_w=2), (oracle.BF16,)),
    (dict(n=2, c=64, k=64, h=12, w=12, y=3, x=3, pad_h=1, pad_w=1), (oracle.F32,)),
    (dict(n=1, c=32, k=96, h=10, w=17, y=3, x=3, dil_h=2, dil_w=2, pad_h=2, pad_w=2), (oracle.F32,)),
    (dict(n=5, c=96, k=32, h=3, w=40, y=3, x=3, pad_h=1, pad_w=1), (oracle.F32,)),
    (dict(n=2, c=32, k=128, h=20, w=9, y=5, x=5, pad_h=2, pad_w=2), (oracle.F32,)),
]


@pytest.mark.parametrize("direction", [0, 1])
@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
@pytest.mark.parametrize("case", STREAMED, ids=lambda c: "x".join(str(v) for v in c[0].values()))
def test_streamed_filter_halo_kernel_exact(cuda_device, case, layout, direction):
    """Bit for bit against the oracle on `-rand 1` integer data, and bit for bit against the im2col form of the same
    library (variant bit 26) - the two differ in kernel, tile order and, for f32, in how the three TF32 products are
    summed, none of which may show on data whose sums are exact."""
    from rocmlir_b200 import _lib as L
    shape, codes = case
    for code in codes:
        if layout == "nchw" and code != oracle.F32:
            continue   # channel-major 16-bit tensors take the gather path: not this kernel
        cfg, ocfg = make_cfgs(**shape, **LAYOUTS[layout])
        (ff, fraw), (inf, iraw), (of, oraw) = reference_random([(ocfg.numel("fil"),), (ocfg.numel("in"),),
                                                               (ocfg.numel("out"),)], code, seed=3)
        ref_raw = oracle.from_f32(oracle.conv_f32(ocfg, direction, ff, inf, of, threads=oracle.max_threads()), code)
        n0 = L.launch_count()
        got = run_conv(cfg, direction, code, {"fil": fraw, "in": iraw, "out": oraw})
        np.testing.assert_array_equal(got.ravel(), ref_raw.ravel())
        if code == oracle.F32 and direction == 0:   # image planes, filter planes, kernel: what rbConvKernelCount reports
            import ctypes
            import torch
            assert L.launch_count() - n0 == 3 == L.lib().rbConvKernelCount(ctypes.byref(cfg.to_c(torch.float32, 0, 0)))
        L.lib().rbSetGemmVariant(1 << 26)
        try:
            other = run_conv(cfg, direction, code, {"fil": fraw, "in": iraw, "out": oraw})
        finally:
            L.lib().rbSetGemmVariant(0)
        np.testing.assert_array_equal(got.ravel(), other.ravel())


# Backward data with a stride runs as one unit-stride problem per class of input pixels (h mod stride, w mod stride):
# classes without any tap (1x1 filter, stride 2), more classes than taps (stride 3 under a 2x2 filter), different
# strides per axis, odd extents, groups, a padding larger than the stride.
STRIDED = [
    dict(n=2, c=64, k=128, h=14, w=14, y=1, x=1, stride_h=2, stride_w=2),
    dict(n=2, c=64, k=64, h=15, w=13, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1),
    dict(n=1, c=64, k=64, h=17, w=16, y=2, x=2, stride_h=3, stride_w=3),
    dict(n=2, c=8, k=16, h=12, w=11, y=3, x=5, stride_h=2, stride_w=3, pad_h=1, pad_w=2),
    dict(n=2, c=8, k=8, g=2, h=9, w=9, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1),
    dict(n=1, c=64, k=64, h=12, w=12, y=7, x=7, stride_h=2, stride_w=2, pad_h=3, pad_w=3),
    dict(n=1, c=16, k=16, h=10, w=10, y=3, x=3, stride_h=4, stride_w=4, pad_h=1, pad_w=1),
]


@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
@pytest.mark.parametrize("code", [oracle.F16, oracle.F32, oracle.BF16])
@pytest.mark.parametrize("shape", STRIDED, ids=lambda s: "x".join(str(v) for v in s.values()))
def test_strided_backward_data_exact(cuda_device, shape, code, layout):
    cfg, ocfg = make_cfgs(**shape, **LAYOUTS[layout])
    (ff, fraw), (inf, iraw), (of, oraw) = reference_random([(ocfg.numel("fil"),), (ocfg.numel("in"),),
                                                           (ocfg.numel("out"),)], code, seed=1)
    ref_raw = oracle.from_f32(oracle.conv_f32(ocfg, 1, ff, inf, of, threads=oracle.max_threads()), code)
    got = run_conv(cfg, 1, code, {"fil": fraw, "in": iraw, "out": oraw})
    np.testing.assert_array_equal(got.ravel(), ref_raw.ravel())


@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
def test_int8_forward_bit_exact(cuda_device, layout):
    """i8 forward -> i32. The reference's CPU loop multiplies in i8 before widening (rocmlir-gen.cpp:1955-1960);
    with -rand 1 data (values in [-5,4]) no product exceeds 127, so both readings agree and parity is exact."""
    cfg, ocfg = make_cfgs(n=2, c=32, k=48, h=12, w=12, y=3, x=3, pad_h=1, pad_w=1, **LAYOUTS[layout])
    (ff, fraw), (inf, iraw) = reference_random([(ocfg.numel("fil"),), (ocfg.numel("in"),)], oracle.I8, seed=1)
    ref = oracle.conv_i8(ocfg, fraw, iraw, wrap_product=True, threads=oracle.max_threads())
    assert np.array_equal(ref, oracle.conv_i8(ocfg, fraw, iraw, wrap_product=False))
    got = run_conv(cfg, 0, oracle.I8, {"fil": fraw, "in": iraw, "out": np.zeros(ocfg.numel("out"), np.int32)})
    assert oracle.verify_int(got, ref)[0] == [1, 1, 1]


@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
@pytest.mark.parametrize("code", [oracle.F8E4M3, oracle.F8E5M2])
def test_fp8_forward_exact_on_reference_integer_data(cuda_device, code, layout):
    """-t fp8 / bf8 forward -> f32 (rocmlir-gen.cpp:430-455). -rand 1 values are small integers, exact in both 8-bit
    formats, so the f32 result must match the oracle bit for bit (NHWC C=128 takes the implicit-GEMM path)."""
    cfg, ocfg = make_cfgs(n=2, c=128, k=48, h=12, w=12, y=3, x=3, pad_h=1, pad_w=1, **LAYOUTS[layout])
    (ff, fraw), (inf, iraw) = reference_random([(ocfg.numel("fil"),), (ocfg.numel("in"),)], code, seed=1)
    ref = oracle.conv_f32(ocfg, 0, ff, inf, None, threads=oracle.max_threads())
    import torch
    from rocmlir_b200.conv import conv
    t = {"fil": to_device(fraw, code), "in": to_device(iraw, code),
         "out": torch.zeros(ocfg.numel("out"), dtype=torch.float32, device="cuda")}
    got = conv(cfg, 0, t["fil"], t["in"], t["out"]).cpu().numpy()
    np.testing.assert_array_equal(got.ravel(), ref.ravel())


def test_fp32_nchw_forward_headline_config(cuda_device):
    """BASELINE config 1: fp32 NCHW/KCYX, N=16 C=64 56x56 K=64 3x3 s1 p1, input and filter uniform[-1,1) from a seed;
    judged by the reference verifier with its default RMS threshold 3e-5 (relDiff disabled: summation order)."""
    cfg, ocfg = make_cfgs(n=16, c=64, k=64, h=56, w=56, y=3, x=3, pad_h=1, pad_w=1, **LAYOUTS["nchw"])
    fil = uniform_f32((ocfg.numel("fil"),), seed=1, lo=-1.0, hi=1.0)
    inp = uniform_f32((ocfg.numel("in"),), seed=2, lo=-1.0, hi=1.0)
    ref = oracle.conv_f32(ocfg, 0, fil, inp, None, threads=oracle.max_threads())
    got = run_conv(cfg, 0, oracle.F32, {"fil": fil, "in": inp, "out": np.zeros(ocfg.numel("out"), np.float32)})
    verdict, info = oracle.verify_float(got, ref, RMS[oracle.F32], 100.0, 100.0)
    assert verdict == [1, 1, 1], info


RESNET = [dict(c=64, k=64, h=56, w=56, y=3, x=3, pad_h=1, pad_w=1),
          dict(c=256, k=64, h=56, w=56, y=1, x=1),
          dict(c=128, k=128, h=28, w=28, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1),
          dict(c=512, k=2048, h=7, w=7, y=1, x=1)]


@pytest.mark.parametrize("direction", [0, 1, 2])
@pytest.mark.parametrize("shape", RESNET, ids=lambda s: f"c{s['c']}k{s['k']}h{s['h']}y{s['y']}")
def test_fp16_nhwc_resnet_shapes_reduced_batch(cuda_device, shape, direction):
    """BASELINE config 4 shapes (fp16 NHWC, tensors ~ 0.05 * N(0,1)) at batch 4 instead of 256 so that the
    sequential oracle finishes in seconds; reference verifier, RMS 1e-3 (PrResnet50.toml:3)."""
    cfg, ocfg = make_cfgs(n=4, **shape, **LAYOUTS["nhwc"])
    ff, fraw = normal_data((ocfg.numel("fil"),), oracle.F16, seed=1, scale=0.05)
    inf, iraw = normal_data((ocfg.numel("in"),), oracle.F16, seed=2, scale=0.05)
    of, oraw = normal_data((ocfg.numel("out"),), oracle.F16, seed=3, scale=0.05)
    ref = oracle.round_to(oracle.conv_f32(ocfg, direction, ff, inf, of, threads=oracle.max_threads()), oracle.F16)
    got = oracle.to_f32(run_conv(cfg, direction, oracle.F16, {"fil": fraw, "in": iraw, "out": oraw}), oracle.F16)
    verdict, info = oracle.verify_float(got, ref, RMS[oracle.F16], 100.0, 100.0)
    assert verdict == [1, 1, 1], info


def test_fp16_nhwc_full_batch_forward_sampled_images(cuda_device):
    """Full BASELINE size N=256 (C=64 -> K=64, 56x56, 3x3): images are independent, so the oracle is evaluated on
    two seeded images of the batch and compared with the same images of the full-batch result."""
    shape = RESNET[0]
    cfg, ocfg = make_cfgs(n=256, **shape, **LAYOUTS["nhwc"])
    ff, fraw = normal_data((ocfg.numel("fil"),), oracle.F16, seed=1, scale=0.05)
    inf, iraw = normal_data((ocfg.numel("in"),), oracle.F16, seed=2, scale=0.05)
    got = oracle.to_f32(run_conv(cfg, 0, oracle.F16, {"fil": fraw, "in": iraw,
                                                       "out": np.zeros(ocfg.numel("out"), np.uint16)}), oracle.F16)
    got = got.reshape(256, -1)
    _, ocfg1 = make_cfgs(n=1, **shape, **LAYOUTS["nhwc"])
    per_img = inf.size // 256
    for img in (0, 171):
        ref = oracle.round_to(oracle.conv_f32(ocfg1, 0, ff, inf[img * per_img:(img + 1) * per_img], None,
                                              threads=oracle.max_threads()), oracle.F16)
        verdict, info = oracle.verify_float(got[img], ref, RMS[oracle.F16], 100.0, 100.0)
        assert verdict == [1, 1, 1], (img, info)
