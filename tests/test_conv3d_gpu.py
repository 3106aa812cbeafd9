"""GPU parity tests of rbConv3d (three image dimensions) against the CPU oracle: -rand 1 integer data must match
bit for bit in every direction, element type and layout; float data goes through the reference verifier."""
import numpy as np
import pytest

import oracle
from helpers import from_device, normal_data, reference_random, to_device

pytestmark = pytest.mark.gpu

RMS = {oracle.F32: 3e-5, oracle.F16: 1e-3, oracle.BF16: 8e-3}
SHAPES = [
    dict(n=2, c=16, k=24, d=5, h=6, w=7, z=3, y=3, x=3, pad_d=1, pad_h=1, pad_w=1),
    dict(n=1, c=64, k=32, d=6, h=8, w=8, z=2, y=3, x=3, stride_d=2, stride_h=1, stride_w=2, pad_d=1, pad_h=1, pad_w=1),
    dict(n=2, c=6, k=4, g=2, d=7, h=5, w=4, z=3, y=1, x=2, dil_d=2, pad_d=2, pad_d_r=1),
    dict(n=3, c=5, k=7, d=1, h=9, w=8, z=1, y=3, x=3, pad_h=1, pad_w=1),          # unit depth: the 2-D pass-through
]
LAYOUTS = {"channels_last": dict(fil_layout="kzyxc", in_layout="ndhwc", out_layout="ndhwk"),
           "channels_first": dict(fil_layout="kczyx", in_layout="ncdhw", out_layout="nkdhw"),
           "digits": dict(fil_layout="kc012", in_layout="nc012", out_layout="nk012")}


def make_cfgs(**kw):
    from rocmlir_b200.conv import Conv3dConfig
    cfg = Conv3dConfig(**kw)
    ocfg = oracle.Conv3d(n=cfg.n, c=cfg.c, k=cfg.k, d=cfg.d, h=cfg.h, w=cfg.w, z=cfg.z, y=cfg.y, x=cfg.x, g=cfg.g,
                         stride_d=cfg.stride_d, stride_h=cfg.stride_h, stride_w=cfg.stride_w, dil_d=cfg.dil_d,
                         dil_h=cfg.dil_h, dil_w=cfg.dil_w, pad_d=cfg.pad_d, pad_h=cfg.pad_h, pad_w=cfg.pad_w,
                         pad_d_r=cfg.pad_d_r, pad_h_r=cfg.pad_h_r, pad_w_r=cfg.pad_w_r, fil_layout=cfg.fil_layout,
                         in_layout=cfg.in_layout, out_layout=cfg.out_layout)
    assert (ocfg.dout, ocfg.ho, ocfg.wo) == (cfg.dout, cfg.ho, cfg.wo)
    return cfg, ocfg


def run_conv3d(cfg, direction, code, raws, f32_mode=0):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.conv import conv3d
    out_code = oracle.I32 if code == oracle.I8 else code
    t = {k: to_device(v, out_code if (k == "out" and code == oracle.I8) else code) for k, v in raws.items()}
    res = conv3d(cfg, direction, t["fil"], t["in"], t["out"], f32_mode=f32_mode)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return from_device(res, out_code if direction == 0 else code)


@pytest.mark.parametrize("direction", [0, 1, 2])
@pytest.mark.parametrize("layout", list(LAYOUTS))
@pytest.mark.parametrize("code", [oracle.F16, oracle.F32, oracle.BF16])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(str(v) for v in s.values()))
def test_conv3d_exact_on_reference_integer_data(cuda_device, shape, code, layout, direction):
    cfg, ocfg = make_cfgs(**shape, **LAYOUTS[layout])
    (ff, fraw), (inf, iraw), (of, oraw) = reference_random([(ocfg.numel("fil"),), (ocfg.numel("in"),),
                                                           (ocfg.numel("out"),)], code, seed=1)
    ref = oracle.conv3d_f32(ocfg, direction, ff, inf, of, threads=oracle.max_threads())
    ref_raw = oracle.from_f32(ref, code)
    got = run_conv3d(cfg, direction, code, {"fil": fraw, "in": iraw, "out": oraw})
    np.testing.assert_array_equal(got.ravel(), ref_raw.ravel())


@pytest.mark.parametrize("layout", ["channels_last", "channels_first"])
def test_conv3d_int8_forward_bit_exact(cuda_device, layout):
    cfg, ocfg = make_cfgs(n=2, c=32, k=24, d=4, h=6, w=6, z=3, y=3, x=3, pad_d=1, pad_h=1, pad_w=1, **LAYOUTS[layout])
    (ff, fraw), (inf, iraw) = reference_random([(ocfg.numel("fil"),), (ocfg.numel("in"),)], oracle.I8, seed=1)
    ref = oracle.conv3d_i8(ocfg, fraw, iraw, threads=oracle.max_threads())
    got = run_conv3d(cfg, 0, oracle.I8, {"fil": fraw, "in": iraw, "out": np.zeros(ocfg.numel("out"), np.int32)})
    assert oracle.verify_int(got, ref)[0] == [1, 1, 1]


@pytest.mark.parametrize("direction", [0, 1, 2])
@pytest.mark.parametrize("code", [oracle.F16, oracle.F32])
def test_conv3d_float_data_reference_verifier(cuda_device, code, direction):
    """Video-model-like layer in miniature (C=64 -> K=64, 3x3x3, pad 1) on 0.05 * N(0,1) data, judged like the
    reference judges its float runs: RMS threshold of the element type, relDiff off (summation order)."""
    cfg, ocfg = make_cfgs(n=2, c=64, k=64, d=6, h=14, w=14, z=3, y=3, x=3, pad_d=1, pad_h=1, pad_w=1,
                          **LAYOUTS["channels_last"])
    ff, fraw = normal_data((ocfg.numel("fil"),), code, seed=1, scale=0.05)
    inf, iraw = normal_data((ocfg.numel("in"),), code, seed=2, scale=0.05)
    of, oraw = normal_data((ocfg.numel("out"),), code, seed=3, scale=0.05)
    ref = oracle.round_to(oracle.conv3d_f32(ocfg, direction, ff, inf, of, threads=oracle.max_threads()), code)
    got = oracle.to_f32(run_conv3d(cfg, direction, code, {"fil": fraw, "in": iraw, "out": oraw}), code)
    verdict, info = oracle.verify_float(got, ref, RMS[code], 100.0, 100.0)
    assert verdict == [1, 1, 1], info


def test_conv3d_rejects_bad_problems(cuda_device):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.conv import Conv3dConfig, conv3d
    cfg = Conv3dConfig(n=1, c=4, k=4, d=2, h=4, w=4, z=3, y=1, x=1)      # filter depth does not fit: dout <= 0
    t = torch.zeros(max(1, cfg.numel("in")), dtype=torch.float16, device="cuda")
    with pytest.raises(L.RbError):
        conv3d(cfg, 0, torch.zeros(cfg.numel("fil"), dtype=torch.float16, device="cuda"), t,
               torch.zeros(max(1, abs(cfg.numel("out"))), dtype=torch.float16, device="cuda"))
    cfg = Conv3dConfig(n=1, c=4, k=4, d=3, h=4, w=4, z=3, y=1, x=1)
    i8 = torch.zeros(cfg.numel("in"), dtype=torch.int8, device="cuda")
    with pytest.raises(L.RbError):                                          # i8 exists forward only
        conv3d(cfg, 1, torch.zeros(cfg.numel("fil"), dtype=torch.int8, device="cuda"), i8,
               torch.zeros(cfg.numel("out"), dtype=torch.int8, device="cuda"))
