"""GPU parity of the fused elementwise tails against op-by-op oracle restatements of the reference's own fusion tests:

  convolution + broadcast add + clip          mlir/test/fusion/pr-e2e/mixr-conv-bias-clipped-relu.mlir:5-13
  quant_convolution -> dequantizelinear -> add -> relu -> quantizelinear (with zero points)
                                              mlir/test/fusion/pr-e2e/tosa-to-rock-quantization.e2e.mlir:5-18
  dot + same-shape add                        mlir/test/fusion/pr-e2e/mixr-gemm/mixr-gemm-add.e2e.mlir
  dot + add broadcast along M / scalar add    MIGraphXToTosa.cpp:393-424 (multibroadcast strides 0)
  C += A.B (--store-method=atomic_add)        mlir/test/e2e/gemm_with_atomic_add.toml:6-9

Bars: exact on the reference's integer-valued `-rand 1` data and for every integer result; the reference verifier
with its default thresholds on `-rand 1 -rand_type float` data.
"""
import numpy as np
import pytest

import oracle
from helpers import from_device, normal_data, reference_random, to_device, torch_dtype, uniform_f32, uniform_int8

pytestmark = pytest.mark.gpu

NHWC = dict(fil_layout="kyxc", in_layout="nhwc", out_layout="nhwk")
NCHW = dict(fil_layout="kcyx", in_layout="nchw", out_layout="nkhw")


def _cfgs(**kw):
    from rocmlir_b200.conv import ConvConfig
    cfg = ConvConfig(**kw)
    ocfg = oracle.Conv(n=cfg.n, c=cfg.c, k=cfg.k, h=cfg.h, w=cfg.w, y=cfg.y, x=cfg.x, g=cfg.g, stride_h=cfg.stride_h,
                       stride_w=cfg.stride_w, dil_h=cfg.dil_h, dil_w=cfg.dil_w, pad_h=cfg.pad_h, pad_w=cfg.pad_w,
                       fil_layout=cfg.fil_layout, in_layout=cfg.in_layout, out_layout="nhwgk")
    return cfg, ocfg


def _to_layout(ref_nhwk, cfg):
    """Oracle results are computed in [n][h][w][k] order (the epilogue indexes the channel last); the library writes the
    tensor's own layout."""
    x = ref_nhwk.reshape(cfg.n, cfg.ho, cfg.wo, cfg.k)
    return x if cfg.out_layout == "nhwgk" else np.ascontiguousarray(x.transpose(0, 3, 1, 2))


@pytest.mark.parametrize("layout", [NHWC, NCHW], ids=["nhwc", "nchw"])
@pytest.mark.parametrize("code", [oracle.F32, oracle.F16])
@pytest.mark.parametrize("shape", [dict(n=4, c=3, k=4, h=3, w=3, y=3, x=3),                       # the reference's test
                                   dict(n=2, c=64, k=96, h=14, w=14, y=3, x=3, pad_h=1, pad_w=1)],  # implicit-GEMM path
                         ids=["mixr_4x3x3x3", "c64k96"])
def test_convolution_bias_clip(cuda_device, shape, code, layout):
    """out = clip(conv(in, fil) + bias[k], 0, 6)."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.conv import conv_fused
    from rocmlir_b200.gemm import Epilogue
    cfg, ocfg = _cfgs(**shape, **layout)
    (bf, braw), (ff, fraw), (inf, iraw) = reference_random([(cfg.k,), (cfg.numel("fil"),), (cfg.numel("in"),)], code, seed=1)
    # the oracle takes the tensors in the library's layouts except the output, which it produces as [n][h][w][k]
    acc = oracle.conv_f32(ocfg, 0, ff, inf, None, threads=oracle.max_threads())
    mid = None if code == oracle.F32 else code
    ref = oracle.from_f32(_to_layout(oracle.epilogue(acc, cfg.k, bias=bf, clip=(0.0, 6.0), mid_type=mid), cfg), code)
    out = torch.empty(cfg.numel("out"), dtype=torch_dtype(code), device="cuda")
    epi = Epilogue(bias=to_device(braw, code), clip=(0.0, 6.0), mid_type=mid)
    conv_fused(cfg, to_device(fraw, code), to_device(iraw, code), out, epi)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    got = from_device(out, code)
    np.testing.assert_array_equal(got.ravel(), ref.ravel())
    assert got.size and (oracle.to_f32(got, code) >= 0).all() and (oracle.to_f32(got, code) <= 6).all()


@pytest.mark.parametrize("zp_in,zp_out", [(0, 0), (3, -5)])
@pytest.mark.parametrize("layout", [NHWC, NCHW], ids=["nhwc", "nchw"])
def test_quant_convolution_dequant_add_relu_quant(cuda_device, layout, zp_in, zp_out):
    """i8 conv -> i32 -> (f32(acc) - zp_in) * s -> + bias[k] -> relu -> * 1/s_out -> rne -> + zp_out -> clamp -> i8,
    with the dequantisation scale of the reference's test (2^-13) and an output scale at which a percent or two of the
    outputs saturate, bit-exact."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.conv import conv_fused
    from rocmlir_b200.gemm import Epilogue
    cfg, ocfg = _cfgs(n=2, c=64, k=48, h=10, w=10, y=3, x=3, pad_h=1, pad_w=1, **layout)
    fil = uniform_int8((cfg.numel("fil"),), seed=31)
    inp = uniform_int8((cfg.numel("in"),), seed=32)
    bias = uniform_f32((cfg.k,), seed=33, lo=-2.0, hi=2.0)
    s_deq, s_out = 1.22070313e-4, 0.25
    acc = oracle.conv_i8(ocfg, fil, inp, wrap_product=False, threads=oracle.max_threads())
    x = oracle.epilogue(acc.reshape(-1, cfg.k), cfg.k, alpha=s_deq, bias=bias, relu=True, requant_scale=s_out,
                        in_zero=float(zp_in) if zp_in else None)
    ref = _to_layout(oracle.quantize_i8(x, zp_out), cfg)
    assert 0.001 < np.mean(ref == 127) < 0.1 and np.mean(ref == zp_out) > 0.05   # both the clamp and the rectifier bite
    epi = Epilogue(alpha=s_deq, bias=to_device(bias, oracle.F32), relu=True, requant_scale=s_out,
                   in_zero=float(zp_in) if zp_in else None, out_zero=zp_out if zp_out else None)
    out = torch.empty(cfg.numel("out"), dtype=torch.int8, device="cuda")
    conv_fused(cfg, to_device(fil, oracle.I8), to_device(inp, oracle.I8), out, epi)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    np.testing.assert_array_equal(out.cpu().numpy().ravel(), ref.ravel())


def _gemm(araw, braw, code, out_code, **kw):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import gemm
    out = gemm(to_device(araw, code), to_device(braw, code), out_dtype=torch_dtype(out_code), **kw)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return from_device(out, out_code)


@pytest.mark.parametrize("tc", [False, True], ids=["c", "trans_c"])
@pytest.mark.parametrize("code", [oracle.F16, oracle.F32, oracle.BF16])
@pytest.mark.parametrize("g,m,n,k", [(1, 5, 3, 4), (2, 300, 200, 456), (1, 64, 576, 8192)],
                         ids=["mixr_5x4x3", "ragged", "k_split"])
def test_dot_plus_same_shape_add(cuda_device, g, m, n, k, code, tc):
    """migraphx.dot then migraphx.add with an operand of the result's shape; the dot result is rounded to its declared
    type before the add. The third shape cuts K into ranges, where the add happens in the reduction pass."""
    from rocmlir_b200.gemm import Epilogue
    (af, araw), (bf, braw), (rf, rraw) = reference_random([(g, m, k), (g, k, n), (g, m, n)], code, seed=1)
    acc = oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads())
    mid = None if code == oracle.F32 else code
    ref = oracle.from_f32(oracle.epilogue(acc, n, residual=rf, mid_type=mid), code)
    res_dev = to_device(np.ascontiguousarray(np.swapaxes(rraw, 1, 2)) if tc else rraw, code)
    got = _gemm(araw, braw, code, code, trans_c=tc, epilogue=Epilogue(residual=res_dev, mid_type=mid))
    got = np.swapaxes(got.reshape(g, n, m), 1, 2) if tc else got.reshape(g, m, n)
    np.testing.assert_array_equal(got, ref.reshape(g, m, n))


@pytest.mark.parametrize("mode", ["row", "scalar"])
@pytest.mark.parametrize("g,m,n,k", [(2, 130, 100, 192), (1, 64, 576, 8192)], ids=["ragged", "k_split"])
def test_dot_plus_bias_broadcast_along_n_or_scalar(cuda_device, g, m, n, k, mode):
    from rocmlir_b200.gemm import Epilogue
    code = oracle.F16
    (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], code, seed=1)
    bias = ((np.arange(m if mode == "row" else 1) % 11) - 5).astype(np.float32)
    acc = oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads())
    # rows are counted over all leading dimensions in the oracle: the per-row bias repeats for every batch
    ref = oracle.from_f32(oracle.epilogue(acc, n, bias=np.tile(bias, g) if mode == "row" else bias, bias_mode=mode,
                                          relu=True, mid_type=code), code)
    epi = Epilogue(bias=to_device(oracle.from_f32(bias, code), code), bias_mode=mode, relu=True, mid_type=code)
    got = _gemm(araw, braw, code, code, epilogue=epi)
    np.testing.assert_array_equal(got.reshape(ref.shape), ref)


@pytest.mark.parametrize("code,rms", [(oracle.F32, 3e-5), (oracle.F16, 1e-3)])
def test_gemm_accumulate_store_method(cuda_device, code, rms):
    """--store-method=atomic_add at the reference's shape (-g 3 -m 1024 -k 769 -n 1024): C = C_old + A.B. Exact on
    integer-valued data; on float data the reference verifier with the suite's thresholds (f16: RMS 1e-3)."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import gemm
    g, m, n, k = 3, 1024, 1024, 769
    for float_data in (False, True):
        (af, araw), (bf, braw), (cf, craw) = reference_random([(g, m, k), (g, k, n), (g, m, n)], code, seed=1,
                                                              rand_float=float_data, mn=-1 if float_data else -5,
                                                              mx=1 if float_data else 5)
        acc = oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads())
        ref = oracle.epilogue(acc, n, residual=cf, mid_type=code)
        c = to_device(craw, code).clone()
        gemm(to_device(araw, code), to_device(braw, code), out=c, accumulate=True)
        torch.cuda.synchronize()
        assert L.kernel_status() == 0
        got = from_device(c, code)
        if not float_data:
            np.testing.assert_array_equal(got.reshape(g, m, n), oracle.from_f32(ref, code).reshape(g, m, n))
        else:
            verdict, info = oracle.verify_float(oracle.to_f32(got, code), oracle.round_to(ref, code), rms, 100.0, 100.0)
            assert verdict == [1, 1, 1], info


@pytest.mark.parametrize("code", [oracle.F16, oracle.F32])
@pytest.mark.parametrize("fn", ["abs", "ceil", "erf", "exp", "floor", "log", "neg", "recip", "rsqrt", "sigmoid", "sqrt", "tanh"])
def test_gemm_bias_unary(cuda_device, fn, code):
    """dot -> add(bias) -> one MIGraphX unary elementwise op (MIGraphX.td:134-181), each step in the declared type.
    Operands are positive so that log / sqrt / rsqrt / recip see their domain. The oracle evaluates the function with
    the C library in f32; the device's own f32 routines may differ in the last bit, which after the rounding to f16
    shows as an occasional one-step difference (as does the summation order of the GEMM itself on such data): the
    reference verifier with its RMS bar decides; ceil / floor are compared exactly away from their steps."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import Epilogue, gemm
    m, n, k = 300, 200, 96
    rng = np.random.Generator(np.random.PCG64(sum(map(ord, fn))))   # (not hash(): that differs from process to process)
    a32 = rng.uniform(0.05, 0.5, size=(m, k)).astype(np.float32)
    b32 = rng.uniform(0.05, 0.5, size=(k, n)).astype(np.float32)
    bias32 = rng.uniform(-0.5, 0.5, size=(n,)).astype(np.float32)
    if fn in ("log", "sqrt", "rsqrt", "recip"):
        bias32 = np.abs(bias32) + np.float32(0.1)
    araw, braw, biasraw = (oracle.from_f32(x, code) for x in (a32, b32, bias32))
    af, bf, biasf = (oracle.to_f32(x, code) for x in (araw, braw, biasraw))
    mid = None if code == oracle.F32 else code
    acc = oracle.gemm_f32(af[None], bf[None], 1, m, n, k, threads=oracle.max_threads())
    ref = oracle.from_f32(oracle.epilogue(acc, n, bias=biasf, mid_type=mid, unary=fn), code)
    out = gemm(to_device(araw, code), to_device(braw, code), out_dtype=torch_dtype(code),
               epilogue=Epilogue(bias=to_device(biasraw, code), mid_type=mid, unary=fn), f32_mode=0)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    got = from_device(out, code).reshape(ref.shape)
    bar = 1e-3 if code == oracle.F16 else 3e-5
    if fn in ("ceil", "floor"):
        # a step function turns a last-bit difference of the sum into a whole unit: compare where the argument is not
        # within two f16 steps of an integer (the sums reach 16, where a step is 2^-7)
        pre = oracle.to_f32(oracle.from_f32(oracle.epilogue(acc, n, bias=biasf, mid_type=mid), code), code).reshape(ref.shape)
        keep = np.abs(pre - np.rint(pre)) > 0.02
        assert keep.mean() > 0.9
        np.testing.assert_array_equal(oracle.to_f32(got, code)[keep], oracle.to_f32(ref, code)[keep])
        return
    verdict, info = oracle.verify_float(oracle.to_f32(got, code), oracle.to_f32(ref, code), bar, 1e30, 1e30)
    assert verdict[0] == 1, (fn, info)
