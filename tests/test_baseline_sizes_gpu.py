"""The benchmark configurations at their stated sizes against the CPU oracle.

The sequential oracle cannot evaluate these problems whole in test time, so each case compares a seeded sample on
which the oracle is exact work for exact work - rows of a GEMM (rows are independent), images of a forward or
backward-data convolution (images are independent), output channels of a backward-weight convolution (each filter
gradient entry is a reduction over the WHOLE batch, so the sample still covers every K range of the split) - and adds
size-independent properties over the whole result: bitwise determinism of a second run and, for the integer GEMM,
row and column checksums that must hold exactly.

Bars: integer results bit-exact; float results by the reference's verifier with the RMS thresholds of its own suites
(f16 1e-3: mlir/test/e2e/PrResnet50.toml:3, rocmlir-gen.cpp:2850-2861; bf16 and fp8 -> bf16 8e-3 from the 8-bit
mantissa of the result), relDiff disabled as the reference does for 16-bit types (summation order differs).
"""
import numpy as np
import pytest

import oracle
from helpers import from_device, normal_data, to_device, uniform_f32, uniform_int8

pytestmark = pytest.mark.gpu

RMS = {oracle.F16: 1e-3, oracle.BF16: 8e-3, oracle.F8E4M3: 8e-3}


def _gemm(a_raw, b_raw, code, out_code, tb=False, epilogue=None):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import gemm
    from helpers import torch_dtype
    out = gemm(to_device(a_raw, code), to_device(b_raw, code), trans_b=tb, out_dtype=torch_dtype(out_code),
               epilogue=epilogue)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return from_device(out, out_code)


def _rows(m, count, seed):
    """Sampled rows: the first and last row of the matrix, the rows either side of the CTA-pair tile edges that the
    ragged last wave computes, and seeded random ones."""
    fixed = [0, 127, 128, 255, 256, m - 129, m - 128, m - 1]
    rnd = np.random.Generator(np.random.PCG64(seed)).choice(m, size=count - len(fixed), replace=False)
    return np.unique(np.concatenate([np.asarray(fixed), rnd]))


# ---- config 3: quantised LLM-linear GEMM, M = 2048 tokens, N = 11008, K = 4096 --------------------------------------
C3 = (2048, 11008, 4096)


@pytest.fixture(scope="module")
def c3_int8():
    m, n, k = C3
    return uniform_int8((1, m, k), seed=101), uniform_int8((1, n, k), seed=102)     # weight stored [out, in]: transB


def test_int8_llm_linear_full_size_bit_exact(cuda_device, c3_int8):
    m, n, k = C3
    a, b = c3_int8
    got = _gemm(a, b, oracle.I8, oracle.I32, tb=True).reshape(m, n)
    rows = _rows(m, 64, seed=7)
    ref = oracle.gemm_i8(a[:, rows, :], b, 1, len(rows), n, k, tb=True, threads=oracle.max_threads())
    verdict, info = oracle.verify_int(got[rows], ref)
    assert verdict == [1, 1, 1] and info["overflows"] == 0, info
    # whole-tensor checksums, exact in integers: 1^T C = (1^T A) B^T and C 1 = A (B^T 1)
    a64, b64 = a[0].astype(np.int64), b[0].astype(np.int64)
    np.testing.assert_array_equal(got.astype(np.int64).sum(0), a64.sum(0) @ b64.T)
    np.testing.assert_array_equal(got.astype(np.int64).sum(1), a64 @ b64.sum(0))
    again = _gemm(a, b, oracle.I8, oracle.I32, tb=True).reshape(m, n)
    np.testing.assert_array_equal(again, got)


def test_int8_llm_linear_full_size_dequant_requant_bit_exact(cuda_device, c3_int8):
    """i32 -> f32 -> x s_col[n] -> x 1/s_out -> round half even -> saturate -> i8, at 2048 x 11008 x 4096 with
    per-column scales ~ U(0.001, 0.01) and an output scale at which about 1 % of the outputs saturate."""
    from rocmlir_b200.gemm import Epilogue
    m, n, k = C3
    a, b = c3_int8
    s_col = uniform_f32((n,), seed=103, lo=0.001, hi=0.01)
    rows = _rows(m, 64, seed=8)
    acc = oracle.gemm_i8(a[:, rows, :], b, 1, len(rows), n, k, tb=True, threads=oracle.max_threads())
    deq = oracle.epilogue(acc, n, col_scale=s_col)
    s_out = float(np.float32(np.quantile(np.abs(deq), 0.99) / 127.0))
    ref = oracle.from_f32(oracle.epilogue(acc, n, col_scale=s_col, requant_scale=s_out), oracle.I8, sat_int=True)
    assert 0.001 < np.mean(np.abs(ref.astype(np.int32)) >= 127) < 0.05
    epi = Epilogue(col_scale=to_device(s_col, oracle.F32), requant_scale=s_out)
    got = _gemm(a, b, oracle.I8, oracle.I8, tb=True, epilogue=epi).reshape(m, n)
    np.testing.assert_array_equal(got[rows], ref.reshape(len(rows), n))
    again = _gemm(a, b, oracle.I8, oracle.I8, tb=True, epilogue=epi).reshape(m, n)
    np.testing.assert_array_equal(again, got)


def test_fp8_llm_linear_full_size_bf16_out(cuda_device):
    """fp8-e4m3 x fp8-e4m3 with per-tensor scales amax/448, f32 accumulate, x (sA sB), bf16 out, full size."""
    from rocmlir_b200.gemm import Epilogue
    m, n, k = C3
    xa = normal_data((1, m, k), oracle.F32, seed=111, scale=1.0)[0]
    xb = normal_data((1, n, k), oracle.F32, seed=112, scale=1.0)[0]
    sa, sb = np.float32(np.abs(xa).max() / 448.0), np.float32(np.abs(xb).max() / 448.0)
    araw, braw = oracle.from_f32(xa / sa, oracle.F8E4M3), oracle.from_f32(xb / sb, oracle.F8E4M3)
    alpha = np.float32(sa * sb)
    got = oracle.to_f32(_gemm(araw, braw, oracle.F8E4M3, oracle.BF16, tb=True, epilogue=Epilogue(alpha=float(alpha))),
                        oracle.BF16).reshape(m, n)
    rows = _rows(m, 32, seed=9)
    af, bf = oracle.to_f32(araw[:, rows, :], oracle.F8E4M3), oracle.to_f32(braw, oracle.F8E4M3)
    acc = oracle.gemm_f32(af, bf, 1, len(rows), n, k, tb=True, threads=oracle.max_threads())
    ref = oracle.round_to(oracle.epilogue(acc, n, alpha=alpha), oracle.BF16)
    verdict, info = oracle.verify_float(got[rows], ref, RMS[oracle.F8E4M3], 100.0, 100.0)
    assert verdict == [1, 1, 1], info


# ---- config 2: 4096^3, bf16 variant and the fused relu(C + bias[N]) --------------------------------------------------
def test_bf16_gemm_4096_cubed_sampled_rows(cuda_device):
    m = n = k = 4096
    af, araw = normal_data((1, m, k), oracle.BF16, seed=1, scale=0.1)
    bf, braw = normal_data((1, k, n), oracle.BF16, seed=2, scale=0.1)
    got_raw = _gemm(araw, braw, oracle.BF16, oracle.BF16)
    got = oracle.to_f32(got_raw, oracle.BF16).reshape(m, n)
    rows = _rows(m, 24, seed=3)
    ref = oracle.round_to(oracle.gemm_f32(af[:, rows, :], bf, 1, len(rows), n, k, threads=oracle.max_threads()), oracle.BF16)
    verdict, info = oracle.verify_float(got[rows], ref, RMS[oracle.BF16], 100.0, 100.0)
    assert verdict == [1, 1, 1], info
    np.testing.assert_array_equal(_gemm(araw, braw, oracle.BF16, oracle.BF16), got_raw)


@pytest.mark.parametrize("bias_code", [oracle.F16, oracle.F32], ids=["bias_f16", "bias_f32"])
def test_fp16_gemm_4096_cubed_bias_relu_sampled_rows(cuda_device, bias_code):
    """C' = relu(C + bias[N]), bias ~ N(0, 0.1), f16 or f32 bias vector; the dot result is rounded to f16 before the
    add (the MIGraphX form dot -> add -> relu, MIGraphXToTosa.cpp:1009-1018)."""
    from rocmlir_b200.gemm import Epilogue
    m = n = k = 4096
    af, araw = normal_data((1, m, k), oracle.F16, seed=1, scale=0.1)
    bf, braw = normal_data((1, k, n), oracle.F16, seed=2, scale=0.1)
    biasf, biasraw = normal_data((n,), bias_code, seed=4, scale=0.1)
    epi = Epilogue(bias=to_device(biasraw, bias_code), relu=True, mid_type=oracle.F16)
    got = oracle.to_f32(_gemm(araw, braw, oracle.F16, oracle.F16, epilogue=epi), oracle.F16).reshape(m, n)
    rows = _rows(m, 24, seed=5)
    acc = oracle.gemm_f32(af[:, rows, :], bf, 1, len(rows), n, k, threads=oracle.max_threads())
    ref = oracle.round_to(oracle.epilogue(acc, n, bias=biasf, relu=True, mid_type=oracle.F16), oracle.F16)
    verdict, info = oracle.verify_float(got[rows], ref, RMS[oracle.F16], 100.0, 100.0)
    assert verdict == [1, 1, 1], info
    assert (got >= 0).all()
    assert 0.3 < np.mean(got[rows] == 0) < 0.7      # the rectifier is really at work on zero-mean data


# ---- config 4: fp16 NHWC ResNet-50 layers at batch 256, three directions ---------------------------------------------
RESNET = {"a": dict(c=64, k=64, h=56, w=56, y=3, x=3, pad_h=1, pad_w=1),
          "b": dict(c=256, k=64, h=56, w=56, y=1, x=1),
          "c": dict(c=128, k=128, h=28, w=28, y=3, x=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1),
          "d": dict(c=512, k=2048, h=7, w=7, y=1, x=1)}
NHWC = dict(fil_layout="kyxc", in_layout="nhwc", out_layout="nhwk")
BATCH = 256
IMAGES = (0, 171, 255)
_DATA = {}


def _cfgs(n, shape, k=None):
    from rocmlir_b200.conv import ConvConfig
    kw = dict(RESNET[shape])
    if k is not None:
        kw["k"] = k
    cfg = ConvConfig(n=n, **kw, **NHWC)
    ocfg = oracle.Conv(n=n, c=cfg.c, k=cfg.k, h=cfg.h, w=cfg.w, y=cfg.y, x=cfg.x, stride_h=cfg.stride_h,
                       stride_w=cfg.stride_w, pad_h=cfg.pad_h, pad_w=cfg.pad_w, fil_layout=cfg.fil_layout,
                       in_layout=cfg.in_layout, out_layout=cfg.out_layout)
    return cfg, ocfg


def _data(shape):
    """Filter, input and output(-gradient) tensors ~ 0.05 N(0,1) in f16, made once per layer shape."""
    if shape not in _DATA:
        _, ocfg = _cfgs(BATCH, shape)
        _DATA[shape] = {w: normal_data((ocfg.numel(w),), oracle.F16, seed=s, scale=0.05)
                        for w, s in (("fil", 1), ("in", 2), ("out", 3))}
    return _DATA[shape]


def _conv(cfg, direction, raws):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.conv import conv
    t = {k: to_device(v, oracle.F16) for k, v in raws.items()}
    res = conv(cfg, direction, t["fil"], t["in"], t["out"])
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return oracle.to_f32(from_device(res, oracle.F16), oracle.F16)


@pytest.mark.parametrize("direction", [0, 1], ids=["fwd", "bwd_data"])
@pytest.mark.parametrize("shape", list(RESNET))
def test_fp16_nhwc_resnet_batch_256_sampled_images(cuda_device, shape, direction):
    cfg, ocfg = _cfgs(BATCH, shape)
    d = _data(shape)
    res_name = "out" if direction == 0 else "in"
    raws = {w: d[w][1] for w in ("fil", "in", "out")}
    raws[res_name] = np.zeros(ocfg.numel(res_name), np.uint16)
    got = _conv(cfg, direction, raws).reshape(BATCH, -1)
    _, ocfg1 = _cfgs(1, shape)
    per_in, per_out = ocfg1.numel("in"), ocfg1.numel("out")
    for img in IMAGES:
        inp = d["in"][0][img * per_in:(img + 1) * per_in]
        out = d["out"][0][img * per_out:(img + 1) * per_out]
        ref = oracle.round_to(oracle.conv_f32(ocfg1, direction, d["fil"][0], inp if direction == 0 else None,
                                              out if direction == 1 else None, threads=oracle.max_threads()), oracle.F16)
        verdict, info = oracle.verify_float(got[img], ref, RMS[oracle.F16], 100.0, 100.0)
        assert verdict == [1, 1, 1], (img, info)


@pytest.mark.parametrize("shape", list(RESNET))
def test_fp16_nhwc_resnet_batch_256_backward_weight(cuda_device, shape):
    """The filter gradient reduces over all N Ho Wo = up to 802 816 output pixels (49 K ranges with f32 planes and a
    fixed-order reduction on the GPU). Sampled output channels are compared over the WHOLE batch: the gradient of
    channel k only needs channel k of the output gradient, so the oracle runs the same convolution with the sampled
    channels as its K."""
    cfg, ocfg = _cfgs(BATCH, shape)
    d = _data(shape)
    raws = {"fil": np.zeros(ocfg.numel("fil"), np.uint16), "in": d["in"][1], "out": d["out"][1]}
    got = _conv(cfg, 2, raws).reshape(cfg.k, -1)
    nsel = {"a": 6, "b": 6, "c": 12, "d": 96}[shape]   # sized so that the sequential oracle needs seconds
    ksel = np.unique(np.concatenate([[0, cfg.k - 1], np.random.Generator(np.random.PCG64(11)).choice(cfg.k, nsel - 2, replace=False)]))
    _, osub = _cfgs(BATCH, shape, k=len(ksel))
    out_sub = np.ascontiguousarray(d["out"][0].reshape(-1, cfg.k)[:, ksel]).ravel()
    ref = oracle.round_to(oracle.conv_f32(osub, 2, None, d["in"][0], out_sub, threads=oracle.max_threads()), oracle.F16)
    verdict, info = oracle.verify_float(got[ksel].ravel(), ref, RMS[oracle.F16], 100.0, 100.0)
    assert verdict == [1, 1, 1], info
    # accuracy against a float64 reduction of the same entries: the GPU's range-wise f32 sums are no worse than the
    # oracle's single sequential f32 chain (plus one f16 output ulp)
    ref64 = oracle.conv_f32(osub, 2, None, d["in"][0], out_sub, threads=oracle.max_threads(), f64=True)
    err_gpu = np.abs(got[ksel].ravel().astype(np.float64) - ref64).max()
    err_ref = np.abs(ref.astype(np.float64) - ref64).max()
    assert err_gpu <= err_ref + 2.0 ** -10 * np.abs(ref64).max(), (err_gpu, err_ref)
    again = _conv(cfg, 2, raws).reshape(cfg.k, -1)
    np.testing.assert_array_equal(again, got)    # deterministic: no atomics
