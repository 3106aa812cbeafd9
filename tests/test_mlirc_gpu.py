"""The MLIR C API surface end to end on the GPU: module text -> high-level / backend pipelines -> launch, checked
against op-by-op oracle restatements; and the same kernel launched by the client itself from mlirGetBinary's cubin."""
import numpy as np
import pytest

import oracle
from helpers import from_device, reference_random, to_device, uniform_f32, uniform_int8
from test_mlirc_cpu import CONV_1D, CONV_BIAS_CLIP_NHWC, DOT_INT4, DOT_SHARED_B, DOT_ADD, DOT_TRANSB_BIAS_RELU, QUANT_CONV

pytestmark = pytest.mark.gpu


def _launch(text, tensors):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.mlirc import Module
    with Module(text) as m:
        m.high_level()
        m.backend("sm_100a")
        m.launch(tensors)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0


def test_dot_add_f32(cuda_device):
    import torch
    (af, araw), (bf, braw), (cf, craw) = reference_random([(1, 5, 4), (1, 4, 3), (1, 5, 3)], oracle.F32, seed=1)
    out = torch.zeros((1, 5, 3), dtype=torch.float32, device="cuda")
    _launch(DOT_ADD, [to_device(araw, oracle.F32), to_device(braw, oracle.F32), to_device(craw, oracle.F32), out])
    ref = oracle.epilogue(oracle.gemm_f32(af, bf, 1, 5, 3, 4), 3, residual=cf)
    np.testing.assert_array_equal(out.cpu().numpy(), ref)


def test_dot_transposed_b_bias_relu_f16(cuda_device):
    import torch
    g, m, n, k = 2, 384, 520, 256
    (af, araw), (bf, braw), (biasf, biasraw) = reference_random([(g, m, k), (g, n, k), (n,)], oracle.F16, seed=1)   # B stored [g][n][k]
    out = torch.zeros((g, m, n), dtype=torch.float16, device="cuda")
    _launch(DOT_TRANSB_BIAS_RELU, [to_device(araw, oracle.F16), to_device(braw, oracle.F16), to_device(biasraw, oracle.F16), out])
    acc = oracle.gemm_f32(af, bf, g, m, n, k, tb=True, threads=oracle.max_threads())
    ref = oracle.from_f32(oracle.epilogue(acc, n, bias=biasf, relu=True, mid_type=oracle.F16), oracle.F16)
    np.testing.assert_array_equal(from_device(out, oracle.F16).reshape(ref.shape), ref)


def _conv_case():
    ocfg = oracle.Conv(n=2, c=64, k=96, h=14, w=14, y=3, x=3, pad_h=1, pad_w=1, fil_layout="gkyxc", in_layout="nhwgc", out_layout="nhwgk")
    (bf, braw), (xf, xraw), (wf, wraw) = reference_random([(96,), (ocfg.numel("in"),), (ocfg.numel("fil"),)], oracle.F16, seed=1)
    acc = oracle.conv_f32(ocfg, 0, wf, xf, None, threads=oracle.max_threads())
    ref = oracle.from_f32(oracle.epilogue(acc, 96, bias=bf, clip=(0.0, 6.0), mid_type=oracle.F16), oracle.F16)
    return ocfg, (braw, xraw, wraw), ref


def test_convolution_bias_clip_nhwc_f16(cuda_device):
    import torch
    ocfg, (braw, xraw, wraw), ref = _conv_case()
    out = torch.zeros(ocfg.numel("out"), dtype=torch.float16, device="cuda")
    _launch(CONV_BIAS_CLIP_NHWC, [to_device(braw, oracle.F16), to_device(xraw, oracle.F16), to_device(wraw, oracle.F16), out])
    np.testing.assert_array_equal(from_device(out, oracle.F16).ravel(), ref.ravel())


def test_one_dimensional_convolution_bias_relu(cuda_device):
    """Rank-3 tensors (n, c, w), channels last, stride 2, padding 2: the unit-height 2-D problem against the oracle."""
    import torch
    ocfg = oracle.Conv(n=4, c=64, k=128, h=1, w=100, y=1, x=5, stride_w=2, pad_w=2, fil_layout="gkyxc", in_layout="nhwgc",
                       out_layout="nhwgk")
    (xf, xraw), (wf, wraw), (bf, braw) = reference_random([(ocfg.numel("in"),), (ocfg.numel("fil"),), (128,)], oracle.F16, seed=3)
    acc = oracle.conv_f32(ocfg, 0, wf, xf, None, threads=oracle.max_threads())
    ref = oracle.from_f32(oracle.epilogue(acc, 128, bias=bf, relu=True, mid_type=oracle.F16), oracle.F16)
    out = torch.zeros(ocfg.numel("out"), dtype=torch.float16, device="cuda")
    _launch(CONV_1D, [to_device(xraw, oracle.F16), to_device(wraw, oracle.F16), to_device(braw, oracle.F16), out])
    np.testing.assert_array_equal(from_device(out, oracle.F16).ravel(), ref.ravel())


def _unpack_int4(packed: np.ndarray, signed: bool) -> np.ndarray:
    """MIGraphX.td:190-193: out[..., 2i] = in & 0xf, out[..., 2i+1] = in >> 4 (arithmetic when signed)."""
    b = packed.astype(np.uint8)
    lo, hi = (b & 0xF).astype(np.int16), (b >> 4).astype(np.int16)
    if signed:
        lo = np.where(lo > 7, lo - 16, lo)
        hi = np.where(hi > 7, hi - 16, hi)
    out = np.empty(packed.shape[:-1] + (2 * packed.shape[-1],), dtype=np.int16)
    out[..., 0::2], out[..., 1::2] = lo, hi
    return out


def test_int4_weights_unpack_dequantize_dot(cuda_device):
    """The graph of mlir/test/fusion/pr-e2e/mixr-dot-int4-f16.mlir: packed signed int4 operand -> unpack along the
    reduction dimension -> x 0.25 (f16) -> dot with an f16 matrix, against numpy + the GEMM oracle."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.mlirc import Module
    rng = np.random.Generator(np.random.PCG64(11))
    packed = rng.integers(0, 256, size=(1, 96, 64), dtype=np.uint8)
    (bf, braw), = reference_random([(1, 128, 80)], oracle.F16, seed=2)
    a = (_unpack_int4(packed, signed=True).astype(np.float32) * np.float32(0.25)).astype(np.float16).astype(np.float32)
    ref = oracle.from_f32(oracle.gemm_f32(a, bf, 1, 96, 80, 128), oracle.F16)
    out = torch.zeros((1, 96, 80), dtype=torch.float16, device="cuda")
    with Module(DOT_INT4) as m:
        m.high_level()
        m.backend("sm_100a")
        ws = torch.empty(m.workspace_size, dtype=torch.uint8, device="cuda")
        m.launch([torch.from_numpy(packed.view(np.int8)).cuda(), to_device(braw, oracle.F16), out], workspace=ws)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    np.testing.assert_array_equal(from_device(out, oracle.F16).reshape(ref.shape), ref)


@pytest.mark.parametrize("unsigned,out", [(0, "i8"), (1, "i8"), (0, "f16"), (1, "bf16"), (0, "f32")])
def test_unpack_int4_entry_point(cuda_device, unsigned, out):
    import ctypes as C
    import torch
    from rocmlir_b200 import _lib as L
    rng = np.random.Generator(np.random.PCG64(5))
    packed = rng.integers(0, 256, size=(7, 33), dtype=np.uint8)       # odd sizes: no vector assumptions
    vals = _unpack_int4(packed, signed=not unsigned).astype(np.float32)
    dt = {"i8": torch.int8, "f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[out]
    code = {"i8": L.I8, "f16": L.F16, "bf16": L.BF16, "f32": L.F32}[out]
    scale, zero = (1.0, 0) if out == "i8" else (0.37, 3)
    dst = torch.zeros((7, 66), dtype=dt, device="cuda")
    src = torch.from_numpy(packed).cuda()
    L.check(L.lib().rbUnpackInt4(src.data_ptr(), dst.data_ptr(), packed.size, unsigned, code, C.c_float(scale), zero, None))
    torch.cuda.synchronize()
    want = torch.from_numpy(vals if out == "i8" else (vals - zero) * np.float32(scale)).to(dt)
    assert torch.equal(dst.cpu(), want)


def test_shared_second_operand_runs_as_one_group(cuda_device):
    import torch
    (af, araw), (bf, braw) = reference_random([(8, 96, 64), (1, 64, 80)], oracle.F16, seed=4)
    out = torch.zeros((8, 96, 80), dtype=torch.float16, device="cuda")
    _launch(DOT_SHARED_B, [to_device(araw, oracle.F16), to_device(braw, oracle.F16), out])
    ref = oracle.from_f32(oracle.gemm_f32(af.reshape(1, 768, 64), bf, 1, 768, 80, 64), oracle.F16)
    np.testing.assert_array_equal(from_device(out, oracle.F16).reshape(ref.shape), ref)


def test_client_launches_the_modules_kernel_from_the_binary(cuda_device):
    """mlirGetBinary + mlirGetKernelAttrs + rbModuleGetKernelLaunch, then cuModuleLoadData / cuLaunchKernelEx by the
    client: the fused convolution + bias + clip in one kernel out of the cubin."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.mlirc import Module
    from test_cubin_gpu import driver_launch
    ocfg, (braw, xraw, wraw), ref = _conv_case()
    out = torch.zeros(ocfg.numel("out"), dtype=torch.float16, device="cuda")
    tensors = [to_device(braw, oracle.F16), to_device(xraw, oracle.F16), to_device(wraw, oracle.F16), out]
    with Module(CONV_BIAS_CLIP_NHWC) as m:
        m.high_level()
        m.backend("sm_100a")
        block, grid = m.kernel_attrs()
        image = m.binary()
        kl = m.kernel_launch(tensors)
    assert (kl.block, kl.grid) == (block, grid)
    torch.cuda.synchronize()
    driver_launch(image, kl, torch.cuda.current_stream().cuda_stream)
    assert L.kernel_status() == 0
    np.testing.assert_array_equal(from_device(out, oracle.F16).ravel(), ref.ravel())


def test_quant_convolution_chain_nchw(cuda_device):
    import torch
    ocfg = oracle.Conv(n=2, c=64, k=48, h=10, w=10, y=3, x=3, pad_h=1, pad_w=1, fil_layout="gkcyx", in_layout="ngchw", out_layout="nhwgk")
    bias = uniform_f32((48,), seed=33, lo=-2.0, hi=2.0)
    x = uniform_int8((ocfg.numel("in"),), seed=32)
    w = uniform_int8((ocfg.numel("fil"),), seed=31)
    acc = oracle.conv_i8(ocfg, w, x, wrap_product=False, threads=oracle.max_threads())
    y = oracle.epilogue(acc.reshape(-1, 48), 48, alpha=1.22070313e-4, bias=bias, relu=True, requant_scale=0.25)
    ref = oracle.quantize_i8(y, -5).reshape(2, 10, 10, 48).transpose(0, 3, 1, 2)     # the function returns NCHW
    out = torch.zeros(ocfg.numel("out"), dtype=torch.int8, device="cuda")
    _launch(QUANT_CONV, [to_device(bias, oracle.F32), to_device(x, oracle.I8), to_device(w, oracle.I8), out])
    np.testing.assert_array_equal(out.cpu().numpy().reshape(2, 48, 10, 10), ref)
