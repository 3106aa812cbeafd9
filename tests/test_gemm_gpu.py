"""GPU parity tests of rbGemm (through the C ABI) against the CPU oracle.

Bars: integer results bit-exact; float results judged by the reference's verifier
(conv-validation-wrappers.cpp:104-216) with the thresholds stated beside each case, and exactly
equal on the reference's integer-valued random data (`-rand 1 -rand_type int`: values in [-5,4],
rocmlir-gen.cpp:1346-1349) where every partial sum is exactly representable.
"""
import numpy as np
import pytest

import oracle
from helpers import from_device, normal_data, reference_random, to_device, uniform_f32, uniform_int8

pytestmark = pytest.mark.gpu

# RMS thresholds: f32 / f16 are the reference's defaults (rocmlir-gen.cpp:709-721, 2850-2861);
# bf16 and fp8-in/bf16-out follow from the 8-bit mantissa of the output type (2^-9 relative rounding).
RMS = {oracle.F32: 3e-5, oracle.F16: 1e-3, oracle.BF16: 8e-3, oracle.F8E4M3: 8e-3}


def run_gemm(a_raw, b_raw, code, out_code, ta=False, tb=False, tc=False, epilogue=None, variant=None, f32_mode=0):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import gemm
    from helpers import torch_dtype
    a = to_device(a_raw, code)
    b = to_device(b_raw, code)
    out = gemm(a, b, trans_a=ta, trans_b=tb, trans_c=tc, out_dtype=torch_dtype(out_code), epilogue=epilogue,
               variant=variant, f32_mode=f32_mode)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0, "a bounded device-side wait ran out"
    return from_device(out, out_code)


def stored(x, trans):
    """Logical [G, rows, cols] -> storage order ([G, cols, rows] when transposed)."""
    return np.ascontiguousarray(np.swapaxes(x, 1, 2)) if trans else x


# Shapes from the reference's own GEMM suites (mlir/test/e2e/PrGemm.toml:28-53): default 1024x769x512
# (odd K -> padding path), G = 3 batches, 1x1x1, plus tile-edge cases of this kernel (128 / 256 / 64 +-1).
SHAPES = [(1, 1024, 512, 769), (3, 64, 96, 128), (1, 1, 1, 1), (1, 129, 257, 65), (2, 255, 130, 72),
          (1, 128, 256, 64)]


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("ta,tb,tc", [(0, 0, 0), (1, 0, 0), (0, 1, 0), (1, 1, 1)])
@pytest.mark.parametrize("code", [oracle.F16, oracle.BF16, oracle.F8E4M3, oracle.F32])
@pytest.mark.parametrize("g,m,n,k", SHAPES[1:])
def test_float_gemm_exact_on_reference_integer_data(cuda_device, g, m, n, k, code, ta, tb, tc, variant):
    (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], code, seed=1)
    out_code = oracle.F32 if code == oracle.F8E4M3 else code   # rocmlir-gen: -t fp8 => f32 result
    ref = oracle.gemm_f32(stored(af, ta), stored(bf, tb), g, m, n, k, ta, tb, tc, threads=oracle.max_threads())
    ref_raw = oracle.from_f32(ref, out_code)
    got = run_gemm(stored(araw, ta), stored(braw, tb), code, out_code, ta, tb, tc, variant=variant)
    np.testing.assert_array_equal(got.reshape(ref_raw.shape), ref_raw)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("ta,tb,tc", [(0, 0, 0), (1, 0, 0), (0, 1, 0), (1, 1, 1)])
@pytest.mark.parametrize("g,m,n,k", SHAPES)
def test_int8_gemm_bit_exact(cuda_device, g, m, n, k, ta, tb, tc, variant):
    a = uniform_int8((g, m, k), seed=11)
    b = uniform_int8((g, k, n), seed=12)
    ref = oracle.gemm_i8(stored(a, ta), stored(b, tb), g, m, n, k, ta, tb, tc, threads=oracle.max_threads())
    got = run_gemm(stored(a, ta), stored(b, tb), oracle.I8, oracle.I32, ta, tb, tc, variant=variant)
    verdict, info = oracle.verify_int(got, ref)
    assert verdict == [1, 1, 1], info
    assert info["overflows"] == 0


# K blocks per barrier round (variant bits 28-29: 1, 2, 4 blocks) x tile width x CTA grouping, with a K that leaves
# a partial last round (7 or 13 blocks) and ragged M, N: every configuration must give the same exact result.
@pytest.mark.parametrize("kpr", [1, 2, 3])
@pytest.mark.parametrize("bn", [1, 2, 3])
@pytest.mark.parametrize("ctas", [1, 2])
def test_k_blocks_per_round_configurations_exact(cuda_device, kpr, bn, ctas):
    variant = ctas | (bn << 12) | (kpr << 28)
    g, m, n, k = 2, 300, 200, 64 * 7 + 8
    (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], oracle.F16, seed=1)
    ref = oracle.from_f32(oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads()), oracle.F16)
    got = run_gemm(araw, braw, oracle.F16, oracle.F16, variant=variant)
    np.testing.assert_array_equal(got.reshape(ref.shape), ref)
    k = 128 * 13
    a = uniform_int8((g, m, k), seed=21)
    b = uniform_int8((g, n, k), seed=22)
    refi = oracle.gemm_i8(a, b, g, m, n, k, False, True, False, threads=oracle.max_threads())
    goti = run_gemm(a, b, oracle.I8, oracle.I32, tb=True, variant=variant)
    assert oracle.verify_int(goti, refi)[0] == [1, 1, 1]


# Few output tiles and a long reduction: the library cuts K into ranges (partial planes + fixed-order reduction),
# and narrow N selects the 64- and 128-column tiles. Shapes of the ResNet bwd-weight GEMMs in miniature.
SPLITK_SHAPES = [(1, 64, 576, 8192), (1, 200, 64, 4096), (2, 130, 100, 2048), (1, 576, 64, 6272)]


@pytest.mark.parametrize("ta,tb,tc", [(0, 0, 0), (1, 0, 1), (0, 1, 0)])
@pytest.mark.parametrize("g,m,n,k", SPLITK_SHAPES)
def test_split_k_and_narrow_tiles_exact(cuda_device, g, m, n, k, ta, tb, tc):
    from rocmlir_b200 import _lib as L
    import ctypes as C
    prob = L.RbGemmProblem(g, m, n, k, ta, tb, tc, L.F16, L.F16, 0)
    assert L.lib().rbGemmWorkspaceSize(C.byref(prob)) > 0, "expected a K split (workspace for partial planes)"
    (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], oracle.F16, seed=1)
    ref = oracle.from_f32(oracle.gemm_f32(stored(af, ta), stored(bf, tb), g, m, n, k, ta, tb, tc,
                                          threads=oracle.max_threads()), oracle.F16)
    got = run_gemm(stored(araw, ta), stored(braw, tb), oracle.F16, oracle.F16, ta, tb, tc)
    np.testing.assert_array_equal(got.reshape(ref.shape), ref)
    a = uniform_int8((g, m, k), seed=41)
    b = uniform_int8((g, k, n), seed=42)
    refi = oracle.gemm_i8(stored(a, ta), stored(b, tb), g, m, n, k, ta, tb, tc, threads=oracle.max_threads())
    goti = run_gemm(stored(a, ta), stored(b, tb), oracle.I8, oracle.I32, ta, tb, tc)
    assert oracle.verify_int(goti, refi)[0] == [1, 1, 1]


@pytest.mark.parametrize("code,scale", [(oracle.F16, 0.1), (oracle.BF16, 0.1), (oracle.F32, 1.0)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0)])
def test_float_gemm_normal_data_reference_verifier(cuda_device, code, scale, ta, tb):
    g, m, n, k = 1, 384, 520, 1024
    af, araw = normal_data((g, m, k), code, seed=1, scale=scale)
    bf, braw = normal_data((g, k, n), code, seed=2, scale=scale)
    ref = oracle.gemm_f32(stored(af, ta), stored(bf, tb), g, m, n, k, ta, tb, False, threads=oracle.max_threads())
    ref = oracle.round_to(ref, code)
    got = oracle.to_f32(run_gemm(stored(araw, ta), stored(braw, tb), code, code, ta, tb), code)
    # relDiff is disabled (100) as the reference does for f16 (rocmlir-gen.cpp:2860-2861): summation order differs.
    verdict, info = oracle.verify_float(got, ref, RMS[code], 100.0, 100.0)
    assert verdict == [1, 1, 1], info
    # accuracy against the double-precision oracle: same class as the sequential f32 reference. 16-bit inputs:
    # no worse than it + 1 output ulp. f32 inputs (3xTF32 split, terms below 2^-22 dropped): within 4x of it.
    ref64 = oracle.gemm_f64(stored(af, ta), stored(bf, tb), g, m, n, k, ta, tb, False, threads=oracle.max_threads())
    err_kernel = np.abs(got.astype(np.float64) - ref64).max()
    err_ref = np.abs(ref.astype(np.float64) - ref64).max()
    ulp = {oracle.F32: 2.0 ** -23, oracle.F16: 2.0 ** -10, oracle.BF16: 2.0 ** -7}[code] * np.abs(ref64).max()
    factor = 4.0 if code == oracle.F32 else 1.0
    assert err_kernel <= factor * err_ref + ulp, (err_kernel, err_ref, ulp)


def test_f32_single_pass_tf32_mode_states_its_tolerance(cuda_device):
    """f32_mode = 1 (one TF32 pass) is the fast mode: 10-bit mantissa inputs -> RMS 1e-3 class, not fp32 class."""
    g, m, n, k = 1, 256, 256, 576
    af, araw = normal_data((g, m, k), oracle.F32, seed=3, scale=1.0)
    bf, braw = normal_data((g, k, n), oracle.F32, seed=4, scale=1.0)
    ref = oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads())
    got = run_gemm(araw, braw, oracle.F32, oracle.F32, f32_mode=1)
    verdict, info = oracle.verify_float(got, ref, 1e-3, 100.0, 100.0)
    assert verdict == [1, 1, 1], info
    got3 = run_gemm(araw, braw, oracle.F32, oracle.F32, f32_mode=0)
    _, info3 = oracle.verify_float(got3, ref, 3e-5, 100.0, 100.0)
    assert info3["rms"] < info["rms"] / 50, (info3, info)


def test_fp16_gemm_bias_relu_epilogue_matches_op_by_op_oracle(cuda_device):
    """C' = relu(C + bias[N]) in f16 (BASELINE config 2): the dot result is rounded to f16 first, the add is an
    f16 add, as the MIGraphX form dot -> add -> relu computes it (MIGraphXToTosa.cpp:1009-1018)."""
    import torch
    from rocmlir_b200.gemm import Epilogue
    g, m, n, k = 1, 256, 512, 512
    af, araw = normal_data((g, m, k), oracle.F16, seed=5, scale=0.1)
    bf, braw = normal_data((g, k, n), oracle.F16, seed=6, scale=0.1)
    biasf, biasraw = normal_data((n,), oracle.F16, seed=7, scale=0.1)
    acc = oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads())
    ref = oracle.epilogue(acc, n, bias=biasf, relu=True, mid_type=oracle.F16)
    epi = Epilogue(bias=to_device(biasraw, oracle.F16), relu=True, mid_type=oracle.F16)
    got = oracle.to_f32(run_gemm(araw, braw, oracle.F16, oracle.F16, epilogue=epi), oracle.F16)
    verdict, info = oracle.verify_float(got, oracle.round_to(ref, oracle.F16), 1e-3, 100.0, 100.0)
    assert verdict == [1, 1, 1], info
    assert (got >= 0).all()
    # same epilogue on integer-valued data: exact
    (ai, airaw), (bi, biraw) = reference_random([(g, m, k), (g, k, n)], oracle.F16, seed=1)
    bint = np.arange(n, dtype=np.float32) % 7 - 3
    acc = oracle.gemm_f32(ai, bi, g, m, n, k, threads=oracle.max_threads())
    ref = oracle.from_f32(oracle.epilogue(acc, n, bias=bint, relu=True, mid_type=oracle.F16), oracle.F16)
    epi = Epilogue(bias=to_device(oracle.from_f32(bint, oracle.F16), oracle.F16), relu=True, mid_type=oracle.F16)
    got = run_gemm(airaw, biraw, oracle.F16, oracle.F16, epilogue=epi)
    np.testing.assert_array_equal(got.reshape(ref.shape), ref)


@pytest.mark.parametrize("variant", [1, 2])
def test_int8_dequant_requant_epilogue_bit_exact(cuda_device, variant):
    """acc:i32 -> f32 -> x s_col[n] -> x (1/s_out) -> round-half-even -> saturate -> i8 (BASELINE config 3):
    quant_dot -> dequantizelinear -> quantizelinear (MIGraphXToTosa.cpp:876-982)."""
    from rocmlir_b200.gemm import Epilogue
    g, m, n, k = 1, 256, 768, 1024
    a = uniform_int8((g, m, k), seed=21)
    b = uniform_int8((g, n, k), seed=22)          # LLM-linear weight [out, in]: transB
    s_col = uniform_f32((n,), seed=23, lo=0.001, hi=0.01)
    acc = oracle.gemm_i8(a, b, g, m, n, k, tb=True, threads=oracle.max_threads())
    deq = oracle.epilogue(acc, n, col_scale=s_col)
    s_out = float(np.float32(np.quantile(np.abs(deq), 0.99) / 127.0))  # about 1 % of the outputs saturate
    ref = oracle.from_f32(oracle.epilogue(acc, n, col_scale=s_col, requant_scale=s_out), oracle.I8, sat_int=True)
    assert 0.001 < np.mean(np.abs(ref.astype(np.int32)) >= 127) < 0.05
    epi = Epilogue(col_scale=to_device(s_col, oracle.F32), requant_scale=s_out)
    got = run_gemm(a, b, oracle.I8, oracle.I8, tb=True, epilogue=epi, variant=variant)
    np.testing.assert_array_equal(got.reshape(ref.shape), ref)


def test_fp8_gemm_per_tensor_scales_bf16_out(cuda_device):
    """fp8-e4m3 x fp8-e4m3, f32 accumulate, x (sA*sB), bf16 out (BASELINE config 3, fp8 variant)."""
    from rocmlir_b200.gemm import Epilogue
    g, m, n, k = 1, 256, 512, 1024
    xa = normal_data((g, m, k), oracle.F32, seed=31, scale=1.0)[0]
    xb = normal_data((g, n, k), oracle.F32, seed=32, scale=1.0)[0]
    sa = np.float32(np.abs(xa).max() / 448.0)
    sb = np.float32(np.abs(xb).max() / 448.0)
    araw = oracle.from_f32(xa / sa, oracle.F8E4M3)
    braw = oracle.from_f32(xb / sb, oracle.F8E4M3)
    af, bf = oracle.to_f32(araw, oracle.F8E4M3), oracle.to_f32(braw, oracle.F8E4M3)
    alpha = np.float32(sa * sb)
    acc = oracle.gemm_f32(af, bf, g, m, n, k, tb=True, threads=oracle.max_threads())
    ref = oracle.round_to(oracle.epilogue(acc, n, alpha=alpha), oracle.BF16)
    got = oracle.to_f32(run_gemm(araw, braw, oracle.F8E4M3, oracle.BF16, tb=True, epilogue=Epilogue(alpha=float(alpha))),
                        oracle.BF16)
    verdict, info = oracle.verify_float(got, ref, RMS[oracle.F8E4M3], 100.0, 100.0)
    assert verdict == [1, 1, 1], info


def test_fp16_gemm_4096_cubed_sampled_rows_and_linearity(cuda_device):
    """BASELINE config 2 at full size: the oracle is evaluated on a seeded sample of rows (the full
    sequential reference would take minutes), plus size-independent properties on the whole result."""
    import torch
    m = n = k = 4096
    af, araw = normal_data((1, m, k), oracle.F16, seed=1, scale=0.1)
    bf, braw = normal_data((1, k, n), oracle.F16, seed=2, scale=0.1)
    got_raw = run_gemm(araw, braw, oracle.F16, oracle.F16)
    got = oracle.to_f32(got_raw, oracle.F16).reshape(m, n)
    rows = np.random.Generator(np.random.PCG64(3)).choice(m, size=24, replace=False)
    ref = oracle.round_to(oracle.gemm_f32(af[:, rows, :], bf, 1, len(rows), n, k, threads=oracle.max_threads()), oracle.F16)
    verdict, info = oracle.verify_float(got[rows], ref, RMS[oracle.F16], 100.0, 100.0)
    assert verdict == [1, 1, 1], info
    # determinism: a second run is bitwise identical (no races on shared memory / TMEM)
    again = run_gemm(araw, braw, oracle.F16, oracle.F16)
    np.testing.assert_array_equal(again, got_raw)
    # column checksum: sum_m C[m,n] == (sum_m A[m,:]) . B[:,n] within f16 output rounding
    colsum_ref = af[0].astype(np.float64).sum(0) @ bf[0].astype(np.float64)
    colsum = got.astype(np.float64).sum(0)
    tol = 4096 * 2.0 ** -11 * np.abs(got).max()
    assert np.abs(colsum - colsum_ref).max() < tol


@pytest.mark.parametrize("m,k1,n1,n2", [(256, 192, 320, 128), (4096, 1024, 1024, 1024),
                                        # k1, n2 <= 128: one launch, intermediate on the SM (attention skeleton)
                                        (256, 64, 320, 128), (4096, 128, 1024, 128), (300, 72, 200, 40), (96, 128, 128, 64)])
def test_gemm_gemm_matches_oracle(cuda_device, m, k1, n1, n2):
    """O = (A.B1).B2, intermediate rounded to f16 (BASELINE config 5b at full size: M 4096, K1 = N1 = N2 = 1024).
    The full-size oracle is evaluated on a seeded sample of rows (rows are independent)."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import gemm_gemm
    af, araw = normal_data((m, k1), oracle.F16, seed=51, scale=0.1)
    b1f, b1raw = normal_data((k1, n1), oracle.F16, seed=52, scale=0.1)
    b2f, b2raw = normal_data((n1, n2), oracle.F16, seed=53, scale=0.1)
    out = gemm_gemm(to_device(araw, oracle.F16), to_device(b1raw, oracle.F16), to_device(b2raw, oracle.F16))
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    got = oracle.to_f32(from_device(out, oracle.F16), oracle.F16)
    rows = np.arange(m) if m <= 256 else np.random.Generator(np.random.PCG64(5)).choice(m, 64, replace=False)
    ref = oracle.round_to(oracle.gemm_gemm(af[rows], b1f, b2f, oracle.F16, threads=oracle.max_threads()), oracle.F16)
    verdict, info = oracle.verify_float(got[rows], ref, 1e-3, 100.0, 1e30)
    assert verdict == [1, 1, 1], info


def test_gemm_gemm_on_chip_equals_two_launches(cuda_device):
    """Batched bf16 GEMM+GEMM of attention-like extents: the one-launch form (intermediate in tensor memory) against
    the two-launch form (variant bit 27) on the same inputs - both round the intermediate to bf16 - and the launch count."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import gemm_gemm
    g, m, k1, n1, n2 = 3, 640, 128, 896, 128
    gen = torch.Generator(device="cuda").manual_seed(77)
    a = (torch.randn((g, m, k1), device="cuda", generator=gen) * 0.1).bfloat16()
    b1 = (torch.randn((g, k1, n1), device="cuda", generator=gen) * 0.1).bfloat16()
    b2 = (torch.randn((g, n1, n2), device="cuda", generator=gen) * 0.1).bfloat16()
    lib = L.lib()
    n0 = L.launch_count()
    fused = gemm_gemm(a, b1, b2)
    torch.cuda.synchronize()
    assert L.launch_count() - n0 == 1
    lib.rbSetGemmVariant(1 << 27)
    try:
        plain = gemm_gemm(a, b1, b2)
        torch.cuda.synchronize()
    finally:
        lib.rbSetGemmVariant(0)
    assert L.kernel_status() == 0
    ref = (a.float() @ b1.float()).bfloat16().float() @ b2.float()
    scale = ref.abs().max().item()
    assert (fused.float() - ref).abs().max().item() <= 2.0 ** -7 * scale
    assert (fused.float() - plain.float()).abs().max().item() <= 2.0 ** -7 * scale


@pytest.mark.parametrize("variant", [0, 1 | (3 << 12), 2 | (3 << 12), 1 | (2 << 12), 1 | (1 << 12)])
@pytest.mark.parametrize("m,k,dtype", [(4096, 1024, "float16"), (1000, 512, "bfloat16"), (300, 192, "float16"),
                                       (2304, 320, "float16")])
def test_gemm_gemm_chained_launch_equals_two_launches(cuda_device, m, k, dtype, variant):
    """k1 = n1 = n2: one launch of the GEMM kernel over two groups, the second reading the first one's result as its
    tiles' row blocks complete - bit for bit the two-launch form (variant bit 27), with either tensor of each operand
    at the lower address (the group coordinate of the tensor maps flips), for every tile shape."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import gemm_gemm
    dt = getattr(torch, dtype)
    gen = torch.Generator(device="cuda").manual_seed(m + k)
    lib = L.lib()
    for ws_first in (False, True):
        ws = torch.empty(32 << 20, dtype=torch.uint8, device="cuda") if ws_first else None
        a = (torch.randn((m, k), device="cuda", generator=gen) * 0.1).to(dt)
        bx = (torch.randn((k, k), device="cuda", generator=gen) * 0.1).to(dt)
        by = (torch.randn((k, k), device="cuda", generator=gen) * 0.1).to(dt)
        b1, b2 = (by, bx) if ws_first else (bx, by)
        o = torch.zeros((m, k), device="cuda", dtype=dt)
        if ws is None:
            ws = torch.empty(32 << 20, dtype=torch.uint8, device="cuda")
        try:
            lib.rbSetGemmVariant(variant)
            n0 = L.launch_count()
            chained = gemm_gemm(a, b1, b2, out=o, workspace=ws).clone()
            torch.cuda.synchronize()
            assert L.launch_count() - n0 == 1
            lib.rbSetGemmVariant(variant | (1 << 27))
            plain = gemm_gemm(a, b1, b2, out=o, workspace=ws)
            torch.cuda.synchronize()
        finally:
            lib.rbSetGemmVariant(0)
        assert L.kernel_status() == 0
        assert torch.equal(chained, plain)
        ref = (a.float() @ b1.float()).to(dt).float() @ b2.float()
        assert (chained.float() - ref).abs().max().item() <= 2.0 ** -6 * ref.abs().max().item()


@pytest.mark.parametrize("code,shape", [(oracle.F16, (1, 2304, 2560, 1024)), (oracle.I8, (1, 1300, 3000, 2048)),
                                        (oracle.F16, (2, 1200, 1100, 640))])
@pytest.mark.parametrize("ctas", [1, 2])
def test_stream_k_tail_exact(cuda_device, code, shape, ctas):
    """Opt-in stream-K tail (variant bit 9): tiles of the last waves are dealt out by K blocks, partial tiles are
    summed by the owning CTA in unit order. Integer-valued data: must equal the oracle (and the plain schedule) exactly."""
    import ctypes as C
    from rocmlir_b200 import _lib as L
    g, m, n, k = shape
    variant = 0x200 | ctas
    L.lib().rbSetGemmVariant(variant)
    prob = L.RbGemmProblem(g, m, n, k, 0, 0, 0, code, oracle.I32 if code == oracle.I8 else code, 0)
    assert L.lib().rbGemmWorkspaceSize(C.byref(prob)) > 0, "the shape must trigger the stream-K tail"
    L.lib().rbSetGemmVariant(0)
    if code == oracle.I8:
        a = uniform_int8((g, m, k), seed=61)
        b = uniform_int8((g, k, n), seed=62)
        ref = oracle.gemm_i8(a, b, g, m, n, k, threads=oracle.max_threads())
        got = run_gemm(a, b, oracle.I8, oracle.I32, variant=variant)
        assert oracle.verify_int(got, ref)[0] == [1, 1, 1]
    else:
        (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], code, seed=1)
        ref = oracle.from_f32(oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads()), code)
        got = run_gemm(araw, braw, code, code, variant=variant)
        np.testing.assert_array_equal(got.reshape(ref.shape), ref)
