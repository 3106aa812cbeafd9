"""GPU parity tests of rbAttention against the CPU oracle.

Two oracles (oracle.attention): the faithful one evaluates every op in the element type like the reference's
generated CPU attention (rocmlir-gen.cpp:2507-2638) and is judged with the thresholds of the reference's own f16
attention suite, -absDiff 0.02 -RMS 0.015 (mlir/test/e2e/PrAttentionF16.toml:3; relDiff is forced to 100 for f16,
rocmlir-gen.cpp:2860-2861 - here it is switched off outright, because N(0,1) data put references arbitrarily close to 0);
the double-precision one bounds the kernel's true error far more tightly.
"""
import math

import numpy as np
import pytest

import oracle
from helpers import from_device, normal_data, to_device

pytestmark = pytest.mark.gpu


def run_attention(qraw, kraw, vraw, code, **kw):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.attention import attention
    bias = kw.pop("bias_raw", None)
    mask = kw.pop("mask", None)
    if bias is not None:
        kw["bias"] = to_device(bias, code)
    if mask is not None:
        kw["mask"] = torch.from_numpy(mask).cuda()
    o = attention(to_device(qraw, code), to_device(kraw, code), to_device(vraw, code), **kw)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return oracle.to_f32(from_device(o, code), code)


def make_qkv(g, sq, sk, d, dv, code, seed=1):
    q, qraw = normal_data((g, sq, d), code, seed, 1.0)
    k, kraw = normal_data((g, d, sk), code, seed + 1, 1.0)
    v, vraw = normal_data((g, sk, dv), code, seed + 2, 1.0)
    return (q, qraw), (k, kraw), (v, vraw)


# shapes of the reference's PR attention suite (PrAttentionF16.toml:19-66): seq 64..384, head 64 / 128, plus ragged
# sequence lengths (tails of the 128-row / 128-key tiles)
SHAPES = [(2, 384, 384, 64, 64), (3, 128, 256, 128, 128), (1, 64, 64, 64, 64), (2, 100, 200, 128, 64),
          (1, 256, 128, 64, 128), (1, 257, 136, 128, 128),
          # head dimensions that are not 64 / 128 (rocmlir-gen's -p default is 32, rocmlir-gen.cpp:1018-1020)
          (2, 384, 256, 32, 32), (1, 200, 136, 96, 40), (1, 130, 264, 72, 128)]


@pytest.mark.parametrize("code", [oracle.F16, oracle.BF16])
@pytest.mark.parametrize("g,sq,sk,d,dv", SHAPES)
def test_attention_with_scale_both_oracles(cuda_device, g, sq, sk, d, dv, code):
    (q, qraw), (k, kraw), (v, vraw) = make_qkv(g, sq, sk, d, dv, code)
    scale = 1.0 / math.sqrt(d)
    got = run_attention(qraw, kraw, vraw, code, scale=scale)
    ref64 = oracle.attention(q, k, v, elem_type=oracle.F64, scale_scalar=scale, threads=oracle.max_threads())
    # kernel error: P and O carry one rounding to the element type each (2^-11 f16, 2^-8 bf16, relative)
    ulp = 2.0 ** -10 if code == oracle.F16 else 2.0 ** -7
    err = np.abs(got - ref64).max()
    assert err <= 2.0 * ulp * max(1.0, np.abs(ref64).max()), err
    verdict, info = oracle.verify_float(got, ref64, 1e-3 if code == oracle.F16 else 8e-3, 100.0, 1e30)
    assert verdict == [1, 1, 1], info
    if code == oracle.F16:
        faithful = oracle.attention(q, k, v, elem_type=oracle.F16, scale_scalar=oracle.round_to(np.float32([scale]), code)[0],
                                    threads=oracle.max_threads())
        verdict, info = oracle.verify_float(got, faithful, 0.015, 0.02, 1e30)
        assert verdict == [1, 1, 1], info


def test_trans_k_matches_default_layout(cuda_device):
    g, sq, sk, d, dv = 2, 256, 384, 128, 128
    (q, qraw), (k, kraw), (v, vraw) = make_qkv(g, sq, sk, d, dv, oracle.F16)
    a = run_attention(qraw, kraw, vraw, oracle.F16, scale=0.1)
    b = run_attention(qraw, np.ascontiguousarray(np.swapaxes(kraw, 1, 2)), vraw, oracle.F16, scale=0.1, trans_k=True)
    np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("sq,sk", [(384, 384), (200, 200)])
def test_causal_equals_mask_tensor_form_and_oracle(cuda_device, sq, sk):
    """The analytic causal path must agree bit for bit with the reference's own way of masking,
    where(mask_i8, s, -inf) with a lower-triangular mask tensor (test/fusion/pr-e2e/attention/mixr-attn-where.mlir)."""
    g, d, dv = 2, 128, 128
    (q, qraw), (k, kraw), (v, vraw) = make_qkv(g, sq, sk, d, dv, oracle.F16, seed=5)
    scale = 1.0 / math.sqrt(d)
    causal = run_attention(qraw, kraw, vraw, oracle.F16, scale=scale, causal=True)
    mask = np.broadcast_to(np.tril(np.ones((sq, sk), np.int8)), (g, sq, sk)).copy()
    masked = run_attention(qraw, kraw, vraw, oracle.F16, scale=scale, mask=mask, mask_fill=float("-inf"))
    np.testing.assert_array_equal(causal, masked)
    ref64 = oracle.attention(q, k, v, elem_type=oracle.F64, scale_scalar=scale, causal=True, threads=oracle.max_threads())
    verdict, info = oracle.verify_float(causal, ref64, 1e-3, 100.0, 1e30)
    assert verdict == [1, 1, 1], info
    ref_mask = oracle.attention(q, k, v, elem_type=oracle.F64, scale_scalar=scale, mask=mask, mask_fill=float("-inf"),
                                threads=oracle.max_threads())
    np.testing.assert_allclose(ref64, ref_mask, rtol=0, atol=0)


def test_bias_and_finite_mask_fill(cuda_device):
    g, sq, sk, d, dv = 2, 128, 256, 64, 64
    (q, qraw), (k, kraw), (v, vraw) = make_qkv(g, sq, sk, d, dv, oracle.F16, seed=9)
    bias, braw = normal_data((g, sq, sk), oracle.F16, 11, 0.5)
    rng = np.random.Generator(np.random.PCG64(12))
    mask = (rng.random((g, sq, sk)) > 0.3).astype(np.int8)
    scale = 0.125
    got = run_attention(qraw, kraw, vraw, oracle.F16, scale=scale, bias_raw=braw, mask=mask, mask_fill=-1000.0)
    ref64 = oracle.attention(q, k, v, elem_type=oracle.F64, scale_scalar=scale, bias=bias, mask=mask, mask_fill=-1000.0,
                             threads=oracle.max_threads())
    verdict, info = oracle.verify_float(got, ref64, 1e-3, 100.0, 1e30)
    assert verdict == [1, 1, 1], info


@pytest.mark.parametrize("causal", [False, True])
def test_headline_size_sampled_groups(cuda_device, causal):
    """BASELINE config 5 at full size (batch 16 x 32 heads = 512 groups, S = 2048, D = 128, Q/K/V ~ N(0,1)); groups are
    independent, so the double-precision oracle is evaluated on two seeded groups and compared with the same groups
    of the full result. Reduced to 64 groups of inputs (repeated) would change nothing: all 512 are computed."""
    g, s, d = 512, 2048, 128
    (q, qraw), (k, kraw), (v, vraw) = make_qkv(g, s, s, d, d, oracle.F16, seed=1)
    scale = 1.0 / math.sqrt(d)
    got = run_attention(qraw, kraw, vraw, oracle.F16, scale=scale, causal=causal)
    for grp in (0, 377):
        ref = oracle.attention(q[grp:grp + 1], k[grp:grp + 1], v[grp:grp + 1], elem_type=oracle.F64, scale_scalar=scale,
                               causal=causal, threads=oracle.max_threads())
        verdict, info = oracle.verify_float(got[grp], ref[0], 1e-3, 100.0, 1e30)
        assert verdict == [1, 1, 1], (grp, info)
        assert np.abs(got[grp] - ref[0]).max() < 4e-3


@pytest.mark.parametrize("trans_k", [False, True])
@pytest.mark.parametrize("with_side", [False, True])
def test_first_gemm_quantised_attention(cuda_device, trans_k, with_side):
    """rocmlir-gen -t i8: Q and K int8, (i32(Q.K) - quant_bias) -> f16, * quant_scale, then the f16 chain. Judged
    like the reference judges an f16 result by default (RMS 1e-3) against the oracle that rounds every step to f16."""
    import torch
    from rocmlir_b200.attention import attention
    g, sq, sk, d, dv = 2, 200, 136, 64, 64
    rng = np.random.default_rng(7)
    q = rng.integers(-5, 5, (g, sq, d)).astype(np.int8)
    k = rng.integers(-5, 5, (g, d, sk)).astype(np.int8)
    v = oracle.round_to((rng.standard_normal((g, sk, dv))).astype(np.float32), oracle.F16)
    qb, qs = 3, oracle.round_to(np.float32([0.0625]), oracle.F16)[0]
    sc = bi = None
    if with_side:
        sc = oracle.round_to(rng.uniform(0.5, 1.5, (g, sq, sk)).astype(np.float32), oracle.F16)
        bi = oracle.round_to(rng.standard_normal((g, sq, sk)).astype(np.float32), oracle.F16)
    want = oracle.attention_i8(q, k, v, qb, float(qs), scale=sc, bias=bi, threads=oracle.max_threads())
    kd = np.ascontiguousarray(k.transpose(0, 2, 1)) if trans_k else k
    dev = lambda a, t: torch.from_numpy(np.ascontiguousarray(a)).to("cuda").to(t)
    o = attention(dev(q, torch.int8), dev(kd, torch.int8), dev(v, torch.float16), trans_k=trans_k,
                  quant_bias=dev(np.int8([qb]), torch.int8), quant_scale=dev(np.float32([qs]), torch.float16),
                  scale_tensor=None if sc is None else dev(sc, torch.float16),
                  bias=None if bi is None else dev(bi, torch.float16))
    torch.cuda.synchronize()
    got = o.float().cpu().numpy()
    verdict, info = oracle.verify_float(got, oracle.round_to(want, oracle.F16), 1e-3, 100.0, 100.0)
    assert verdict == [1, 1, 1], info


@pytest.mark.parametrize("tq,tk,tv,to", [(True, False, False, False), (False, True, True, False),
                                         (False, False, False, True), (True, True, True, True)])
def test_transposed_operand_forms(cuda_device, tq, tk, tv, to):
    """rocmlir-gen's -transQ / -transK / -transV / -transO (rocmlir-gen.cpp:2149-2200): the same operation on operands
    stored transposed must give the same bits as on the plain ones, and so must K stored G x D x Sk with Sk = 27,
    whose rows do not start on 16-byte boundaries."""
    import torch
    from rocmlir_b200.attention import attention
    g, sq, sk, d, dv = 2, 150, 27, 64, 32
    (q, qraw), (k, kraw), (v, vraw) = make_qkv(g, sq, sk, d, dv, oracle.F16)
    from helpers import to_device
    dev = lambda a: to_device(np.ascontiguousarray(a), oracle.F16)
    scale = 1.0 / math.sqrt(d)
    base = attention(dev(qraw), dev(kraw.transpose(0, 2, 1)), dev(vraw), trans_k=True, scale=scale)   # K [G,Sk,D]
    got = attention(dev(qraw.transpose(0, 2, 1)) if tq else dev(qraw),
                    dev(kraw.transpose(0, 2, 1)) if tk else dev(kraw),
                    dev(vraw.transpose(0, 2, 1)) if tv else dev(vraw),
                    trans_q=tq, trans_k=tk, trans_v=tv, trans_o=to, scale=scale)
    torch.cuda.synchronize()
    if to:
        got = got.transpose(1, 2)
    assert torch.equal(got.contiguous(), base)
    ref64 = oracle.attention(q, k, v, elem_type=oracle.F64, scale_scalar=scale, threads=oracle.max_threads())
    assert np.abs(base.float().cpu().numpy() - ref64).max() <= 2.0 ** -9 * max(1.0, np.abs(ref64).max())


@pytest.mark.parametrize("g,sq,sk,d,dv", [(2, 384, 384, 64, 64), (1, 128, 27, 64, 32), (2, 77, 200, 40, 24)])
def test_f32_attention_unfused(cuda_device, g, sq, sk, d, dv):
    """-t f32: two 3xTF32 GEMMs around a row softmax. On the reference's -rand 1 integer data the scores are exact, and
    the result must pass the reference verifier at the thresholds of its f32 PR suite (RMS 3e-5 default, relDiff 5e-6:
    PrAttentionF32.toml:3); with scale and bias tensors as well."""
    import torch
    from rocmlir_b200.attention import attention
    from helpers import reference_random
    (q, _), (k, _), (v, _), (sc, _), (bi, _) = reference_random([(g, sq, d), (g, d, sk), (g, sk, dv), (g, sq, sk),
                                                                  (g, sq, sk)], oracle.F32, seed=1)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to("cuda")
    for side in (False, True):
        want = oracle.attention(q, k, v, elem_type=oracle.F32, scale=sc if side else None, bias=bi if side else None,
                                threads=oracle.max_threads())
        got = attention(dev(q), dev(k), dev(v), scale_tensor=dev(sc) if side else None, bias=dev(bi) if side else None)
        torch.cuda.synchronize()
        verdict, info = oracle.verify_float(got.cpu().numpy(), want, 3e-5, 100.0, 5e-6)
        assert verdict == [1, 1, 1], info
    # a scalar scale and the analytic causal mask against the float64 oracle
    qn, kn, vn = (np.random.default_rng(s).standard_normal(x.shape).astype(np.float32) for s, x in ((1, q), (2, k), (3, v)))
    ref64 = oracle.attention(qn, kn, vn, elem_type=oracle.F64, scale_scalar=0.125, causal=True, threads=oracle.max_threads())
    got = attention(dev(qn), dev(kn), dev(vn), scale=0.125, causal=True).cpu().numpy()
    assert np.abs(got - ref64).max() <= 2e-5 * max(1.0, np.abs(ref64).max())


def test_negative_scale_takes_the_general_kernel_and_matches_the_oracle(cuda_device):
    """A negative scale cannot be folded into the row maximum: the call must still be right (it runs the one-tile
    kernel), and a problem without a scale must not be dispatched on whatever its unused `scale` field holds."""
    import ctypes as C
    import torch
    from rocmlir_b200 import _lib as L
    g, sq, sk, d, dv = 2, 300, 264, 64, 64
    (q, qraw), (k, kraw), (v, vraw) = make_qkv(g, sq, sk, d, dv, oracle.F16)
    got = run_attention(qraw, kraw, vraw, oracle.F16, scale=-0.125)
    ref64 = oracle.attention(q, k, v, elem_type=oracle.F64, scale_scalar=-0.125, threads=oracle.max_threads())
    verdict, info = oracle.verify_float(got, ref64, 1e-3, 100.0, 1e30)
    assert verdict == [1, 1, 1], info
    # has_scale = 0 with a garbage negative `scale` field: same result as the clean call
    tq, tk, tv = to_device(qraw, oracle.F16), to_device(kraw, oracle.F16), to_device(vraw, oracle.F16)
    outs = []
    for junk in (0.0, -7.0):
        o = torch.empty((g, sq, dv), dtype=torch.float16, device="cuda")
        p = L.RbAttentionProblem(g, sq, sk, d, dv, 0, 0, 0, 0, L.F16, 0, junk, 0, 0.0, None, None, None, None, None)
        L.check(L.lib().rbAttention(C.byref(p), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        outs.append(o)
    assert torch.equal(outs[0], outs[1])


def test_caller_workspace_entry_point_equals_thread_scratch_entry_point(cuda_device):
    """rbAttentionWs (scratch from the caller, nothing allocated) and rbAttention (scratch owned by the calling
    thread) run the same kernels: identical results on a form that stages three operands (transposed Q, V and O)."""
    import ctypes as C
    import torch
    from rocmlir_b200 import _lib as L
    g, sq, sk, d, dv = 2, 200, 136, 64, 64
    (q, qraw), (k, kraw), (v, vraw) = make_qkv(g, sq, sk, d, dv, oracle.F16)
    tq = to_device(np.ascontiguousarray(np.swapaxes(qraw, 1, 2)), oracle.F16)
    tv = to_device(np.ascontiguousarray(np.swapaxes(vraw, 1, 2)), oracle.F16)
    tk = to_device(kraw, oracle.F16)
    p = L.RbAttentionProblem(g, sq, sk, d, dv, 1, 0, 1, 1, L.F16, 1, 0.125, 0, 0.0, None, None, None, None, None)
    need = L.lib().rbAttentionWorkspaceSize(C.byref(p))
    assert need >= 2 * (g * sq * d + g * sk * dv + g * sq * dv)
    stream = torch.cuda.current_stream().cuda_stream
    o1 = torch.zeros((g, dv, sq), dtype=torch.float16, device="cuda")
    o2 = torch.zeros((g, dv, sq), dtype=torch.float16, device="cuda")
    st = L.lib().rbAttentionWs(C.byref(p), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o1.data_ptr(), None, 0, stream)
    assert st == L.WORKSPACE_TOO_SMALL and str(need) in L.lib().rbGetLastError().decode()
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    L.check(L.lib().rbAttentionWs(C.byref(p), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o1.data_ptr(), ws.data_ptr(), need, stream))
    L.check(L.lib().rbAttention(C.byref(p), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o2.data_ptr(), stream))
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    assert torch.equal(o1, o2)
    ref64 = oracle.attention(q, k, v, elem_type=oracle.F64, scale_scalar=0.125, threads=oracle.max_threads())
    got = oracle.to_f32(from_device(o1, oracle.F16), oracle.F16).reshape(g, dv, sq).swapaxes(1, 2)
    verdict, info = oracle.verify_float(got, ref64, 1e-3, 100.0, 1e30)
    assert verdict == [1, 1, 1], info
