"""The oracle's 8-bit float conversions against an independent implementation (torch's CPU casts): decoding of all
256 codes, and encoding (round-to-nearest-even) of in-range values; out-of-range values saturate, which is where
the reference's truncation (saturateFP8Truncf, mlir/lib/Dialect/Rock/Pipelines/Pipelines.cpp:238) and torch's
IEEE-style cast differ by design."""
import numpy as np
import pytest
import torch

import oracle

CASES = [(oracle.F8E4M3, torch.float8_e4m3fn, 448.0), (oracle.F8E5M2, torch.float8_e5m2, 57344.0)]


@pytest.mark.parametrize("code,tdt,maxv", CASES)
def test_decode_all_codes(code, tdt, maxv):
    raw = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(raw.copy()).view(tdt).float().numpy()
    got = oracle.to_f32(raw, code)
    finite = np.isfinite(want)
    np.testing.assert_array_equal(got[finite], want[finite])
    assert np.isnan(got[np.isnan(want)]).all()


@pytest.mark.parametrize("code,tdt,maxv", CASES)
def test_encode_round_to_nearest_even_and_saturate(code, tdt, maxv):
    rng = np.random.Generator(np.random.PCG64(5))
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-4, 1e-2, 1.0, 30.0)])
    x = x[np.abs(x) < maxv * 0.95]
    # every exact tie between neighbouring codes, too
    codes = oracle.to_f32(np.arange(256, dtype=np.uint8), code)
    pos = np.sort(codes[np.isfinite(codes) & (codes >= 0)])
    ties = ((pos[:-1] + pos[1:]) / 2).astype(np.float32)
    x = np.concatenate([x, ties, -ties]).astype(np.float32)
    want = torch.from_numpy(x).to(tdt).view(torch.uint8).numpy()
    got = oracle.from_f32(x, code)
    np.testing.assert_array_equal(got & 0x7f, want & 0x7f)          # magnitude bits (the sign of zero may differ)
    big = np.array([maxv, maxv * 1.5, 1e30, np.inf, -maxv * 2], np.float32)
    sat = oracle.to_f32(oracle.from_f32(big, code), code)
    np.testing.assert_array_equal(sat, np.array([maxv, maxv, maxv, maxv, -maxv], np.float32))


def test_quantised_attention_oracle_reduces_to_the_f16_one():
    """With a zero quantisation bias, scale 1 and scores small enough to be exact in f16 (|sum| <= 16 * 25), the
    first-GEMM-quantised oracle must agree bit for bit with the f16 oracle, which the reference's attention
    structure test pins (mlir/test/rocmlir-gen/attention-kernel.mlir); and the bias / scale enter as
    f16((s - b)) * qs."""
    import oracle
    rng = np.random.default_rng(11)
    g, sq, sk, d, dv = 2, 9, 13, 16, 8
    q = rng.integers(-5, 5, (g, sq, d)).astype(np.int8)
    k = rng.integers(-5, 5, (g, d, sk)).astype(np.int8)
    v = oracle.round_to(rng.standard_normal((g, sk, dv)).astype(np.float32), oracle.F16)
    a = oracle.attention_i8(q, k, v, 0, 1.0)
    b = oracle.attention(q.astype(np.float32), k.astype(np.float32), v, elem_type=oracle.F16)
    np.testing.assert_array_equal(a, b)
    # (s - 3) * 0.5 == the f16 oracle on pre-shifted scores expressed through a bias tensor and a scalar scale
    s = np.einsum("gid,gdj->gij", q.astype(np.int32), k.astype(np.int32))
    shifted = oracle.round_to(oracle.round_to((s - 3).astype(np.float32), oracle.F16) * np.float32(0.5), oracle.F16)
    c = oracle.attention_i8(q, k, v, 3, 0.5)
    # same softmax input => same result as feeding `shifted` as a bias over zero scores
    zq = np.zeros((g, sq, d), np.float32)
    e = oracle.attention(zq, k.astype(np.float32), v, elem_type=oracle.F16, bias=shifted)
    np.testing.assert_array_equal(c, e)
