"""Pins the oracle's attention and GEMM functions on the op sequences the reference itself holds.

The reference's CPU validator is a generated program; its lit tests keep that program's structure as FileCheck lines
(mlir/test/rocmlir-gen/attention-kernel.mlir, `@host_naive_attention`; mlir/test/rocmlir-gen/gemm-kernel.mlir,
`@host_naive_gemm`). tests/golden/make_validator_structure.py turns those lines into tests/golden/
validator_structure.json, and this file EXECUTES that description with numpy - every op typed with the element type,
tosa.matmul and tosa.reduce_sum accumulating in that type with the reduction index ascending (the lowering the
reference uses, external/llvm-project/mlir/lib/Conversion/TosaToLinalg/TosaToLinalgNamed.cpp:645-657) - and compares
with oracle.attention / oracle.gemm_f32 on seeded data. The oracle is thereby tied to the reference's op order and
typing, not only to a reading of the generator's source.

Bars: GEMM bit-exact. Attention bit-exact up to the exponential, whose last bit differs between libm (the oracle) and
numpy: results agree within 2 units in the last place of the element type (taken at the magnitude of the output
row) on every element and are identical on most; a control that accumulates in a wider type instead is measurably
further away.
"""
import json
import os

import numpy as np
import pytest

import oracle

FIX = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "validator_structure.json")))
NP_T = {"f32": np.float32, "f16": np.float16}
ORC_T = {"f32": oracle.F32, "f16": oracle.F16}


def test_fixture_holds_the_reference_op_sequence():
    scale, plain = FIX["cases"]
    assert [o["op"].split(".")[1] for o in scale["ops"]] == ["matmul", "mul", "reduce_max", "sub", "exp", "reduce_sum",
                                                             "reciprocal", "mul", "matmul"]
    assert [o["op"].split(".")[1] for o in plain["ops"]] == ["matmul", "reduce_max", "sub", "exp", "reduce_sum",
                                                             "reciprocal", "mul", "matmul"]
    # every op works on the score matrix or its row reduction: nothing widens on the way
    for case in FIX["cases"]:
        assert case["element_type"] == "f32"
        for o in case["ops"][1:-1]:
            assert set(o["operand_shapes"]) <= {"squareShape", "reducedShape"}
            assert o["result_shape"] in ("squareShape", "reducedShape")


def _matmul_T(a, b, T, acc_T=None):
    """tosa.matmul lowered to linalg.batch_matmul with a zero-filled result of the RESULT type: k ascending, the
    product and the sum rounded separately to that type."""
    acc_T = acc_T or T
    acc = np.zeros((a.shape[0], a.shape[1], b.shape[2]), acc_T)
    for k in range(a.shape[2]):
        prod = (a[:, :, k, None].astype(acc_T) * b[:, k, None, :].astype(acc_T)).astype(acc_T)
        acc = (acc + prod).astype(acc_T)
    return acc.astype(T)


def _reduce_sum_T(x, T, acc_T=None):
    acc_T = acc_T or T
    acc = np.zeros(x.shape[:2] + (1,), acc_T)
    for k in range(x.shape[2]):
        acc = (acc + x[:, :, k, None].astype(acc_T)).astype(acc_T)
    return acc.astype(T)


def interpret(case, inputs, T, acc_T=None):
    env = dict(inputs)
    for o in case["ops"]:
        a = [env[n] for n in o["operands"]]
        kind = o["op"]
        if kind == "tosa.matmul":
            r = _matmul_T(a[0], a[1], T, acc_T)
        elif kind == "tosa.mul":
            r = (a[0] * a[1]).astype(T)
        elif kind == "tosa.sub":
            r = (a[0] - a[1]).astype(T)
        elif kind == "tosa.reduce_max":
            r = a[0].max(axis=2, keepdims=True)
        elif kind == "tosa.reduce_sum":
            r = _reduce_sum_T(a[0], T, acc_T)
        elif kind == "tosa.exp":
            r = np.exp(a[0].astype(np.float64)).astype(np.float32).astype(T)   # exp evaluated in f32, like the oracle's expf
        elif kind == "tosa.reciprocal":
            r = (T(1.0) / a[0]).astype(T)
        else:
            raise AssertionError(f"op {kind} is not part of the reference's attention validator")
        assert r.dtype == T
        env[o["result"]] = r
    return env[case["ops"][-1]["result"]]


def _ulps(got, ref, T):
    """Difference in units of the last place of the largest magnitude of each output row (an output element is a
    sum of Sk signed terms: one that cancels to near zero keeps the absolute uncertainty of its terms)."""
    eps = np.finfo(T).eps
    scale = np.abs(ref.astype(np.float64)).max(axis=-1, keepdims=True)
    return np.abs(got.astype(np.float64) - ref.astype(np.float64)) / (scale * eps)


@pytest.mark.parametrize("elem", ["f32", "f16"])
@pytest.mark.parametrize("case", FIX["cases"], ids=lambda c: c["prefix"])
def test_oracle_attention_follows_the_reference_op_sequence(case, elem):
    T = NP_T[elem]
    G, Sq, Sk, D, Dv = 2, 24, 40, 16, 8
    rng = np.random.Generator(np.random.PCG64(5))
    q = rng.standard_normal((G, Sq, D), dtype=np.float32).astype(T)
    k = rng.standard_normal((G, D, Sk), dtype=np.float32).astype(T)
    v = rng.standard_normal((G, Sk, Dv), dtype=np.float32).astype(T)
    inputs = {"queriesTensor": q, "keysTensor": k, "valuesTensor": v}
    scale = None
    if "--with-attn-scale" in case["flags"]:
        scale = (rng.random((G, Sq, Sk), dtype=np.float32) * 0.5 + 0.25).astype(T)
        inputs["scaleTensor"] = scale
    want = interpret(case, inputs, T)
    got = oracle.attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), elem_type=ORC_T[elem],
                           scale=None if scale is None else scale.astype(np.float32)).astype(T)
    u = _ulps(got, want, T)
    assert u.max() <= 2.0, f"oracle and interpreted reference program differ by {u.max():.1f} ulp"
    assert np.mean(u == 0) > 0.9
    if elem == "f16":
        # control: the same program with f32 accumulators in matmul / reduce_sum is NOT what the oracle computes
        wide = interpret(case, inputs, T, acc_T=np.float32)
        assert _ulps(wide, want, T).max() > 2.0


@pytest.mark.parametrize("tc", ["NOTRC", "TRC"])
@pytest.mark.parametrize("tb", ["NOTRB", "TRB"])
@pytest.mark.parametrize("ta", ["NOTRA", "TRA"])
def test_oracle_gemm_follows_the_reference_loop_nest(ta, tb, tc):
    gm = FIX["gemm"]
    assert gm["iterator_types"] == ["parallel", "parallel", "parallel", "reduction"] and gm["fill"] == 0.0
    assert [b["op"] for b in gm["body"]] == ["arith.mulf", "arith.addf"] and gm["yield"] == "add"
    assert gm["body"][0]["operands"] == ["aElem", "bElem"] and gm["body"][1]["operands"] == ["mul", "cElem"]
    # shapes of the check file, scaled down: d0 = g, d1 = m, d2 = n, d3 = k (reduction, innermost)
    ext = {"d0": 2, "d1": 9, "d2": 7, "d3": 33}
    big = {"d0": gm["sizes"]["g"], "d1": gm["sizes"]["m"], "d2": gm["sizes"]["n"], "d3": gm["sizes"]["k"]}
    for name, pref in (("A", ta), ("B", tb), ("C", tc)):
        assert gm["shapes"][name][pref] == [big[d] for d in gm["maps"][name][pref]]
    rng = np.random.Generator(np.random.PCG64(6))
    a = rng.standard_normal([ext[d] for d in gm["maps"]["A"][ta]], dtype=np.float32)
    b = rng.standard_normal([ext[d] for d in gm["maps"]["B"][tb]], dtype=np.float32)
    c = np.full([ext[d] for d in gm["maps"]["C"][tc]], np.float32(gm["fill"]))

    def view(x, dims):     # x indexed by its map -> array indexed (d0, d1, d2) or (d0, d1|d2, d3) in domain order
        order = sorted(range(3), key=lambda i: dims[i])
        return np.transpose(x, order)
    av, bv, cv = view(a, gm["maps"]["A"][ta]), view(b, gm["maps"]["B"][tb]), view(c, gm["maps"]["C"][tc])
    # av [g, m, k], bv [g, n, k], cv [g, m, n]; the reduction index runs innermost and ascending
    for kk in range(ext["d3"]):
        mul = (av[:, :, None, kk] * bv[:, None, :, kk]).astype(np.float32)     # arith.mulf
        cv[...] = (mul + cv).astype(np.float32)                                  # arith.addf
    got = oracle.gemm_f32(a, b, ext["d0"], ext["d1"], ext["d2"], ext["d3"], ta == "TRA", tb == "TRB", tc == "TRC")
    np.testing.assert_array_equal(got, c)
