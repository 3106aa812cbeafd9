"""The known answers the reference's fusion end-to-end tests print for all-ones inputs
(tests/golden/fusion_known_answers.json, from the CHECK lines of mlir/test/fusion/pr-e2e): the oracle must reproduce
them on the CPU, and the library on the GPU (dot and quant_dot; the convolution with its broadcast add through the
oracle only, since the library has no fused add on convolutions)."""
import json
import os

import numpy as np
import pytest

import oracle

CASES = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "fusion_known_answers.json")))["cases"]
IDS = [os.path.basename(c["file"]) for c in CASES]


def expected(c):
    return np.asarray(c["printed"], np.float64)


@pytest.mark.parametrize("c", CASES, ids=IDS)
def test_oracle_reproduces_the_printed_result(c):
    if c["op"] in ("dot", "quant_dot"):
        g, m, k, n = c["g"], c["m"], c["k"], c["n"]
        if c["type"] == "i8":
            got = oracle.gemm_i8(np.ones((g, m, k), np.int8), np.ones((g, k, n), np.int8), g, m, n, k, 0, 0, 0)
        else:
            got = oracle.gemm_f32(np.ones((g, m, k), np.float32), np.ones((g, k, n), np.float32), g, m, n, k, 0, 0, 0)
        got = got.astype(np.float64).ravel() + (1.0 if c["add"] else 0.0)
        assert got.size == c["m"] * c["n"]
    else:
        p = oracle.Conv(n=c["n"], c=c["c"], k=c["k"], h=c["h"], w=c["w"], y=c["y"], x=c["x"])
        got = oracle.conv_f32(p, 0, np.ones(p.numel("fil"), np.float32), np.ones(p.numel("in"), np.float32), None)
        got = got.astype(np.float64).ravel() + (1.0 if c["add"] else 0.0)
    want = expected(c)
    np.testing.assert_array_equal(got[: want.size], want)       # some CHECK lines print only the first values


@pytest.mark.gpu
@pytest.mark.parametrize("c", [c for c in CASES if c["op"] in ("dot", "quant_dot")],
                         ids=[i for i, c in zip(IDS, CASES) if c["op"] in ("dot", "quant_dot")])
def test_library_reproduces_the_printed_result(cuda_device, c):
    import torch
    from rocmlir_b200.gemm import gemm
    g, m, k, n = c["g"], c["m"], c["k"], c["n"]
    dt = torch.int8 if c["type"] == "i8" else torch.float32
    a = torch.ones((g, m, k), dtype=dt, device="cuda")
    b = torch.ones((g, k, n), dtype=dt, device="cuda")
    out = gemm(a, b)
    torch.cuda.synchronize()
    got = out.double().cpu().numpy().ravel() + (1.0 if c["add"] else 0.0)
    np.testing.assert_array_equal(got, expected(c))
