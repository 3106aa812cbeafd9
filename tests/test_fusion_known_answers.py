"""The known answers the reference's fusion end-to-end tests print for all-ones inputs
(tests/golden/fusion_known_answers.json, from the CHECK lines of mlir/test/fusion/pr-e2e): the oracle must reproduce
them on the CPU, and the library on the GPU. The adds of the `+ add` cases are computed where the reference fuses
them: mixr-gemm-add is a same-shape add (RB_EPI_RESIDUAL), mixr-gemm-bcast-add a vector broadcast along the rows
(bias[n]), mixr-bcast-add a per-output-channel add behind a convolution (rbConvEpi)."""
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
        if c["add"] and "bcast" in c["file"]:
            got = oracle.epilogue(got.astype(np.float32), n, bias=np.ones(n, np.float32))
        elif c["add"]:
            got = oracle.epilogue(got.astype(np.float32), n, residual=np.ones((g, m, n), np.float32))
        got = got.astype(np.float64).ravel()
        assert got.size == c["m"] * c["n"]
    else:
        p = oracle.Conv(n=c["n"], c=c["c"], k=c["k"], h=c["h"], w=c["w"], y=c["y"], x=c["x"], out_layout="nhwgk")
        got = oracle.conv_f32(p, 0, np.ones(p.numel("fil"), np.float32), np.ones(p.numel("in"), np.float32), None)
        assert c["add"]
        got = oracle.epilogue(got, c["k"], bias=np.ones(c["k"], np.float32)).astype(np.float64).ravel()
    want = expected(c)
    np.testing.assert_array_equal(got[: want.size], want)       # some CHECK lines print only the first values


@pytest.mark.gpu
@pytest.mark.parametrize("c", CASES, ids=IDS)
def test_library_reproduces_the_printed_result(cuda_device, c):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import Epilogue, gemm
    if c["op"] in ("dot", "quant_dot"):
        g, m, k, n = c["g"], c["m"], c["k"], c["n"]
        dt = torch.int8 if c["type"] == "i8" else torch.float32
        a = torch.ones((g, m, k), dtype=dt, device="cuda")
        b = torch.ones((g, k, n), dtype=dt, device="cuda")
        epi = None
        if c["add"] and "bcast" in c["file"]:
            epi = Epilogue(bias=torch.ones(n, dtype=torch.float32, device="cuda"))
        elif c["add"]:
            epi = Epilogue(residual=torch.ones((g, m, n), dtype=torch.float32, device="cuda"))
        out = gemm(a, b, epilogue=epi)
    else:
        from rocmlir_b200.conv import ConvConfig, conv_fused
        cfg = ConvConfig(n=c["n"], c=c["c"], k=c["k"], h=c["h"], w=c["w"], y=c["y"], x=c["x"], fil_layout="kcyx",
                         in_layout="nchw", out_layout="nkhw")
        t = {w: torch.ones(cfg.numel(w), dtype=torch.float32, device="cuda") for w in ("fil", "in", "out")}
        out = conv_fused(cfg, t["fil"], t["in"], t["out"], Epilogue(bias=torch.ones(c["k"], dtype=torch.float32, device="cuda")))
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    got = out.double().cpu().numpy().ravel()
    want = expected(c)
    np.testing.assert_array_equal(got[: want.size], want)
