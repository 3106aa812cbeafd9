"""The string-configured handle API on the GPU: launching through a handle and through a stored launch
descriptor gives the oracle's result (exactly, on the reference's integer-valued `-rand 1` data), for the three
convolution directions, a GEMM and attention; and the tuning loop measures a space and fills a table."""
import numpy as np
import pytest

import oracle
from helpers import from_device, normal_data, reference_random, to_device

pytestmark = pytest.mark.gpu

CONV = (" --operation {op} --arch sm_100a --in_type {t} --fil_type {t} --out_type {t} --fil_layout {fl} --in_layout {il} "
        "--out_layout {ol} --batchsize 4 --groupsize 1 --in_channels 64 --out_channels 32 --in_h 14 --in_w 14 --out_h 14 "
        "--out_w 14 --fil_h 3 --fil_w 3 --padding_h 1 --padding_w 1 --conv_stride_h 1 --conv_stride_w 1")
LAYOUTS = {"nchw": ("GNCHW", "NGCHW", "NGCHW", "gkcyx", "ngchw", "ngkhw"),
           "nhwc": ("GNHWC", "NHWGC", "NHWGC", "gkyxc", "nhwgc", "nhwgk")}


@pytest.mark.parametrize("op,direction", [("conv", 0), ("conv_bwd_data", 1), ("conv_bwd_weight", 2)])
@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("via", ["handle", "buffer"])
def test_conv_through_the_handle_api(cuda_device, op, direction, layout, via):
    import torch
    from rocmlir_b200 import miir
    fl, il, ol, ofl, oil, ool = LAYOUTS[layout]
    ocfg = oracle.Conv(n=4, c=64, k=32, h=14, w=14, y=3, x=3, pad_h=1, pad_w=1, fil_layout=ofl, in_layout=oil,
                       out_layout=ool)
    (fil_f, fil_r), (in_f, in_r), (out_f, out_r) = reference_random(
        [(ocfg.numel("fil"),), (ocfg.numel("in"),), (ocfg.numel("out"),)], oracle.F16, seed=1)
    want = oracle.conv_f32(ocfg, direction, fil_f, in_f, out_f)
    t = {"fil": to_device(fil_r, oracle.F16), "in": to_device(in_r, oracle.F16), "out": to_device(out_r, oracle.F16)}
    with miir.Handle(CONV.format(op=op, t="fp16", fl=fl, il=il, ol=ol)) as h:
        assert h.kernel_count == 1
        ws = torch.empty(max(1, h.workspace_size), dtype=torch.uint8, device="cuda")
        h.lower_bin()
        if via == "handle":
            h.launch(t["fil"], t["in"], t["out"], workspace=ws)
        else:
            blob = h.descriptor()
    if via == "buffer":   # the handle is gone: the descriptor alone is enough
        miir.launch_from_buffer(blob, t["fil"], t["in"], t["out"], workspace=ws)
    torch.cuda.synchronize()
    got = oracle.to_f32(from_device(t[{0: "out", 1: "in", 2: "fil"}[direction]], oracle.F16), oracle.F16)
    np.testing.assert_array_equal(got.ravel(), oracle.round_to(want, oracle.F16).ravel())


def test_gemm_and_attention_through_the_handle_api(cuda_device):
    import torch
    from rocmlir_b200 import miir
    G, M, N, K = 2, 192, 160, 128
    (a_f, a_r), (b_f, b_r) = reference_random([(G, M, K), (G, K, N)], oracle.F16, seed=1)
    want = oracle.round_to(oracle.gemm_f32(a_f, b_f, G, M, N, K), oracle.F16)
    a, b = to_device(a_r, oracle.F16), to_device(b_r, oracle.F16)
    c = torch.zeros(G, M, N, dtype=torch.float16, device="cuda")
    with miir.Handle(f"--operation gemm --arch sm_100a -t f16 -g {G} -m {M} -n {N} -k {K}") as h:
        h.lower_tuning_params()
        ws = torch.empty(max(1, h.workspace_size), dtype=torch.uint8, device="cuda")
        h.launch(a, b, c, workspace=ws)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(oracle.to_f32(from_device(c, oracle.F16), oracle.F16), want)

    g, sq, sk, d = 3, 256, 320, 64
    q_f, q_r = normal_data((g, sq, d), oracle.F16, 11, 1.0)
    k_f, k_r = normal_data((g, sk, d), oracle.F16, 12, 1.0)
    v_f, v_r = normal_data((g, sk, d), oracle.F16, 13, 1.0)
    scale = float(1.0 / np.sqrt(d))
    from rocmlir_b200.attention import attention
    q, k, v = to_device(q_r, oracle.F16), to_device(k_r, oracle.F16), to_device(v_r, oracle.F16)
    direct = attention(q, k, v, scale=scale, trans_k=True)
    o = torch.zeros(g, sq, d, dtype=torch.float16, device="cuda")
    with miir.Handle(f"--operation attention --arch sm_100a -t f16 -g {g} -seq_len_q {sq} -seq_len_k {sk} -head_dim_qk {d} "
                     f"-head_dim_v {d} -transK true --with-attn-scale {scale!r}") as h:
        h.lower_bin()
        h.launch(q, k, v, extra=o)
    torch.cuda.synchronize()
    assert torch.equal(o, direct)     # same kernel, same problem: bit-identical to the struct API


def test_tuning_loop_measures_a_space_and_fills_a_table(cuda_device, tmp_path):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200 import tuning
    from rocmlir_b200.gemm import gemm
    M = N = K = 1024
    a = torch.randn(M, K, device="cuda").half()
    b = torch.randn(K, N, device="cuda").half()
    ref = None
    prob = tuning.Problem(f"--operation gemm --arch sm_100a -t f16 -m {M} -n {N} -k {K}")
    table = tuning.Table()
    outs = {}

    def run(variant):
        outs[variant] = gemm(a, b, variant=variant)

    results = tuning.tune(prob, run, kind=tuning.QUICK, iters=3, table=table)
    assert len(results) == len(prob.space(tuning.QUICK)) >= 2
    assert all(ms > 0 for _, ms in results) and results == sorted(results, key=lambda r: r[1])
    # every configuration computes the same GEMM (K is not split in the quick set of this problem: bit-identical)
    vals = list(outs.values())
    for o in vals[1:]:
        torch.testing.assert_close(o.float(), vals[0].float(), rtol=2e-3, atol=2e-2)
    assert prob.set_from_table(table) and prob.perf_config == results[0][0]
    tuning.write_tsv(str(tmp_path / "tuned.tsv"), [(prob.key, results[0][0], results[0][1])])
    line = open(tmp_path / "tuned.tsv").read().rstrip("\n").split("\t")
    assert line[0] == "sm_100a" and line[-2] == results[0][0]
    assert L.kernel_status() == 0
