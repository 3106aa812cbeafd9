"""The reference's end-to-end matrices (mlir/test/e2e/*.toml, expanded by tests/golden/make_e2e_configs.py into
tests/golden/e2e_configs.json) run through oracle/harness.py: every command line must end in the verdict
`[1 1 1]`, exactly what the reference's generated lit tests CHECK for.

By default the PR suites run in full and every 4th line of the large regression matrices; set RB_E2E_ALL=1 to run
all 1335 lines (about half an hour, dominated by the CPU validator)."""
import json
import os

import pytest

from oracle import harness as rocmlir_gen

pytestmark = pytest.mark.gpu

CASES = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "e2e_configs.json")))["cases"]
FULL_FILES = {"PrGemm.toml", "PrGemmSplitK.toml", "PrResnet50.toml", "PrAttentionF16.toml", "PrAttentionI8.toml", "PrAttentionF32.toml", "gemm_split_k_f16.toml",
              "gemm_split_k_f32.toml", "conv_wrw_perf_config.toml", "gemm_with_atomic_add.toml"}


def selected():
    run_all = os.environ.get("RB_E2E_ALL", "0") == "1"
    out = []
    for i, c in enumerate(CASES):
        if run_all or c["file"] in FULL_FILES or i % 4 == 0:
            out.append(c)
    return out


@pytest.mark.parametrize("case", selected(), ids=lambda c: f"{c['file'][:-5]}-{c['suite']}-{c['test']}-{c['variant']}")
def test_reference_e2e_line_gives_111(cuda_device, case):
    try:
        verdict = rocmlir_gen.run(case["flags"])
    except rocmlir_gen.Unsupported as e:
        pytest.skip(f"no kernel: {e}")
    assert verdict == [1, 1, 1], case["flags"]


@pytest.mark.parametrize("line", [
    "--operation gemm -t f16 -g 3 -m 1024 -k 769 -n 1024 --arch sm_100a -ph -pv -rand 1",
    "--operation conv -t f16 --fil_layout gkyxc --in_layout nhwgc --out_layout nhwgk --batchsize 4 --in_channels 64 "
    "--out_channels 64 --in_h 14 --in_w 14 --fil_h 3 --fil_w 3 --padding_h 1 --padding_w 1 --arch sm_100a -ph -pv -rand 1",
    "--operation attention -t f16 -seq_len_q 256 -seq_len_k 256 -head_dim_qk 64 -head_dim_v 64 --arch sm_100a -ph -pv -rand 1 "
    "-rand_type float -RMS_threshold 0.015 -absDiff_threshold 0.02",
])
def test_tools_pipeline_prints_the_verdict(cuda_device, line):
    """`rocmlir-gen <flags> -ph -pv | rocmlir-driver -c` with this repository's tools of those names."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    gen = subprocess.run([sys.executable, os.path.join(root, "oracle", "bin", "rocmlir-gen")] + line.split(),
                         capture_output=True, text=True, check=True)
    drv = subprocess.run([sys.executable, os.path.join(root, "oracle", "bin", "rocmlir-driver"), "-c"], input=gen.stdout,
                         capture_output=True, text=True, timeout=600)
    assert drv.returncode == 0 and drv.stdout.strip().endswith("[1 1 1]"), drv.stdout + drv.stderr
