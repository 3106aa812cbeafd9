"""The reference's end-to-end matrices (mlir/test/e2e/*.toml, expanded by tests/golden/make_e2e_configs.py into
tests/golden/e2e_configs.json) run through tests/rocmlir_gen.py: every command line must end in the verdict
`[1 1 1]`, exactly what the reference's generated lit tests CHECK for.

By default the PR suites run in full and every 4th line of the large regression matrices; set RB_E2E_ALL=1 to run
all 1335 lines (about half an hour, dominated by the CPU validator)."""
import json
import os

import pytest

import rocmlir_gen

pytestmark = pytest.mark.gpu

CASES = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "e2e_configs.json")))["cases"]
FULL_FILES = {"PrGemm.toml", "PrGemmSplitK.toml", "PrResnet50.toml", "PrAttentionF16.toml", "PrAttentionI8.toml", "PrAttentionF32.toml", "gemm_split_k_f16.toml",
              "gemm_split_k_f32.toml", "conv_wrw_perf_config.toml"}


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
