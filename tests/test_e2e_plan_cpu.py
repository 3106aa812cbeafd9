"""Every command line of the reference's end-to-end matrices (tests/golden/e2e_configs.json) must be parsed, typed
and sized by the driver without a GPU: a line the library cannot run is a planning-time `Unsupported`, never a
surprise on the device. Keeps the fixture, the driver and the Python mirror consistent on CPU-only machines."""
import collections
import json
import os
import sys

sys.path.insert(0, os.path.dirname(__file__))
from oracle import harness as rocmlir_gen  # noqa: E402

CASES = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "e2e_configs.json")))["cases"]


def test_every_line_plans():
    reasons = collections.Counter()
    for c in CASES:
        try:
            assert rocmlir_gen.plan(c["flags"]) is None
        except rocmlir_gen.Unsupported as e:
            reasons[str(e)] += 1
    # the only lines left out: results whose CPU validation alone would take the test budget
    assert sum(reasons.values()) == 2, reasons
    assert all("2 GiB" in r for r in reasons), reasons


def test_fixture_covers_the_suites():
    files = collections.Counter(c["file"] for c in CASES)
    assert len(CASES) == 1375 and files["gemm_with_atomic_add.toml"] == 4
    for name in ("PrGemm.toml", "PrResnet50.toml", "PrAttentionF16.toml", "PrAttentionI8.toml", "PrAttentionF32.toml",
                 "conv_regression_fwd.toml", "conv_regression_bwd.toml", "MixedConvLayouts.toml"):
        assert files[name] > 0, name


def test_rocmlir_gen_tool_writes_a_harness_description_and_refuses_bad_lines():
    """oracle/bin/rocmlir-gen: stage one of `rocmlir-gen ... -pv | rocmlir-driver -c` needs no GPU."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    gen = os.path.join(root, "oracle", "bin", "rocmlir-gen")
    drv = os.path.join(root, "oracle", "bin", "rocmlir-driver")
    line = "--operation gemm -t f16 -g 3 -m 1024 -k 769 -n 1024 --arch sm_100a -ph -pv -rand 1"
    r = subprocess.run([sys.executable, gen] + line.split(), capture_output=True, text=True)
    assert r.returncode == 0 and json.loads(r.stdout)["flags"] == line
    r = subprocess.run([sys.executable, gen] + line.replace("sm_100a", "gfx942").split(), capture_output=True, text=True)
    assert r.returncode == 2 and "not this hardware" in r.stderr
    r = subprocess.run([sys.executable, drv, "-c"], input="not a description", capture_output=True, text=True)
    assert r.returncode == 2
    r = subprocess.run([sys.executable, drv], input="{}", capture_output=True, text=True)
    assert r.returncode == 2 and "nothing to do" in r.stderr
