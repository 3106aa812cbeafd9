"""Every command line of the reference's end-to-end matrices (tests/golden/e2e_configs.json) must be parsed, typed
and sized by the driver without a GPU: a line the library cannot run is a planning-time `Unsupported`, never a
surprise on the device. Keeps the fixture, the driver and the Python mirror consistent on CPU-only machines."""
import collections
import json
import os
import sys

sys.path.insert(0, os.path.dirname(__file__))
import rocmlir_gen  # noqa: E402

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
    assert len(CASES) == 1371
    for name in ("PrGemm.toml", "PrResnet50.toml", "PrAttentionF16.toml", "PrAttentionI8.toml", "PrAttentionF32.toml",
                 "conv_regression_fwd.toml", "conv_regression_bwd.toml", "MixedConvLayouts.toml"):
        assert files[name] > 0, name
