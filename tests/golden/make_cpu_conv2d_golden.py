"""Extracts the known-answer tensors of the reference's CPU convolution tests into a JSON fixture.

Source: mlir/test/rocmlir-driver/cpu_conv2d/*.mlir of the reference checkout. Each RUN line gives the
rocmlir-gen flags of one case (`-prc -rand=none`: all inputs 1, only the CPU reference runs) and the
CHECK-NEXT line under the same prefix gives the printed result tensor.
Run where the reference checkout is available (its root is the first argument, or $ROCMLIR_REFERENCE_DIR):
    python tests/golden/make_cpu_conv2d_golden.py <reference root>
"""
import glob
import json
import os
import re
import sys

ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ROCMLIR_REFERENCE_DIR") or sys.exit("usage: pass the root of the reference checkout as the first argument (or set ROCMLIR_REFERENCE_DIR)")
SRC = os.path.join(ROOT, "mlir", "test", "rocmlir-driver", "cpu_conv2d")
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpu_conv2d.json")

FLAG = re.compile(r"-{1,2}([A-Za-z_]+)[= ]([^\s|]+)")


def main():
    cases = []
    for path in sorted(glob.glob(os.path.join(SRC, "*.mlir"))):
        lines = open(path).read().splitlines()
        expected, unchecked = {}, set()
        for i, l in enumerate(lines):
            # One case spells the directive "LITERAY" and spreads the tensor over several lines; FileCheck
            # ignores such lines, so that tensor is kept but flagged as not enforced by the reference.
            m = re.match(r"//\s*(CHECK\w*)-NEXT\{LITERA([LY])\}:(.*)$", l)
            if m:
                nums = [float(v) for v in re.findall(r"-?\d+(?:\.\d+)?", m.group(3))]
                expected.setdefault(m.group(1), []).extend(nums)
                if m.group(2) == "Y":
                    unchecked.add(m.group(1))
        for l in lines:
            if "RUN:" not in l:
                continue
            gen = l.split("|")[0]
            prefix = re.search(r"--check-prefix=(\w+)", l).group(1)
            flags = {k: v for k, v in FLAG.findall(gen)}
            op = flags.get("operation", "conv")
            cases.append({
                "file": os.path.basename(path),
                "prefix": prefix,
                "operation": op,
                "dtype": flags.get("t", "f32"),
                "fil_layout": flags["fil_layout"], "in_layout": flags["in_layout"], "out_layout": flags["out_layout"],
                "n": int(flags["batchsize"]), "c": int(flags["in_channels"]), "k": int(flags["out_channels"]),
                "h": int(flags["in_h"]), "w": int(flags["in_w"]), "y": int(flags["fil_h"]), "x": int(flags["fil_w"]),
                "dil_h": int(flags["dilation_h"]), "dil_w": int(flags["dilation_w"]),
                "pad_h": int(flags["padding_h"]), "pad_w": int(flags["padding_w"]),
                "stride_h": int(flags["conv_stride_h"]), "stride_w": int(flags["conv_stride_w"]),
                "expected": expected[prefix],
                "enforced_by_reference": prefix not in unchecked,
            })
    with open(OUT, "w") as f:
        json.dump({"source": "mlir/test/rocmlir-driver/cpu_conv2d/*.mlir", "cases": cases}, f, separators=(",", ":"))
    print(len(cases), "cases ->", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
