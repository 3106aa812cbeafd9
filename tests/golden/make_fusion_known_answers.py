"""Known answers the reference's fusion end-to-end tests print for all-ones inputs (`-rand none`), as a JSON fixture.

Source: mlir/test/fusion/pr-e2e/**.mlir of the reference checkout (root = first argument or $ROCMLIR_REFERENCE_DIR).
Each listed file holds one function and one CHECK line with the printed result; the operation and its sizes are
read from the function signature by the patterns below. Only files whose function is a plain dot / quant_dot
(optionally followed by an add of a same-shape tensor or a transpose / reshape, which do not change the values)
or a convolution followed by a broadcast add are taken.
    python tests/golden/make_fusion_known_answers.py <reference root>
"""
import json
import os
import re
import sys

ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ROCMLIR_REFERENCE_DIR") or sys.exit("usage: pass the root of the reference checkout as the first argument (or set ROCMLIR_REFERENCE_DIR)")
DIR = os.path.join(ROOT, "mlir", "test", "fusion", "pr-e2e")
FILES = ["mixr-gemm/mixr-gemm-add.e2e.mlir", "mixr-gemm/mixr-gemm-bcast-add.e2e.mlir",
         "mixr-gemm/mixr-gemm-reshape-case1.e2e.mlir", "mixr-gemm/mixr-gemm-reshape-case1-quant.e2e.mlir",
         "mixr-gemm/mixr-gemm-reshape-case2.e2e.mlir", "mixr-gemm/mixr-gemm-transpose.e2e.mlir",
         "mixr-bcast-add.e2e.mlir"]


def main():
    cases = []
    for rel in FILES:
        text = open(os.path.join(DIR, rel)).read()
        check = re.search(r"//\s*CHECK:\s*\[?([0-9.,\s]+)\]?", text)
        values = [float(v) for v in re.findall(r"\d+(?:\.\d+)?", check.group(1))]
        line = text[:check.start()].count("\n") + 1
        case = {"file": "mlir/test/fusion/pr-e2e/" + rel, "line": line, "printed": values}
        dot = re.search(r"migraphx\.(quant_dot|dot) [^:]*: <(\d+)x(\d+)x(\d+)x(\w+),[^>]*>, <(\d+)x(\d+)x(\d+)x(\w+),", text)
        conv = re.search(r"migraphx\.convolution [^:]*\{([^}]*)\} : <(\d+)x(\d+)x(\d+)x(\d+)x(\w+),[^>]*>, <(\d+)x(\d+)x(\d+)x(\d+)x", text)
        if dot:
            case.update(op=dot.group(1), g=int(dot.group(2)), m=int(dot.group(3)), k=int(dot.group(4)), n=int(dot.group(8)),
                        type=dot.group(5), add=bool(re.search(r"migraphx\.add", text)))
        elif conv:
            case.update(op="convolution", n=int(conv.group(2)), c=int(conv.group(3)), h=int(conv.group(4)), w=int(conv.group(5)),
                        type=conv.group(6), k=int(conv.group(7)), y=int(conv.group(9)), x=int(conv.group(10)),
                        add=bool(re.search(r"migraphx\.add", text)))
        else:
            raise SystemExit("no operation recognised in " + rel)
        cases.append(case)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fusion_known_answers.json")
    with open(out, "w") as fh:
        json.dump({"source": "CHECK lines of mlir/test/fusion/pr-e2e (all inputs 1)", "cases": cases}, fh, indent=1)
    print(len(cases), "cases")


if __name__ == "__main__":
    main()
