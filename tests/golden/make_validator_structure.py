"""The op sequence of the reference's CPU attention validator, as a JSON fixture.

Source: mlir/test/rocmlir-gen/attention-kernel.mlir of the reference checkout (root = first argument or
$ROCMLIR_REFERENCE_DIR). Its FileCheck lines under `func.func @host_naive_attention` hold, op by op, the TOSA program
that rocmlir-gen emits as the CPU reference of rock.attention (with and without the scale operand): which op, which
operands, which result shape class. This script parses those lines into a small dataflow list:

    {"prefix": "CHECK_SCALE", "element_type": "f32", "ops": [{"result": "qkTensor", "op": "tosa.matmul",
      "operands": ["queriesTensor", "keysTensor"], "operand_shapes": [...], "result_shape": "squareShape"}, ...]}

tests/test_oracle_structure.py interprets the list with numpy, every op in the element type, and compares
with the oracle. The same is done for the GEMM validator (mlir/test/rocmlir-gen/gemm-kernel.mlir: fill, indexing maps
per transposition, iterator types, mulf then addf).     python tests/golden/make_validator_structure.py <reference root>
"""
import json
import os
import re
import sys

ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ROCMLIR_REFERENCE_DIR") or sys.exit(
    "usage: pass the root of the reference checkout as the first argument (or set ROCMLIR_REFERENCE_DIR)")
SRC = os.path.join(ROOT, "mlir", "test", "rocmlir-gen", "attention-kernel.mlir")
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "validator_structure.json")

VAR = r"%\[\[(\w+)(?::[^\]]*)?\]\]"      # %[[name]] or %[[name:.*]]
SHAPE = r"\[\[(\w+)(?::[^\]]*)?\]\]"     # [[name]] or [[name:tensor<.*>]]


def parse(prefix, lines):
    run = next(l for l in lines if l.startswith("// RUN:") and prefix in l)
    elem = re.search(r"-t (\w+)", run).group(1)
    flags = re.findall(r"(--with-attn-\w+|-transK|-transQ|-transV|-transO)", run)
    body, inside = [], False
    for l in lines:
        if l.startswith(f"// {prefix}-LABEL: func.func @host_naive_attention"):
            inside = True
            continue
        if inside and re.match(rf"// {prefix}(-DAG|-NEXT)?: ", l):
            text = l.split(": ", 1)[1].strip()
            if text == "return":
                break
            body.append((l.split(":")[0].replace("// ", ""), text))
    ops = []
    for directive, text in body:
        m = re.match(rf"{VAR} = (tosa\.\w+) (.*?) : \((.*?)\) -> (.*)$", text)
        assert m, text
        result, op, operand_text, in_shapes, out_shape = m.groups()
        ops.append({"result": result, "op": op, "operands": re.findall(VAR, operand_text),
                    "operand_shapes": re.findall(SHAPE, in_shapes), "result_shape": re.findall(SHAPE, out_shape)[0],
                    "directive": directive})
    return {"prefix": prefix, "element_type": elem, "flags": flags, "ops": ops}


def parse_gemm(lines):
    """mlir/test/rocmlir-gen/gemm-kernel.mlir, `func.func @host_naive_gemm`: the fill value, the indexing maps of A, B
    and C per transposition prefix, the iterator types and the two-op body of the linalg.generic."""
    out = {"maps": {}, "shapes": {}}
    inside = False
    body = []
    for l in lines:
        m = re.match(r"// (\w+)-DAG:\s+#\[\[\$map([ABC])Host:\.\*\]\] = affine_map<\((.*?)\) -> \((.*?)\)>", l)
        if m:
            out["maps"].setdefault(m.group(2), {})[m.group(1)] = [d.strip() for d in m.group(4).split(",")]
            out["domain"] = [d.strip() for d in m.group(3).split(",")]
        if l.startswith("// CHECK-LABEL: func.func @host_naive_gemm"):
            inside = True
            continue
        if not inside:
            continue
        m = re.match(r"// CHECK-NEXT: %\[\[cst:\.\*\]\] = arith.constant ([0-9.]+)", l)
        if m:
            out["fill"] = float(m.group(1))
        m = re.match(r"// CHECK-NEXT: %\[\[([abc]):\.\*\]\] = memref.expand_shape", l)
        if m:
            last = m.group(1).upper()
        m = re.match(r"// (\w+)-SAME:\s+into memref<([0-9x]+)xf32>", l)
        if m:
            out["shapes"].setdefault(last, {})[m.group(1)] = [int(v) for v in m.group(2).split("x")]
        m = re.match(r"// CHECK-SAME: iterator_types = \[(.*)\]", l)
        if m:
            out["iterator_types"] = [t.strip().strip('"') for t in m.group(1).split(",")]
        m = re.match(r"// CHECK-NEXT: %\[\[(\w+):\.\*\]\] = (arith\.\w+) %\[\[(\w+)\]\], %\[\[(\w+)\]\]", l)
        if m:
            body.append({"result": m.group(1), "op": m.group(2), "operands": [m.group(3), m.group(4)]})
        m = re.match(r"// CHECK-NEXT: linalg.yield %\[\[(\w+)\]\]", l)
        if m:
            out["yield"] = m.group(1)
            break
    out["body"] = body
    run = next(l for l in lines if l.startswith("// RUN:") and "--operation gemm" in l)
    out["sizes"] = {k: int(v) for k, v in re.findall(r"-([gmkn]) (\d+)", run)}
    return out


def main():
    lines = open(SRC).read().splitlines()
    cases = [parse(p, lines) for p in ("CHECK_SCALE", "CHECK_NO_SCALE")]
    gemm_src = os.path.join(ROOT, "mlir", "test", "rocmlir-gen", "gemm-kernel.mlir")
    gemm = parse_gemm(open(gemm_src).read().splitlines())
    json.dump({"source": "mlir/test/rocmlir-gen/attention-kernel.mlir", "cases": cases,
               "gemm_source": "mlir/test/rocmlir-gen/gemm-kernel.mlir", "gemm": gemm}, open(OUT, "w"), indent=1)
    print(f"{OUT}: {[len(c['ops']) for c in cases]} attention ops, gemm body {[b['op'] for b in gemm['body']]}")


if __name__ == "__main__":
    main()
