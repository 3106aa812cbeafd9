"""Expands the reference's end-to-end test matrices (mlir/test/e2e/*.toml) into flat command lines, the way
mlir/test/e2e/generateE2ETest.py:113-157 does (axes x suite tests, minus each test's exclusions), and stores
them as tests/golden/e2e_configs.json. Every line is a rocmlir-gen flag string whose run must end in the verdict
`[1 1 1]`. Run in a checkout that has the reference tree: python tests/golden/make_e2e_configs.py <reference root>
"""
import itertools
import json
import os
import re
import sys
import tomllib

# matrices that exercise the path of this library (PR suites + regression lists); the nightly model sweeps
# (Resnet50Config, Resnet101Config, Resnext101Config) repeat the same kernels on ~100 more shapes each
FILES = ["PrGemm.toml", "PrGemmSplitK.toml", "PrResnet50.toml", "PrAttentionF16.toml", "PrAttentionI8.toml", "PrAttentionF32.toml",
         "PaddedGemmConfig.toml",
         "GemmVariants.toml", "MixedConvLayouts.toml", "conv_regression_fwd.toml", "conv_regression_bwd.toml",
         "gemm_split_k_f16.toml", "gemm_split_k_f32.toml", "conv_wrw_perf_config.toml", "gemm_with_atomic_add.toml"]

# lit substitutions of the reference's default configuration (mlir/test/e2e/lit.site.cfg.py.in:22-23,
# mlir/test/lit.cfg.py:35-38): validation on the CPU, random data seed 1
SUBST = {"%pv": "-pv", "%random_data": "-rand 1", "%rocmlir_gen_flags": "", "%arch": "%arch"}


def option_list(prefixes, table, key1, key2):
    lists = []
    for item in table.get(key1, []):
        lists.append([prefixes.get(item["name"], "") + v for v in item[key2]])
    return list(itertools.product(*lists))


def expand(path):
    t = tomllib.load(open(path, "rb"))
    prefixes = {a["name"]: a["prefix"] for a in t.get("axis", []) if "prefix" in a}
    combos = option_list(prefixes, t, "axis", "values")
    gen_part = t["suffix"].split("|")[0]
    for k, v in SUBST.items():
        gen_part = gen_part.replace(k, v)
    out = []
    for suite in t["suite"]:
        for ti, test in enumerate(suite["test"], 1):
            excl = option_list(prefixes, test, "exclude", "values") if "exclude" in test else []
            for oi, opt in enumerate(combos, 1):
                if len(opt) >= 3 and "i8" in opt[2] and ("conv_bwd_data" in opt[0] or "conv_bwd_weight" in opt[0]):
                    continue
                if any(all(x in opt for x in e) for e in excl):
                    continue
                line = " ".join((test["config"] + " " + " ".join(opt) + " " + gen_part).split())
                out.append({"file": os.path.basename(path), "suite": suite["name"], "test": ti, "variant": oi,
                            "flags": line})
    return out


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ROCMLIR_REFERENCE_DIR") or sys.exit("usage: pass the root of the reference checkout as the first argument (or set ROCMLIR_REFERENCE_DIR)")
    cases = []
    for f in FILES:
        cases += expand(os.path.join(root, "mlir", "test", "e2e", f))
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "e2e_configs.json"), "w") as fh:
        json.dump({"source": "mlir/test/e2e/*.toml expanded as generateE2ETest.py does", "cases": cases}, fh, indent=0)
    print(len(cases), "cases")
    by = {}
    for c in cases:
        by[c["file"]] = by.get(c["file"], 0) + 1
    print(by)


if __name__ == "__main__":
    main()
