"""Builds librocmlir_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Usage: python -m rocmlir_b200.build [--force] [--verbose]
The shared library has no dependency on torch; it links the CUDA runtime statically.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "librocmlir_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + [
    "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fvisibility=hidden", "-I", INCLUDE, "-I", CSRC,
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the library cannot be built (there is no CPU fallback)")
    return cand


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


CUBIN_SRC = os.path.join(CSRC, "cubin", "gemm_kernels.cu")


def _deps_digest() -> str:
    h = hashlib.sha256()
    for root in (CSRC, INCLUDE, os.path.join(CSRC, "cubin")):
        for f in sorted(os.listdir(root)):
            if f.endswith((".cu", ".cuh", ".h")):
                with open(os.path.join(root, f), "rb") as fh:
                    h.update(f.encode())
                    h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    stamp = os.path.join(OBJ, "digest.txt")
    digest = _deps_digest()
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read() == digest:
        return LIB
    nvcc = _nvcc()
    srcs = sources()

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, "-c", src, "-o", obj] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    def cubin_object(_=None) -> str:
        """The kernels once more as a cubin (an ELF image for cuModuleLoadData), wrapped into an object file as
        read-only data between the symbols rb_gemm_cubin_start / rb_gemm_cubin_end."""
        cubin = os.path.join(OBJ, "gemm_kernels.cubin")
        cmd = [nvcc, "-cubin", CUBIN_SRC, "-o", cubin] + ARCH_FLAGS + ["-O3", "-std=c++17", "-lineinfo",
                                                                      "--expt-relaxed-constexpr", "-I", INCLUDE, "-I", CSRC]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("nvcc -cubin failed")
        asm = os.path.join(OBJ, "gemm_cubin_blob.S")
        with open(asm, "w") as fh:
            fh.write('.section .rodata\n.balign 64\n.global rb_gemm_cubin_start\nrb_gemm_cubin_start:\n'
                     '.incbin "gemm_kernels.cubin"\n.global rb_gemm_cubin_end\nrb_gemm_cubin_end:\n'
                     '.section .note.GNU-stack,"",@progbits\n')
        obj = os.path.join(OBJ, "gemm_cubin_blob.o")
        r = subprocess.run(["gcc", "-c", "gemm_cubin_blob.S", "-o", obj], cwd=OBJ, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("assembling the cubin blob failed")
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) + 1)) as ex:
        blob = ex.submit(cubin_object)
        objs = list(ex.map(compile_one, srcs))
        objs.append(blob.result())
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ARCH_FLAGS + ["-cudart", "static", "-Xcompiler", "-fPIC"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    with open(stamp, "w") as fh:
        fh.write(digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
