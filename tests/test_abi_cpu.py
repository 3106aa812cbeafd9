"""No-GPU checks of the C ABI: the shared library loads and exports every symbol include/*.h declares,
and argument validation that needs no device behaves like the reference boundary (error codes, no crash)."""
import ctypes as C
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        src = open(h).read()
        names += [n for n in re.findall(r"^(?:RB|MIIR)_EXPORT[^;(]*?\b(\w+)\s*\(", src, re.M)]
    return sorted(set(names))


@pytest.fixture(scope="module")
def lib():
    from rocmlir_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from rocmlir_b200 import build
        build.build()
    return _lib.lib()


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "rbGemm" in syms and "rbGemmWorkspaceSize" in syms and len(syms) >= 6


def test_library_exports_every_declared_symbol(lib):
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_workspace_size_needs_no_device(lib):
    from rocmlir_b200 import _lib as L
    # aligned f16 problem with enough tiles to fill the GPU: no workspace; K = 769 (odd, the reference's default
    # gemm K): a pitched copy of A
    p = L.RbGemmProblem(1, 4096, 4096, 4096, 0, 0, 0, L.F16, L.F16, 0)
    assert lib.rbGemmWorkspaceSize(C.byref(p)) == 0
    lib.rbSetGemmVariant(0x200)          # opt-in stream-K tail: one f32 partial tile per CTA pair plus arrival words
    assert lib.rbGemmWorkspaceSize(C.byref(p)) == 74 * 256 * 256 * 4 + 74 * 8 * 4 + 192  # words rounded up to 256 B
    lib.rbSetGemmVariant(0)
    p = L.RbGemmProblem(1, 1024, 512, 769, 0, 0, 0, L.F16, L.F16, 0)
    assert lib.rbGemmWorkspaceSize(C.byref(p)) >= 1024 * 776 * 2
    # f32 accurate mode needs hi/lo planes of both operands
    p = L.RbGemmProblem(1, 64, 64, 64, 0, 0, 0, L.F32, L.F32, 0)
    assert lib.rbGemmWorkspaceSize(C.byref(p)) >= 4 * 64 * 64 * 4


def test_gemm_gemm_workspace_holds_intermediate_and_flag_words(lib):
    """rbGemmGemmWorkspaceSize: the rounded intermediate, the larger of the two products' own workspaces, and the flag
    words of the chained one-launch form (four per 128-row block and 32-column tile), whatever form then runs."""
    from rocmlir_b200 import _lib as L
    m, k1, n1, n2 = 4096, 1024, 1024, 1024
    need = lib.rbGemmGemmWorkspaceSize(1, m, k1, n1, n2, L.F16)
    flags = (m // 128) * (n1 // 32) * 4 * 4
    assert need >= m * n1 * 2 + flags and need % 256 == 0
    assert lib.rbGemmGemmWorkspaceSize(1, 0, k1, n1, n2, L.F16) == 0          # malformed sizes report 0
    st = lib.rbGemmGemm(1, m, k1, n1, n2, L.F16, None, None, None, None, None, 0, None)
    assert st != L.SUCCESS                                                     # no workspace, no device pointers


def test_invalid_problem_is_rejected_without_device(lib):
    from rocmlir_b200 import _lib as L
    p = L.RbGemmProblem(1, 0, 512, 64, 0, 0, 0, L.F16, L.F16, 0)
    st = lib.rbGemm(C.byref(p), None, None, None, None, None, 0, None)
    assert st == L.INVALID_PARAM
    assert b"positive" in lib.rbGetLastError()
    p = L.RbGemmProblem(1, 8, 8, 8, 0, 0, 0, 99, L.F16, 0)
    assert lib.rbGemm(C.byref(p), None, None, None, None, None, 0, None) == L.INVALID_PARAM


def test_product_does_not_import_oracle():
    """The product package must never route through the CPU oracle."""
    for path in glob.glob(os.path.join(ROOT, "rocmlir_b200", "**", "*"), recursive=True):
        if path.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
            txt = open(path, errors="ignore").read()
            assert "import oracle" not in txt and "from oracle" not in txt and "liboracle" not in txt, path


def test_ctypes_mirror_of_the_launch_description_matches_the_c_layout(tmp_path):
    """RbKernelLaunch is filled by the library: the Python mirror must have the C struct's size and field offsets."""
    import subprocess
    from rocmlir_b200 import _lib as L
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "rocmlir_b200.h"\n'
                   'int main(void) { printf("%zu %zu %zu %zu\\n", sizeof(RbKernelLaunch), offsetof(RbKernelLaunch, params), '
                   'offsetof(RbKernelLaunch, grid), sizeof(RbEpilogue)); return 0; }\n')
    exe = str(tmp_path / "layout")
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-o", exe, str(src)], check=True)
    size, params_off, grid_off, epi = map(int, subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split())
    assert (C.sizeof(L.RbKernelLaunch), L.RbKernelLaunch.params.offset, L.RbKernelLaunch.grid.offset) == (size, params_off, grid_off)
    assert C.sizeof(L.RbEpilogue) == epi
