"""Failure detection of the GEMM kernel without a GPU fault: every device-side wait is bounded, and when one runs
out the kernel records a code, frees its tensor memory and returns, so that the context stays usable.

The failure is injected on the host (rbInjectStall: the producer of the next launch issues no loads, a flag that
nothing sets); nothing traps, faults or spins without a limit. The wait limit is lowered to about a millisecond for
the stalled launch so that the test takes milliseconds, and restored afterwards."""
import ctypes as C

import numpy as np
import pytest

import oracle
from helpers import from_device, reference_random, to_device

pytestmark = pytest.mark.gpu

LIMIT_CYCLES = 2_000_000   # about 1 ms at 1.9 GHz


@pytest.mark.parametrize("variant", [1, 2], ids=["single_cta", "cta_pair"])
def test_bounded_waits_run_out_and_the_next_launch_works(cuda_device, variant):
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import gemm
    lib = L.lib()
    g, m, n, k = 1, 512, 512, 1024
    (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], oracle.F16, seed=1)
    a, b = to_device(araw, oracle.F16), to_device(braw, oracle.F16)
    assert L.kernel_status() == 0
    lib.rbSetWaitLimit(LIMIT_CYCLES)
    lib.rbInjectStall(1)
    try:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        gemm(a, b, variant=variant)                 # the stalled launch: returns, result undefined
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 500.0, "every role must give up after about one wait limit"
        code = L.kernel_status(clear=True)
        assert code != 0, "the status word must say that a wait ran out"
        assert 0x100 <= code < 0x500, hex(code)      # a producer / MMA / epilogue timeout code
    finally:
        lib.rbSetWaitLimit(0)
        lib.rbInjectStall(0)
    # the context is intact: the same problem now computes the exact result
    out = gemm(a, b, variant=variant)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    ref = oracle.from_f32(oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads()), oracle.F16)
    np.testing.assert_array_equal(from_device(out, oracle.F16).reshape(ref.shape), ref)


def test_synchronous_entry_point_returns_kernel_timeout(cuda_device):
    """rbGemmHost waits for its stream, so it is the call that can return RB_KERNEL_TIMEOUT itself."""
    import torch
    from rocmlir_b200 import _lib as L
    lib = L.lib()
    g, m, n, k = 1, 256, 256, 512
    (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], oracle.F16, seed=1)
    a = torch.from_numpy(araw.view(np.int16)).view(torch.float16).pin_memory()
    b = torch.from_numpy(braw.view(np.int16)).view(torch.float16).pin_memory()
    out = torch.empty((g, m, n), dtype=torch.float16).pin_memory()
    prob = L.RbGemmProblem(g, m, n, k, 0, 0, 0, L.F16, L.F16, 0)
    stream = torch.cuda.current_stream().cuda_stream
    lib.rbSetWaitLimit(LIMIT_CYCLES)
    lib.rbInjectStall(1)
    try:
        st = lib.rbGemmHost(C.byref(prob), None, a.data_ptr(), b.data_ptr(), out.data_ptr(), stream)
    finally:
        lib.rbSetWaitLimit(0)
        lib.rbInjectStall(0)
    assert st == L.KERNEL_TIMEOUT, L.STATUS_NAMES[st]
    assert b"wait ran out" in lib.rbGetLastError()
    assert L.kernel_status() == 0, "the call that reported the timeout also cleared the word"
    L.check(lib.rbGemmHost(C.byref(prob), None, a.data_ptr(), b.data_ptr(), out.data_ptr(), stream))
    ref = oracle.from_f32(oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads()), oracle.F16)
    np.testing.assert_array_equal(out.view(torch.int16).numpy().view(np.uint16).reshape(ref.shape), ref)
