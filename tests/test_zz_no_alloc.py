"""rbGemmNoAlloc: the GEMM for callers that may not allocate device memory (allocator callbacks, plugins that
are handed their buffers, loops that must not take the allocator lock). Its scratch is a fixed array inside the
library, so this test checks through the C ABI that (1) it computes exactly what rbGemm computes with a caller
workspace, on two calls in a row that reuse the scratch, and (2) it refuses a problem whose scratch need is larger
than the built-in array. Collected last on purpose: a failure here cannot hide other tests behind `-x`."""
import ctypes as C

import numpy as np
import pytest

import oracle
from helpers import reference_random, to_device, torch_dtype

pytestmark = pytest.mark.gpu

# problems that need scratch: a K split (few tiles, long K), a padded operand (K = 769), f32 hi/lo planes
CASES = [(1, 64, 576, 8192, oracle.F16), (1, 1024, 512, 769, oracle.F16), (1, 200, 300, 256, oracle.F32)]


def _run(entry, prob, a, b, out, ws=None, epi=None):
    import torch
    from rocmlir_b200 import _lib as L
    lib = L.lib()
    stream = torch.cuda.current_stream().cuda_stream
    e = C.byref(epi) if epi is not None else None
    if entry == "noalloc":
        st = lib.rbGemmNoAlloc(C.byref(prob), e, a.data_ptr(), b.data_ptr(), out.data_ptr(), stream)
    else:
        st = lib.rbGemm(C.byref(prob), e, a.data_ptr(), b.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                        stream)
    L.check(st)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0


@pytest.mark.parametrize("g,m,n,k,code", CASES)
def test_no_alloc_matches_workspace_entry_point_twice(cuda_device, g, m, n, k, code):
    import torch
    from rocmlir_b200 import _lib as L
    prob = L.RbGemmProblem(g, m, n, k, 0, 0, 0, code, code, 0)
    need = L.lib().rbGemmWorkspaceSize(C.byref(prob))
    assert 0 < need <= (16 << 20), "the case must exercise the scratch and fit the built-in array"
    (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], code, seed=1)
    a, b = to_device(araw, code), to_device(braw, code)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    want = torch.empty((g, m, n), dtype=torch_dtype(code), device="cuda")
    _run("workspace", prob, a, b, want, ws)
    for call in range(2):  # the second call finds the first call's leftovers in the scratch
        got = torch.full((g, m, n), 7.0, dtype=torch_dtype(code), device="cuda")
        _run("noalloc", prob, a, b, got)
        # same kernels, same order of operations: the tolerance is exact equality
        assert torch.equal(got, want), f"call {call}: rbGemmNoAlloc differs from rbGemm"
    # and both agree with the oracle on this integer-valued data
    ref = oracle.from_f32(oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads()), code)
    from helpers import from_device
    np.testing.assert_array_equal(from_device(want, code).reshape(ref.shape), ref)


def test_no_alloc_carries_the_fused_epilogue(cuda_device):
    """The same entry point with a fused tail, relu(C + bias[N]) rounded through f16, on a problem whose K split puts
    the epilogue into the reduction pass over the built-in scratch: equal to rbGemm with a caller workspace, twice, and
    equal to the oracle's op-by-op restatement on integer-valued data."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200.gemm import Epilogue
    from helpers import from_device
    g, m, n, k = 1, 64, 576, 8192
    prob = L.RbGemmProblem(g, m, n, k, 0, 0, 0, L.F16, L.F16, 0)
    need = L.lib().rbGemmWorkspaceSize(C.byref(prob))
    assert 0 < need <= (16 << 20)
    (af, araw), (bf, braw) = reference_random([(g, m, k), (g, k, n)], oracle.F16, seed=1)
    bias = (np.arange(n, dtype=np.float32) % 9) - 4
    a, b = to_device(araw, oracle.F16), to_device(braw, oracle.F16)
    bias_dev = to_device(oracle.from_f32(bias, oracle.F16), oracle.F16)     # kept alive: the C struct only holds its address
    epi = Epilogue(bias=bias_dev, relu=True, mid_type=oracle.F16).to_c()
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    want = torch.empty((g, m, n), dtype=torch.float16, device="cuda")
    _run("workspace", prob, a, b, want, ws, epi)
    for call in range(2):
        got = torch.full((g, m, n), 7.0, dtype=torch.float16, device="cuda")
        _run("noalloc", prob, a, b, got, epi=epi)
        assert torch.equal(got, want), f"call {call}: rbGemmNoAlloc with an epilogue differs from rbGemm"
    acc = oracle.gemm_f32(af, bf, g, m, n, k, threads=oracle.max_threads())
    ref = oracle.from_f32(oracle.epilogue(acc, n, bias=bias, relu=True, mid_type=oracle.F16), oracle.F16)
    np.testing.assert_array_equal(from_device(want, oracle.F16).reshape(ref.shape), ref)


def test_no_alloc_rejects_oversized_scratch_need(cuda_device):
    from rocmlir_b200 import _lib as L
    prob = L.RbGemmProblem(1, 4096, 4096, 4096, 0, 0, 0, L.F32, L.F32, 0)  # hi/lo planes: 4 x 64 MiB
    assert L.lib().rbGemmWorkspaceSize(C.byref(prob)) > (16 << 20)
    dummy = C.c_void_p(256)
    st = L.lib().rbGemmNoAlloc(C.byref(prob), None, dummy, dummy, dummy, None)
    assert st == L.WORKSPACE_TOO_SMALL
    msg = L.lib().rbGetLastError().decode()
    assert "scratch" in msg and str(16 << 20) in msg
