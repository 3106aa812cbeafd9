"""Compares the oracle's restated RNG and verifier with the reference's own conv-validation-wrappers.cpp,
compiled unmodified into oracle/_ref/ by oracle/Makefile (skipped where that library was not built)."""
import ctypes as C
import os
import tempfile

import numpy as np
import pytest

import oracle

REF = oracle.ref_lib()
pytestmark = pytest.mark.skipif(REF is None, reason="oracle/_ref/libconv-validation-wrappers.so not built")


def _capture_stdout(fn):
    """Runs fn while fd 1 is redirected to a file; returns what C code printed."""
    libc = C.CDLL(None)
    with tempfile.TemporaryFile(mode="w+b") as tmp:
        saved = os.dup(1)
        libc.fflush(None)
        os.dup2(tmp.fileno(), 1)
        try:
            fn()
            libc.fflush(None)
        finally:
            os.dup2(saved, 1)
            os.close(saved)
        tmp.seek(0)
        return tmp.read().decode()


@pytest.mark.parametrize("seed", [1, 2, 12345])
def test_random_streams_match(seed):
    REF.seedRandomValues(seed)
    ref_i = [REF.randomIntegerValue(-5, 5) for _ in range(200)]
    ref_f = [REF.randomFloatValue(-1, 1) for _ in range(200)]
    oracle.seed(seed)
    got_i = oracle.fill_random(200, False, -5, 5)
    got_f = oracle.fill_random(200, True, -1, 1)
    assert np.array_equal(np.asarray(ref_i, np.float32), got_i)
    assert np.array_equal(np.asarray(ref_f, np.float32), got_f)
    assert set(np.unique(got_i)).issubset(set(range(-5, 5)))   # integers in [-5, 4]
    # min == max: the constant (rand_type float scales it by 0.1)
    assert REF.randomIntegerValue(1, 1) == oracle.lib().orc_random_integer_value(1, 1) == 1.0
    assert REF.randomFloatValue(1, 1) == oracle.lib().orc_random_float_value(1, 1)


def _ref_verify_float(gpu, val, rms, ab, rel):
    g = np.ascontiguousarray(gpu, np.float32)
    v = np.ascontiguousarray(val, np.float32)
    fp = C.POINTER(C.c_float)
    REF.mcpuVerifyFloat.argtypes = [fp, fp, C.c_int64, C.c_int64, C.c_int64, fp, fp, C.c_int64, C.c_int64, C.c_int64,
                                    C.c_float, C.c_float, C.c_float, C.c_char]
    out = _capture_stdout(lambda: REF.mcpuVerifyFloat(g.ctypes.data_as(fp), g.ctypes.data_as(fp), 0, g.size, 1,
                                                      v.ctypes.data_as(fp), v.ctypes.data_as(fp), 0, v.size, 1,
                                                      rms, ab, rel, b"\x00"))
    line = [l for l in out.splitlines() if l.startswith("[")][-1]
    return [int(x) for x in line.strip("[]").split()]


@pytest.mark.parametrize("noise,thr", [(0.0, (3e-5, 100.0, 1e-6)), (1e-6, (3e-5, 100.0, 1e-6)), (1e-3, (3e-5, 1e-4, 100.0)),
                                       (1e-3, (1e-2, 100.0, 100.0)), (5e-2, (1e-3, 0.02, 100.0))])
def test_float_verdicts_match(noise, thr):
    rng = np.random.Generator(np.random.PCG64(7))
    val = rng.standard_normal(5000).astype(np.float32)
    val[::97] = 0.0                      # zero references only count in the histogram
    val[5] = np.inf                      # an infinite reference is replaced by +-65504
    gpu = (val + noise * rng.standard_normal(5000)).astype(np.float32)
    gpu[5] = 65504.0
    want = _ref_verify_float(gpu, val, *thr)
    got, _ = oracle.verify_float(gpu, val, *thr)
    assert got == want


def test_int_verdicts_match():
    ip, lp = C.POINTER(C.c_int32), C.POINTER(C.c_int64)
    REF.mcpuVerifyInt32Int64.argtypes = [ip, ip, C.c_int64, C.c_int64, C.c_int64, lp, lp, C.c_int64, C.c_int64,
                                         C.c_int64, C.c_char]
    rng = np.random.Generator(np.random.PCG64(9))
    val = rng.integers(-10**6, 10**6, 1000).astype(np.int64)
    for flip in (False, True):
        gpu = val.astype(np.int32)
        if flip:
            gpu[123] += 1
        out = _capture_stdout(lambda: REF.mcpuVerifyInt32Int64(gpu.ctypes.data_as(ip), gpu.ctypes.data_as(ip), 0,
                                                               gpu.size, 1, val.ctypes.data_as(lp),
                                                               val.ctypes.data_as(lp), 0, val.size, 1, b"\x00"))
        want = [int(x) for x in [l for l in out.replace("]", "]\n").splitlines() if l.startswith("[")][-1].strip("[]").split()]
        got, info = oracle.verify_int(gpu, val)
        assert got == want and info["mismatches"] == (1 if flip else 0)
