"""The code object a client loads itself: the library hands out an sm_100a cubin (rbGetKernelBinary, miirBufferGet)
and a launch description (RbKernelLaunch); a kernel launched from that image with the driver API must write exactly
what the library's own launch writes.

 - tests/cubin_client.c is such a client in plain C (dlopen of libcuda and of the library, cuModuleLoadData,
   cuLaunchKernelEx): compiled and run here for an fp16 GEMM;
 - the same through the Miir handle API for an implicit-GEMM convolution, with the driver calls made through ctypes.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle
from helpers import from_device, reference_random, to_device

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c_client_loads_the_cubin_and_matches_rbgemm(cuda_device, tmp_path):
    from rocmlir_b200 import _lib as L
    exe = str(tmp_path / "cubin_client")
    subprocess.run(["gcc", "-O1", "-I", os.path.join(ROOT, "include"), "-o", exe,
                    os.path.join(ROOT, "tests", "cubin_client.c"), "-ldl"], check=True)
    r = subprocess.run([exe, L.LIB_PATH], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.startswith("MATCH"), r.stdout + r.stderr
    assert "gemm_tcgen05_kernel" in r.stdout


class _LaunchAttr(C.Structure):
    _fields_ = [("id", C.c_int), ("pad", C.c_char * 4), ("x", C.c_uint), ("y", C.c_uint), ("z", C.c_uint), ("rest", C.c_char * 52)]


class _LaunchConfig(C.Structure):
    _fields_ = [("gx", C.c_uint), ("gy", C.c_uint), ("gz", C.c_uint), ("bx", C.c_uint), ("by", C.c_uint), ("bz", C.c_uint),
                ("smem", C.c_uint), ("stream", C.c_void_p), ("attrs", C.POINTER(_LaunchAttr)), ("nattrs", C.c_uint)]


def driver_launch(image: bytes, kl, stream: int):
    """cuModuleLoadData + cuModuleGetFunction + cuLaunchKernelEx of the kernel described by an RbKernelLaunch."""
    cu = C.CDLL("libcuda.so.1")
    mod, fn = C.c_void_p(), C.c_void_p()
    buf = C.create_string_buffer(image, len(image))
    assert cu.cuModuleLoadData(C.byref(mod), buf) == 0
    assert cu.cuModuleGetFunction(C.byref(fn), mod, kl.symbol) == 0, kl.symbol
    assert cu.cuFuncSetAttribute(fn, 8, int(kl.dynamic_smem)) == 0     # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES
    attr = _LaunchAttr(id=4, x=kl.cluster, y=1, z=1)                   # CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION
    cfg = _LaunchConfig(kl.grid, 1, 1, kl.block, 1, 1, kl.dynamic_smem, stream, C.pointer(attr), 1)
    base = C.addressof(kl) + type(kl).params.offset
    params = (C.c_void_p * 4)(*[base + kl.param_offset[i] for i in range(4)])
    assert cu.cuLaunchKernelEx(C.byref(cfg), fn, params, None) == 0
    assert cu.cuCtxSynchronize() == 0
    assert cu.cuModuleUnload(mod) == 0


@pytest.mark.parametrize("op,direction", [("conv", 0), ("conv_bwd_data", 1)])
def test_miir_code_object_launched_by_the_client(cuda_device, op, direction):
    """A forward 3x3 NHWC convolution (implicit GEMM: one kernel, the A tiles fetched by im2col TMA loads) and a
    pointwise backward-data convolution, launched by the client from miirBufferGet's cubin: equal to miirLaunch and to
    the oracle on integer-valued data."""
    import torch
    from rocmlir_b200 import _lib as L
    from rocmlir_b200 import miir
    y = 3 if direction == 0 else 1
    pad = 1 if direction == 0 else 0
    ocfg = oracle.Conv(n=4, c=64, k=64, h=14, w=14, y=y, x=y, pad_h=pad, pad_w=pad, fil_layout="gkyxc", in_layout="nhwgc",
                       out_layout="nhwgk")
    if direction == 1:      # the filter of a pointwise backward-data GEMM is used in place when stored (k, c)
        ocfg.fil_layout = "gyxkc"
    (ff, fraw), (inf, iraw), (of, oraw) = reference_random([(ocfg.numel("fil"),), (ocfg.numel("in"),), (ocfg.numel("out"),)],
                                                           oracle.F16, seed=1)
    want = oracle.from_f32(oracle.conv_f32(ocfg, direction, ff, inf, of, threads=oracle.max_threads()), oracle.F16)
    res = {0: "out", 1: "in"}[direction]
    opts = (f"--operation {op} --arch sm_100a --in_type fp16 --fil_type fp16 --out_type fp16 --fil_layout {ocfg.fil_layout} "
            f"--in_layout nhwgc --out_layout nhwgk --batchsize 4 --groupsize 1 --in_channels 64 --out_channels 64 --in_h 14 "
            f"--in_w 14 --out_h 14 --out_w 14 --fil_h {y} --fil_w {y} --padding_h {pad} --padding_w {pad}")
    t1 = {"fil": to_device(fraw, oracle.F16), "in": to_device(iraw, oracle.F16), "out": to_device(oraw, oracle.F16)}
    t2 = {k: v.clone() for k, v in t1.items()}
    t2[res].fill_(3.0)
    with miir.Handle(opts) as h:
        h.lower_bin()
        assert h.workspace_size == 0
        h.launch(t1["fil"], t1["in"], t1["out"])                      # the library launches
        image = h.buffer()
        kl = h.kernel_launch(t2["fil"], t2["in"], t2["out"])
        glob, loc = h.execution_dims()
    torch.cuda.synchronize()
    assert image[:4] == b"\x7fELF"
    assert (kl.grid * kl.block, kl.block) == (glob, loc)              # attrs[0..1] keep the reference's meaning
    driver_launch(image, kl, torch.cuda.current_stream().cuda_stream)  # the client launches
    assert L.kernel_status() == 0
    assert torch.equal(t1[res], t2[res])
    np.testing.assert_array_equal(from_device(t2[res], oracle.F16).ravel(), want.ravel())


def test_problems_of_several_kernels_have_no_single_kernel_description(cuda_device):
    import torch
    from rocmlir_b200 import _lib as L
    a = torch.zeros((64, 8192), dtype=torch.float16, device="cuda")
    b = torch.zeros((8192, 576), dtype=torch.float16, device="cuda")
    c = torch.zeros((64, 576), dtype=torch.float16, device="cuda")
    p = L.RbGemmProblem(1, 64, 576, 8192, 0, 0, 0, L.F16, L.F16, 0)       # few tiles, long K: a K split + reduction pass
    kl = L.RbKernelLaunch()
    st = L.lib().rbGemmEncodeLaunch(C.byref(p), None, a.data_ptr(), b.data_ptr(), c.data_ptr(), C.byref(kl))
    assert st == L.UNSUPPORTED and b"several kernels" in L.lib().rbGetLastError()
