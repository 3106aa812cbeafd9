"""Python mirror of the MLIR C API surface (include/mlir_c_b200.h): a module of `migraphx.*` ops given as text goes
through the three MIGraphX pipelines and answers the getters MIGraphX uses - the call sequence of
mlir/test/CAPI/mixr_full.c:176-330 - and can be launched on torch CUDA tensors."""
from __future__ import annotations

import ctypes as C
import struct
from typing import List, Optional, Sequence, Tuple

from . import _lib as L


class _Ptr(C.Structure):
    _fields_ = [("ptr", C.c_void_p)]


class _StringRef(C.Structure):
    _fields_ = [("data", C.c_char_p), ("length", C.c_size_t)]


_bound = False


def _lib():
    global _bound
    l = L.lib()
    if not _bound:
        l.mlirContextCreate.restype = _Ptr
        l.mlirContextDestroy.argtypes = [_Ptr]
        l.mlirModuleCreateParse.restype = _Ptr
        l.mlirModuleCreateParse.argtypes = [_Ptr, _StringRef]
        l.mlirModuleGetOperation.restype = _Ptr
        l.mlirModuleGetOperation.argtypes = [_Ptr]
        l.mlirModuleDestroy.argtypes = [_Ptr]
        l.mlirPassManagerCreate.restype = _Ptr
        l.mlirPassManagerCreate.argtypes = [_Ptr]
        l.mlirPassManagerDestroy.argtypes = [_Ptr]
        l.mlirPassManagerRunOnOp.restype = C.c_int8
        l.mlirPassManagerRunOnOp.argtypes = [_Ptr, _Ptr]
        for n in ("mlirMIGraphXAddHighLevelPipeline", "mlirMIGraphXAddApplicabilityPipeline"):
            getattr(l, n).argtypes = [_Ptr]
            getattr(l, n).restype = None
        l.mlirMIGraphXAddBackendPipeline.restype = C.c_bool
        l.mlirMIGraphXAddBackendPipeline.argtypes = [_Ptr, C.c_char_p]
        l.mlirGetKernelInfo.argtypes = [_Ptr, C.POINTER(C.c_int), C.c_void_p]
        l.mlirGetKernelInfo.restype = None
        l.mlirGetKernelAttrs.argtypes = [_Ptr, C.POINTER(C.c_uint32)]
        l.mlirGetKernelAttrs.restype = None
        l.mlirGetBinary.restype = C.c_bool
        l.mlirGetBinary.argtypes = [_Ptr, C.POINTER(C.c_size_t), C.c_char_p]
        l.rbModuleGetDiagnostic.restype = C.c_char_p
        l.rbModuleGetDiagnostic.argtypes = [_Ptr]
        l.rbModuleGetWorkspaceSize.restype = C.c_size_t
        l.rbModuleGetWorkspaceSize.argtypes = [_Ptr]
        l.rbModuleLaunch.restype = C.c_int
        l.rbModuleLaunch.argtypes = [_Ptr, C.POINTER(C.c_void_p), C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]
        l.rbModuleGetKernelLaunch.restype = C.c_int
        l.rbModuleGetKernelLaunch.argtypes = [_Ptr, C.POINTER(C.c_void_p), C.c_size_t, C.POINTER(L.RbKernelLaunch)]
        l.mlirRockTuningGetKey.restype = C.c_size_t
        l.mlirRockTuningGetKey.argtypes = [_Ptr, C.c_char_p, C.c_size_t]
        l.mlirRockTuningSetFromStr.restype = C.c_bool
        l.mlirRockTuningSetFromStr.argtypes = [_Ptr, _StringRef]
        _bound = True
    return l


class PipelineError(RuntimeError):
    pass


class Module:
    """A parsed module. `with Module(text) as m: m.high_level(); m.backend("sm_100a"); m.launch([...tensors...])`."""

    def __init__(self, text: str):
        l = _lib()
        self._ctx = l.mlirContextCreate()
        raw = text.encode()
        self._m = l.mlirModuleCreateParse(self._ctx, _StringRef(raw, len(raw)))
        if not self._m.ptr:
            msg = l.rbGetLastError().decode()
            l.mlirContextDestroy(self._ctx)
            raise ValueError("mlirModuleCreateParse: " + msg)

    def close(self):
        if getattr(self, "_m", None) is not None and self._m.ptr:
            _lib().mlirModuleDestroy(self._m)
            _lib().mlirContextDestroy(self._ctx)
            self._m.ptr = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _run(self, add) -> None:
        l = _lib()
        pm = l.mlirPassManagerCreate(self._ctx)
        try:
            add(pm)
            ok = l.mlirPassManagerRunOnOp(pm, l.mlirModuleGetOperation(self._m))
        finally:
            l.mlirPassManagerDestroy(pm)
        if not ok:
            raise PipelineError(l.rbModuleGetDiagnostic(self._m).decode())

    def high_level(self) -> None:
        self._run(_lib().mlirMIGraphXAddHighLevelPipeline)

    def applicability(self) -> None:
        self._run(_lib().mlirMIGraphXAddApplicabilityPipeline)

    def backend(self, arch: str = "sm_100a") -> None:
        def add(pm):
            if not _lib().mlirMIGraphXAddBackendPipeline(pm, arch.encode()):
                raise PipelineError(f"architecture {arch!r} is not accepted")
        self._run(add)

    def set_perf_config(self, perf: str) -> bool:
        raw = perf.encode()
        return bool(_lib().mlirRockTuningSetFromStr(self._m, _StringRef(raw, len(raw))))

    @property
    def key(self) -> Optional[str]:
        buf = C.create_string_buffer(2048)
        n = _lib().mlirRockTuningGetKey(self._m, buf, 2048)
        return None if n == C.c_size_t(-1).value else buf.raw[:n].decode()

    def kernel_info(self) -> Tuple[List[List[int]], str]:
        """([dims of argument 0 in memory order, ..., dims of the result], kernel name): the blob of mlirGetKernelInfo."""
        size = C.c_int(0)
        _lib().mlirGetKernelInfo(self._m, C.byref(size), None)
        buf = C.create_string_buffer(size.value)
        _lib().mlirGetKernelInfo(self._m, None, buf)
        raw = buf.raw
        nargs = struct.unpack_from("<i", raw, 0)[0]
        pos, args = 4, []
        for _ in range(nargs):
            rank = struct.unpack_from("<i", raw, pos)[0]
            pos += 4
            args.append(list(struct.unpack_from(f"<{rank}i", raw, pos)))
            pos += 4 * rank
        return args, raw[pos:].decode()

    def kernel_attrs(self) -> Tuple[int, int]:
        a = (C.c_uint32 * 2)(0, 0)
        _lib().mlirGetKernelAttrs(self._m, a)
        return int(a[0]), int(a[1])      # block size, grid size

    def binary(self) -> bytes:
        size = C.c_size_t(0)
        if not _lib().mlirGetBinary(self._m, C.byref(size), None):
            raise PipelineError("mlirGetBinary: run the backend pipeline first")
        buf = C.create_string_buffer(size.value)
        assert _lib().mlirGetBinary(self._m, None, buf)
        return buf.raw

    @property
    def workspace_size(self) -> int:
        return int(_lib().rbModuleGetWorkspaceSize(self._m))

    def _args(self, tensors: Sequence):
        return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])

    def launch(self, tensors: Sequence, workspace=None) -> None:
        """tensors: CUDA tensors in kernel-argument order (the function's arguments, then its result)."""
        import torch
        need = self.workspace_size
        if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
            workspace = torch.empty(need, dtype=torch.uint8, device=tensors[0].device)
        stream = torch.cuda.current_stream(tensors[0].device).cuda_stream
        L.check(_lib().rbModuleLaunch(self._m, self._args(tensors), len(tensors), workspace.data_ptr() if need else None,
                                      workspace.numel() * workspace.element_size() if need else 0, stream))

    def kernel_launch(self, tensors: Sequence) -> "L.RbKernelLaunch":
        out = L.RbKernelLaunch()
        L.check(_lib().rbModuleGetKernelLaunch(self._m, self._args(tensors), len(tensors), C.byref(out)))
        return out
