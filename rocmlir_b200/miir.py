"""Python mirror of the string-configured handle API (include/miir_b200.h), the counterpart of
mlir/tools/rocmlir-lib/Miir.h:50-101 as exercised by mlir/tools/rocmlir-lib/rocmlir-lib-test.cpp:30-110."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

from . import _lib as L

SUCCESS, INVALID_PARAM, INVALID_MODULE, BUILD_FAILURE = range(4)
VERSION_FLAT = 6


class MiirError(RuntimeError):
    def __init__(self, status: int, what: str):
        names = ["MIIR_SUCCESS", "MIIR_INVALID_PARAM", "MIIR_INVALID_MODULE", "MIIR_BUILD_FAILURE"]
        super().__init__(f"{what}: {names[status] if 0 <= status < 4 else status}")
        self.status = status


class Handle:
    """One operation configured by an option string. `Handle(options)` raises ValueError where the C call returns
    NULL (missing keys, inconsistent dimensions, foreign architecture, no kernel)."""

    def __init__(self, options: str):
        self._h = L.lib().miirCreateHandle(options.encode())
        if not self._h:
            raise ValueError("miirCreateHandle returned NULL for: " + options)

    def close(self) -> None:
        if self._h:
            L.lib().miirDestroyHandle(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def kernel_count(self) -> int:
        return L.lib().miirGetKernelCount(self._h)

    @property
    def workspace_size(self) -> int:
        return L.lib().miirGetWorkspaceSize(self._h)

    def lower_tuning_params(self) -> None:
        st = L.lib().miirLowerTuningParams(self._h)
        if st != SUCCESS:
            raise MiirError(st, "miirLowerTuningParams")

    def lower_bin(self) -> None:
        st = L.lib().miirLowerBin(self._h)
        if st != SUCCESS:
            raise MiirError(st, "miirLowerBin")

    def _two_call(self, fn, what: str) -> bytes:
        size = C.c_size_t(0)
        st = fn(self._h, None, C.byref(size))
        if st != SUCCESS:
            raise MiirError(st, what + "(size)")
        buf = C.create_string_buffer(size.value)
        st = fn(self._h, buf, C.byref(size))
        if st != SUCCESS:
            raise MiirError(st, what + "(copy)")
        return buf.raw[: size.value]

    def buffer(self) -> bytes:
        """The code object (an sm_100a cubin). Two-call protocol: size first, then the bytes."""
        return self._two_call(L.lib().miirBufferGet, "miirBufferGet")

    def descriptor(self) -> bytes:
        """The relocatable launch descriptor for launch_from_buffer."""
        return self._two_call(L.lib().miirDescriptorGet, "miirDescriptorGet")

    def kernel_launch(self, arg0, arg1, arg2) -> "L.RbKernelLaunch":
        """Name, cluster size, shared memory and parameter block of the handle's kernel for these device buffers."""
        out = L.RbKernelLaunch()
        ptr = lambda t: None if t is None else t.data_ptr()
        st = L.lib().miirGetKernelLaunch(self._h, ptr(arg0), ptr(arg1), ptr(arg2), C.byref(out))
        if st != SUCCESS:
            raise MiirError(st, "miirGetKernelLaunch (" + L.lib().rbGetLastError().decode() + ")")
        return out

    def arg_sizes(self) -> Tuple[int, int, int, int]:
        """Bytes of the operation's tensors in argument order (the fourth is attention's O, else 0)."""
        sizes = (C.c_size_t * 4)()
        st = L.lib().miirGetArgSizes(self._h, sizes)
        if st != SUCCESS:
            raise MiirError(st, "miirGetArgSizes")
        return tuple(int(v) for v in sizes)

    def execution_dims(self) -> Tuple[int, int]:
        g, l = C.c_size_t(0), C.c_size_t(0)
        st = L.lib().miirGetExecutionDims(self._h, C.byref(g), C.byref(l))
        if st != SUCCESS:
            raise MiirError(st, "miirGetExecutionDims")
        return g.value, l.value

    def launch(self, arg0, arg1, arg2, extra=None, workspace=None, stream: Optional[int] = None) -> None:
        """Tensors are torch CUDA tensors (or None); order = the reference's kernel arguments."""
        import torch
        ptr = lambda t: None if t is None else t.data_ptr()
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        st = L.lib().miirLaunch(self._h, ptr(arg0), ptr(arg1), ptr(arg2), ptr(extra), ptr(workspace), ws_bytes, s)
        if st != SUCCESS:
            raise MiirError(st, "miirLaunch (" + L.lib().rbGetLastError().decode() + ")")


def launch_from_buffer(blob: bytes, arg0, arg1, arg2, extra=None, workspace=None, stream: Optional[int] = None) -> None:
    import torch
    ptr = lambda t: None if t is None else t.data_ptr()
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    s = torch.cuda.current_stream().cuda_stream if stream is None else stream
    st = L.lib().miirLaunchFromBuffer(blob, len(blob), ptr(arg0), ptr(arg1), ptr(arg2), ptr(extra), ptr(workspace),
                                      ws_bytes, s)
    if st != SUCCESS:
        raise MiirError(st, "miirLaunchFromBuffer (" + L.lib().rbGetLastError().decode() + ")")
