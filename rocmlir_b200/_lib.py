"""ctypes binding of librocmlir_b200.so (the C ABI declared in include/rocmlir_b200.h).

There is no CPU path: importing works anywhere, but every compute call needs the built
library and an sm_100 GPU and raises otherwise.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librocmlir_b200.so")

# RbDType
F32, F16, BF16, I8, I32, F8E4M3, F8E5M2, F8E4M3_E5M2, F8E5M2_E4M3 = range(9)
DTYPE_NAMES = {F32: "f32", F16: "f16", BF16: "bf16", I8: "i8", I32: "i32", F8E4M3: "fp8", F8E5M2: "bf8", F8E4M3_E5M2: "fp8_bf8",
               F8E5M2_E4M3: "bf8_fp8"}
DTYPE_BYTES = {F32: 4, F16: 2, BF16: 2, I8: 1, I32: 4, F8E4M3: 1, F8E5M2: 1, F8E4M3_E5M2: 1, F8E5M2_E4M3: 1}

# RbStatus
SUCCESS, INVALID_PARAM, UNSUPPORTED, WORKSPACE_TOO_SMALL, CUDA_ERROR, KERNEL_TIMEOUT = range(6)
STATUS_NAMES = ["RB_SUCCESS", "RB_INVALID_PARAM", "RB_UNSUPPORTED", "RB_WORKSPACE_TOO_SMALL", "RB_CUDA_ERROR",
                "RB_KERNEL_TIMEOUT"]

EPI_ALPHA, EPI_COL_SCALE, EPI_BIAS, EPI_RELU, EPI_REQUANT, EPI_ROUND_MID = 1, 2, 4, 8, 16, 32
EPI_CLIP, EPI_RESIDUAL, EPI_BIAS_ROW, EPI_BIAS_SCALAR, EPI_ZP_IN, EPI_ZP_OUT = 64, 128, 256, 512, 1024, 2048
EPI_UNARY = 4096
# RbUnary
UNARY = {n: i + 1 for i, n in enumerate(("abs", "ceil", "erf", "exp", "floor", "log", "neg", "recip", "rsqrt", "sigmoid",
                                          "sqrt", "tanh"))}


class RbEpilogue(C.Structure):
    _fields_ = [("flags", C.c_uint32), ("alpha", C.c_float), ("out_recip", C.c_float), ("mid_type", C.c_int32),
                ("bias_type", C.c_int32), ("col_scale", C.c_void_p), ("bias", C.c_void_p), ("clip_lo", C.c_float),
                ("clip_hi", C.c_float), ("in_zero", C.c_float), ("out_zero", C.c_int32), ("residual", C.c_void_p),
                ("res_type", C.c_int32), ("unary", C.c_int32)]


class RbGemmProblem(C.Structure):
    _fields_ = [("g", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("trans_a", C.c_int32),
                ("trans_b", C.c_int32), ("trans_c", C.c_int32), ("ab_type", C.c_int32), ("c_type", C.c_int32),
                ("f32_mode", C.c_int32), ("store_method", C.c_int32)]


class RbConvProblem(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n", "g", "c", "k", "h", "w", "y", "x", "stride_h", "stride_w", "dil_h",
                                         "dil_w", "pad_h", "pad_w", "pad_h_r", "pad_w_r", "ho", "wo", "data_type",
                                         "direction", "f32_mode")] + \
               [("fil_layout", C.c_char * 8), ("in_layout", C.c_char * 8), ("out_layout", C.c_char * 8)]


class RbConv3dProblem(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n", "g", "c", "k", "d", "h", "w", "z", "y", "x", "stride_d", "stride_h",
                                         "stride_w", "dil_d", "dil_h", "dil_w", "pad_d", "pad_h", "pad_w", "pad_d_r",
                                         "pad_h_r", "pad_w_r", "dout", "ho", "wo", "data_type", "direction",
                                         "f32_mode")] + \
               [("fil_layout", C.c_char * 8), ("in_layout", C.c_char * 8), ("out_layout", C.c_char * 8)]


class RbAttentionProblem(C.Structure):
    _fields_ = [("g", C.c_int32), ("seq_q", C.c_int32), ("seq_k", C.c_int32), ("head_qk", C.c_int32),
                ("head_v", C.c_int32), ("trans_q", C.c_int32), ("trans_k", C.c_int32), ("trans_v", C.c_int32),
                ("trans_o", C.c_int32), ("data_type", C.c_int32), ("has_scale", C.c_int32), ("scale", C.c_float),
                ("causal", C.c_int32), ("mask_fill", C.c_float), ("bias", C.c_void_p), ("mask", C.c_void_p),
                ("scale_tensor", C.c_void_p), ("quant_bias", C.c_void_p), ("quant_scale", C.c_void_p)]


class RbGemmConfigInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("tile_m", "tile_n", "tile_k", "ctas", "stages", "splits", "stream_k")] + \
               [(n, C.c_uint32) for n in ("grid", "block", "dynamic_smem", "variant")] + \
               [("kpr", C.c_int32), ("stages_epi_vec", C.c_int32), ("dynamic_smem_epi_vec", C.c_uint32)]


class RbKernelLaunch(C.Structure):
    _fields_ = [("symbol", C.c_char * 160), ("grid", C.c_uint32), ("block", C.c_uint32), ("cluster", C.c_uint32),
                ("dynamic_smem", C.c_uint32), ("param_count", C.c_uint32), ("param_offset", C.c_uint32 * 4),
                ("param_size", C.c_uint32 * 4), ("reserved", C.c_uint32 * 3),
                ("_pad", C.c_ubyte * 32),      # the C struct aligns `params` to 64 bytes: offset 256
                ("params", C.c_ubyte * 2048)]


class _Handle(C.Structure):
    """The one-pointer opaque structs of the tuning API (RbProblem, RbTuningSpace, RbTuningParam, RbTuningTable)."""
    _fields_ = [("ptr", C.c_void_p)]


class RbError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"{STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else status}: {msg}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m rocmlir_b200.build` (no CPU fallback exists)")
        l = C.CDLL(LIB_PATH)
        l.rbGemmWorkspaceSize.restype = C.c_size_t
        l.rbGemmWorkspaceSize.argtypes = [C.POINTER(RbGemmProblem)]
        l.rbGemm.restype = C.c_int
        l.rbGemm.argtypes = [C.POINTER(RbGemmProblem), C.POINTER(RbEpilogue), C.c_void_p, C.c_void_p, C.c_void_p,
                             C.c_void_p, C.c_size_t, C.c_void_p]
        l.rbGemmNoAlloc.restype = C.c_int
        l.rbGemmNoAlloc.argtypes = [C.POINTER(RbGemmProblem), C.POINTER(RbEpilogue), C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p]
        l.rbGemmHost.restype = C.c_int
        l.rbGemmHost.argtypes = [C.POINTER(RbGemmProblem), C.POINTER(RbEpilogue), C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p]
        l.rbConvWorkspaceSize.restype = C.c_size_t
        l.rbConvWorkspaceSize.argtypes = [C.POINTER(RbConvProblem)]
        l.rbConvKernelCount.restype = C.c_int
        l.rbConvKernelCount.argtypes = [C.POINTER(RbConvProblem)]
        l.rbConv.restype = C.c_int
        l.rbConv.argtypes = [C.POINTER(RbConvProblem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                             C.c_void_p]
        l.rbConvEpiWorkspaceSize.restype = C.c_size_t
        l.rbConvEpiWorkspaceSize.argtypes = [C.POINTER(RbConvProblem), C.c_int32]
        l.rbConvEpi.restype = C.c_int
        l.rbConvEpi.argtypes = [C.POINTER(RbConvProblem), C.POINTER(RbEpilogue), C.c_int32, C.c_void_p, C.c_void_p,
                                C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        l.rbConv3dWorkspaceSize.restype = C.c_size_t
        l.rbConv3dWorkspaceSize.argtypes = [C.POINTER(RbConv3dProblem)]
        l.rbConv3d.restype = C.c_int
        l.rbConv3d.argtypes = [C.POINTER(RbConv3dProblem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                               C.c_void_p]
        l.rbAttention.restype = C.c_int
        l.rbAttention.argtypes = [C.POINTER(RbAttentionProblem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_void_p]
        l.rbAttentionWorkspaceSize.restype = C.c_size_t
        l.rbAttentionWorkspaceSize.argtypes = [C.POINTER(RbAttentionProblem)]
        l.rbAttentionWs.restype = C.c_int
        l.rbAttentionWs.argtypes = [C.POINTER(RbAttentionProblem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_size_t, C.c_void_p]
        l.rbUnpackInt4.restype = C.c_int
        l.rbUnpackInt4.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_void_p]
        l.rbGemmGemmWorkspaceSize.restype = C.c_size_t
        l.rbGemmGemmWorkspaceSize.argtypes = [C.c_int32] * 6
        l.rbGemmGemm.restype = C.c_int
        l.rbGemmGemm.argtypes = [C.c_int32] * 6 + [C.c_void_p] * 5 + [C.c_size_t, C.c_void_p]
        l.rbSetGemmVariant.restype = None
        l.rbSetGemmVariant.argtypes = [C.c_int]
        l.rbGetGemmVariant.restype = C.c_int
        l.rbGetGemmVariant.argtypes = []
        l.rbGemmGetConfig.restype = C.c_int
        l.rbGemmGetConfig.argtypes = [C.POINTER(RbGemmProblem), C.POINTER(RbGemmConfigInfo)]
        l.rbConvGetGemmProblem.restype = C.c_int
        l.rbConvGetGemmProblem.argtypes = [C.POINTER(RbConvProblem), C.POINTER(RbGemmProblem)]
        # include/miir_b200.h
        l.miirCreateHandle.restype = C.c_void_p
        l.miirCreateHandle.argtypes = [C.c_char_p]
        for name in ("miirGetKernelCount", "miirGetWorkspaceSize", "miirLowerTuningParams", "miirLowerBin",
                     "miirDestroyHandle"):
            getattr(l, name).restype = C.c_int
            getattr(l, name).argtypes = [C.c_void_p]
        l.miirBufferGet.restype = C.c_int
        l.miirBufferGet.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_size_t)]
        l.miirGetArgSizes.restype = C.c_int
        l.miirGetArgSizes.argtypes = [C.c_void_p, C.POINTER(C.c_size_t)]
        l.miirGetExecutionDims.restype = C.c_int
        l.miirGetExecutionDims.argtypes = [C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        l.miirDescriptorGet.restype = C.c_int
        l.miirDescriptorGet.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_size_t)]
        l.miirGetKernelLaunch.restype = C.c_int
        l.miirGetKernelLaunch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(RbKernelLaunch)]
        l.rbGetKernelBinary.restype = C.c_int
        l.rbGetKernelBinary.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]
        l.rbGemmEncodeLaunch.restype = C.c_int
        l.rbGemmEncodeLaunch.argtypes = [C.POINTER(RbGemmProblem), C.POINTER(RbEpilogue), C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.POINTER(RbKernelLaunch)]
        l.rbConvEncodeLaunch.restype = C.c_int
        l.rbConvEncodeLaunch.argtypes = [C.POINTER(RbConvProblem), C.POINTER(RbEpilogue), C.c_int32, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.POINTER(RbKernelLaunch)]
        l.miirLaunch.restype = C.c_int
        l.miirLaunch.argtypes = [C.c_void_p] * 6 + [C.c_size_t, C.c_void_p]
        l.miirLaunchFromBuffer.restype = C.c_int
        l.miirLaunchFromBuffer.argtypes = [C.c_char_p, C.c_size_t] + [C.c_void_p] * 5 + [C.c_size_t, C.c_void_p]
        # include/rocmlir_b200_tuning.h
        l.rbProblemCreate.restype = _Handle
        l.rbProblemCreate.argtypes = [C.c_char_p]
        l.rbProblemFromGemm.restype = _Handle
        l.rbProblemFromGemm.argtypes = [C.POINTER(RbGemmProblem)]
        l.rbProblemFromConv.restype = _Handle
        l.rbProblemFromConv.argtypes = [C.POINTER(RbConvProblem)]
        l.rbProblemFromAttention.restype = _Handle
        l.rbProblemFromAttention.argtypes = [C.POINTER(RbAttentionProblem)]
        l.rbProblemDestroy.restype = None
        l.rbProblemDestroy.argtypes = [_Handle]
        l.rbProblemGetPerfConfig.restype = C.c_size_t
        l.rbProblemGetPerfConfig.argtypes = [_Handle, C.c_char_p, C.c_size_t]
        l.rbProblemGetVariant.restype = C.c_uint32
        l.rbProblemGetVariant.argtypes = [_Handle]
        l.rbTuningSpaceCreate.restype = _Handle
        l.rbTuningSpaceCreate.argtypes = [_Handle, C.c_int]
        l.rbTuningGetNumParams.restype = C.c_uint
        l.rbTuningGetNumParams.argtypes = [_Handle]
        l.rbTuningParamCreate.restype = _Handle
        l.rbTuningParamCreate.argtypes = []
        l.rbTuningParamDestroy.restype = None
        l.rbTuningParamDestroy.argtypes = [_Handle]
        l.rbTuningSpaceDestroy.restype = None
        l.rbTuningSpaceDestroy.argtypes = [_Handle]
        l.rbTuningParamGet.restype = C.c_bool
        l.rbTuningParamGet.argtypes = [_Handle, C.c_uint, _Handle]
        l.rbTuningParamGetQuick.restype = C.c_bool
        l.rbTuningParamGetQuick.argtypes = [_Handle, C.c_uint, _Handle]
        l.rbTuningParamToString.restype = C.c_size_t
        l.rbTuningParamToString.argtypes = [_Handle, C.c_char_p, C.c_size_t]
        l.rbTuningSetParam.restype = C.c_bool
        l.rbTuningSetParam.argtypes = [_Handle, _Handle]
        l.rbTuningSetFromStr.restype = C.c_bool
        l.rbTuningSetFromStr.argtypes = [_Handle, C.c_char_p, C.c_size_t]
        l.rbTuningTableCreate.restype = _Handle
        l.rbTuningTableCreate.argtypes = []
        l.rbTuningTableDestroy.restype = None
        l.rbTuningTableDestroy.argtypes = [_Handle]
        l.rbTuningUpdateTable.restype = C.c_bool
        l.rbTuningUpdateTable.argtypes = [_Handle, C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t, C.c_float]
        l.rbTuningSetFromTable.restype = C.c_bool
        l.rbTuningSetFromTable.argtypes = [_Handle, _Handle]
        l.rbTuningTableLoad.restype = C.c_int
        l.rbTuningTableLoad.argtypes = [_Handle, C.c_char_p]
        l.rbTuningTableSave.restype = C.c_int
        l.rbTuningTableSave.argtypes = [_Handle, C.c_char_p, C.c_char_p]
        l.rbTuningDbLoad.restype = C.c_int
        l.rbTuningDbLoad.argtypes = [C.c_char_p]
        l.rbTuningDbClear.restype = None
        l.rbTuningDbClear.argtypes = []
        l.rbTuningDbSize.restype = C.c_int
        l.rbTuningDbSize.argtypes = []
        l.rbTuningDbLookup.restype = C.c_uint32
        l.rbTuningDbLookup.argtypes = [_Handle]
        l.rbTuningGetKey.restype = C.c_size_t
        l.rbTuningGetKey.argtypes = [_Handle, C.c_char_p, C.c_size_t]
        l.rbIsSplitKFaster.restype = C.c_int
        l.rbIsSplitKFaster.argtypes = [C.c_int64] * 5 + [C.c_int]
        l.rbIsProblemFusible.restype = C.c_bool
        l.rbIsProblemFusible.argtypes = [_Handle, C.c_char_p, C.c_size_t]
        l.rbGetNumPrefillArgs.restype = C.c_size_t
        l.rbGetNumPrefillArgs.argtypes = [_Handle]
        l.rbGetNumAuxBuffers.restype = C.c_size_t
        l.rbGetNumAuxBuffers.argtypes = [_Handle]
        l.rbSetTraceBuffer.restype = None
        l.rbSetTraceBuffer.argtypes = [C.c_void_p, C.c_size_t]
        l.rbReadKernelStatus.restype = C.c_int
        l.rbReadKernelStatus.argtypes = [C.POINTER(C.c_uint32), C.c_int]
        l.rbSetWaitLimit.restype = None
        l.rbSetWaitLimit.argtypes = [C.c_uint64]
        l.rbInjectStall.restype = None
        l.rbInjectStall.argtypes = [C.c_int]
        l.rbLaunchCount.restype = C.c_uint64
        l.rbGetLastError.restype = C.c_char_p
        _lib = l
    return _lib


def check(status: int) -> None:
    if status != SUCCESS:
        raise RbError(status, lib().rbGetLastError().decode())


def kernel_status(clear: bool = True) -> int:
    v = C.c_uint32(0)
    check(lib().rbReadKernelStatus(C.byref(v), 1 if clear else 0))
    return v.value


def launch_count() -> int:
    return int(lib().rbLaunchCount())
