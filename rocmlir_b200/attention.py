"""Host-side mirror of rock.attention (mlir/include/mlir/Dialect/Rock/IR/RockOps.td:208-254) over the C ABI.

Q [G,Sq,D], K [G,D,Sk] (trans_k: [G,Sk,D]), V [G,Sk,Dv] -> O [G,Sq,Dv]; argument names follow rocmlir-gen's
attention flags (-seq_len_q, -seq_len_k, -head_dim_qk, -head_dim_v, -transK, --with-attn-scale, --with-attn-bias).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib as L
from .gemm import rb_dtype


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, trans_k: bool = False, trans_q: bool = False,
              trans_v: bool = False, trans_o: bool = False,
              scale: Optional[float] = None, bias: Optional[torch.Tensor] = None,
              mask: Optional[torch.Tensor] = None, mask_fill: float = float("-inf"), causal: bool = False,
              out: Optional[torch.Tensor] = None, scale_tensor: Optional[torch.Tensor] = None,
              quant_bias: Optional[torch.Tensor] = None, quant_scale: Optional[torch.Tensor] = None,
              workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """With int8 `q` and `k` this is the first-GEMM-quantised form (rocmlir-gen -t i8): `v`, the result and the
    side tensors are f16, and `quant_bias` (one int8) and `quant_scale` (one f16), both CUDA tensors, are required."""
    for t in (q, k, v):
        if not t.is_cuda or not t.is_contiguous():
            raise L.RbError(L.INVALID_PARAM, "q, k, v must be contiguous CUDA tensors (the library has no CPU path)")
    # stored shapes: Q [G,Sq,D] (trans_q: [G,D,Sq]), V [G,Sk,Dv] (trans_v: [G,Dv,Sk]), O [G,Sq,Dv] (trans_o: [G,Dv,Sq])
    g = q.shape[0]
    d, sq = (q.shape[1], q.shape[2]) if trans_q else (q.shape[2], q.shape[1])
    dv, sk = (v.shape[1], v.shape[2]) if trans_v else (v.shape[2], v.shape[1])
    kshape = (g, sk, d) if trans_k else (g, d, sk)
    if tuple(k.shape) != kshape or v.shape[0] != g:
        raise L.RbError(L.INVALID_PARAM, f"shape mismatch: Q {tuple(q.shape)} K {tuple(k.shape)} V {tuple(v.shape)}")
    side_dtype = v.dtype          # the element type of everything but a quantised Q and K
    if out is None:
        out = torch.empty((g, dv, sq) if trans_o else (g, sq, dv), dtype=side_dtype, device=q.device)
    p = L.RbAttentionProblem(g, sq, sk, d, dv, int(trans_q), int(trans_k), int(trans_v), int(trans_o), rb_dtype(q.dtype),
                             int(scale is not None),
                             float(scale or 0.0), int(causal), float(mask_fill), None, None, None, None, None)
    if q.dtype == torch.int8:
        if quant_bias is None or quant_scale is None or quant_bias.dtype != torch.int8 or \
                quant_scale.dtype != torch.float16 or v.dtype != torch.float16 or k.dtype != torch.int8:
            raise L.RbError(L.INVALID_PARAM, "the i8 form takes i8 q, k, f16 v, an i8 quant_bias and an f16 quant_scale")
        assert quant_bias.is_cuda and quant_scale.is_cuda and quant_bias.numel() == 1 and quant_scale.numel() == 1
        p.quant_bias = quant_bias.data_ptr()
        p.quant_scale = quant_scale.data_ptr()
    if scale_tensor is not None:
        assert scale_tensor.is_cuda and scale_tensor.is_contiguous() and scale_tensor.dtype == side_dtype and \
            tuple(scale_tensor.shape) == (g, sq, sk)
        p.scale_tensor = scale_tensor.data_ptr()
    if bias is not None:
        assert bias.is_cuda and bias.is_contiguous() and bias.dtype == side_dtype and tuple(bias.shape) == (g, sq, sk)
        p.bias = bias.data_ptr()
    if mask is not None:
        assert mask.is_cuda and mask.is_contiguous() and mask.dtype == torch.int8 and tuple(mask.shape) == (g, sq, sk)
        p.mask = mask.data_ptr()
    stream = torch.cuda.current_stream(q.device).cuda_stream
    # scratch for staged operands comes from the caller's side (rbAttentionWs): the library allocates nothing
    need = int(L.lib().rbAttentionWorkspaceSize(C.byref(p)))
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    L.check(L.lib().rbAttentionWs(C.byref(p), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                  workspace.data_ptr() if need else None,
                                  workspace.numel() * workspace.element_size() if need else 0, stream))
    return out


def flops(g: int, sq: int, sk: int, d: int, dv: int, causal: bool = False) -> float:
    """perfRunner.py:759-777: matmul FLOPs only; under a causal mask only unmasked score entries count."""
    if causal:
        return 2.0 * g * (d + dv) * sq * (sk + 1) / 2
    return 2.0 * g * sq * sk * d + 2.0 * g * sq * sk * dv
