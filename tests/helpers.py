"""Shared helpers for the parity tests: seeded inputs with identical bits on the oracle side (numpy)
and on the device side (torch tensors used as plain device buffers)."""
from __future__ import annotations

import numpy as np

import oracle

NP_STORAGE = {oracle.F32: np.float32, oracle.F16: np.uint16, oracle.BF16: np.uint16, oracle.I8: np.int8,
              oracle.I32: np.int32, oracle.F8E4M3: np.uint8, oracle.F8E5M2: np.uint8}


def torch_dtype(code):
    import torch
    return {oracle.F32: torch.float32, oracle.F16: torch.float16, oracle.BF16: torch.bfloat16, oracle.I8: torch.int8,
            oracle.I32: torch.int32, oracle.F8E4M3: torch.float8_e4m3fn, oracle.F8E5M2: torch.float8_e5m2}[code]


def to_device(raw: np.ndarray, code: int, device="cuda"):
    """Raw storage bits (as produced by oracle.from_f32) -> torch tensor of the matching dtype."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(raw).view(np.int16) if raw.dtype == np.uint16 else np.ascontiguousarray(raw))
    return t.to(device).view(torch_dtype(code))


def from_device(t, code: int) -> np.ndarray:
    """Torch tensor -> raw storage bits as numpy."""
    import torch
    if code in (oracle.F16, oracle.BF16):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    if code in (oracle.F8E4M3, oracle.F8E5M2):
        return t.contiguous().view(torch.uint8).cpu().numpy()
    return t.contiguous().cpu().numpy()


def reference_random(shapes, code: int, seed: int, rand_float=False, mn=-5, mx=5):
    """rocmlir-gen `-rand <seed>` data: srand(seed), tensors filled in argument order, one rand() per
    element, converted to the element type (rocmlir-gen.cpp:3157-3218). Returns (f32 values, raw bits) per tensor."""
    oracle.seed(seed)
    out = []
    for shp in shapes:
        n = int(np.prod(shp))
        f = oracle.fill_random(n, rand_float, mn, mx)
        raw = oracle.from_f32(f, code)
        out.append((oracle.to_f32(raw, code).reshape(shp), raw.reshape(shp)))
    return out


def normal_data(shape, code: int, seed: int, scale: float):
    """scale * N(0,1) from a seeded PCG64 stream, rounded to the element type (RNE; fp8 saturating)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    f = (rng.standard_normal(int(np.prod(shape)), dtype=np.float32) * np.float32(scale)).astype(np.float32)
    raw = oracle.from_f32(f, code)
    return oracle.to_f32(raw, code).reshape(shape), raw.reshape(shape)


def uniform_int8(shape, seed: int, lo=-127, hi=127):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(lo, hi + 1, size=shape, dtype=np.int8)


def uniform_f32(shape, seed: int, lo: float, hi: float):
    rng = np.random.Generator(np.random.PCG64(seed))
    return (rng.random(int(np.prod(shape)), dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).reshape(shape)
