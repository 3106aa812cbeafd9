"""Python mirror of the tuning surface (include/rocmlir_b200_tuning.h), the counterpart of the mlirRockTuning*
functions (mlir/include/mlir-c/Dialect/Rock.h:39-166), plus the measuring loop of the reference's tuning driver
(mlir/tools/rocmlir-tuning-driver/rocmlir-tuning-driver.cpp:234-400): time every configuration of a tuning space
and keep the fastest per problem key in a table / .tsv file."""
from __future__ import annotations

import ctypes as C
from typing import Callable, Iterable, List, Optional, Tuple

from . import _lib as L

QUICK, FULL, EXHAUSTIVE = 0, 1, 2
NEVER, MAYBE, ALWAYS = 0, 1, 2
PARAM_STRING_BUFSZ = 64
KEY_BUFSZ = 2048
SIZE_MAX = C.c_size_t(-1).value


def _string(call, handle, bufsz: int) -> Optional[str]:
    buf = C.create_string_buffer(bufsz)
    n = call(handle, buf, bufsz)
    if n == SIZE_MAX:
        return None
    if n >= bufsz:   # strncpy semantics: the buffer was too small and is not terminated
        buf = C.create_string_buffer(n + 1)
        call(handle, buf, n + 1)
    return buf.value.decode()


class Problem:
    """The role of the reference's MlirModule holding one rock op."""

    def __init__(self, options: Optional[str] = None, *, gemm=None, conv=None, attention=None):
        lib = L.lib()
        if options is not None:
            self._p = lib.rbProblemCreate(options.encode())
        elif gemm is not None:
            self._p = lib.rbProblemFromGemm(C.byref(gemm))
        elif conv is not None:
            self._p = lib.rbProblemFromConv(C.byref(conv))
        elif attention is not None:
            self._p = lib.rbProblemFromAttention(C.byref(attention))
        else:
            raise ValueError("Problem needs options or a problem struct")
        if not self._p.ptr:
            raise ValueError("no kernel for this problem (NULL problem handle)")

    def close(self):
        if self._p.ptr:
            L.lib().rbProblemDestroy(self._p)
            self._p.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def key(self) -> Optional[str]:
        return _string(L.lib().rbTuningGetKey, self._p, KEY_BUFSZ)

    @property
    def perf_config(self) -> str:
        return _string(L.lib().rbProblemGetPerfConfig, self._p, PARAM_STRING_BUFSZ) or ""

    @property
    def variant(self) -> int:
        return int(L.lib().rbProblemGetVariant(self._p))

    def set_from_str(self, perf: str) -> bool:
        b = perf.encode()
        return bool(L.lib().rbTuningSetFromStr(self._p, b, len(b)))

    def set_from_table(self, table: "Table") -> bool:
        return bool(L.lib().rbTuningSetFromTable(table._t, self._p))

    def is_fusible(self, perf: str) -> bool:
        b = perf.encode()
        return bool(L.lib().rbIsProblemFusible(self._p, b, len(b)))

    @property
    def num_prefill_args(self) -> int:
        return int(L.lib().rbGetNumPrefillArgs(self._p))

    @property
    def num_aux_buffers(self) -> int:
        return int(L.lib().rbGetNumAuxBuffers(self._p))

    def space(self, kind: int = FULL) -> List[str]:
        """The perf_config strings of the tuning space, in the space's order."""
        lib = L.lib()
        sp = lib.rbTuningSpaceCreate(self._p, kind)
        par = lib.rbTuningParamCreate()
        out = []
        try:
            for i in range(lib.rbTuningGetNumParams(sp)):
                if not lib.rbTuningParamGet(sp, i, par):
                    break
                out.append(_string(lib.rbTuningParamToString, par, PARAM_STRING_BUFSZ))
        finally:
            lib.rbTuningParamDestroy(par)
            lib.rbTuningSpaceDestroy(sp)
        return out

    def quick_space(self) -> List[str]:
        lib = L.lib()
        sp = lib.rbTuningSpaceCreate(self._p, FULL)
        par = lib.rbTuningParamCreate()
        out = []
        try:
            i = 0
            while lib.rbTuningParamGetQuick(sp, i, par):
                out.append(_string(lib.rbTuningParamToString, par, PARAM_STRING_BUFSZ))
                i += 1
        finally:
            lib.rbTuningParamDestroy(par)
            lib.rbTuningSpaceDestroy(sp)
        return out


class Table:
    def __init__(self):
        self._t = L.lib().rbTuningTableCreate()

    def close(self):
        if self._t.ptr:
            L.lib().rbTuningTableDestroy(self._t)
            self._t.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def update(self, key: str, perf: str, time: float) -> bool:
        k, p = key.encode(), perf.encode()
        return bool(L.lib().rbTuningUpdateTable(self._t, k, len(k), p, len(p), float(time)))

    def load(self, path: str) -> int:
        """Reads a tuning database in the reference's 3-, 4- or 5-column text form; returns the entries taken."""
        return int(L.lib().rbTuningTableLoad(self._t, path.encode()))

    def save(self, path: str, space_name: str = "full") -> int:
        """Writes `arch <tab> numCUs <tab> problem <tab> perf_config` lines (tuningRunner.py's 4-column form)."""
        return int(L.lib().rbTuningTableSave(self._t, path.encode(), space_name.encode()))


def db_load(path: str) -> int:
    """Adds a database file to the process-wide table every launch with variant 0 consults."""
    return int(L.lib().rbTuningDbLoad(path.encode()))


def db_clear() -> None:
    L.lib().rbTuningDbClear()


def db_size() -> int:
    return int(L.lib().rbTuningDbSize())


def db_lookup(problem: "Problem") -> int:
    return int(L.lib().rbTuningDbLookup(problem._p))


def is_split_k_faster(g: int, m: int, n: int, k: int, num_cus: int = 148, level: int = FULL) -> int:
    return int(L.lib().rbIsSplitKFaster(g, m, n, k, num_cus, level))


def tune(problem: Problem, run: Callable[[int], None], kind: int = FULL, iters: int = 10,
         table: Optional[Table] = None) -> List[Tuple[str, float]]:
    """Times `run(variant)` (which must launch the problem's kernel on the current CUDA stream with that variant
    word) for every configuration of the space; returns (perf_config, milliseconds) sorted fastest first and
    records the winner in `table`."""
    import torch
    results = []
    saved = L.lib().rbGetGemmVariant()   # `run` may set the thread's variant word: the caller's value is put back
    try:
        for perf in problem.space(kind):
            if not problem.set_from_str(perf):
                continue
            v = problem.variant
            for _ in range(2):
                run(v)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(iters):
                run(v)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            results.append((perf, ms))
            if table is not None and problem.key is not None:
                table.update(problem.key, perf, ms)
    finally:
        L.lib().rbSetGemmVariant(saved)
    results.sort(key=lambda r: r[1])
    return results


def write_tsv(path: str, rows: Iterable[Tuple[str, str, float]]) -> None:
    """One line per problem: key <tab> perf_config <tab> milliseconds (the reference's tuning database text form,
    mlir/utils/performance/tuningRunner.py)."""
    with open(path, "w") as f:
        for key, perf, ms in rows:
            f.write(f"{key}\t{perf}\t{ms:.6f}\n")
