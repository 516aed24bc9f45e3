"""ctypes access to the CPU oracle. TEST INFRASTRUCTURE: used by tests/, the smoke check and
the CPU-baseline legs of bench.py only; never by the product path."""
import ctypes as C
import os
import subprocess

import numpy as np

ORACLE_DIR = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(ORACLE_DIR, "_build", "liboracle.so")
KAT = os.path.join(ORACLE_DIR, "_build", "kat")


class OrcDecision(C.Structure):
    _fields_ = [("found", C.c_int32), ("action", C.c_uint32), ("main", C.c_uint32), ("depth", C.c_uint32),
                ("peaks", C.c_uint64 * 4)]


DEC_DTYPE = np.dtype([("found", "<i4"), ("action", "<u4"), ("main", "<u4"), ("depth", "<u4"), ("peaks", "<u8", (4,))])


def build():
    res = subprocess.run(["make", "-C", ORACLE_DIR, "-j4"], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + res.stdout + res.stderr)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        self.h = lib.orc_create()

    def close(self):
        if self.h:
            self.lib.orc_destroy(self.h)
            self.h = None

    def precompute(self, size, through=2, dtype_mask=3, threads=1, budget_s=0.0, cache=False):
        sec = C.c_double()
        puts, lspecs, solves = C.c_uint64(), C.c_uint64(), C.c_uint64()
        fin = C.c_int()
        busy = C.c_double()
        rc = self.lib.orc_precompute(self.h, size, through, dtype_mask, threads, budget_s, int(cache), C.byref(sec),
                                     C.byref(puts), C.byref(lspecs), C.byref(solves), C.byref(fin), C.byref(busy))
        if rc != 0:
            raise RuntimeError("oracle precompute failed")
        return {"seconds": sec.value, "puts": puts.value, "logical_specs": lspecs.value, "solves": solves.value,
                "finished": bool(fin.value), "busy_seconds": busy.value}

    def precompute_phases(self, size, phase_budgets_s, through=2, dtype_mask=3, threads=1):
        """The driver with one time budget per phase (Move, Zero, Matmul): a sample that reaches every
        phase. Returns totals and, per phase, seconds / goal Specs completed / puts / finished."""
        n = through + 1
        budgets = (C.c_double * 3)(*(list(phase_budgets_s) + [0.0] * 3)[:3])
        sec, busy = C.c_double(), C.c_double()
        puts, lspecs = C.c_uint64(), C.c_uint64()
        psec, pspecs, pputs, pfin = (C.c_double * 3)(), (C.c_uint64 * 3)(), (C.c_uint64 * 3)(), (C.c_int * 3)()
        rc = self.lib.orc_precompute_phases(self.h, size, through, dtype_mask, threads, budgets, C.byref(sec), C.byref(busy),
                                            C.byref(puts), C.byref(lspecs), psec, pspecs, pputs, pfin)
        if rc != 0:
            raise RuntimeError("oracle precompute failed")
        names = ["move", "zero", "matmul"]
        return {"seconds": sec.value, "busy_seconds": busy.value, "puts": puts.value, "logical_specs": lspecs.value,
                "phases": [{"phase": names[k], "seconds": psec[k], "goal_specs_completed": int(pspecs[k]),
                            "puts": int(pputs[k]), "finished": bool(pfin[k])} for k in range(n)]}

    def top_down(self, key: bytes, limits):
        lim = (C.c_uint64 * 4)(*limits)
        out = OrcDecision()
        rc = self.lib.orc_top_down(self.h, key, len(key), lim, C.byref(out))
        if rc != 0:
            raise RuntimeError(f"oracle top_down failed ({rc})")
        return out

    def get_impl(self, key: bytes, limits) -> str:
        """The optimal implementation of (Spec, limits) as text, one line per node."""
        lim = (C.c_uint64 * 4)(*limits)
        buf = C.create_string_buffer(1 << 20)
        self.lib.orc_get_impl.restype = C.c_long
        n = self.lib.orc_get_impl(self.h, key, len(key), lim, buf, len(buf))
        if n < 0:
            raise RuntimeError(f"oracle get_impl failed ({n})")
        return buf.raw[:n].decode()

    def num_puts(self):
        return int(self.lib.orc_num_puts(self.h))

    def dominance_conflicts(self):
        return int(self.lib.orc_num_dominance_conflicts(self.h))

    def dump(self):
        """All puts: (keys bytes, key_off[n+1], rect[n,8] lattice codes lo|hi, decisions[n])."""
        n, kb = C.c_uint64(), C.c_uint64()
        self.lib.orc_dump(self.h, C.byref(n), C.byref(kb), None, None, None, None)
        n, kb = n.value, kb.value
        keys = np.zeros(max(kb, 1), dtype=np.uint8)
        key_off = np.zeros(n + 1, dtype=np.uint64)
        rect = np.zeros((n, 8), dtype=np.uint8)
        dec = np.zeros(n, dtype=DEC_DTYPE)
        self.lib.orc_dump(self.h, None, None, keys.ctypes.data_as(C.POINTER(C.c_uint8)),
                          key_off.ctypes.data_as(C.POINTER(C.c_uint64)), rect.ctypes.data_as(C.POINTER(C.c_uint8)),
                          dec.ctypes.data_as(C.POINTER(OrcDecision)))
        return keys[:kb], key_off, rect, dec


def load():
    build()
    lib = C.CDLL(LIB)
    lib.orc_create.restype = C.c_void_p
    lib.orc_destroy.argtypes = [C.c_void_p]
    lib.orc_precompute.argtypes = [C.c_void_p, C.c_uint32, C.c_int, C.c_int, C.c_int, C.c_double, C.c_int,
                                   C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                                   C.POINTER(C.c_uint64), C.POINTER(C.c_int), C.POINTER(C.c_double)]
    lib.orc_precompute_phases.argtypes = [C.c_void_p, C.c_uint32, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double),
                                          C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_uint64),
                                          C.POINTER(C.c_uint64), C.POINTER(C.c_double), C.POINTER(C.c_uint64),
                                          C.POINTER(C.c_uint64), C.POINTER(C.c_int)]
    lib.orc_top_down.argtypes = [C.c_void_p, C.c_char_p, C.c_uint32, C.POINTER(C.c_uint64), C.POINTER(OrcDecision)]
    lib.orc_num_puts.restype = C.c_uint64
    lib.orc_num_puts.argtypes = [C.c_void_p]
    lib.orc_num_dominance_conflicts.restype = C.c_uint64
    lib.orc_num_dominance_conflicts.argtypes = [C.c_void_p]
    lib.orc_dump.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint8),
                             C.POINTER(C.c_uint64), C.POINTER(C.c_uint8), C.POINTER(OrcDecision)]

    class _Factory:
        def new(self):
            return Oracle(lib)
        kat_path = KAT
    return _Factory()


def codes_to_limits(codes):
    """Lattice codes (registers raw, caches bit length) -> decoded limits."""
    c = np.asarray(codes, dtype=np.uint64)
    out = c.copy()
    for k in (2, 3):
        out[..., k] = np.where(c[..., k] == 0, 0, np.uint64(1) << (np.maximum(c[..., k], 1) - np.uint64(1)))
    return out
