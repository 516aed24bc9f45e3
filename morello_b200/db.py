"""Host-side mirror of the reference's search / database interface for the fill path."""
import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

from . import _lib as L

KIND_MOVE, KIND_FILL_ZERO, KIND_MATMUL_ACCUM, KIND_MATMUL = 0, 1, 2, 3
DTYPE_U32, DTYPE_F32 = 4, 6
RF, VRF, L1, GL = 0, 1, 2, 3
THROUGH_MOVE, THROUGH_ZERO, THROUGH_MATMUL = 0, 1, 2
# Avx2Target::max_mem() (morello/src/target/avx2.rs:59-65): RF, VRF registers; L1, GL lines.
MAX_MEM = (16, 16, 1024, 33554432)


@dataclass(frozen=True)
class Decision:
    """One ActionCostVec entry with k = 1 (morello/src/db/mod.rs:54,171)."""
    found: int            # 1 optimum, 0 unsatisfiable, -1 not in the tables
    action: int = 0
    main_cost: int = 0
    depth: int = 0
    peaks: Tuple[int, int, int, int] = (0, 0, 0, 0)

    @staticmethod
    def from_c(d) -> "Decision":
        if d.found != 1:
            return Decision(found=int(d.found))
        return Decision(1, int(d.action), int(d.main_cost), int(d.depth), tuple(int(x) for x in d.peaks))


def simple_spec(kind: int, dtype: int, spec_shape: Sequence[int], memory: int = GL) -> bytes:
    """Blob of a serial Spec with every operand row-major in `memory` (the goal Specs of
    frontend/src/main.rs:192-204 and the bounds of precompute/src/main.rs:651-736)."""
    lib = L.load()
    shape = (C.c_uint32 * len(spec_shape))(*spec_shape)
    buf = C.create_string_buffer(256)
    n = lib.mrl_spec_simple(kind, dtype, shape, len(spec_shape), memory, buf, 256)
    if n < 0:
        raise ValueError(f"cannot build Spec (status {n})")
    return buf.raw[:n]


def describe_spec(blob: bytes) -> str:
    lib = L.load()
    buf = C.create_string_buffer(512)
    n = lib.mrl_spec_describe(blob, len(blob), buf, 512)
    if n < 0:
        raise ValueError("bad Spec blob")
    return buf.value.decode()


def tabulate(blob: bytes):
    """[(ActionNum, combine kind, immediate, memory, units, [sub-Spec blobs])]: the applicable actions
    of a Spec as the fill tabulates them, in the reference's enumeration order."""
    lib = L.load()
    buf = C.create_string_buffer(1 << 18)
    n = lib.mrl_tabulate(blob, len(blob), buf, len(buf))
    if n < 0:
        raise ValueError(f"cannot tabulate Spec (status {n})")
    raw, p, out = buf.raw[:n], 0, []
    while p < n:
        action = int.from_bytes(raw[p:p + 2], "little")
        kind, nchild = raw[p + 2], raw[p + 3]
        imm = int.from_bytes(raw[p + 4:p + 8], "little")
        level = raw[p + 8]
        units = int.from_bytes(raw[p + 12:p + 16], "little")
        p += 16
        children = []
        for _ in range(nchild):
            ln = int.from_bytes(raw[p:p + 2], "little")
            children.append(raw[p + 2:p + 2 + ln])
            p += 2 + ln
        out.append((action, kind, imm, level, units, children))
    return out


def _pack(blobs: Sequence[bytes], limits: Optional[Sequence[Sequence[int]]]):
    off = (C.c_uint64 * (len(blobs) + 1))()
    pos = 0
    for i, b in enumerate(blobs):
        off[i] = pos
        pos += len(b)
    off[len(blobs)] = pos
    data = b"".join(blobs)
    lim = None
    if limits is not None:
        lim = (C.c_uint64 * (4 * len(blobs)))()
        for i, l in enumerate(limits):
            for k in range(4):
                lim[4 * i + k] = l[k]
    return data, off, lim


class SynthesisDatabase:
    """An in-memory synthesis database living on one GPU.

    Mirrors, for the fill path, FilesDatabase (morello/src/db/mod.rs:350-380, 481-503) together
    with search::top_down_many (morello/src/search/mod.rs:21-42) and the precompute driver
    (precompute/src/main.rs:172-386). Everything is computed by the CUDA extension; there is
    no CPU path, and construction fails when no GPU or no built extension is present.
    """

    def __init__(self, device: int = 0, threads: int = 0):
        self._lib = L.load()
        self._ctx = C.c_void_p()
        rc = self._lib.mrl_ctx_create(device, threads, C.byref(self._ctx))
        if rc != 0:
            msg = self._lib.mrl_last_error(self._ctx).decode() if self._ctx else "context creation failed"
            if self._ctx:
                self._lib.mrl_ctx_destroy(self._ctx)
                self._ctx = None
            raise RuntimeError(msg)

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.mrl_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != 0:
            err = RuntimeError(self._lib.mrl_last_error(self._ctx).decode() or f"status {rc}")
            err.status = rc
            raise err

    def set_plan_flags(self, no_twins: bool = False, no_memo: bool = False):
        """Cross-check modes of the host planner: the same plan built the slow way."""
        self._check(self._lib.mrl_set_plan_flags(self._ctx, int(no_twins) | (int(no_memo) << 1)))

    # --- search::top_down_many / top_down ---
    def top_down_many(self, goals: Sequence[bytes], limits: Optional[Sequence[Sequence[int]]] = None) -> List[Decision]:
        if limits is None:
            limits = [MAX_MEM] * len(goals)
        data, off, lim = _pack(goals, limits)
        out = (L.Decision * len(goals))()
        self._check(self._lib.mrl_top_down_many(self._ctx, data, off, len(goals), lim, out))
        return [Decision.from_c(d) for d in out]

    def top_down_many_noalloc(self, goals: Sequence[bytes],
                              limits: Optional[Sequence[Sequence[int]]] = None) -> List[Decision]:
        """top_down_many for callers that must not allocate device memory: the fill runs inside a
        fixed 32 MiB device array and is refused (RuntimeError) when it needs more. One call at a
        time per GPU; make the first call before any stream capture."""
        if limits is None:
            limits = [MAX_MEM] * len(goals)
        data, off, lim = _pack(goals, limits)
        out = (L.Decision * len(goals))()
        self._check(self._lib.mrl_top_down_many_noalloc(self._ctx, data, off, len(goals), lim, out))
        return [Decision.from_c(d) for d in out]

    def top_down(self, goal: bytes, limits: Sequence[int] = MAX_MEM) -> Decision:
        return self.top_down_many([goal], [limits])[0]

    # --- the precompute driver ---
    def precompute(self, size: int, through: int = THROUGH_MATMUL, dtypes: Sequence[int] = (DTYPE_U32, DTYPE_F32)):
        self._check(self._lib.mrl_precompute(self._ctx, size, through, self._dtype_mask(dtypes)))
        return self.stats()

    # --- the stages, for measurement ---
    def plan_precompute(self, size: int, through: int = THROUGH_MATMUL, dtypes: Sequence[int] = (DTYPE_U32, DTYPE_F32)):
        self._check(self._lib.mrl_plan_precompute(self._ctx, size, through, self._dtype_mask(dtypes)))

    def plan_goals(self, goals: Sequence[bytes]):
        data, off, _ = _pack(goals, None)
        self._check(self._lib.mrl_plan_goals(self._ctx, data, off, len(goals)))

    def upload(self):
        self._check(self._lib.mrl_upload(self._ctx))

    def fill(self):
        self._check(self._lib.mrl_fill(self._ctx))

    # --- FilesDatabase::get ---
    def get_many(self, specs: Sequence[bytes], limits: Sequence[Sequence[int]]) -> List[Decision]:
        data, off, lim = _pack(specs, limits)
        out = (L.Decision * len(specs))()
        self._check(self._lib.mrl_get_many(self._ctx, data, off, len(specs), lim, out))
        return [Decision.from_c(d) for d in out]

    def get(self, spec: bytes, limits: Sequence[int] = MAX_MEM) -> Decision:
        return self.get_many([spec], [limits])[0]

    # --- multi-GPU: shard ownership and the per-stage fill (see morello_b200/sharded.py) ---
    def set_shard(self, rank: int, world: int):
        self._check(self._lib.mrl_set_shard(self._ctx, rank, world))

    def plan_share(self):
        """[(host pointer, bytes)] x 8: this context's plan as flat byte ranges."""
        ptrs, sizes = (C.c_void_p * 8)(), (C.c_uint64 * 8)()
        self._check(self._lib.mrl_plan_share(self._ctx, ptrs, sizes))
        return [(int(ptrs[k] or 0), int(sizes[k])) for k in range(8)]

    def plan_adopt(self, sizes: Sequence[int], cands_on_device_only: bool = False):
        """Allocates an empty plan of the given range sizes; returns the pointers to fill (0 for
        the candidate records when they will only be copied device to device)."""
        ptrs, sz = (C.c_void_p * 8)(), (C.c_uint64 * 8)(*sizes)
        self._check(self._lib.mrl_plan_adopt(self._ctx, sz, ptrs, int(cands_on_device_only)))
        return [int(ptrs[k] or 0) for k in range(8)]

    def device_cands(self):
        """(device pointer, bytes) of the uploaded candidate records."""
        ptr, n = C.c_void_p(), C.c_uint64()
        if self._lib.mrl_device_cands(self._ctx, C.byref(ptr), C.byref(n)) != 0:
            raise RuntimeError("plan not uploaded")
        return int(ptr.value or 0), int(n.value)

    def cands_arrived(self):
        """After the candidate records were written into device_cands(): checks them on the device."""
        self._check(self._lib.mrl_cands_arrived(self._ctx))

    def plan_adopt_done(self, plan_seconds: float = 0.0):
        self._check(self._lib.mrl_plan_adopt_done(self._ctx, plan_seconds))

    def set_stream(self, cuda_stream: int):
        self._check(self._lib.mrl_set_stream(self._ctx, C.c_void_p(cuda_stream)))

    def num_stages(self) -> int:
        return int(self._lib.mrl_num_stages(self._ctx))

    def stages(self):
        """[(first Spec id, end Spec id, first family, end family)] in plan order."""
        out = []
        a, b, c, d = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        for s in range(self.num_stages()):
            if self._lib.mrl_stage_info(self._ctx, s, C.byref(a), C.byref(b), C.byref(c), C.byref(d)) != 0:
                raise IndexError(s)
            out.append((int(a.value), int(b.value), int(c.value), int(d.value)))
        return out

    def families(self):
        """[(stage, owner rank, first Spec id, end Spec id)] in plan order."""
        out = []
        g, o, lo, hi = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        for f in range(int(self._lib.mrl_num_families(self._ctx))):
            if self._lib.mrl_family_info(self._ctx, f, C.byref(g), C.byref(o), C.byref(lo), C.byref(hi)) != 0:
                raise IndexError(f)
            out.append((int(g.value), int(o.value), int(lo.value), int(hi.value)))
        return out

    def spec_owners(self) -> bytes:
        """One byte per Spec id: the rank that computes it (all zero when not sharded)."""
        n = self.num_specs()
        buf = C.create_string_buffer(max(n, 1))
        if self._lib.mrl_spec_owners(self._ctx, buf, n) != 0:
            raise RuntimeError("nothing planned")
        return buf.raw[:n]

    def device_rows(self):
        """(device pointer, row count) of the finished table (mrl_row_bytes() bytes per row)."""
        ptr, n = C.c_void_p(), C.c_uint64()
        if self._lib.mrl_device_rows(self._ctx, C.byref(ptr), C.byref(n)) != 0:
            raise RuntimeError("no table on the device")
        return int(ptr.value or 0), int(n.value)

    def fill_begin(self):
        self._check(self._lib.mrl_fill_begin(self._ctx))

    def fill_stage_solve(self, stage: int):
        """Solves this rank's share of a stage; (device pointer, bytes) of the stage's breakpoint masks."""
        ptr, n = C.c_void_p(), C.c_uint64()
        self._check(self._lib.mrl_fill_stage_solve(self._ctx, stage, C.byref(ptr), C.byref(n)))
        return int(ptr.value or 0), int(n.value)

    def fill_stage_place(self, stage: int):
        """Appends the stage to the table; (device pointer, bytes) of the stage's rows."""
        ptr, n = C.c_void_p(), C.c_uint64()
        self._check(self._lib.mrl_fill_stage_place(self._ctx, stage, C.byref(ptr), C.byref(n)))
        return int(ptr.value or 0), int(n.value)

    def fill_end(self):
        self._check(self._lib.mrl_fill_end(self._ctx))

    # --- FilesDatabase::get_impl ---
    def get_impl(self, spec: bytes, limits: Sequence[int] = MAX_MEM) -> str:
        """The optimal implementation of (Spec, limits) reconstructed from the tables, as text."""
        lim = (C.c_uint64 * 4)(*limits)
        buf = C.create_string_buffer(1 << 20)
        n = self._lib.mrl_get_impl(self._ctx, spec, len(spec), lim, buf, len(buf))
        if n < 0:
            self._check(int(n))
        return buf.raw[:n].decode()

    def verify(self, n_samples: int = 0, seed: int = 1):
        """(points checked, mismatches): recomputes the decision from the children's tables at
        n_samples pseudo-random (Spec, limits) points - all of them when n_samples is 0 - and
        compares with the table."""
        checked, bad = C.c_uint64(), C.c_uint64()
        self._check(self._lib.mrl_verify(self._ctx, n_samples, seed, C.byref(checked), C.byref(bad)))
        return int(checked.value), int(bad.value)

    # --- export / stats ---
    def stats(self) -> dict:
        s = L.Stats()
        self._check(self._lib.mrl_get_stats(self._ctx, C.byref(s)))
        out = {name: getattr(s, name) for name, _ in L.Stats._fields_}
        out["phase_ms"] = [float(x) for x in s.phase_ms]
        out["plan_layout_step_seconds"] = [float(x) for x in s.plan_layout_step_seconds]
        return out

    def num_specs(self) -> int:
        return int(self._lib.mrl_num_specs(self._ctx))

    def spec_blob(self, spec_id: int) -> bytes:
        buf = C.create_string_buffer(256)
        n = self._lib.mrl_spec_blob(self._ctx, spec_id, buf, 256)
        if n < 0:
            raise IndexError(spec_id)
        return buf.raw[:n]

    def spec_grid(self, spec_id: int):
        masks = (C.c_uint32 * 4)()
        n = C.c_uint64()
        if self._lib.mrl_spec_grid(self._ctx, spec_id, masks, C.byref(n)) != 0:
            raise IndexError(spec_id)
        return [int(m) for m in masks], int(n.value)

    def export_rows(self, spec_id: int) -> List[Decision]:
        _, n = self.spec_grid(spec_id)
        out = (L.Decision * n)()
        self._check(self._lib.mrl_export_rows(self._ctx, spec_id, out, n))
        return [Decision.from_c(d) for d in out]

    def checksum(self) -> int:
        """64-bit checksum of the filled tables (Spec ids, masks, rows in cell order)."""
        out = C.c_uint64()
        self._check(self._lib.mrl_checksum(self._ctx, C.byref(out)))
        return int(out.value)

    def export_all(self):
        """The whole table in two device-to-host copies: (masks[n_specs, 4] uint32,
        first_row[n_specs + 1] uint64, rows[n_rows, 4] uint32 = main, peak codes, depth << 16 | action, 0)."""
        import numpy as np
        n, n_rows = self.num_specs(), int(self.stats()["n_rows"])
        masks = np.zeros((n, 4), dtype=np.uint32)
        first = np.zeros(n + 1, dtype=np.uint64)
        rows = np.zeros((max(n_rows, 1), 4), dtype=np.uint32)
        self._check(self._lib.mrl_export_all(self._ctx, masks.ctypes.data, first.ctypes.data, rows.ctypes.data, n_rows))
        return masks, first, rows[:n_rows]

    def export_rects(self, spec_id: int):
        """[(lo codes, hi codes, Decision)]: the Spec's table as rectangles over the four limit
        dimensions, equal neighbours merged (the reference's logical page contents)."""
        _, cells = self.spec_grid(spec_id)
        lo = C.create_string_buffer(4 * cells)
        hi = C.create_string_buffer(4 * cells)
        out = (L.Decision * cells)()
        n = self._lib.mrl_export_rects(self._ctx, spec_id, lo, hi, out, cells)
        if n < 0:
            self._check(int(n))
        return [(tuple(lo.raw[4 * i:4 * i + 4]), tuple(hi.raw[4 * i:4 * i + 4]), Decision.from_c(out[i])) for i in range(n)]

    def save(self, path: str):
        """FilesDatabase::save: the filled tables to one file (written to a temporary, then renamed)."""
        self._check(self._lib.mrl_save(self._ctx, path.encode()))

    def load(self, path: str):
        """Reopens a saved database. Lookups work afterwards; with the job's plan already in this
        context (plan_precompute / plan_goals of the same job) so do verify and fill."""
        self._check(self._lib.mrl_load(self._ctx, path.encode()))

    def put(self, spec: bytes, limits: Sequence[int], decision: "Decision"):
        """FilesDatabase::put as a check: succeeds when the tables hold exactly this decision."""
        d = L.Decision()
        d.found = 1 if decision.found == 1 else 0
        d.action, d.main_cost, d.depth = decision.action, decision.main_cost, decision.depth
        for k in range(4):
            d.peaks[k] = decision.peaks[k]
        lim = (C.c_uint64 * 4)(*limits)
        self._check(self._lib.mrl_put(self._ctx, spec, len(spec), lim, C.byref(d)))

    @staticmethod
    def _dtype_mask(dtypes):
        mask = 0
        for d in dtypes:
            mask |= {DTYPE_U32: 1, DTYPE_F32: 2}[d]
        return mask
