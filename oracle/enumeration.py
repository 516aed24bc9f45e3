"""TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT PATH.

A second, deliberately plain restatement of how the reference enumerates the actions of a logical
Spec and what each applicable action asks for, written from the Rust sources and from nothing in
this repository's C++ model (morello_b200/csrc/model/), so that tests can compare the two. Pure
Python, no caches, no sharing between Specs, no dtype or kind shortcuts.

For the Avx2 target with default features, serial-only Specs, kinds Move / Fill(Zero) / Matmul:

  morello/src/layout.rs:318-343,455-527,602-810,1234-1279   layouts (expansion, tiling, merging, packings)
  morello/src/tensorspec.rs:140-173,232-236,370-387,608-637  tensor specs, vector-size checks
  morello/src/spec.rs:467-583,1704-1747,3194-3214            parameter shapes, canonicalize, dim_range
  morello/src/target/cpu.rs:300-315,399-453,455-823          memories, destination layouts, Target::actions
  morello/src/target/cpu.rs:896-1031,1694-1745,1812-1856     kernel applicability
  morello/src/target/cpu.rs:1881-1998,2000-2380,2719-2808    kernel memory and cost, broadcast side
  morello/src/target/cpu.rs:2878-3012                        packed / odd-even layout generators
  morello/src/target/common_actions.rs:37-121,123-249,301-376  tile-outs, splits, moves
  morello/src/scheduling/moves.rs:118-138,275-381,383-528    the Move solver
  morello/src/scheduling/tiling.rs:132-228,478-541           the TileOut / Split solvers
  morello/src/scheduling/to_accum.rs:12-62, scheduling/mod.rs:526-546   ToAccum
  morello/src/imp/allocs.rs:156-173                          move_cost

`enumerate_actions(spec)` returns the applicable actions in the reference's order, each with its
ActionNum (position among ALL enumerated actions, applicable or not: search/spectask.rs:66), how its
cost combines (leaf / loop / move / block), its immediates and its sub-Specs as canonical blobs in
the byte format of include/morello_b200.h.
"""
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

RF, VRF, L1, GL = 0, 1, 2, 3
DYNAMIC, PACKED, ODDEVEN = 0, 1, 2
MOVE, FILL_ZERO, MATMUL_ACCUM, MATMUL = 0, 1, 2, 3
LEAF, LOOP, MOVE_KIND, BLOCK = 0, 1, 2, 3
U8, S8, U16, S16, U32, S32, F32, BF16 = range(8)
DTYPE_SIZE = {U8: 1, S8: 1, U16: 2, S16: 2, U32: 4, S32: 4, F32: 4, BF16: 2}
LINE_SIZE = 64
HIT_COST = {RF: 0, VRF: 0, L1: 2, GL: 20}        # avx2.rs:29-40, default features
VECTOR_BYTES = {RF: (), VRF: (16, 32), L1: (), GL: ()}
ALL_VECTOR_BYTES = (16, 32)                          # over all memories, in memory order


def has_layout(mem): return mem != RF
def is_addressed(mem): return mem != L1
def counts_registers(mem): return mem in (RF, VRF)
def rf_or_l1(mem): return mem in (RF, L1)


def possible_destination_memories(mem):             # cpu.rs:304-315
    return {RF: [RF], VRF: [VRF], L1: [L1, RF, VRF], GL: [GL, L1]}[mem]


@dataclass
class Layout:
    dims: List[Tuple[int, int, int]] = field(default_factory=list)   # (logical dim, kind, strip size or 0)
    contig: int = 0

    def copy(self):
        return Layout(list(self.dims), self.contig)

    def fully_contiguous(self):
        return self.contig == len(self.dims)

    def is_row_major(self):
        return all(k == DYNAMIC for _, k, _ in self.dims) and all(
            self.dims[i][0] <= self.dims[i + 1][0] for i in range(len(self.dims) - 1))

    def is_col_major(self):
        return all(k == DYNAMIC for _, k, _ in self.dims) and all(
            self.dims[i + 1][0] < self.dims[i][0] for i in range(len(self.dims) - 1))

    def __eq__(self, other):
        return self.dims == other.dims and self.contig == other.contig


def expand_physical_shape(layout, shape):           # layout.rs:769-810; None = does not apply
    remaining = list(shape)
    tiled = [False] * len(shape)
    out = []
    for ldim, kind, size in reversed(layout.dims):
        rem = remaining[ldim]
        if kind == DYNAMIC:
            assert rem != 0, "two Dynamic dims for one logical dim"
            out.append(rem)
            remaining[ldim] = 0
        elif rem < size:
            allowed = kind == PACKED or rem == 1
            if not allowed or tiled[ldim]:
                return None
            assert rem != 0
            out.append(rem)
            remaining[ldim] = 1
            tiled[ldim] = True
        elif rem % size != 0:
            return None
        else:
            out.append(size)
            remaining[ldim] = rem // size
    if any(d > 1 for d in remaining):
        return None
    out.reverse()
    return out


def merge_consecutive_dimensions(layout):           # layout.rs:602-669
    if not layout.dims:
        return
    first_contig = len(layout.dims) - layout.contig
    new_contig = layout.contig
    out = [layout.dims[0]]
    for idx in range(1, len(layout.dims)):
        ldim, kind, size = layout.dims[idx]
        last_ldim, last_kind, last_size = out[-1]
        if ldim != last_ldim:
            out.append((ldim, kind, size))
            continue
        if last_kind == PACKED and kind == PACKED:
            if idx == first_contig:
                out.append((ldim, kind, size))
            else:
                out[-1] = (last_ldim, PACKED, last_size * size)
                if idx >= first_contig:
                    new_contig -= 1
        elif last_kind == DYNAMIC and kind == PACKED:
            if idx <= first_contig:
                out.append((ldim, kind, size))
            else:
                new_contig -= 1
        elif ODDEVEN in (last_kind, kind) and not (last_kind == ODDEVEN and kind == ODDEVEN):
            out.append((ldim, kind, size))
        else:
            raise AssertionError("layout the reference treats as unreachable")
    layout.dims = out
    layout.contig = new_contig


def prune_size_one(layout, shape, contig):          # layout.rs:455-472
    first_contig = len(layout.dims) - contig
    kept = []
    for idx, d in enumerate(layout.dims):
        if shape[d[0]] != 1:
            kept.append(d)
        elif idx >= first_contig:
            contig -= 1
    layout.dims = kept
    return contig


def drop_unneeded_packings(layout, tile_shape):     # layout.rs:674-766
    dims = layout.dims
    contig = layout.contig
    first_contig = len(dims) - contig
    seen_oe = [False] * len(tile_shape)
    outer_oe = []
    for ldim, kind, _ in dims:
        outer_oe.append(seen_oe[ldim])
        if kind == ODDEVEN:
            seen_oe[ldim] = True
    remaining = list(tile_shape)
    noneified = [None] * len(tile_shape)
    for idx in range(len(dims) - 1, -1, -1):
        ldim, kind, size = dims[idx]
        rem = remaining[ldim]
        if kind == PACKED:
            if rem % size == 0:
                if not outer_oe[idx] and rem == size:
                    dims[idx] = (ldim, DYNAMIC, 0)
                    if noneified[ldim] is None:
                        noneified[ldim] = idx
                remaining[ldim] = rem // size
            elif rem != 0 and size >= rem:
                if not outer_oe[idx]:
                    dims[idx] = (ldim, DYNAMIC, 0)
                    if noneified[ldim] is None:
                        noneified[ldim] = idx
                remaining[ldim] = 1
        elif kind == ODDEVEN:
            if rem % size == 0:
                remaining[ldim] = rem // size
            elif rem != 0 and size % rem == 0:
                remaining[ldim] = 1
    kept = []
    drops = 0
    for idx, (ldim, kind, size) in enumerate(dims):
        skip = False
        if noneified[ldim] is not None and idx < noneified[ldim]:
            skip = True
        elif kept and kept[-1][0] == ldim and kept[-1][1] == DYNAMIC and kind == DYNAMIC:
            skip = True
        if not skip:
            kept.append((ldim, kind, size))
        elif idx >= first_contig:
            drops += 1
    layout.dims = kept
    layout.contig = min(max(contig - drops, 0), len(kept))


def update_for_tiling(layout, parent_shape, tile_shape):   # layout.rs:486-527
    pp = expand_physical_shape(layout, parent_shape)
    tp = expand_physical_shape(layout, tile_shape)
    if pp is None or tp is None:
        return None
    matching = None
    for k in range(len(pp)):
        if pp[len(pp) - 1 - k] != tp[len(tp) - 1 - k]:
            matching = k
            break
    lowered = min(matching + 1 if matching is not None else len(layout.dims), layout.contig)
    new = layout.copy()
    new.contig = lowered
    new.contig = prune_size_one(new, tile_shape, new.contig)
    merge_consecutive_dimensions(new)
    drop_unneeded_packings(new, tile_shape)
    return new


def canonicalize_layout(layout, shape):             # layout.rs:474-484
    if expand_physical_shape(layout, shape) is None:
        return None
    new = layout.copy()
    new.contig = min(new.contig, len(new.dims))
    new.contig = prune_size_one(new, shape, new.contig)
    merge_consecutive_dimensions(new)
    drop_unneeded_packings(new, shape)
    return new


def layout_new(dims):                               # layout.rs:205-217
    l = Layout(list(dims), len(dims))
    merge_consecutive_dimensions(l)
    return l


def row_major(shape):
    return layout_new([(d, DYNAMIC, 0) for d in range(len(shape)) if shape[d] != 1])


def col_major(shape):
    l = row_major(shape)
    l.dims.reverse()
    return l


def nhwc(shape):
    dims = [(d, DYNAMIC, 0) for d in (0, 2, 3, 1) if shape[d] != 1]
    return Layout(dims, len(dims))


def estimate_cache_lines(layout, shape, dtype):     # layout.rs:318-343
    phys = expand_physical_shape(layout, shape)
    assert phys is not None
    first_contig = len(layout.dims) - layout.contig
    lines = 1
    for p in phys[:first_contig]:
        lines *= p
    inner = 1
    for p in phys[first_contig:]:
        inner *= p
    return lines * -(-(inner * DTYPE_SIZE[dtype]) // LINE_SIZE)


@dataclass
class Tensor:
    shape: Tuple[int, ...]
    dtype: int
    mem: int
    layout: Layout
    vs: int            # values per vector register; 0 = none

    def volume(self):
        v = 1
        for d in self.shape:
            v *= d
        return v

    def is_contiguous(self):
        return self.layout.fully_contiguous()

    def same_as(self, o):
        return (tuple(self.shape) == tuple(o.shape) and self.dtype == o.dtype and self.mem == o.mem and
                self.layout == o.layout and self.vs == o.vs)


def check_tensor_vector_size(shape, dtype, mem, vs):   # tensorspec.rs:608-637; "" = ok
    allowed = VECTOR_BYTES[mem]
    if not allowed:
        return ""
    assert vs, "vector memory without a vector size"
    if vs * DTYPE_SIZE[dtype] not in allowed:
        return "invalid"
    volume = 1
    for d in shape:
        volume *= d
    if not any((volume * DTYPE_SIZE[dtype]) % vb == 0 for vb in allowed):
        return "invalid"
    if volume % vs != 0:
        return "volume"
    return ""


def canonicalize_tensor(t):                         # tensorspec.rs:232-236,370-377; False = not canonicalizable
    if check_tensor_vector_size(t.shape, t.dtype, t.mem, t.vs):
        return False
    if not has_layout(t.mem):
        t.layout = Layout()
        return True
    new = update_for_tiling(t.layout, t.shape, t.shape)
    if new is None:
        return False
    t.layout = new
    return True


def memory_units(t):                                # tensorspec.rs:161-173
    if counts_registers(t.mem):
        return -(-t.volume() // t.vs) if t.vs else t.volume()
    return estimate_cache_lines(t.layout, t.shape, t.dtype)


def move_cost(t):                                   # imp/allocs.rs:156-173
    cost = 0
    if has_layout(t.mem):
        cost = HIT_COST[t.mem] * estimate_cache_lines(t.layout, t.shape, t.dtype)
    if not t.is_contiguous():
        cost *= 2
    return cost


@dataclass
class Spec:
    kind: int
    dtype: int
    serial: bool
    shape: Tuple[int, ...]                 # Move / Fill: the tensor shape; Matmul: (b, m, k, n)
    auxes: List[Tuple[int, int, Layout]]   # per operand: (memory, vector size, layout)

    def copy(self):
        return Spec(self.kind, self.dtype, self.serial, tuple(self.shape), [(m, v, l.copy()) for m, v, l in self.auxes])

    def parameter_shapes(self):            # spec.rs:467-583
        if self.kind == MOVE:
            return [tuple(self.shape), tuple(self.shape)]
        if self.kind == FILL_ZERO:
            return [tuple(self.shape)]
        b, m, k, n = self.shape
        return [(b, m, k), (b, k, n), (b, m, n)]

    def operands(self):
        return [Tensor(s, self.dtype, mem, lay.copy(), vs) for s, (mem, vs, lay) in zip(self.parameter_shapes(), self.auxes)]

    def output_index(self):
        return {MOVE: 1, FILL_ZERO: 0, MATMUL_ACCUM: 2, MATMUL: 2}[self.kind]

    def direction(self, idx):              # spec.rs:1204-1246: "in", "out", "inout"
        if self.kind == MOVE:
            return "in" if idx == 0 else "out"
        if self.kind == FILL_ZERO:
            return "out"
        if idx < 2:
            return "in"
        return "inout" if self.kind == MATMUL_ACCUM else "out"

    def blob(self):
        out = bytearray([self.kind, self.dtype, 1 if self.serial else 0, len(self.shape)])
        for d in self.shape:
            out += int(d).to_bytes(2, "little")
        for mem, vs, lay in self.auxes:
            out += bytes([mem, vs, len(lay.dims), lay.contig])
            for ldim, kind, size in lay.dims:
                out += bytes([ldim, kind]) + int(size).to_bytes(2, "little")
        return bytes(out)


def parse_blob(blob):
    kind, dtype, serial, rank = blob[0], blob[1], blob[2] != 0, blob[3]
    p = 4
    shape = []
    for _ in range(rank):
        shape.append(int.from_bytes(blob[p:p + 2], "little"))
        p += 2
    auxes = []
    for _ in range({MOVE: 2, FILL_ZERO: 1, MATMUL_ACCUM: 3, MATMUL: 3}[kind]):
        mem, vs, n, contig = blob[p], blob[p + 1], blob[p + 2], blob[p + 3]
        p += 4
        dims = []
        for _ in range(n):
            dims.append((blob[p], blob[p + 1], int.from_bytes(blob[p + 2:p + 4], "little")))
            p += 4
        auxes.append((mem, vs, Layout(dims, contig)))
    assert p == len(blob)
    return Spec(kind, dtype, serial, tuple(shape), auxes)


def move_symmetry_break(spec):                      # spec.rs:1717-1735; moves.rs:447-467
    first = spec.auxes[0][2]
    if all(lay == first and lay.fully_contiguous() for _, _, lay in spec.auxes):
        spec.auxes = [(mem, vs, row_major(spec.shape) if has_layout(mem) else lay) for mem, vs, lay in spec.auxes]


def canonicalize_spec(spec):                        # spec.rs:1704-1747; False = not canonicalizable
    new_auxes = []
    for shp, (mem, vs, lay) in zip(spec.parameter_shapes(), spec.auxes):
        t = Tensor(shp, spec.dtype, mem, lay.copy(), vs)
        if not canonicalize_tensor(t):
            return False
        new_auxes.append((mem, vs, t.layout))
    spec.auxes = new_auxes
    if spec.kind == MOVE:
        move_symmetry_break(spec)
    return True


def dim_range(dim, include_end):                    # spec.rs:3194-3214, TileScale::PowerOfTwo
    out = []
    x = 1
    while x < dim:
        out.append(x)
        x *= 2
    if include_end:
        out.append(dim)
    return out


def pack_sizes_all(dtype):                          # cpu.rs:2894-2907
    return [2] + [b // DTYPE_SIZE[dtype] for b in ALL_VECTOR_BYTES if b % DTYPE_SIZE[dtype] == 0]


def oddeven_sizes_all(dtype):                       # cpu.rs:2938-2951
    return [2 * b // DTYPE_SIZE[dtype] for b in ALL_VECTOR_BYTES if (2 * b) % DTYPE_SIZE[dtype] == 0]


def move_destination_layouts(shape, dtype):         # cpu.rs:399-453, 2878-3012
    base = [row_major(shape)]
    if not all(d == 1 for d in shape):
        if len(shape) == 2:
            c = col_major(shape)
            if c != base[0]:
                base.append(c)
        elif len(shape) == 4:
            c = nhwc(shape)
            if c != base[0]:
                base.append(c)
    result = list(base)
    for oddeven in (False, True):
        sizes = oddeven_sizes_all(dtype) if oddeven else pack_sizes_all(dtype)
        for orig in base:
            if not orig.dims:
                end = 0
            else:
                d = len(orig.dims) - 1
                while d > 0 and shape[d] == 1:      # the reference indexes the LOGICAL shape with a physical index here
                    d -= 1
                end = d + 1 if oddeven else d
            for ldim, _, _ in orig.dims[:end]:
                if shape[ldim] == 1:
                    continue
                for s in sizes:
                    ok = (s <= shape[ldim]) if oddeven else (s < shape[ldim])
                    if ok and shape[ldim] % s == 0:
                        result.append(layout_new(orig.dims + [(ldim, ODDEVEN if oddeven else PACKED, s)]))
    return result


@dataclass
class Action:
    number: int
    kind: int                  # LEAF / LOOP / MOVE_KIND / BLOCK
    imm: int                   # LEAF: kernel cost; LOOP: iterations; MOVE: base cost
    level: int                 # memory the action allocates in
    units: int                 # MOVE: units consumed; LEAF: the kernel's allocation
    children: List[bytes]      # canonical blobs of the sub-Specs, in request order
    what: str


def broadcastvecmult_side(ops):                     # cpu.rs:2719-2808
    out = ops[2]
    if out.mem != VRF or not out.is_contiguous():
        return False
    if not ops[0].is_contiguous() or not ops[1].is_contiguous():
        return False
    if ops[0].shape[0] != out.shape[0] or ops[1].shape[0] != out.shape[0]:
        return False
    if not out.vs or out.volume() % out.vs != 0:
        return False
    for si, bi in ((0, 1), (1, 0)):
        scalar, bcast = ops[si], ops[bi]
        if not rf_or_l1(scalar.mem) or not scalar.is_contiguous() or bcast.mem != VRF or not bcast.is_contiguous():
            continue
        if any(d != 1 for d in scalar.shape):
            continue
        if bcast.vs != out.vs or bcast.volume() % out.vs != 0:
            continue
        b1, b2 = bcast.shape[1], bcast.shape[2]
        s1, s2 = scalar.shape[1], scalar.shape[2]
        o1, o2 = out.shape[1], out.shape[2]
        if s1 == o1 and s2 == 1 and b1 == 1 and b2 == o2:
            return True
        if s1 == 1 and s2 == o2 and b1 == o1 and b2 == 1:
            return True
    return False


def kernels_for(spec):
    """(name, main cost, allocation level, allocation units) of every kernel of the Spec's list that
    applies, in list order (cpu.rs:477-611, 896-1879, 1881-1998, 2000-2380). Kernels that only take
    dtypes outside {u32, f32} are left out: they never apply here and take no action number."""
    ops = spec.operands()
    out = []
    io_cost = lambda: sum(move_cost(o) for o in ops)
    if spec.kind == MATMUL_ACCUM:
        if all(rf_or_l1(o.mem) and all(d == 1 for d in o.shape) for o in ops):            # MultAdd
            out.append(("MultAdd", (1 if spec.dtype == F32 else 2) + io_cost(), 0, 0))
        if spec.dtype in (U32, S32, F32, U16, S16, U8, S8) and broadcastvecmult_side(ops):   # BroadcastVecMultAdd
            out.append(("BroadcastVecMultAdd", (ops[2].volume() // ops[2].vs) * 2 + 1, VRF, 1))
        lhs, rhs, o = ops                                                                    # DotProductLoop
        if (spec.dtype == F32 and lhs.shape[0] == 1 and lhs.shape[1] == 1 and lhs.shape[2] % 8 == 0 and
                tuple(o.shape) == (1, 1, 1) and lhs.layout.is_row_major() and rhs.layout.is_col_major() and
                lhs.is_contiguous() and rhs.is_contiguous() and lhs.vs in (0, 8) and rhs.vs in (0, 8) and
                (lhs.mem == L1 or (lhs.mem == VRF and lhs.vs == 8)) and rhs.mem == L1 and rf_or_l1(o.mem)):
            out.append(("DotProductLoop", 8 * lhs.shape[2] // (8 * 4) + move_cost(o), VRF, 1))
    elif spec.kind == MOVE:
        src, dst = ops
        scalar = all(d == 1 for d in src.shape) and all(d == 1 for d in dst.shape)
        if scalar:
            if src.layout == dst.layout and rf_or_l1(src.mem) and rf_or_l1(dst.mem):
                out.append(("Assign", io_cost() + 1, 0, 0))
        elif src.is_contiguous() and dst.is_contiguous() and src.layout == dst.layout:
            has_vrf, ok = False, True
            for o in ops:
                if o.mem == VRF:
                    has_vrf = True
                    if o.volume() % o.vs != 0:
                        ok = False
            if has_vrf and ok:
                vs = src.vs if src.vs else dst.vs
                out.append(("Assign", src.volume() // vs, 0, 0))
    elif spec.kind == FILL_ZERO:
        t = ops[0]
        if t.mem not in (RF, VRF) and t.is_contiguous():
            out.append(("MemsetZero", 1, 0, 0))
        if t.volume() == 1 and rf_or_l1(t.mem):
            out.append(("ValueZero", io_cost() + 1, 0, 0))
        if t.is_contiguous() and t.mem == VRF and t.vs and t.vs == t.volume():
            out.append(("VectorZero", 1, 0, 0))
    return out


def plan_move(src, dest_mem, dest_layout, dest_vs):   # moves.rs:275-381; None = not applicable
    if not has_layout(dest_mem):
        lay, miss = Layout(), False
    elif not is_addressed(dest_mem):
        lay = canonicalize_layout(dest_layout, src.shape)
        assert lay is not None
        miss = src.layout == lay
        if not miss:
            lay.contig = len(lay.dims)
    else:
        lay = dest_layout.copy()
        lay.contig = len(lay.dims)
        miss = False
    new = Tensor(tuple(src.shape), src.dtype, dest_mem, lay, dest_vs)
    if not miss and not canonicalize_tensor(new):
        return None
    if src.same_as(new):
        return None
    return new, miss, memory_units(new)


def move_spec(left, right, serial):                 # moves.rs:383-413
    s = Spec(MOVE, left.dtype, serial, tuple(left.shape), [(left.mem, left.vs, left.layout.copy()),
                                                           (right.mem, right.vs, right.layout.copy())])
    move_symmetry_break(s)
    return s


def tiled_body(spec, new_shape):                    # tiling.rs:177-220, 506-533; None = not applicable
    body = spec.copy()
    body.shape = tuple(new_shape)
    new_auxes = []
    for old, shp, (mem, vs, lay) in zip(spec.operands(), body.parameter_shapes(), body.auxes):
        if has_layout(old.mem):
            lay = update_for_tiling(old.layout, old.shape, shp)
            if lay is None:
                return None   # the slow path then rejects the tile shape for this operand (tiling.rs:1044-1048)
        new_auxes.append((mem, vs, lay))
    body.auxes = new_auxes
    return body if canonicalize_spec(body) else None


def enumerate_actions(spec) -> List[Action]:        # cpu.rs:455-823
    assert spec.serial
    ops = spec.operands()
    actions = []
    number = 0
    # 1. Moves (common_actions.rs:301-376)
    for i, op in enumerate(ops):
        dest_layouts = move_destination_layouts(op.shape, op.dtype)
        dest_mems = possible_destination_memories(op.mem)
        proposals = []
        contains_source_layout = False
        for layout in dest_layouts:
            if not contains_source_layout and layout == op.layout:
                contains_source_layout = True
            for mem in dest_mems:
                vss = [b // DTYPE_SIZE[op.dtype] for b in VECTOR_BYTES[mem]] or [0]
                for vs in vss:
                    proposals.append((mem, layout, vs))
        if not contains_source_layout:
            for mem in dest_mems:
                if not is_addressed(mem):
                    proposals.append((mem, op.layout, 0))
        for mem, layout, vs in proposals:
            this = number
            number += 1
            plan = plan_move(op, mem, layout, vs)
            if plan is None:
                continue
            new, miss, units = plan
            direction = spec.direction(i)
            children = []
            if not miss and direction in ("in", "inout"):
                children.append(move_spec(op, new, spec.serial).blob())
            body = spec.copy()
            body.auxes[i] = (new.mem, new.vs, new.layout.copy())
            if body.kind == MOVE:
                move_symmetry_break(body)
            children.append(body.blob())
            if not miss and direction in ("out", "inout"):
                children.append(move_spec(new, op, spec.serial).blob())
            actions.append(Action(this, MOVE_KIND, move_cost(op) + move_cost(new), mem, units, children,
                                  f"move operand {i} to memory {mem}"))
    # 2. Serial single-loop tile-outs (common_actions.rs:37-121; tiling.rs:132-228)
    oi = spec.output_index()
    out = ops[oi]
    for size in dim_range(max(out.shape), True):
        for dim in range(len(out.shape)):
            this = number
            number += 1
            if out.shape[dim] == size or size > out.shape[dim]:
                continue
            tile = list(out.shape)
            tile[dim] = size
            if has_layout(out.mem) and expand_physical_shape(out.layout, tile) is None:
                continue
            assert out.shape[dim] % size == 0
            if spec.kind in (MATMUL, MATMUL_ACCUM):
                new_shape = (tile[0], tile[1], spec.shape[2], tile[2])
            else:
                new_shape = tuple(tile)
            body = tiled_body(spec, new_shape)
            if body is None:
                continue
            iters = 1
            for a, b in zip(spec.shape, body.shape):
                iters *= a // b
            actions.append(Action(this, LOOP, iters, 0, 0, [body.blob()], f"tile out dim {dim} to {size}"))
    # 3. Kernels that apply (inapplicable ones take no number)
    for name, cost, level, units in kernels_for(spec):
        actions.append(Action(number, LEAF, cost, level, units, [], name))
        number += 1
    # 4. Kind-specific tail
    if spec.kind == MATMUL:      # ToAccum (to_accum.rs:12-62): zero the output, then accumulate
        acc = spec.copy()
        acc.kind = MATMUL_ACCUM
        assert canonicalize_spec(acc)
        o = acc.operands()[2]
        fill = Spec(FILL_ZERO, spec.dtype, spec.serial, tuple(o.shape), [(o.mem, o.vs, o.layout.copy())])
        assert canonicalize_spec(fill)
        actions.append(Action(number, BLOCK, 0, 0, 0, [fill.blob(), acc.blob()], "to accum"))
        number += 1
    elif spec.kind == MATMUL_ACCUM:   # Split (common_actions.rs:123-249; tiling.rs:478-541)
        b, m, K, n = spec.shape
        for k in dim_range(K, False):
            ok0 = not has_layout(ops[0].mem) or expand_physical_shape(ops[0].layout, (b, m, k)) is not None
            ok1 = not has_layout(ops[1].mem) or expand_physical_shape(ops[1].layout, (b, k, n)) is not None
            if not (ok0 and ok1):
                continue
            this = number
            number += 1
            assert K % k == 0
            body = tiled_body(spec, (b, m, k, n))
            if body is None:
                continue
            actions.append(Action(this, LOOP, K // k, 0, 0, [body.blob()], f"split k to {k}"))
    return actions
