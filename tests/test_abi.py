"""CPU tests of the boundary: the library loads and exports what the header declares, and the
host-only entry points (Spec blobs, canonicalisation) behave like the reference's."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "morello_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mrl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_extension):
    lib = C.CDLL(built_extension)
    names = _declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_the_header(built_extension):
    from morello_b200 import _lib
    assert sorted(_lib.EXPORTS) == _declared_functions()


def test_python_structs_match_the_header(built_extension, tmp_path):
    """The ctypes mirrors of the header's structs have the sizes and field offsets a C compiler
    gives them (the statistics struct grows with the kernels; a field added on one side only would
    shift everything behind it)."""
    import shutil
    import subprocess
    from morello_b200 import _lib
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    fields = [name for name, _ in _lib.Stats._fields_]
    src = tmp_path / "sizes.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "morello_b200.h"', "int main(void) {",
             '  printf("%zu\\n", sizeof(mrl_stats));']
    lines += ['  printf("%%zu\\n", offsetof(mrl_stats, %s));' % f for f in fields]
    lines += ['  printf("%zu %zu\\n", sizeof(mrl_decision), sizeof(mrl_row));', "  return 0;", "}"]
    src.write_text("\n".join(lines))
    exe = tmp_path / "sizes"
    subprocess.run([cc, "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) == C.sizeof(_lib.Stats)
    for k, f in enumerate(fields):
        assert int(out[1 + k]) == getattr(_lib.Stats, f).offset, f
    assert int(out[-2]) == C.sizeof(_lib.Decision) and int(out[-1]) == C.sizeof(_lib.Row)


def test_spec_blobs_roundtrip_and_canonicalise(built_extension):
    import morello_b200 as m
    goal = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 2, 2, 2], m.GL)
    assert m.describe_spec(goal) == "Matmul(1x2x2x2, (u32, GL, [1, 2]), (u32, GL, [1, 2]), (u32, GL, [1, 2]), serial)"
    # all-ones operands have empty layouts after canonicalisation (layout.rs:455-472)
    one = m.simple_spec(m.KIND_MATMUL, m.DTYPE_F32, [1, 1, 1, 1], m.L1)
    assert "(f32, L1, [])" in m.describe_spec(one)
    # RF has no layout (tensorspec.rs:371-372)
    rf = m.simple_spec(m.KIND_MOVE, m.DTYPE_U32, [2, 2], m.RF)
    assert m.describe_spec(rf) == "Move(2x2, (u32, RF), (u32, RF), serial)"
    with pytest.raises(ValueError):
        m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 2, 2], m.GL)  # Matmul needs rank 4


def test_no_cpu_fallback(built_extension):
    """Without a CUDA device the context refuses to exist; nothing is computed on the host."""
    import torch
    import morello_b200 as m
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="no usable CUDA device"):
        m.SynthesisDatabase()
