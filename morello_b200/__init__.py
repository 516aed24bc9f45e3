"""B200-native fill of Morello's synthesis database (one hot path, behind a C ABI).

Python mirror of the reference's search/database interface for this path:
`SynthesisDatabase.top_down_many` ~ morello::search::top_down_many,
`SynthesisDatabase.precompute` ~ the `precompute` binary,
`SynthesisDatabase.get` ~ FilesDatabase::get.
"""
from .db import (Decision, SynthesisDatabase, MAX_MEM, KIND_MOVE, KIND_FILL_ZERO, KIND_MATMUL_ACCUM, KIND_MATMUL,
                 DTYPE_U32, DTYPE_F32, RF, VRF, L1, GL, THROUGH_MOVE, THROUGH_ZERO, THROUGH_MATMUL, simple_spec,
                 describe_spec, tabulate)

__all__ = ["Decision", "SynthesisDatabase", "MAX_MEM", "simple_spec", "describe_spec", "tabulate", "KIND_MOVE", "KIND_FILL_ZERO",
           "KIND_MATMUL_ACCUM", "KIND_MATMUL", "DTYPE_U32", "DTYPE_F32", "RF", "VRF", "L1", "GL", "THROUGH_MOVE",
           "THROUGH_ZERO", "THROUGH_MATMUL"]
