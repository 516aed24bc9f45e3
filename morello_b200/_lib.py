"""ctypes binding of the C ABI declared in include/morello_b200.h."""
import ctypes as C
import os

from .build import LIB_PATH


class Decision(C.Structure):
    _fields_ = [("found", C.c_int32), ("action", C.c_uint32), ("main_cost", C.c_uint32), ("depth", C.c_uint32),
                ("peaks", C.c_uint64 * 4)]


class Row(C.Structure):
    _fields_ = [("main_cost", C.c_uint32), ("peak_codes", C.c_uint32), ("depth_action", C.c_uint32),
                ("reserved", C.c_uint32)]


class Stats(C.Structure):
    _fields_ = [("n_specs", C.c_uint64), ("n_goal_specs", C.c_uint64), ("n_candidates", C.c_uint64),
                ("n_stages", C.c_uint64), ("n_rows", C.c_uint64), ("n_cells_solved", C.c_uint64),
                ("n_candidates_evaluated", C.c_uint64), ("n_rows_gathered", C.c_uint64),
                ("n_passes", C.c_uint64), ("n_launches", C.c_uint64), ("n_grid_syncs", C.c_uint64),
                ("algorithmic_bytes", C.c_uint64), ("h2d_bytes", C.c_uint64), ("d2h_bytes", C.c_uint64),
                ("plan_seconds", C.c_double), ("upload_seconds", C.c_double), ("fill_ms", C.c_double),
                ("combine_ms", C.c_double), ("early_ms", C.c_double), ("n_sweeps", C.c_uint64), ("plan_goal_seconds", C.c_double), ("plan_discover_seconds", C.c_double),
                ("plan_layout_seconds", C.c_double), ("plan_layout_step_seconds", C.c_double * 8),
                ("n_cells_unordered", C.c_uint64),
                ("n_candidates_swept", C.c_uint64), ("n_items_swept", C.c_uint64), ("n_buffer_growths", C.c_uint64),
                ("phase_ms", C.c_double * 8)]


EXPORTS = {
    "mrl_ctx_create": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "mrl_ctx_destroy": (None, [C.c_void_p]),
    "mrl_last_error": (C.c_char_p, [C.c_void_p]),
    "mrl_spec_simple": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_uint32), C.c_int, C.c_int, C.c_char_p, C.c_size_t]),
    "mrl_spec_canonicalize": (C.c_int, [C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]),
    "mrl_spec_describe": (C.c_int, [C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]),
    "mrl_max_mem": (None, [C.POINTER(C.c_uint64)]),
    "mrl_top_down_many": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64), C.c_size_t, C.POINTER(C.c_uint64),
                                    C.POINTER(Decision)]),
    "mrl_top_down_many_noalloc": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64), C.c_size_t,
                                            C.POINTER(C.c_uint64), C.POINTER(Decision)]),
    "mrl_precompute": (C.c_int, [C.c_void_p, C.c_uint32, C.c_int, C.c_int]),
    "mrl_plan_precompute": (C.c_int, [C.c_void_p, C.c_uint32, C.c_int, C.c_int]),
    "mrl_plan_goals": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64), C.c_size_t]),
    "mrl_upload": (C.c_int, [C.c_void_p]),
    "mrl_fill": (C.c_int, [C.c_void_p]),
    "mrl_set_shard": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32]),
    "mrl_plan_share": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "mrl_plan_adopt": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_void_p), C.c_int]),
    "mrl_device_cands": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "mrl_plan_adopt_done": (C.c_int, [C.c_void_p, C.c_double]),
    "mrl_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mrl_num_stages": (C.c_uint64, [C.c_void_p]),
    "mrl_num_families": (C.c_uint64, [C.c_void_p]),
    "mrl_stage_info": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                 C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "mrl_family_info": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                  C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "mrl_spec_owners": (C.c_int, [C.c_void_p, C.c_char_p, C.c_uint64]),
    "mrl_device_rows": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "mrl_row_bytes": (C.c_uint32, []),
    "mrl_fill_begin": (C.c_int, [C.c_void_p]),
    "mrl_fill_stage_solve": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "mrl_fill_stage_place": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "mrl_fill_end": (C.c_int, [C.c_void_p]),
    "mrl_get_many": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64), C.c_size_t, C.POINTER(C.c_uint64),
                               C.POINTER(Decision)]),
    "mrl_get_impl": (C.c_long, [C.c_void_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_uint64), C.c_char_p, C.c_size_t]),
    "mrl_verify": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "mrl_get_stats": (C.c_int, [C.c_void_p, C.POINTER(Stats)]),
    "mrl_num_specs": (C.c_uint64, [C.c_void_p]),
    "mrl_spec_blob": (C.c_int, [C.c_void_p, C.c_uint64, C.c_char_p, C.c_size_t]),
    "mrl_spec_grid": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]),
    "mrl_export_rows": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(Decision), C.c_size_t]),
    "mrl_tabulate": (C.c_long, [C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]),
    "mrl_set_plan_flags": (C.c_int, [C.c_void_p, C.c_uint32]),
    "mrl_cands_arrived": (C.c_int, [C.c_void_p]),
    "mrl_checksum": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "mrl_export_all": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64]),
    "mrl_decode_row": (None, [C.POINTER(Row), C.POINTER(Decision)]),
    "mrl_export_rects": (C.c_long, [C.c_void_p, C.c_uint64, C.c_char_p, C.c_char_p, C.POINTER(Decision), C.c_size_t]),
    "mrl_save": (C.c_int, [C.c_void_p, C.c_char_p]),
    "mrl_load": (C.c_int, [C.c_void_p, C.c_char_p]),
    "mrl_put": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_uint64), C.POINTER(Decision)]),
}

_lib = None


def load():
    """Loads the CUDA extension. There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    path = LIB_PATH
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build the CUDA extension first (python -c 'import __graft_entry__ as g; g.build()')")
    lib = C.CDLL(path)
    for name, (restype, argtypes) in EXPORTS.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
