"""ctypes loader for libtei_b200.so.

The library is built in-tree by `text-embeddings-inference_b200/build.py`.  There is no fallback:
if the shared object is missing, `load()` raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_longlong, POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_size_t, c_uint32, c_uint64, c_void_p
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent.parent
LIB_PATH = PKG_ROOT / "lib" / "libtei_b200.so"

_lib = None

# name -> (restype, argtypes); mirrors include/tei_b200_ops.h and include/tei_b200.h
_OPS_PROTOTYPES = {
    "tei_b200_op_linear": (c_int, [c_void_p] * 5 + [c_int] * 8 + [c_void_p, c_void_p]),
    "tei_b200_op_linear_rope": (
        c_int, [c_void_p] * 4 + [c_int] * 5 + [c_void_p] * 5 + [c_int] * 3 + [c_float, c_int, c_void_p, c_void_p]),
    "tei_b200_attention_plan": (c_int, [POINTER(c_int32), c_int, c_int, POINTER(c_int32), c_int]),
    "tei_b200_attention_plan_windowed": (
        c_int, [POINTER(c_int32), c_int, c_int, c_int, c_int, POINTER(c_int32), c_int]),
    "tei_b200_op_attention": (
        c_int,
        [c_void_p] * 5 + [c_int] * 10 + [c_float, c_void_p, c_int, c_void_p, c_void_p],
    ),
    "tei_b200_op_attention_windowed": (
        c_int,
        [c_void_p] * 5 + [c_int] * 12 + [c_float, c_void_p, c_int, c_void_p, c_void_p],
    ),
    "tei_b200_op_embed_layernorm": (c_int, [c_void_p] * 9 + [c_int, c_int, c_float, c_int, c_void_p]),
    "tei_b200_op_add_norm": (c_int, [c_void_p] * 6 + [c_int, c_int, c_float, c_int, c_int, c_void_p]),
    "tei_b200_op_qk_norm_rope": (c_int, [c_void_p] * 7 + [c_int] * 6 + [c_float, c_int, c_void_p]),
    "tei_b200_op_pool": (c_int, [c_void_p] * 4 + [c_int] * 5 + [c_void_p]),
    "tei_b200_op_gather_rows_f32": (c_int, [c_void_p] * 3 + [c_int] * 3 + [c_void_p]),
    "tei_b200_op_head_linear": (c_int, [c_void_p] * 4 + [c_int] * 5 + [c_void_p]),
    "tei_b200_op_linear_rows_dev": (c_int, [c_void_p] * 4 + [c_int] * 7 + [c_void_p, c_void_p, c_void_p]),
    "tei_b200_op_moe_route": (c_int, [c_void_p, c_int, c_int, c_int, c_int] + [c_void_p] * 4 + [c_int, c_void_p]),
    "tei_b200_op_moe_route_noalloc": (
        c_int, [c_void_p, c_int, c_int, c_int, c_int] + [c_void_p] * 4 + [c_int, c_void_p, c_char_p, c_size_t]),
    "tei_b200_op_bounded_wait_probe": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    "tei_b200_gemm_tiling": (c_int, [c_int, c_int, c_int, c_int]),
    "tei_b200_op_moe_gather": (c_int, [c_void_p] * 4 + [c_int] * 3 + [c_longlong, c_int, c_void_p]),
    "tei_b200_op_moe_combine": (c_int, [c_void_p] * 6 + [c_int] * 3 + [c_longlong, c_int, c_void_p]),
}

_BATCH = [POINTER(c_uint32), POINTER(c_uint32), POINTER(c_uint32), c_size_t, POINTER(c_uint32), c_size_t,
          c_uint32]

_BACKEND_PROTOTYPES = {
    "tei_b200_create": (
        c_int,
        [c_char_p, c_char_p, c_int, c_int, POINTER(c_int), c_int, POINTER(c_void_p), c_char_p, c_size_t],
    ),
    "tei_b200_add_dense": (c_int, [c_void_p, c_char_p, c_char_p, c_size_t]),
    "tei_b200_destroy": (None, [c_void_p]),
    "tei_b200_health": (c_int, [c_void_p]),
    "tei_b200_is_padded": (c_int, [c_void_p]),
    "tei_b200_max_batch_size": (c_int, [c_void_p]),
    "tei_b200_output_dim": (c_int, [c_void_p]),
    "tei_b200_hidden_size": (c_int, [c_void_p]),
    "tei_b200_num_classes": (c_int, [c_void_p]),
    "tei_b200_position_offset": (c_int, [c_void_p]),
    "tei_b200_embed": (
        c_int,
        [c_void_p] + _BATCH + [POINTER(c_uint32), c_size_t, POINTER(c_uint32), c_size_t, c_int,
                               POINTER(c_float), POINTER(c_float), c_char_p, c_size_t],
    ),
    "tei_b200_predict": (c_int, [c_void_p] + _BATCH + [POINTER(c_float), c_char_p, c_size_t]),
    "tei_b200_num_replicas": (c_int, [c_void_p]),
    "tei_b200_embed_on": (
        c_int,
        [c_void_p, c_int] + _BATCH + [POINTER(c_uint32), c_size_t, POINTER(c_uint32), c_size_t, c_int,
                                      POINTER(c_float), POINTER(c_float), c_char_p, c_size_t],
    ),
    "tei_b200_predict_on": (c_int, [c_void_p, c_int] + _BATCH + [POINTER(c_float), c_char_p, c_size_t]),
    "tei_b200_stage": (
        c_int,
        [c_void_p] + _BATCH + [POINTER(c_uint32), c_size_t, POINTER(c_uint32), c_size_t, c_int, c_int,
                               c_char_p, c_size_t],
    ),
    "tei_b200_run_staged": (c_int, [c_void_p, c_char_p, c_size_t]),
    "tei_b200_sync": (c_int, [c_void_p, c_char_p, c_size_t]),
    "tei_b200_fetch": (
        c_int,
        [c_void_p, POINTER(c_float), POINTER(c_float), POINTER(c_float), c_char_p, c_size_t],
    ),
    "tei_b200_run_staged_timed": (c_int, [c_void_p, c_int, POINTER(c_double), c_char_p, c_size_t]),
    "tei_b200_set_profiling": (c_int, [c_void_p, c_int]),
    "tei_b200_kernel_times": (c_int, [c_void_p, POINTER(c_double), POINTER(c_double), c_int]),
    "tei_b200_stats": (c_int, [c_void_p, POINTER(c_double), c_int]),
    "tei_b200_set_last_layer_shortcut": (c_int, [c_void_p, c_int]),
    "tei_b200_set_fused_rope": (c_int, [c_void_p, c_int]),
    "tei_b200_set_fused_residual": (c_int, [c_void_p, c_int]),
    "tei_b200_selftest_report_timeout": (c_int, [c_void_p, c_int, c_int]),
    "tei_b200_split_echo": (
        c_int,
        [POINTER(c_uint32), POINTER(c_uint32), POINTER(c_uint32), c_size_t, POINTER(c_uint32), c_size_t,
         POINTER(c_uint32), c_size_t, POINTER(c_uint32), c_size_t, c_int, c_int, c_double, c_double, c_int,
         POINTER(c_float), POINTER(c_float), POINTER(c_float), POINTER(c_int)],
    ),
    "tei_b200_compile_compute_cap": (c_int, []),
    "tei_b200_compute_cap_matching": (c_int, [c_int, c_int]),
    "tei_b200_plan_shards": (
        c_int,
        [POINTER(c_uint32), c_size_t, c_int, c_double, c_double, POINTER(c_int)],
    ),
}


_U32P = POINTER(c_uint32)
_SZP = POINTER(c_size_t)

# mirrors include/tei_b200_queue.h
_QUEUE_PROTOTYPES = {
    "tei_b200_queue_create": (c_int, [c_int, c_size_t, c_size_t, POINTER(c_void_p)]),
    "tei_b200_queue_destroy": (None, [c_void_p]),
    "tei_b200_queue_append": (c_int, [c_void_p, _U32P, _U32P, _U32P, c_size_t, c_uint32, c_int, c_uint64]),
    "tei_b200_queue_cancel": (c_int, [c_void_p, c_uint64, _SZP]),
    "tei_b200_queue_len": (c_size_t, [c_void_p]),
    "tei_b200_queue_next_batch": (
        c_int,
        [c_void_p, _U32P, _U32P, _U32P, c_size_t, _U32P, _U32P, _U32P, POINTER(c_uint64), c_size_t,
         _SZP, _SZP, _SZP, _SZP, _U32P],
    ),
}


def prototypes() -> dict:
    out = dict(_OPS_PROTOTYPES)
    out.update(_BACKEND_PROTOTYPES)
    out.update(_QUEUE_PROTOTYPES)
    return out


def load() -> ctypes.CDLL:
    """Loads the shared library and attaches prototypes.  Raises if it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {PKG_ROOT / 'build.py'}`. "
            "There is no CPU or library fallback for this path."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in prototypes().items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
