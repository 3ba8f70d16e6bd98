"""ctypes declarations of the C ABI in include/vkml_b200.h and the library loader.

The CUDA library is the only implementation behind this package: if
``vkml_b200/lib/libvkml_b200.so`` is missing or cannot be loaded, importing the
loader raises -- there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

MAX_DIMS = 4
MAX_SRC = 4
PARAM_BYTES = 64
UNIQUE_ID_BYTES = 128


class Tensor(C.Structure):
    """b200_tensor"""
    _fields_ = [
        ("data", C.c_void_p),
        ("dims", C.c_int64 * MAX_DIMS),
        ("strides", C.c_int64 * MAX_DIMS),
        ("ndim", C.c_int32),
        ("dtype", C.c_int32),
    ]


class Node(C.Structure):
    """b200_node"""
    _fields_ = [
        ("op", C.c_uint32),
        ("n_src", C.c_uint32),
        ("out", Tensor),
        ("src", Tensor * MAX_SRC),
        ("params", C.c_uint8 * PARAM_BYTES),
    ]


class Copy(C.Structure):
    """b200_copy"""
    _fields_ = [("dst", C.c_void_p), ("src", C.c_void_p), ("nbytes", C.c_size_t)]


class Caps(C.Structure):
    """b200_caps"""
    _fields_ = [
        ("name", C.c_char * 128),
        ("cc_major", C.c_int32),
        ("cc_minor", C.c_int32),
        ("sm_count", C.c_uint32),
        ("warp_size", C.c_uint32),
        ("max_threads_per_block", C.c_uint32),
        ("max_shared_memory_bytes", C.c_size_t),
        ("total_memory_bytes", C.c_size_t),
        ("min_buffer_alignment", C.c_size_t),
    ]


class Stats(C.Structure):
    """b200_stats"""
    _fields_ = [(n, C.c_uint64) for n in (
        "reserved_bytes", "in_use_bytes", "peak_in_use_bytes", "live_allocations",
        "total_allocations", "driver_allocations", "compute_calls", "kernel_launches",
        "nodes_computed", "comm_bytes")]


class ProfileRecord(C.Structure):
    """b200_profile_record"""
    _fields_ = [("label", C.c_char * 48), ("ms", C.c_float), ("op", C.c_uint32), ("submission", C.c_uint32)]


# Every symbol include/vkml_b200.h declares: name -> (restype, argtypes).
_P = C.c_void_p
SYMBOLS = {
    "b200_abi_version": (C.c_int, []),
    "b200_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "b200_create": (C.c_int, [C.c_int, C.POINTER(_P)]),
    "b200_destroy": (None, [_P]),
    "b200_get_caps": (C.c_int, [_P, C.POINTER(Caps)]),
    "b200_alloc": (C.c_int, [_P, C.c_size_t, C.POINTER(_P)]),
    "b200_free": (C.c_int, [_P, _P]),
    "b200_trim": (C.c_int, [_P]),
    "b200_supports": (C.c_int, [C.POINTER(Node)]),
    "b200_compute": (C.c_int, [_P, C.POINTER(Node), C.c_size_t, C.c_uint32]),
    "b200_copy_from_host": (C.c_int, [_P, _P, _P, C.c_size_t]),
    "b200_copy_to_host": (C.c_int, [_P, _P, _P, C.c_size_t]),
    "b200_copy_device_to_device": (C.c_int, [_P, C.POINTER(Copy), C.c_size_t]),
    "b200_synchronize": (C.c_int, [_P]),
    "b200_last_error": (C.c_char_p, [_P]),
    "b200_status_name": (C.c_char_p, [C.c_int]),
    "b200_get_stats": (C.c_int, [_P, C.POINTER(Stats)]),
    "b200_profile_enable": (C.c_int, [_P, C.c_int]),
    "b200_profile_read": (C.c_int, [_P, C.POINTER(ProfileRecord), C.c_size_t, C.POINTER(C.c_size_t)]),
    "b200_timer_begin": (C.c_int, [_P]),
    "b200_timer_end": (C.c_int, [_P, C.POINTER(C.c_float)]),
    "b200_alloc_host": (C.c_int, [_P, C.c_size_t, C.POINTER(_P)]),
    "b200_free_host": (C.c_int, [_P, _P]),
    "b200_set_gemm_precision": (C.c_int, [_P, C.c_int]),
    "b200_get_gemm_precision": (C.c_int, [_P]),
    "b200_matmul_kernel": (C.c_int, [_P, C.POINTER(Node), C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]),
    "b200_stream": (_P, [_P]),
    "b200_debug_expire_wait": (C.c_int, [_P, C.c_uint64]),
    "b200_span_graph_stats": (C.c_int, [_P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "b200_dist_unique_id": (C.c_int, [_P]),
    "b200_dist_init": (C.c_int, [_P, C.c_int, C.c_int, _P]),
    "b200_dist_init_deadline": (C.c_int, [_P, C.c_int, C.c_int, _P, C.c_int]),
    "b200_dist_destroy": (C.c_int, [_P]),
    "b200_dist_all_reduce_mean": (C.c_int, [_P, _P, C.c_size_t]),
    "b200_dist_wait": (C.c_int, [_P]),
    "b200_dist_mark_grad": (C.c_int, [_P, _P, C.c_size_t]),
    "b200_dist_clear_grads": (C.c_int, [_P]),
    "b200_tape_create": (C.c_int, [_P, C.c_int, C.POINTER(_P)]),
    "b200_tape_add_template": (C.c_int, [_P, C.POINTER(C.c_int64), C.c_size_t, C.c_int, C.POINTER(C.c_int)]),
    "b200_tape_run": (C.c_int, [_P, C.c_int, C.POINTER(_P), C.c_size_t, C.POINTER(_P), C.c_size_t, C.c_uint32]),
    "b200_tape_enable_graphs": (C.c_int, [_P, C.c_int]),
    "b200_tape_stats": (C.c_int, [_P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "b200_tape_destroy": (None, [_P]),
    "b200_sum_columns_f32_noalloc": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, _P, _P, C.c_char_p, C.c_size_t]),
}

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libvkml_b200.so")

_lib = None


def load() -> C.CDLL:
    """Load libvkml_b200.so and bind every declared symbol. Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"vkml_b200: the CUDA library {LIB_PATH} has not been built "
            "(run `python -c 'import __graft_entry__ as g; g.build()'` or `make -C vkml_b200/csrc`); "
            "there is no CPU fallback")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the export is missing
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
