"""ctypes binding of libtenferro_b200.so (the C ABI declared in include/tenferro_b200.h).

This is the layer a Rust `tenferro-device` FFI module would occupy.  There is no CPU
path behind it: if the shared library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG.parent / "lib" / "libtenferro_b200.so"

c_size_p = C.POINTER(C.c_size_t)
c_ssize_p = C.POINTER(C.c_ssize_t)
c_u32_p = C.POINTER(C.c_uint32)


class TfbDesc(C.Structure):
    _fields_ = [
        ("op", C.c_int32),
        ("reduce_op", C.c_int32),
        ("modes_a", c_u32_p),
        ("n_modes_a", C.c_size_t),
        ("modes_b", c_u32_p),
        ("n_modes_b", C.c_size_t),
        ("modes_c", c_u32_p),
        ("n_modes_c", C.c_size_t),
        ("paired", c_u32_p),
        ("n_pairs", C.c_size_t),
        ("batch_dims", c_size_p),
        ("n_batch_dims", C.c_size_t),
        ("m", C.c_size_t),
        ("n", C.c_size_t),
        ("k", C.c_size_t),
    ]


class TfbView(C.Structure):
    _fields_ = [
        ("base", C.c_void_p),
        ("rank", C.c_size_t),
        ("dims", c_size_p),
        ("strides", c_ssize_p),
        ("offset", C.c_ssize_t),
        ("flags", C.c_uint32),
    ]


class TfbComputeDevice(C.Structure):
    _fields_ = [("kind", C.c_int32), ("device_id", C.c_int32)]


class TfbGemmProblem(C.Structure):
    _fields_ = [
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("a", C.c_void_p), ("a_rs", C.c_int64), ("a_cs", C.c_int64),
        ("b", C.c_void_p), ("b_rs", C.c_int64), ("b_cs", C.c_int64),
        ("c", C.c_void_p), ("c_rs", C.c_int64), ("c_cs", C.c_int64),
    ]


# Every exported symbol with (restype, argtypes).  tests/test_abi.py checks this table
# against the header, so a symbol cannot be declared and then forgotten here.
_VP = C.c_void_p
_VPP = C.POINTER(C.c_void_p)
PROTOTYPES = {
    "tfb_last_error": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "tfb_version": (C.c_char_p, []),
    "tfb_ctx_create": (C.c_int, [C.c_int, _VPP]),
    "tfb_ctx_destroy": (C.c_int, [_VP]),
    "tfb_ctx_device": (C.c_int, [_VP, C.POINTER(C.c_int)]),
    "tfb_ctx_stream": (C.c_int, [_VP, _VPP]),
    "tfb_ctx_set_stream": (C.c_int, [_VP, _VP]),
    "tfb_ctx_synchronize": (C.c_int, [_VP]),
    "tfb_ctx_properties": (C.c_int, [_VP, C.POINTER(C.c_int), c_size_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "tfb_alloc": (C.c_int, [_VP, C.c_size_t, _VPP]),
    "tfb_free": (C.c_int, [_VP, _VP]),
    "tfb_pool_stats": (C.c_int, [_VP, c_size_p, c_size_p]),
    "tfb_memcpy_h2d_async": (C.c_int, [_VP, _VP, _VP, C.c_size_t]),
    "tfb_memcpy_d2h_async": (C.c_int, [_VP, _VP, _VP, C.c_size_t]),
    "tfb_memcpy_d2d_async": (C.c_int, [_VP, _VP, _VP, C.c_size_t]),
    "tfb_memcpy_h2d_2d_async": (C.c_int, [_VP, _VP, C.c_size_t, _VP, C.c_size_t, C.c_size_t, C.c_size_t]),
    "tfb_memcpy_d2h_2d_async": (C.c_int, [_VP, _VP, C.c_size_t, _VP, C.c_size_t, C.c_size_t, C.c_size_t]),
    "tfb_memcpy_p2p_async": (C.c_int, [_VP, _VP, C.c_int, _VP, C.c_int, C.c_size_t]),
    "tfb_memset_async": (C.c_int, [_VP, _VP, C.c_int, C.c_size_t]),
    "tfb_host_alloc": (C.c_int, [C.c_size_t, _VPP]),
    "tfb_host_free": (C.c_int, [_VP]),
    "tfb_kernel_launch_count": (C.c_ulonglong, []),
    "tfb_ctx_profile_begin": (C.c_int, [_VP]),
    "tfb_ctx_profile_read": (C.c_int, [_VP, C.c_char_p, c_size_p, C.POINTER(C.c_double)]),
    "tfb_ctx_profile_end": (C.c_int, [_VP]),
    "tfb_probe_fp64_tflops": (C.c_int, [_VP, C.POINTER(C.c_double)]),
    "tfb_probe_hbm_gbs": (C.c_int, [_VP, C.POINTER(C.c_double)]),
    "tfb_probe_tf32_tflops": (C.c_int, [_VP, C.POINTER(C.c_double)]),
    "tfb_probe_tf32_tflops_sustained": (C.c_int, [_VP, C.c_double, C.POINTER(C.c_double)]),
    "tfb_selftest_wait_expiry": (C.c_int, [_VP, C.c_uint]),
    "tfb_ctx_capture_begin": (C.c_int, [_VP]),
    "tfb_ctx_capture_end": (C.c_int, [_VP, C.POINTER(_VP)]),
    "tfb_graph_launch": (C.c_int, [_VP]),
    "tfb_graph_destroy": (None, [_VP]),
    "tfb_probe_mma_issue_cycles": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "tfb_event_record": (C.c_int, [_VP, _VPP]),
    "tfb_event_wait": (C.c_int, [_VP, _VP]),
    "tfb_event_synchronize": (C.c_int, [_VP]),
    "tfb_event_query": (C.c_int, [_VP, C.POINTER(C.c_int)]),
    "tfb_event_elapsed_ms": (C.c_int, [_VP, _VP, C.POINTER(C.c_float)]),
    "tfb_event_destroy": (C.c_int, [_VP]),
    "tfb_preferred_compute_devices": (
        C.c_int, [C.c_int32, C.c_size_t, C.c_int32, C.POINTER(TfbComputeDevice), C.c_size_t, c_size_p]),
    "tfb_compute_device_format": (C.c_size_t, [TfbComputeDevice, C.c_char_p, C.c_size_t]),
    "tfb_has_extension": (C.c_int, [C.c_int32, C.c_int32]),
    "tfb_plan_create": (
        C.c_int, [_VP, C.POINTER(TfbDesc), C.c_int32, C.c_size_t, c_size_p, C.POINTER(c_size_p), _VPP]),
    "tfb_plan_destroy": (C.c_int, [_VP]),
    "tfb_plan_kernel_name": (C.c_char_p, [_VP]),
    "tfb_plan_force_kernel": (C.c_int, [_VP, C.c_int]),
    "tfb_plan_set_algebra": (C.c_int, [_VP, C.c_int32]),
    "tfb_has_extension_for_algebra": (C.c_int, [C.c_int32, C.c_int32, C.c_int32]),
    "tfb_execute": (C.c_int, [_VP, _VP, C.c_size_t, C.POINTER(TfbView), _VP, C.POINTER(TfbView)]),
    "tfb_reduce_static": (
        C.c_int, [_VP, C.c_int32, C.c_int32, c_u32_p, C.c_size_t, C.POINTER(TfbView), c_u32_p, C.c_size_t,
                  C.POINTER(TfbView), _VP, _VP]),
    "tfb_grouped_gemm": (C.c_int, [_VP, C.c_int32, C.c_size_t, C.POINTER(TfbGemmProblem), _VP, _VP]),
    "tfb_grouped_plan_create": (C.c_int, [_VP, C.c_int32, C.c_size_t, C.POINTER(TfbGemmProblem), C.POINTER(_VP)]),
    "tfb_grouped_plan_execute": (C.c_int, [_VP, _VP, _VP]),
    "tfb_grouped_plan_destroy": (None, [_VP]),
    "tfb_subscripts_new": (C.c_int, [C.c_size_t, c_size_p, C.POINTER(c_u32_p), C.c_size_t, c_u32_p, _VPP]),
    "tfb_subscripts_parse": (C.c_int, [C.c_char_p, _VPP]),
    "tfb_subscripts_destroy": (C.c_int, [_VP]),
    "tfb_subscripts_n_inputs": (C.c_size_t, [_VP]),
    "tfb_subscripts_input": (C.c_size_t, [_VP, C.c_size_t, c_u32_p, C.c_size_t]),
    "tfb_subscripts_output": (C.c_size_t, [_VP, c_u32_p, C.c_size_t]),
    "tfb_subscripts_has_order": (C.c_int, [_VP]),
    "tfb_tree_optimize": (C.c_int, [_VP, c_size_p, C.POINTER(c_size_p), _VPP]),
    "tfb_tree_from_pairs": (C.c_int, [_VP, c_size_p, C.POINTER(c_size_p), C.c_size_t, c_size_p, _VPP]),
    "tfb_tree_destroy": (C.c_int, [_VP]),
    "tfb_tree_n_steps": (C.c_size_t, [_VP]),
    "tfb_tree_pairs": (C.c_size_t, [_VP, c_size_p, C.c_size_t]),
    "tfb_tree_macs": (C.c_double, [_VP]),
    "tfb_tree_output_dims": (C.c_size_t, [_VP, c_size_p, C.c_size_t]),
    "tfb_einsum_with_plan_into": (
        C.c_int, [_VP, _VP, C.c_int32, C.c_size_t, C.POINTER(TfbView), _VP, _VP, C.POINTER(TfbView)]),
}


def _load() -> C.CDLL:
    path = os.environ.get("TENFERRO_B200_LIB", str(LIB_PATH))
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `make -C tenferro-rs_b200/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). "
            "There is no CPU path to fall back to."
        )
    lib = C.CDLL(path)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    n = lib.tfb_last_error(None, 0)
    buf = C.create_string_buffer(n + 1)
    lib.tfb_last_error(buf, n + 1)
    return buf.value.decode("utf-8", "replace")
