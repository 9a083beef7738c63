"""Loader of the native library (same role as the reference's qtensor/cextension.py:21-29).

The reference picks `libqtensor_cuda{torch CUDA version}.so`; this build ships one
sm_100a library, `libqtensor_b200.so`, next to this file.  There is no fallback: when
the library is absent get_lib() raises, and every CUDA entry point of
qtensor.functional then fails with a RuntimeError.
"""
import ctypes as ct
from pathlib import Path

LIBRARY_NAME = "libqtensor_b200.so"

# every symbol the library must export: the sixteen that the reference's
# qtensor/functional.py:17-60 dereferences at import time, then the additive ones
LEGACY_SYMBOLS = tuple(
    f"c{op}_blockwise_{kind}{bits}bit_{dt}"
    for op in ("quantize", "dequantize")
    for kind in ("", "diagreal_")
    for bits in (8, 4)
    for dt in ("fp32", "bf16")
)
EXTRA_SYMBOLS = (
    "qt_version", "qt_launch_count", "qt_note_graph_replay", "qt_last_error", "qt_error_string", "qt_set_stream",
    "qt_quantize_blockwise", "qt_dequantize_blockwise", "qt_dequantize_planes", "qt_householder_panel", "qt_merge_t", "qt_selftest_division", "qt_split_bf16", "qt_split_bf16_rows", "qt_gemm_bf16x3", "qt_split_bf16_3", "qt_gemm_bf16x6", "qt_gemm_bf16x3_q4", "qt_gemm_bf16x6_q4", "qt_matmul_f32", "qt_matmul_f32_scratch_bytes", "qt_matmul_f32_static", "qt_device_error", "qt_adamw_tail", "qt_selftest_wait_timeout", "qt_gemm_ex", "qt_gemm_force_tile", "qt_panel_force_form", "qt_column_dot", "qt_power_iter",
    "qt_inverse_root_newton", "qt_inverse_root_newton_workspace_bytes", "qt_split_f16", "qt_dequantize_planes_f16", "qt_householder_panel_fused", "qt_state_exponents",
)

_lib = None


class GemmDesc(ct.Structure):
    """Mirror of qt_gemm_desc (include/qtensor_b200.h)."""
    _fields_ = [("A", ct.c_void_p * 3), ("lda", ct.c_longlong), ("strideA", ct.c_longlong), ("a_mn", ct.c_int), ("a_entries", ct.c_int),
                ("B", ct.c_void_p * 3), ("ldb", ct.c_longlong), ("strideB", ct.c_longlong), ("b_mn", ct.c_int), ("b_entries", ct.c_int),
                ("M", ct.c_int), ("N", ct.c_int), ("K", ct.c_int), ("batch", ct.c_int), ("alpha", ct.c_float), ("beta", ct.c_float),
                ("C", ct.c_void_p), ("ldc", ct.c_longlong), ("strideC", ct.c_longlong),
                ("D", ct.c_void_p), ("ldd", ct.c_longlong), ("strideD", ct.c_longlong),
                ("P", ct.c_void_p * 3), ("ldp", ct.c_longlong), ("strideP", ct.c_longlong),
                ("T", ct.c_void_p * 3), ("t_c0", ct.c_float), ("t_c1", ct.c_float),
                ("maxdev", ct.c_void_p),
                ("a_slot", ct.c_void_p), ("b_slot", ct.c_void_p), ("d_slot", ct.c_void_p), ("active", ct.c_void_p),
                ("f16", ct.c_int), ("ab_exp0", ct.c_int), ("out_exp0", ct.c_int), ("out_rel", ct.c_int), ("kc", ct.c_int),
                ("a_exp", ct.c_void_p), ("b_exp", ct.c_void_p), ("out_exp", ct.c_void_p), ("out_exp_w", ct.c_void_p),
                ("q_code", ct.c_void_p), ("q_in", ct.c_void_p), ("q_absmax_in", ct.c_void_p), ("q_diag_in", ct.c_void_p),
                ("q_out", ct.c_void_p), ("q_absmax_out", ct.c_void_p), ("q_diag_out", ct.c_void_p),
                ("q_stride_codes", ct.c_longlong), ("q_stride_absmax", ct.c_longlong), ("q_stride_diag", ct.c_longlong),
                ("oq_code", ct.c_void_p),
                ("aq_codes", ct.c_void_p), ("aq_absmax", ct.c_void_p), ("aq_diag", ct.c_void_p), ("aq_slots", ct.c_void_p),
                ("aq_stride_codes", ct.c_longlong), ("aq_stride_absmax", ct.c_longlong), ("aq_stride_diag", ct.c_longlong),
                ("bq_codes", ct.c_void_p), ("bq_absmax", ct.c_void_p), ("bq_diag", ct.c_void_p), ("bq_slots", ct.c_void_p),
                ("bq_stride_codes", ct.c_longlong), ("bq_stride_absmax", ct.c_longlong), ("bq_stride_diag", ct.c_longlong),
                ("max_ctas", ct.c_int), ("c_follows_d", ct.c_int)]


def library_path() -> Path:
    return (Path(__file__).parent / LIBRARY_NAME).resolve()


def _declare(lib):
    vp, i32, i64 = ct.c_void_p, ct.c_int, ct.c_longlong
    lib.qt_version.restype = i32
    lib.qt_last_error.restype = i32
    lib.qt_launch_count.restype = ct.c_ulonglong
    lib.qt_note_graph_replay.restype = None
    lib.qt_note_graph_replay.argtypes = [ct.c_ulonglong]
    lib.qt_error_string.restype = ct.c_char_p
    lib.qt_error_string.argtypes = [i32]
    lib.qt_set_stream.restype = None
    lib.qt_set_stream.argtypes = [vp]
    lib.qt_quantize_blockwise.restype = i32
    lib.qt_quantize_blockwise.argtypes = [vp, i32, i64, vp, i32, i32, vp, i64, vp, i64, vp, i64, i32, i32, vp]
    lib.qt_dequantize_blockwise.restype = i32
    lib.qt_dequantize_blockwise.argtypes = [vp, i64, vp, i32, i32, vp, i64, vp, i64, vp, i32, i64, i32, i32, vp]
    lib.qt_selftest_division.restype = i32
    lib.qt_selftest_division.argtypes = [ct.c_ulonglong, ct.c_ulonglong, vp, vp]
    lib.qt_householder_panel.restype = i32
    lib.qt_householder_panel.argtypes = [vp, i64, i32, i32, i32, i32, vp, i64, vp, i64, vp]
    f32 = ct.c_float
    lib.qt_split_bf16.restype = i32
    lib.qt_split_bf16.argtypes = [vp, i64, i64, i32, i32, i32, vp, vp, i64, i64, vp]
    lib.qt_gemm_bf16x3.restype = i32
    lib.qt_gemm_bf16x3.argtypes = [vp, vp, i64, i64, i32, vp, vp, i64, i64, i32, i32, i32, i32, i32, f32, f32,
                                   vp, i64, i64, vp, i64, i64, vp, vp, i64, i64, vp]
    lib.qt_split_bf16_3.restype = i32
    lib.qt_split_bf16_3.argtypes = [vp, i64, i64, i32, i32, i32, vp, vp, vp, i64, i64, vp]
    lib.qt_gemm_bf16x6.restype = i32
    lib.qt_gemm_bf16x6.argtypes = [vp, vp, vp, i64, i64, i32, vp, vp, vp, i64, i64, i32, i32, i32, i32, i32, f32, f32,
                                   vp, i64, i64, vp, i64, i64, vp]
    lib.qt_adamw_tail.restype = i32
    lib.qt_adamw_tail.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, vp, f32, f32, f32, f32, f32, vp]
    lib.qt_merge_t.restype = i32
    lib.qt_merge_t.argtypes = [vp, i64, i64, vp, i64, i32, i32, vp, i64, vp]
    lib.qt_split_bf16_rows.restype = i32
    lib.qt_split_bf16_rows.argtypes = [vp, i64, i64, i32, i32, i32, vp, i64, vp, i64, vp, vp, i64, i64, vp]
    lib.qt_dequantize_planes.restype = i32
    lib.qt_dequantize_planes.argtypes = [vp, i64, vp, i32, i32, vp, i64, vp, i64, vp, vp, vp, i64, i64, i32, i32, vp]
    lib.qt_gemm_bf16x3_q4.restype = i32
    lib.qt_gemm_bf16x3_q4.argtypes = [vp, vp, i64, i64, i32, vp, vp, i64, i64, i32, i32, i32, i32, f32, f32, vp,
                                      vp, vp, vp, vp, vp, vp, i64, i64, i64, vp]
    lib.qt_gemm_bf16x6_q4.restype = i32
    lib.qt_gemm_bf16x6_q4.argtypes = [vp, vp, vp, i64, i64, i32, vp, vp, vp, i64, i64, i32, i32, i32, i32, f32, f32, vp,
                                      vp, vp, vp, vp, vp, vp, i64, i64, i64, vp]
    lib.qt_matmul_f32_scratch_bytes.restype = ct.c_ulonglong
    lib.qt_matmul_f32_scratch_bytes.argtypes = [i32, i32, i32, i32, i32, i32]
    lib.qt_matmul_f32.restype = i32
    lib.qt_matmul_f32.argtypes = [vp, i64, i64, i32, vp, i64, i64, i32, i32, i32, i32, i32, f32, f32,
                                  vp, i64, i64, vp, i64, i64, vp, ct.c_ulonglong, vp]
    lib.qt_matmul_f32_static.restype = i32
    lib.qt_matmul_f32_static.argtypes = [vp, i64, i64, i32, vp, i64, i64, i32, i32, i32, i32, i32, f32, f32,
                                         vp, i64, i64, vp, i64, i64, vp]
    lib.qt_device_error.restype = i32
    lib.qt_device_error.argtypes = [i32]
    lib.qt_gemm_ex.restype = i32
    lib.qt_gemm_ex.argtypes = [ct.POINTER(GemmDesc), vp]
    lib.qt_split_f16.restype = i32
    lib.qt_split_f16.argtypes = [vp, i64, i64, i32, i32, i32, vp, i64, vp, i64, vp, i32, vp, i32, vp, vp, vp, i64, i64, vp]
    lib.qt_dequantize_planes_f16.restype = i32
    lib.qt_dequantize_planes_f16.argtypes = [vp, i64, vp, i32, i32, vp, i64, vp, i64, vp, vp, i32, vp, vp, vp, i64, i64, i32, i32, vp]
    lib.qt_state_exponents.restype = i32
    lib.qt_state_exponents.argtypes = [vp, i64, i32, vp, i64, i32, vp, i32, i32, vp, vp]
    lib.qt_householder_panel_fused.restype = i32
    lib.qt_householder_panel_fused.argtypes = [vp, i64, i32, i32, i32, i32, vp, i64, vp, i64, i32, vp, i32, vp]
    lib.qt_column_dot.restype = i32
    lib.qt_column_dot.argtypes = [vp, vp, i64, i64, i32, i32, i32, vp, i64, vp]
    lib.qt_panel_force_form.restype = None
    lib.qt_panel_force_form.argtypes = [i32]
    lib.qt_gemm_force_tile.restype = None
    lib.qt_gemm_force_tile.argtypes = [i32]
    lib.qt_power_iter.restype = i32
    lib.qt_power_iter.argtypes = [vp, i64, i32, i32, vp, f32, i32, vp, vp, vp, vp]
    lib.qt_inverse_root_newton_workspace_bytes.restype = ct.c_ulonglong
    lib.qt_inverse_root_newton_workspace_bytes.argtypes = [i32, i32]
    lib.qt_inverse_root_newton.restype = i32
    lib.qt_inverse_root_newton.argtypes = [vp, i64, i32, i32, i32, i32, f32, f32, vp, vp, ct.c_ulonglong, vp, i64, vp, vp, vp]
    lib.qt_selftest_wait_timeout.restype = i32
    lib.qt_selftest_wait_timeout.argtypes = [vp, vp]
    for name in LEGACY_SYMBOLS:
        getattr(lib, name).restype = None
    return lib


def get_lib():
    global _lib
    if _lib is None:
        path = library_path()
        if not path.is_file():
            raise FileNotFoundError(
                f"Quantization library not found at {path}; build it with csrc/build.py (nvcc, sm_100a).")
        lib = ct.cdll.LoadLibrary(str(path))
        missing = [s for s in LEGACY_SYMBOLS + EXTRA_SYMBOLS if not hasattr(lib, s)]
        if missing:
            raise RuntimeError(f"{path} lacks symbols: {missing}")
        _lib = _declare(lib)
    return _lib
