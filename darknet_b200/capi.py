"""ctypes view of libxnor_b200.so -- the C ABI declared in include/xnor_b200.h.

This module only loads the shared library and declares argument types; it holds no
arithmetic.  If the library has not been built, importing ``lib()`` raises: there is no
fallback implementation of any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libxnor_b200.so")

OK = 0
LINEAR = 0
LEAKY = 1
STATIC_SCRATCH_BYTES = 8 << 20  # XNOR_B200_STATIC_SCRATCH_BYTES

# Every symbol include/xnor_b200.h declares; tests check that the library exports each one.
EXPORTS = (
    "xnor_b200_strerror", "xnor_b200_last_cuda_error", "xnor_b200_set_tuning", "xnor_b200_conv_geometry",
    "xnor_b200_binarize_weights", "xnor_b200_binary_align_weights", "xnor_b200_float_to_bit",
    "xnor_b200_repack_input_bin", "xnor_b200_pack_input", "xnor_b200_pack_words_bytes", "xnor_b200_pack_input_staged", "xnor_b200_gemm_bin_mean_transposed",
    "xnor_b200_gemm_counts", "xnor_b200_scratch_bytes", "xnor_b200_conv_forward",
    "xnor_b200_conv_forward_static", "xnor_b200_take_device_status",
    "xnor_b200_pack_input_pooled", "xnor_b200_conv_forward_pooled", "xnor_b200_float_conv_small", "xnor_b200_float_conv3_io", "xnor_b200_float_conv_map_weights_bytes",
    "xnor_b200_float_conv_map_prepare", "xnor_b200_float_conv_map", "xnor_b200_float_conv_map_yolo", "xnor_b200_float_conv_1x1_tc", "xnor_b200_yolo_activate", "xnor_b200_region_activate", "xnor_b200_conv_forward_io", "xnor_b200_conv_takes_masks", "xnor_b200_tap_major_weights",
    "xnor_b200_yolo_detections", "xnor_b200_nms_sort", "xnor_b200_detection_rows",
    "xnor_b200_measure_popc_peak", "xnor_b200_measure_bmma_peak", "xnor_b200_measure_umma_i8_peak", "xnor_b200_measure_umma_mxf4_peak",
)


class ConvDesc(C.Structure):
    """struct xnor_b200_conv_desc"""
    _fields_ = [(n, C.c_int) for n in ("batch", "c", "h", "w", "n", "size", "stride", "pad", "activation")]


class PoolDesc(C.Structure):
    """struct xnor_b200_pool_desc"""
    _fields_ = [(n, C.c_int) for n in ("size", "stride", "pad", "in_h", "in_w")]


class SignSink(C.Structure):
    """struct xnor_b200_sign_sink"""
    _fields_ = [("consumer", C.POINTER(ConvDesc)), ("consumer_scratch", C.c_void_p), ("channel_offset", C.c_int), ("pool", C.c_int),
                ("upsample", C.c_int), ("consumer_window_major", C.c_int)]


class ConvIO(C.Structure):
    """struct xnor_b200_conv_io"""
    _fields_ = [("input", C.c_void_p), ("input_signs", C.c_void_p), ("pool", C.POINTER(PoolDesc)), ("output", C.c_void_p),
                ("output_signs", C.c_void_p), ("shortcut_in", C.c_void_p), ("shortcut_out", C.c_void_p),
                ("input_packed", C.c_int), ("window_major", C.c_int), ("sinks", C.POINTER(SignSink)), ("n_sinks", C.c_int),
                ("input_masks", C.c_void_p), ("tap_major_weights", C.c_int), ("shortcut_signs", C.c_void_p),
                ("shortcut_sink", C.POINTER(SignSink))]


ROUTE_AUTO, ROUTE_INTEGER, ROUTE_TENSOR, ROUTE_TILED = 0, 1, 2, 3


class Tuning(C.Structure):
    """struct xnor_b200_tuning"""
    _fields_ = [(n, C.c_int) for n in ("gemm_route", "gemm_tile", "gemm_split", "pack_ctas_per_sm", "tc_kernel", "tc_wait_polls", "tc_withhold_arrival", "pack_two_pass")]


class YoloHead(C.Structure):
    """struct xnor_b200_yolo_head"""
    _fields_ = [("output", C.c_void_p), ("w", C.c_int), ("h", C.c_int), ("n", C.c_int), ("classes", C.c_int), ("anchors", C.c_float * 32),
                ("new_coords", C.c_int)]


class Detections(C.Structure):
    """struct xnor_b200_detections"""
    _fields_ = [("boxes", C.c_void_p), ("objectness", C.c_void_p), ("probs", C.c_void_p), ("count", C.c_void_p), ("max_dets", C.c_int),
                ("classes", C.c_int)]


class ConvGeom(C.Structure):
    """struct xnor_b200_conv_geom"""
    _fields_ = [(n, C.c_int) for n in ("out_h", "out_w", "n_out", "k", "new_lda", "bit_align", "word_path")] + \
               [("weights_bytes", C.c_size_t), ("packed_input_bytes", C.c_size_t), ("output_floats", C.c_size_t)]


class XnorError(RuntimeError):
    def __init__(self, code: int, where: str) -> None:
        self.code = code
        msg = lib().xnor_b200_strerror(code).decode()
        if code == 4:
            msg += f" (cudaError {lib().xnor_b200_last_cuda_error()})"
        super().__init__(f"{where}: {msg} [code {code}]")


_lib = None


def lib() -> C.CDLL:
    """Loads libxnor_b200.so once.  Raises if it is missing -- build it with ``python -m darknet_b200.build``."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: the CUDA library has not been built (python -m darknet_b200.build). "
            "There is no CPU or PyTorch fallback for this path.")
    L = C.CDLL(LIB_PATH)
    vp, ci, sz = C.c_void_p, C.c_int, C.c_size_t
    dp, gp = C.POINTER(ConvDesc), C.POINTER(ConvGeom)
    L.xnor_b200_strerror.restype = C.c_char_p
    L.xnor_b200_strerror.argtypes = [ci]
    L.xnor_b200_last_cuda_error.restype = ci
    L.xnor_b200_set_tuning.argtypes = [C.POINTER(Tuning)]
    L.xnor_b200_conv_geometry.argtypes = [dp, gp]
    L.xnor_b200_binarize_weights.argtypes = [vp, ci, ci, vp, vp, vp]
    L.xnor_b200_binary_align_weights.argtypes = [dp, vp, vp, vp, ci, vp]
    L.xnor_b200_float_to_bit.argtypes = [vp, vp, sz, vp]
    L.xnor_b200_repack_input_bin.argtypes = [vp, vp, ci, ci, ci, vp]
    L.xnor_b200_pack_input.argtypes = [dp, vp, vp, vp]
    L.xnor_b200_pack_words_bytes.restype = sz
    L.xnor_b200_pack_words_bytes.argtypes = [dp]
    L.xnor_b200_pack_input_staged.argtypes = [dp, vp, vp, vp, vp]
    L.xnor_b200_gemm_bin_mean_transposed.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, ci, vp, vp, ci, vp, vp, vp]
    L.xnor_b200_gemm_counts.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, vp]
    L.xnor_b200_scratch_bytes.restype = sz
    L.xnor_b200_scratch_bytes.argtypes = [dp]
    L.xnor_b200_conv_forward.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    pp = C.POINTER(PoolDesc)
    L.xnor_b200_pack_input_pooled.argtypes = [dp, pp, vp, vp, vp]
    L.xnor_b200_conv_forward_pooled.argtypes = [dp, pp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    L.xnor_b200_float_conv_small.argtypes = [dp, vp, vp, vp, vp, vp]
    L.xnor_b200_float_conv3_io.argtypes = [dp, ci, vp, vp, vp, vp, vp, vp, vp]
    L.xnor_b200_conv_takes_masks.argtypes = [dp]
    L.xnor_b200_tap_major_weights.argtypes = [dp, vp, vp, vp]
    L.xnor_b200_float_conv_map_weights_bytes.argtypes = [dp]
    L.xnor_b200_float_conv_map_weights_bytes.restype = C.c_size_t
    L.xnor_b200_float_conv_map_prepare.argtypes = [dp, vp, vp, vp]
    L.xnor_b200_float_conv_map.argtypes = [dp, vp, vp, vp, vp, vp]
    L.xnor_b200_float_conv_1x1_tc.argtypes = [dp, vp, vp, vp, vp, vp]
    L.xnor_b200_float_conv_map_yolo.argtypes = [dp, vp, vp, vp, vp, ci, vp]
    L.xnor_b200_yolo_activate.argtypes = [vp, vp, ci, ci, ci, ci, vp]
    L.xnor_b200_region_activate.argtypes = [vp, vp, ci, ci, ci, ci, ci, ci, vp]
    L.xnor_b200_conv_forward_io.argtypes = [dp, C.POINTER(ConvIO), vp, vp, vp, vp, sz, vp]
    L.xnor_b200_yolo_detections.argtypes = [C.POINTER(YoloHead), ci, ci, ci, ci, ci, C.c_float, ci, ci, ci, C.POINTER(Detections), vp]
    L.xnor_b200_nms_sort.argtypes = [C.POINTER(Detections), ci, C.c_float, vp]
    L.xnor_b200_detection_rows.argtypes = [C.POINTER(Detections), ci, vp, ci, vp, vp]
    L.xnor_b200_conv_forward_static.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp]
    L.xnor_b200_take_device_status.argtypes = [C.POINTER(ci)]
    L.xnor_b200_measure_popc_peak.argtypes = [ci, C.POINTER(C.c_double), C.POINTER(C.c_double)]
    L.xnor_b200_measure_bmma_peak.argtypes = [ci, C.POINTER(C.c_double), C.POINTER(C.c_double)]
    L.xnor_b200_measure_umma_i8_peak.argtypes = [ci, C.POINTER(C.c_double), C.POINTER(C.c_double)]
    L.xnor_b200_measure_umma_mxf4_peak.argtypes = [ci, C.POINTER(C.c_double), C.POINTER(C.c_double)]
    _lib = L
    return L


def check(code: int, where: str) -> None:
    if code != OK:
        raise XnorError(code, where)


def set_tuning(**fields) -> None:
    """xnor_b200_set_tuning: pins kernel choices process-wide (tests and benchmarks); no arguments = library defaults."""
    if not fields:
        check(lib().xnor_b200_set_tuning(None), "xnor_b200_set_tuning")
        return
    t = Tuning()
    for k, v in fields.items():
        setattr(t, k, v)
    check(lib().xnor_b200_set_tuning(C.byref(t)), "xnor_b200_set_tuning")


def geometry(desc: ConvDesc) -> ConvGeom:
    g = ConvGeom()
    check(lib().xnor_b200_conv_geometry(C.byref(desc), C.byref(g)), "xnor_b200_conv_geometry")
    return g
