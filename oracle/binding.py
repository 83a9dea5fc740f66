"""TEST INFRASTRUCTURE: ctypes bindings for the two CPU checkers.

``Port``  wraps oracle/_build/liboracle.so  -- the plain-C restatement (xnor_oracle.c).
``Ref``   wraps oracle/_ref/liboracle_ref.so -- the reference's own xnor CPU sources compiled
          unmodified (see the Makefile beside this file); present only where that build ran.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.  The
product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(_HERE, "_build", "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "liboracle_ref.so")
REF_FAST_SO = os.path.join(_HERE, "_ref", "liboracle_ref_fast.so")      # same sources, the reference's own optimisation flags (timing only)


def reference_dir() -> str:
    """Where the darknet tree is mounted when it is present at all: $DARKNET_REFERENCE_DIR, else the default mount.
    The one place this location is written down; the Makefile beside this file receives it as REF=..."""
    return os.environ.get("DARKNET_REFERENCE_DIR", "/root/reference")


def build_ref(target: str = "ref") -> bool:
    """Runs `make <target>` against the mounted reference tree; False when the tree is not there."""
    ref = reference_dir()
    if not os.path.isdir(os.path.join(ref, "src-lib")):
        return False
    subprocess.check_call(["make", "-C", _HERE, target, f"REF={ref}"], stdout=subprocess.DEVNULL)
    return True

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def build_port() -> str:
    """Compile the plain-C restatement if it is missing or stale; returns the .so path."""
    src = os.path.join(_HERE, "xnor_oracle.c")
    if not os.path.exists(PORT_SO) or os.path.getmtime(PORT_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "port"], stdout=subprocess.DEVNULL)
    return PORT_SO


def out_dim(i: int, size: int, stride: int, pad: int) -> int:
    return (i + 2 * pad - size) // stride + 1


def new_lda(k: int) -> int:
    return k + (256 - k % 256)


def bit_align(n: int) -> int:
    return n + (32 - n % 32)


class Port:
    """The plain-C restatement.  All arrays are numpy; bit tensors are uint8 arrays."""

    def __init__(self) -> None:
        self.lib = C.CDLL(build_port())
        L = self.lib
        L.oracle_binarize_weights.argtypes = [_f32p, C.c_int, C.c_int, _f32p]
        L.oracle_float_to_bit.argtypes = [_f32p, _u8p, C.c_size_t]
        L.oracle_binary_align_weights.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, _u8p, _f32p]
        L.oracle_repack_input_bin.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _u32p]
        L.oracle_im2col_words.argtypes = [_u32p] + [C.c_int] * 6 + [_u32p]
        L.oracle_transpose_uint32.argtypes = [_u32p, _u32p] + [C.c_int] * 4
        L.oracle_im2col_bin.argtypes = [_f32p] + [C.c_int] * 7 + [_u8p]
        L.oracle_transpose_bin.argtypes = [_u8p, _u8p] + [C.c_int] * 4
        L.oracle_pack_input.argtypes = [_f32p] + [C.c_int] * 6 + [_u8p]
        L.oracle_gemm_counts.argtypes = [C.c_int] * 3 + [_u8p, C.c_int, _u8p, C.c_int, _i32p]
        L.oracle_gemm_bin_mean_transposed.argtypes = [C.c_int] * 3 + [_u8p, C.c_int, _u8p, C.c_int, _f32p, C.c_int, _f32p]
        L.oracle_add_bias.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.oracle_activate_leaky.argtypes = [_f32p, C.c_size_t]
        L.oracle_conv_forward.argtypes = [_f32p] + [C.c_int] * 4 + [_f32p, _f32p] + [C.c_int] * 5 + [_f32p, C.c_void_p, C.c_void_p]

    def binarize_weights(self, w: np.ndarray) -> np.ndarray:
        n, size = w.shape[0], int(np.prod(w.shape[1:]))
        out = np.empty((n, size), np.float32)
        self.lib.oracle_binarize_weights(np.ascontiguousarray(w.reshape(n, size)), n, size, out)
        return out

    def float_to_bit(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x.reshape(-1), np.float32)
        out = np.empty(x.size // 8 + 1, np.uint8)
        self.lib.oracle_float_to_bit(x, out, x.size)
        return out

    def binary_align_weights(self, w: np.ndarray, invert: bool = False):
        """w [n][c][ks][ks] -> (align_bit_weights uint8[n*new_lda/8 + 1], mean_arr float32[n])."""
        n, c, ks, _ = w.shape
        lda = new_lda(c * ks * ks)
        bits = np.empty(n * lda // 8 + 1, np.uint8)
        mean = np.empty(n, np.float32)
        self.lib.oracle_binary_align_weights(np.ascontiguousarray(w, np.float32).reshape(-1), n, c, ks, int(invert), bits, mean)
        return bits, mean

    def repack_input_bin(self, x: np.ndarray) -> np.ndarray:
        c, h, w = x.shape
        out = np.empty((c // 32, h * w), np.uint32)
        self.lib.oracle_repack_input_bin(np.ascontiguousarray(x, np.float32).reshape(-1), c, h, w, out.reshape(-1))
        return out

    def pack_input(self, x: np.ndarray, ks: int, stride: int, pad: int) -> np.ndarray:
        """x [c][h][w] -> t_bit_input uint8 [N][new_ldb/8]."""
        c, h, w = x.shape
        n = out_dim(h, ks, stride, pad) * out_dim(w, ks, stride, pad)
        ldb = new_lda(ks * ks * c)
        out = np.empty((n, ldb // 8), np.uint8)
        self.lib.oracle_pack_input(np.ascontiguousarray(x, np.float32).reshape(-1), c, h, w, ks, stride, pad, out.reshape(-1))
        return out

    def gemm_counts(self, M, N, K, A, lda, B, ldb) -> np.ndarray:
        counts = np.empty((M, N), np.int32)
        self.lib.oracle_gemm_counts(M, N, K, A.reshape(-1), lda, B.reshape(-1), ldb, counts.reshape(-1))
        return counts

    def gemm_bin_mean_transposed(self, M, N, K, A, lda, B, ldb, mean) -> np.ndarray:
        out = np.empty((M, N), np.float32)
        self.lib.oracle_gemm_bin_mean_transposed(M, N, K, A.reshape(-1), lda, B.reshape(-1), ldb, out.reshape(-1), N, mean)
        return out

    def conv_forward(self, x, w, b, stride, pad, leaky, dumps: bool = False):
        """x [batch][c][h][w], w [n][c][ks][ks], b [n] -> out [batch][n][oh][ow] (+ optional dumps)."""
        batch, c, h, wd = x.shape
        n, _, ks, _ = w.shape
        oh, ow = out_dim(h, ks, stride, pad), out_dim(wd, ks, stride, pad)
        N, K = oh * ow, ks * ks * c
        out = np.empty((batch, n, oh, ow), np.float32)
        tb = cnt = None
        tbp = cntp = None
        if dumps:
            tb = np.empty((batch, N, new_lda(K) // 8), np.uint8)
            cnt = np.empty((batch, n, N), np.int32)
            tbp, cntp = tb.ctypes.data, cnt.ctypes.data
        self.lib.oracle_conv_forward(np.ascontiguousarray(x, np.float32).reshape(-1), batch, c, h, wd,
                                     np.ascontiguousarray(w, np.float32).reshape(-1), np.ascontiguousarray(b, np.float32),
                                     n, ks, stride, pad, int(leaky), out.reshape(-1), tbp, cntp)
        return (out, tb, cnt) if dumps else out


class Ref:
    """The reference's own functions (batch 1 only, as in the reference)."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self, path: str = REF_SO) -> None:
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        L = self.lib
        L.ref_set_gpu_index.argtypes = [C.c_int]
        L.ref_set_num_threads.argtypes = [C.c_int]
        L.ref_max_threads.restype = C.c_int
        L.ref_binarize_weights.argtypes = [_f32p, C.c_int, C.c_int, _f32p]
        L.ref_float_to_bit.argtypes = [_f32p, _u8p, C.c_size_t]
        L.ref_repack_input.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.ref_im2col_cpu_custom.argtypes = [C.c_void_p] + [C.c_int] * 6 + [C.c_void_p]
        L.ref_transpose_uint32.argtypes = [_u32p, _u32p] + [C.c_int] * 4
        L.ref_im2col_cpu_custom_bin.argtypes = [_f32p] + [C.c_int] * 6 + [C.c_void_p, C.c_int]
        L.ref_transpose_bin.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 5
        L.ref_gemm_nn_custom_bin_mean_transposed.argtypes = [C.c_int] * 3 + [_u8p, C.c_int, _u8p, C.c_int, _f32p, C.c_int, _f32p]
        L.ref_add_bias.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.ref_activate_array_cpu_custom.argtypes = [_f32p, C.c_int, C.c_int]
        L.ref_layer_create.restype = C.c_void_p
        L.ref_layer_create.argtypes = [C.c_int] * 8 + [_f32p, _f32p]
        L.ref_layer_geometry.argtypes = [C.c_void_p, _i32p]
        for fn, rt in (("ref_layer_align_bit_weights", C.c_void_p), ("ref_layer_mean_arr", C.c_void_p),
                       ("ref_layer_binary_weights", C.c_void_p), ("ref_layer_t_bit_input", C.c_void_p),
                       ("ref_layer_bin_re_packed_input", C.c_void_p)):
            getattr(L, fn).restype = rt
            getattr(L, fn).argtypes = [C.c_void_p]
        L.ref_layer_forward.argtypes = [C.c_void_p, _f32p, _f32p]
        L.ref_layer_destroy.argtypes = [C.c_void_p]

    def set_gpu_index(self, idx: int) -> None:
        self.lib.ref_set_gpu_index(idx)

    def set_num_threads(self, n: int) -> None:
        self.lib.ref_set_num_threads(n)

    def max_threads(self) -> int:
        return self.lib.ref_max_threads()

    def layer(self, x_shape, w: np.ndarray, b: np.ndarray, stride: int, pad: int, leaky: bool) -> "RefLayer":
        return RefLayer(self, x_shape, w, b, stride, pad, leaky)


class RefLayer:
    """One reference xnor conv layer: reference constructor + binary_align_weights + CPU forward."""

    def __init__(self, ref: Ref, x_shape, w, b, stride, pad, leaky) -> None:
        self.ref = ref
        c, h, wd = x_shape
        n, cw, ks, _ = w.shape
        assert cw == c
        self.c, self.h, self.w, self.n, self.ks, self.stride, self.pad = c, h, wd, n, ks, stride, pad
        self.handle = ref.lib.ref_layer_create(h, wd, c, n, ks, stride, pad, int(leaky),
                                               np.ascontiguousarray(w, np.float32).reshape(-1),
                                               np.ascontiguousarray(b, np.float32))
        g = np.zeros(8, np.int32)
        ref.lib.ref_layer_geometry(self.handle, g)
        self.out_h, self.out_w, self.bit_align, self.new_lda, self.align_bit_weights_size = (int(v) for v in g[:5])
        self.N = self.out_h * self.out_w
        self.K = ks * ks * c

    def _view(self, ptr: int, nbytes: int, dtype) -> np.ndarray:
        buf = (C.c_uint8 * nbytes).from_address(ptr)
        return np.frombuffer(buf, dtype=dtype).copy()

    def align_bit_weights(self) -> np.ndarray:
        return self._view(self.ref.lib.ref_layer_align_bit_weights(self.handle), self.align_bit_weights_size, np.uint8)

    def mean_arr(self) -> np.ndarray:
        return self._view(self.ref.lib.ref_layer_mean_arr(self.handle), 4 * self.n, np.float32)

    def t_bit_input(self) -> np.ndarray:
        """[N][new_ldb/8] bytes as left by the last forward."""
        nbytes = self.N * self.new_lda // 8
        return self._view(self.ref.lib.ref_layer_t_bit_input(self.handle), nbytes, np.uint8).reshape(self.N, self.new_lda // 8)

    def forward(self, x: np.ndarray) -> np.ndarray:
        out = np.empty((self.n, self.out_h, self.out_w), np.float32)
        self.ref.lib.ref_layer_forward(self.handle, np.ascontiguousarray(x, np.float32).reshape(-1), out.reshape(-1))
        return out

    def close(self) -> None:
        if self.handle:
            self.ref.lib.ref_layer_destroy(self.handle)
            self.handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


REFNET_SO = os.path.join(_HERE, "_ref", "liboracle_refnet.so")
REFGPU_SO = os.path.join(_HERE, "_ref", "liboracle_refgpu.so")       # the reference's own GPU xnor kernels (timing baseline only)


class RefNet:
    """The reference's own network code on the CPU (oracle/_ref/liboracle_refnet.so, see build_refnet.py): load_network_custom
    on a .cfg and a .weights file, network_predict, per-layer outputs, get_network_boxes + do_nms_sort."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REFNET_SO)

    _lib = None

    @classmethod
    def lib(cls):
        if cls._lib is None:
            L = C.CDLL(REFNET_SO)
            L.refnet_load.restype = C.c_void_p
            L.refnet_load.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
            L.refnet_free.argtypes = [C.c_void_p]
            L.refnet_layers.argtypes = [C.c_void_p]
            L.refnet_layer_info.argtypes = [C.c_void_p, C.c_int, _i32p]
            L.refnet_predict.argtypes = [C.c_void_p, _f32p]
            L.refnet_layer_output.argtypes = [C.c_void_p, C.c_int, _f32p, C.c_int]
            L.refnet_layer_weights.argtypes = [C.c_void_p, C.c_int, _f32p, C.c_int, _f32p, C.c_int]
            L.refnet_detections.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, _f32p, C.c_int]
            L.refnet_nms_sort.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_float]
            cls._lib = L
        return cls._lib

    def __init__(self, cfg_path: str, weights_path: str, batch: int = 1) -> None:
        if not self.available():
            raise FileNotFoundError(REFNET_SO)
        self.batch = batch
        self.handle = self.lib().refnet_load(cfg_path.encode(), weights_path.encode(), batch)
        if not self.handle:
            raise RuntimeError("the reference could not load the network")
        self.n = self.lib().refnet_layers(self.handle)

    def layer_info(self, i: int) -> dict:
        v = np.zeros(10, np.int32)
        self.lib().refnet_layer_info(self.handle, i, v)
        keys = ("type", "outputs", "out_c", "out_h", "out_w", "xnor", "batch", "n", "activation", "packed")
        return dict(zip(keys, (int(x) for x in v)))

    def predict(self, x: np.ndarray) -> None:
        if self.lib().refnet_predict(self.handle, np.ascontiguousarray(x, np.float32).reshape(-1)) != 0:
            raise RuntimeError("network_predict failed")

    def layer_output(self, i: int) -> np.ndarray:
        info = self.layer_info(i)
        out = np.empty(info["batch"] * info["outputs"], np.float32)
        if self.lib().refnet_layer_output(self.handle, i, out, out.size) != 0:
            raise RuntimeError(f"layer {i} has no output")
        if info["out_c"] * info["out_h"] * info["out_w"] == info["outputs"]:
            return out.reshape(info["batch"], info["out_c"], info["out_h"], info["out_w"])
        return out.reshape(info["batch"], -1)

    def layer_weights(self, i: int, nweights: int, n: int):
        w, b = np.empty(nweights, np.float32), np.empty(n, np.float32)
        if self.lib().refnet_layer_weights(self.handle, i, w, nweights, b, n) != 0:
            raise RuntimeError(f"layer {i} has no weights of that size")
        return w, b

    def detections(self, w: int, h: int, thresh: float, nms: float, letter: int = 0, max_rows: int = 100000) -> np.ndarray:
        """Rows {x, y, w, h, objectness, class, probability} of image 0 after get_network_boxes + do_nms_sort."""
        rows = np.empty((max_rows, 7), np.float32)
        n = self.lib().refnet_detections(self.handle, w, h, thresh, nms, letter, rows.reshape(-1), max_rows)
        return rows[:n].copy()

    def close(self) -> None:
        if self.handle:
            self.lib().refnet_free(self.handle)
            self.handle = None

    @classmethod
    def nms_sort(cls, boxes: np.ndarray, objectness: np.ndarray, probs: np.ndarray, thresh: float) -> np.ndarray:
        """The reference's do_nms_sort on boxes [n][4], objectness [n], probs [n][classes]; returns the probabilities after
        suppression, in the caller's order."""
        out = np.ascontiguousarray(probs, np.float32).copy()
        n, classes = out.shape
        cls.lib().refnet_nms_sort(np.ascontiguousarray(boxes, np.float32).reshape(-1), np.ascontiguousarray(objectness, np.float32),
                                  out.reshape(-1), n, classes, thresh)
        return out
