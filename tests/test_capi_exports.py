"""CPU checks of the boundary: the library loads, exports every symbol the header declares, and its
argument checks answer before anything would be launched (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

from darknet_b200 import build, capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    build.build()
    return capi.lib()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "xnor_b200.h")).read()
    return set(re.findall(r"XNOR_B200_API[^;(]*?\b(xnor_b200_\w+)\s*\(", text))


def test_every_declared_symbol_is_exported(L):
    declared = header_symbols()
    assert declared, "no declarations found in include/xnor_b200.h"
    for name in declared:
        assert hasattr(L, name), f"{name} declared in the header but not exported by libxnor_b200.so"


def test_binding_lists_exactly_the_header(L):
    assert set(capi.EXPORTS) == header_symbols()


def test_geometry_follows_the_reference_rules(L):
    # BASELINE config 1: C=256 -> 512 filters, 26x26, 3x3/s1/p1
    g = capi.geometry(capi.ConvDesc(1, 256, 26, 26, 512, 3, 1, 1, capi.LEAKY))
    assert (g.out_h, g.out_w, g.n_out, g.k, g.new_lda, g.bit_align, g.word_path) == (26, 26, 676, 2304, 2560, 704, 1)
    assert g.weights_bytes == 512 * 2560 // 8 and g.packed_input_bytes == 676 * 2560 // 8
    # K = 675 is not word aligned; stride 2
    g = capi.geometry(capi.ConvDesc(8, 75, 26, 26, 64, 3, 2, 1, capi.LINEAR))
    assert (g.out_h, g.n_out, g.k, g.new_lda, g.word_path) == (13, 169, 675, 768, 0)
    assert g.packed_input_bytes == 8 * 169 * 768 // 8


@pytest.mark.parametrize("desc", [
    (0, 32, 8, 8, 8, 3, 1, 1, 0), (1, 0, 8, 8, 8, 3, 1, 1, 0), (1, 32, 8, 8, 8, 0, 1, 1, 0), (1, 32, 8, 8, 8, 3, 0, 1, 0),
    (1, 32, 8, 8, 8, 3, 1, -1, 0), (1, 32, 8, 8, 8, 3, 1, 1, 7), (1, 32, 2, 2, 8, 5, 1, 0, 0),
])
def test_bad_descriptors_are_rejected(L, desc):
    g = capi.ConvGeom()
    assert L.xnor_b200_conv_geometry(C.byref(capi.ConvDesc(*desc)), C.byref(g)) == 1
    assert L.xnor_b200_scratch_bytes(C.byref(capi.ConvDesc(*desc))) == 0


def test_null_and_alignment_checks_answer_without_a_device(L):
    d = capi.ConvDesc(1, 32, 8, 8, 8, 3, 1, 1, 0)
    assert L.xnor_b200_conv_geometry(None, None) == 2
    assert L.xnor_b200_pack_input(C.byref(d), None, None, None) == 2
    assert L.xnor_b200_conv_forward(C.byref(d), None, None, None, None, None, None, None, None, 0, None) == 2
    assert L.xnor_b200_gemm_counts(8, 8, 256, None, 256, None, 256, None, None) == 2
    # lda must cover K and be a multiple of 128 bits; pointers 16-byte aligned
    assert L.xnor_b200_gemm_counts(8, 8, 300, 16, 256, 16, 512, 16, None) == 1
    assert L.xnor_b200_gemm_counts(8, 8, 256, 16, 300, 16, 512, 16, None) == 1
    assert L.xnor_b200_gemm_counts(8, 8, 256, 20, 256, 16, 256, 16, None) == 5
    # scratch too small is reported before any launch
    assert L.xnor_b200_conv_forward(C.byref(d), 256, 256, 256, 256, 256, None, None, 256, 16, None) == 3
    assert L.xnor_b200_strerror(3).decode() == "scratch buffer too small"
    assert L.xnor_b200_repack_input_bin(256, 256, 8, 8, 33, None) == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", str(tmp_path / "libxnor_b200.so"))
    with pytest.raises(FileNotFoundError, match="no CPU or PyTorch fallback"):
        capi.lib()
