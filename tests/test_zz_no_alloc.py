"""The allocation-free layer entry point against the ordinary one.

xnor_b200_conv_forward_static serves callers that cannot give the library a scratch buffer (they may not
call cudaMalloc at all, or their memory pool is sealed): it keeps the packed activations in a fixed array
inside the library.  This file is collected last on purpose, so a run that stops at the first failure has
already exercised every other test; it also passes when run on its own in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")

from darknet_b200 import capi, layer as L  # noqa: E402


def _static_forward(l, x, out, shortcut_in=None, shortcut_out=None):
    capi.check(capi.lib().xnor_b200_conv_forward_static(
        C.byref(l.desc), x.data_ptr(), l.align_bit_weights_gpu.data_ptr(), l.mean_arr_gpu.data_ptr(),
        l.biases_gpu.data_ptr(), out.data_ptr(), None if shortcut_in is None else shortcut_in.data_ptr(),
        None if shortcut_out is None else shortcut_out.data_ptr(), torch.cuda.current_stream().cuda_stream),
        "xnor_b200_conv_forward_static")


def _layer(seed, batch, c, h, w, n, ks, stride, pad, leaky):
    x, wt, b = synth.conv_case(seed, batch, c, h, w, n, ks)
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, stride, pad, capi.LEAKY if leaky else capi.LINEAR)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    return l, torch.from_numpy(x).cuda()


def _reference_forward(l, xg, shortcut_in=None):
    """xnor_b200_conv_forward with the layer's own scratch: (output, shortcut sum or None)."""
    out = torch.empty(l.batch, l.n, l.geom.out_h, l.geom.out_w, device="cuda")
    sc_out = None if shortcut_in is None else torch.empty_like(out)
    capi.check(capi.lib().xnor_b200_conv_forward(
        C.byref(l.desc), xg.data_ptr(), l.align_bit_weights_gpu.data_ptr(), l.mean_arr_gpu.data_ptr(), l.biases_gpu.data_ptr(),
        out.data_ptr(), None if shortcut_in is None else shortcut_in.data_ptr(), None if sc_out is None else sc_out.data_ptr(),
        l.scratch.data_ptr(), l.scratch.numel(), torch.cuda.current_stream().cuda_stream), "xnor_b200_conv_forward")
    return out, sc_out


@pytest.mark.gpu
def test_static_scratch_entry_point_matches_conv_forward_twice_in_a_row():
    """Two different layers back to back through the shared array: the second call must not see anything the
    first one left behind, and both must equal xnor_b200_conv_forward bit for bit (the tolerance of every
    other layer test here)."""
    cases = [
        (2, 64, 26, 26, 48, 3, 1, 1, 1),     # word path, 2 images
        (1, 75, 13, 13, 24, 3, 1, 1, 0),     # bit path, smaller packed operand than the call before it
        (2, 64, 26, 26, 48, 3, 1, 1, 1),     # the first layer again with fresh inputs
    ]
    for rep, (batch, c, h, w, n, ks, stride, pad, leaky) in enumerate(cases):
        x, wt, b = synth.conv_case(4000 + rep, batch, c, h, w, n, ks)
        l = L.make_convolutional_layer(batch, h, w, c, n, ks, stride, pad, capi.LEAKY if leaky else capi.LINEAR)
        l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
        L.binary_align_weights(l)
        xg = torch.from_numpy(x).cuda()
        want = L.forward_convolutional_layer_gpu(l, xg).clone()
        got = torch.full_like(want, float("nan"))
        _static_forward(l, xg, got)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {rep}: static-scratch output differs from xnor_b200_conv_forward"
        assert np.isfinite(got.cpu().numpy()).all()


@pytest.mark.gpu
def test_static_scratch_entry_point_with_a_fused_shortcut():
    l, xg = _layer(4100, 2, 64, 26, 26, 64, 3, 1, 1, 0)
    sc_in = torch.from_numpy(synth.bell(4101, (2, 64, 26, 26))).cuda()
    want, want_sum = _reference_forward(l, xg, sc_in)
    got, got_sum = torch.full_like(want, float("nan")), torch.full_like(want, float("nan"))
    _static_forward(l, xg, got, sc_in, got_sum)
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(got_sum, want_sum)


@pytest.mark.gpu
def test_static_scratch_entry_point_on_the_tensor_core_route():
    """A layer whose GEMM runs on the tcgen05 kernel (route pinned) reads the library-resident array as its pixel operand:
    8 images of the 256 -> 256 3x3 layer at 26x26 pack into 1.7 MB."""
    l, xg = _layer(4200, 8, 256, 26, 26, 256, 3, 1, 1, 1)
    assert l.geom.packed_input_bytes < capi.STATIC_SCRATCH_BYTES
    try:
        capi.set_tuning(gemm_route=capi.ROUTE_INTEGER)
        want, _ = _reference_forward(l, xg)
        capi.set_tuning(gemm_route=capi.ROUTE_TENSOR)
        got = torch.full_like(want, float("nan"))
        _static_forward(l, xg, got)
        torch.cuda.synchronize()
    finally:
        capi.set_tuning()
    assert torch.equal(got, want)
    st = C.c_int(-1)
    capi.check(capi.lib().xnor_b200_take_device_status(C.byref(st)), "xnor_b200_take_device_status")
    assert st.value == 0


@pytest.mark.gpu
def test_static_scratch_entry_point_just_under_the_limit():
    """219 images of a 21x19 map with 96-byte packed rows fill the array up to 32 bytes short of its end: the last rows and the
    K padding of the last row are read by the GEMM like any other."""
    l, xg = _layer(4300, 219, 64, 21, 19, 32, 3, 1, 1, 1)
    assert 0 <= capi.STATIC_SCRATCH_BYTES - l.geom.packed_input_bytes < l.new_lda // 8
    want, _ = _reference_forward(l, xg)
    got = torch.full_like(want, float("nan"))
    _static_forward(l, xg, got)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # one more image does not fit and is refused before anything is launched
    bigger = capi.ConvDesc(220, 64, 21, 19, 32, 3, 1, 1, capi.LEAKY)
    rc = capi.lib().xnor_b200_conv_forward_static(C.byref(bigger), xg.data_ptr(), l.align_bit_weights_gpu.data_ptr(),
                                                 l.mean_arr_gpu.data_ptr(), l.biases_gpu.data_ptr(), got.data_ptr(), None, None, None)
    assert rc == 6


@pytest.mark.gpu
def test_static_scratch_entry_point_rejects_oversized_layers():
    # 64 images of a 104x104 layer with K = 288 need 64*10816*512/8 = 44 MB of packed activations
    desc = capi.ConvDesc(64, 32, 104, 104, 64, 3, 1, 1, capi.LINEAR)
    assert capi.geometry(desc).packed_input_bytes > capi.STATIC_SCRATCH_BYTES
    dummy = torch.zeros(64, device="cuda")
    rc = capi.lib().xnor_b200_conv_forward_static(C.byref(desc), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                                 dummy.data_ptr(), dummy.data_ptr(), None, None, None)
    assert rc == 6
    with pytest.raises(capi.XnorError, match="exceeds a fixed limit"):
        capi.check(rc, "xnor_b200_conv_forward_static")
