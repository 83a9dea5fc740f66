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


def _static_forward(l, x, out):
    capi.check(capi.lib().xnor_b200_conv_forward_static(
        C.byref(l.desc), x.data_ptr(), l.align_bit_weights_gpu.data_ptr(), l.mean_arr_gpu.data_ptr(),
        l.biases_gpu.data_ptr(), out.data_ptr(), None, None, torch.cuda.current_stream().cuda_stream),
        "xnor_b200_conv_forward_static")


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
