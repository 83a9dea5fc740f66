"""The two-pass pack (sign words first, packed rows from the words) against the CPU oracle and the single kernel.

Bit-exact bar.  The two-pass route is switched on with set_tuning.
"""
import ctypes as C

import numpy as np
import pytest

import synth
from oracle.binding import new_lda, out_dim

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, layer as L  # noqa: E402

CASES = [
    # batch, c, h, w, n, ks, stride, pad
    (2, 64, 13, 11, 32, 3, 1, 1),      # odd plane size: one position per thread
    (3, 32, 7, 9, 16, 1, 1, 0),        # 1x1: rows are the transposed words
    (2, 96, 12, 10, 32, 3, 2, 1),      # stride 2, even plane: two positions per thread
    (1, 128, 16, 16, 64, 5, 1, 2),     # 5x5 taps, plane a multiple of four
    (5, 256, 26, 26, 64, 3, 1, 1),     # several strips and channel groups per image
]


@pytest.fixture(autouse=True)
def default_tuning_afterwards():
    yield
    capi.set_tuning()


@pytest.mark.parametrize("case", CASES, ids=lambda s: "x".join(map(str, s)))
def test_two_pass_pack_matches_oracle(case, port):
    batch, c, h, w, n, ks, stride, pad = case
    x = synth.bell(sum(case), (batch, c, h, w))
    x[0, :, 0, 0] = 0.0                                     # zero is not positive
    x[-1, 1::2, -1, -1] = -0.0
    K = c * ks * ks
    lda = new_lda(K)
    N = out_dim(h, ks, stride, pad) * out_dim(w, ks, stride, pad)
    want = np.stack([port.pack_input(x[b], ks, stride, pad) for b in range(batch)])
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, stride, pad, capi.LINEAR)
    xg = torch.from_numpy(x).cuda()
    capi.set_tuning(pack_two_pass=2)
    got = L.pack_input_staged(l, xg)
    assert np.array_equal(got.cpu().numpy().reshape(batch, N, lda // 8), want)
    assert torch.equal(got, L.pack_input(l, xg))


def test_layer_forward_is_the_same_on_both_routes():
    """xnor_b200_conv_forward with room for the sign words behind its packed rows: two passes, one pass, the default."""
    batch, c, h, w, n, ks = 4, 128, 26, 26, 256, 3
    x, wt, b = synth.conv_case(11, batch, c, h, w, n, ks)
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, 1, 1, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    lib = capi.lib()
    l.scratch = torch.zeros(lib.xnor_b200_scratch_bytes(C.byref(l.desc)) + lib.xnor_b200_pack_words_bytes(C.byref(l.desc)),
                            dtype=torch.uint8, device="cuda")
    xg = torch.from_numpy(x).cuda()
    capi.set_tuning(pack_two_pass=1)
    want = L.forward_convolutional_layer_gpu(l, xg).clone()
    capi.set_tuning(pack_two_pass=2)
    assert torch.equal(L.forward_convolutional_layer_gpu(l, xg), want)
    capi.set_tuning()
    assert torch.equal(L.forward_convolutional_layer_gpu(l, xg), want)


def test_large_input_matches_the_single_kernel():
    batch, c, h, w = 64, 256, 26, 26                        # 44 MB of input, 14 MB of rows
    l = L.make_convolutional_layer(batch, h, w, c, 512, 3, 1, 1, capi.LINEAR)
    xg = torch.from_numpy(synth.bell(3, (batch, c, h, w))).cuda()
    want = L.pack_input(l, xg)
    capi.set_tuning(pack_two_pass=2)
    assert torch.equal(L.pack_input_staged(l, xg), want)
    assert capi.lib().xnor_b200_pack_words_bytes(C.byref(l.desc)) == batch * (c // 32) * h * w * 4
