"""BASELINE configuration 3 (xnor conv layer shape sweep) at sizes the oracle finishes in seconds:
kernel 1x1 and 3x3, C in {32, 64, 75, 128, 256, 512, 1024}, filters in {64, 256, 1024}, spatial 13 and 26, batch 1 and 8.
Layer outputs must equal the oracle bit for bit (C = 75 with a 1x1 kernel has no reference CPU result; the oracle's
closed form defines it).  The larger spatial sizes and batch 64 of the sweep are covered by size-independent
properties in test_gpu_parity.py and by the tensor-core tests."""
import itertools

import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, layer as L  # noqa: E402

CASES = []
for ks, c, n, s in itertools.product((1, 3), (32, 64, 75, 128, 256, 512, 1024), (64, 256, 1024), (13, 26)):
    if n == 1024 and (c >= 512 or s == 26):
        continue                                   # keep the CPU oracle time of the whole file under a minute
    batch = 8 if (c <= 128 and n == 64 and s == 13) else 1
    CASES.append((batch, c, s, n, ks))


@pytest.mark.parametrize("case", CASES, ids=lambda c: "b%d_c%d_s%d_n%d_k%d" % c)
def test_sweep_layer_matches_oracle(port, case):
    batch, c, s, n, ks = case
    x, wt, b = synth.conv_case(hash(case) % 100000, batch, c, s, s, n, ks)
    want = port.conv_forward(x, wt, b, 1, ks // 2, True)
    l = L.make_convolutional_layer(batch, s, s, c, n, ks, 1, ks // 2, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    y = L.forward_convolutional_layer_gpu(l, torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
