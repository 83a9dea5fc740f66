"""BASELINE configuration 3 (xnor conv layer shape sweep) against the oracle, bit for bit:
kernel 1x1 and 3x3, C in {32, 64, 75, 128, 256, 512, 1024}, filters in {64, 256, 1024}, spatial {13, 26, 52, 104, 208},
batch {1, 8, 64}.  The full cross product at spatial 13 and 26 (batch 1, batch 8 on the small ones), and a thinned set of
points at spatial 52 / 104 / 208 and at batch 8 / 64 chosen so that every value of every axis occurs there and both GEMM
routes (integer pipe, tensor cores) are reached.  C = 75 with a 1x1 kernel has no reference CPU result; the oracle's
closed form defines it."""
import itertools

import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, layer as L  # noqa: E402

CASES = []
for ks, c, n, s in itertools.product((1, 3), (32, 64, 75, 128, 256, 512, 1024), (64, 256, 1024), (13, 26)):
    batch = 8 if (c <= 128 and n == 64 and s == 13) else 1
    CASES.append((batch, c, s, n, ks))

# (batch, C, spatial, filters, kernel): the large-spatial and large-batch corner of the sweep
LARGE = [
    (1, 32, 208, 64, 3), (1, 64, 208, 64, 1), (1, 75, 208, 64, 3), (1, 32, 104, 256, 3), (1, 128, 104, 64, 1),
    (1, 75, 104, 256, 1), (1, 256, 104, 64, 3), (1, 64, 52, 1024, 3), (1, 512, 52, 256, 1), (1, 1024, 52, 64, 1),
    (1, 256, 52, 256, 3), (8, 32, 104, 64, 3), (8, 128, 52, 256, 3), (8, 75, 52, 64, 3), (8, 1024, 26, 256, 1),
    (8, 512, 26, 1024, 3), (8, 64, 208, 64, 1), (64, 32, 52, 64, 3), (64, 64, 26, 256, 3), (64, 75, 26, 64, 3),
    (64, 256, 13, 1024, 3), (64, 1024, 13, 256, 1), (64, 128, 26, 64, 1), (64, 512, 13, 64, 3), (64, 75, 13, 256, 1),
]


def run_case(port, case):
    batch, c, s, n, ks = case
    x, wt, b = synth.conv_case(hash(case) % 100000, batch, c, s, s, n, ks)
    want = port.conv_forward(x, wt, b, 1, ks // 2, True)
    l = L.make_convolutional_layer(batch, s, s, c, n, ks, 1, ks // 2, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    y = L.forward_convolutional_layer_gpu(l, torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("case", CASES, ids=lambda c: "b%d_c%d_s%d_n%d_k%d" % c)
def test_sweep_layer_matches_oracle(port, case):
    run_case(port, case)


@pytest.mark.parametrize("case", LARGE, ids=lambda c: "b%d_c%d_s%d_n%d_k%d" % c)
def test_sweep_large_spatial_and_batch_matches_oracle(port, case):
    run_case(port, case)
