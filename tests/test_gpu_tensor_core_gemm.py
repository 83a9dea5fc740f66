"""The tcgen05 (tensor-core) variant of the XNOR GEMM against the oracle and against the integer-pipe kernel.

XNOR_B200_GEMM_TC=1 routes every GEMM call to the tensor-core kernel, =0 to the integer-pipe kernel, so both are
exercised on identical operands.  Integer accumulators and fp32 outputs must be bit-identical to the oracle."""
import os

import numpy as np
import pytest

import synth
from oracle.binding import new_lda

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, layer as L  # noqa: E402


@pytest.fixture
def force_tc():
    old = os.environ.get("XNOR_B200_GEMM_TC")

    def set_mode(v):
        if v is None:
            os.environ.pop("XNOR_B200_GEMM_TC", None)
        else:
            os.environ["XNOR_B200_GEMM_TC"] = v
    yield set_mode
    set_mode(old)


def random_bits(rng, rows, K):
    ld = new_lda(K)
    out = np.zeros((rows, ld // 8), np.uint8)
    bits = rng.integers(0, 2, (rows, K), dtype=np.uint8)
    packed = np.packbits(bits, axis=1, bitorder="little")
    out[:, :packed.shape[1]] = packed
    return out, ld


def device_status():
    import ctypes as C
    st = C.c_int(-1)
    capi.check(capi.lib().xnor_b200_take_device_status(C.byref(st)), "xnor_b200_take_device_status")
    return st.value


@pytest.mark.parametrize("shape", [
    (128, 128, 128), (128, 128, 1024), (256, 384, 2304), (130, 200, 675), (100, 131, 300), (384, 1000, 4608),
    (128, 4097, 1152), (1, 1, 1), (257, 129, 9216),
], ids=lambda s: "M%d_N%d_K%d" % s)
def test_tensor_core_counts_match_oracle(port, force_tc, shape):
    M, N, K = shape
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    A, ld = random_bits(rng, M, K)
    B, _ = random_bits(rng, N, K)
    want = port.gemm_counts(M, N, K, A, ld, B, ld)
    Ag, Bg = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    force_tc("1")
    got_tc = L.gemm_counts(M, N, K, Ag, ld, Bg, ld).cpu().numpy()
    assert device_status() == 0
    force_tc("0")
    got_int = L.gemm_counts(M, N, K, Ag, ld, Bg, ld).cpu().numpy()
    assert np.array_equal(got_int, want)
    assert np.array_equal(got_tc, want), f"tensor-core counts differ in {np.count_nonzero(got_tc != want)} of {want.size} entries"


def test_tensor_core_layer_output_matches_oracle_and_integer_kernel(port, force_tc):
    """Whole layer (batch folded into N, leaky, bias) through both kernels."""
    batch, c, h, w, n, ks, stride, pad, leaky = 3, 128, 20, 20, 160, 3, 1, 1, 1
    x, wt, b = synth.conv_case(555, batch, c, h, w, n, ks)
    want = port.conv_forward(x, wt, b, stride, pad, leaky)
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, stride, pad, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    xg = torch.from_numpy(x).cuda()
    force_tc("1")
    y_tc = L.forward_convolutional_layer_gpu(l, xg).clone().cpu().numpy()
    assert device_status() == 0
    force_tc("0")
    y_int = L.forward_convolutional_layer_gpu(l, xg).clone().cpu().numpy()
    assert np.array_equal(y_int.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(y_tc.view(np.uint32), want.view(np.uint32))


def test_automatic_dispatch_uses_tensor_cores_for_large_layers_and_stays_exact(port, force_tc):
    """A batch-64 BASELINE-sized layer (eligible for the tensor-core kernel) equals the integer kernel bit for bit."""
    batch, c, h, w, n, ks = 64, 256, 26, 26, 512, 3
    x1, wt, b = synth.conv_case(777, 2, c, h, w, n, ks)
    x = np.concatenate([x1] * (batch // 2), 0)
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, 1, 1, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    xg = torch.from_numpy(x).cuda()
    force_tc(None)
    y_auto = L.forward_convolutional_layer_gpu(l, xg).clone()
    assert device_status() == 0
    force_tc("0")
    y_int = L.forward_convolutional_layer_gpu(l, xg).clone()
    assert torch.equal(y_auto, y_int)
    want = port.conv_forward(x1, wt, b, 1, 1, 1)
    assert np.array_equal(y_auto[:2].cpu().numpy().view(np.uint32), want.view(np.uint32))
