"""GPU parity: every stage of the CUDA path, called through the C ABI, against the CPU oracle.

Bar: packed bit tensors, integer accumulators and mean_arr bit-exact; fp32 layer outputs bit-exact too
(the epilogue reproduces the reference CPU rounding order), which is tighter than the stated 1e-5.
"""
import numpy as np
import pytest

import synth
from oracle.binding import new_lda, out_dim

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, layer as L  # noqa: E402


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_layer(batch, c, h, w, n, ks, stride, pad, leaky, wt, b):
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, stride, pad, capi.LEAKY if leaky else capi.LINEAR)
    l.load_weights(dev(wt), dev(b))
    L.binary_align_weights(l)
    return l


def assert_bits_equal(got, want, what):
    got = np.ascontiguousarray(got)
    want = np.ascontiguousarray(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    if not np.array_equal(got.view(np.uint8), want.view(np.uint8)):
        bad = np.flatnonzero(got.reshape(-1).view(np.uint8) != want.reshape(-1).view(np.uint8))
        raise AssertionError(f"{what}: {bad.size} differing bytes, first at {bad[0]}")


def test_golden_vectors_from_the_reference(golden):
    """Packed weights, mean_arr, packed input and layer output against what the reference CPU code produced."""
    cases, data = golden
    for i, (seed, c, h, w, n, ks, stride, pad, leaky) in enumerate(cases):
        x, wt, b = synth.conv_case(seed, 1, c, h, w, n, ks)
        l = make_layer(1, c, h, w, n, ks, stride, pad, leaky, wt, b)
        assert_bits_equal(l.align_bit_weights_gpu.cpu().numpy(), data[f"c{i}_align_bit_weights"], f"case {i} packed weights")
        assert_bits_equal(l.mean_arr_gpu.cpu().numpy(), data[f"c{i}_mean_arr"], f"case {i} mean_arr")
        xg = dev(x)
        assert_bits_equal(L.pack_input(l, xg).cpu().numpy(), data[f"c{i}_t_bit_input"], f"case {i} t_bit_input")
        y = L.forward_convolutional_layer_gpu(l, xg).cpu().numpy()[0]
        assert_bits_equal(y, data[f"c{i}_output"], f"case {i} output")
    seed, c, h, w, n, ks, stride, pad, leaky = cases[0]
    _, wt, b = synth.conv_case(seed, 1, c, h, w, n, ks)
    l = L.make_convolutional_layer(1, h, w, c, n, ks, stride, pad, capi.LINEAR)
    l.load_weights(dev(wt), dev(b))
    L.binary_align_weights(l, invert=True)
    assert_bits_equal(l.align_bit_weights_gpu.cpu().numpy(), data["c0_align_bit_weights_inverted"], "inverted packed weights")


SHAPES = [
    # batch, c, h, w, n, ks, stride, pad, leaky
    (1, 256, 26, 26, 512, 3, 1, 1, 1),     # BASELINE config 1
    (2, 32, 9, 7, 16, 3, 1, 1, 0),
    (3, 64, 8, 8, 32, 1, 1, 0, 1),
    (2, 64, 16, 16, 32, 3, 2, 1, 1),
    (2, 5, 10, 10, 8, 3, 1, 1, 1),
    (2, 75, 13, 13, 64, 3, 1, 1, 1),       # K = 675, bit path
    (2, 75, 13, 13, 64, 1, 1, 0, 1),       # K = 75: no reference CPU result exists, closed form only
    (1, 16, 52, 52, 32, 3, 1, 1, 0),       # first xnor layer of the tiny nets (C = 16), reduced spatial size
    (1, 512, 13, 13, 1024, 3, 1, 1, 0),    # yolov3-tiny layer 12: M = 1024, N = 169, K = 4608
    (1, 1024, 13, 13, 256, 1, 1, 0, 1),
    (1, 384, 26, 26, 256, 3, 1, 1, 1),
    (4, 128, 28, 28, 64, 1, 1, 0, 1),      # darknet53-like 1x1
    (2, 32, 56, 56, 64, 3, 2, 1, 1),       # darknet53-like stride-2
    (5, 96, 7, 9, 17, 3, 1, 1, 1),         # odd M, odd N, batch boundary inside a tile
    (1, 33, 6, 6, 3, 3, 1, 1, 0),          # tiny M, C just over a word
    (8, 64, 13, 13, 64, 3, 1, 1, 1),       # batch folded into N
    (1, 32, 104, 104, 64, 3, 1, 1, 0),     # yolov3-tiny layer 4
    (1, 64, 40, 40, 40, 5, 1, 2, 1),       # 5x5 kernel
    (1, 64, 12, 12, 8, 3, 1, 0, 1),        # no padding
    (1, 32, 5, 5, 8, 3, 1, 3, 0),          # padding larger than the kernel reach: whole rows of padded taps
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "b%d_c%d_%dx%d_n%d_k%d_s%d_p%d_%d" % s)
def test_layer_stages_match_oracle(port, shape):
    batch, c, h, w, n, ks, stride, pad, leaky = shape
    x, wt, b = synth.conv_case(sum(shape), batch, c, h, w, n, ks)
    want_out, want_tb, want_cnt = port.conv_forward(x, wt, b, stride, pad, leaky, dumps=True)
    want_A, want_mean = port.binary_align_weights(wt)
    K = c * ks * ks
    lda = new_lda(K)
    N = out_dim(h, ks, stride, pad) * out_dim(w, ks, stride, pad)

    l = make_layer(batch, c, h, w, n, ks, stride, pad, leaky, wt, b)
    assert_bits_equal(l.align_bit_weights_gpu.cpu().numpy(), want_A[:n * lda // 8], "packed weights")
    assert_bits_equal(l.mean_arr_gpu.cpu().numpy(), want_mean, "mean_arr")
    xg = dev(x)
    tb = L.pack_input(l, xg)
    assert_bits_equal(tb.cpu().numpy().reshape(batch, N, lda // 8), want_tb, "t_bit_input")
    counts = L.gemm_counts(n, batch * N, K, l.align_bit_weights_gpu, lda, tb, lda).cpu().numpy()
    assert_bits_equal(counts.reshape(n, batch, N).transpose(1, 0, 2), want_cnt, "popcount accumulators")
    y = L.forward_convolutional_layer_gpu(l, xg).cpu().numpy()
    assert_bits_equal(y, want_out, "layer output")
    rel = np.abs(y - want_out).max() / max(np.abs(want_out).max(), 1e-30)
    assert rel <= 1e-5


def test_binarize_weights_matches_oracle(port):
    wt = synth.bell(5, (24, 75 * 9), 0.05)
    binary, mean = L.binarize_weights(dev(wt), 24, 75 * 9)
    want = port.binarize_weights(wt)
    assert_bits_equal(binary.cpu().numpy(), want, "binary_weights")
    assert_bits_equal(mean.cpu().numpy(), np.abs(want[:, 0]), "mean")


def test_stage_seams_float_to_bit_and_repack(port):
    x = synth.bell(6, (64, 11, 13), 1.0)
    x.reshape(-1)[:8] = [0.0, -0.0, 1e-45, -1e-45, np.inf, -np.inf, np.nan, 1.0]
    xg = dev(x)
    nbits = x.size
    out = torch.zeros((nbits + 31) // 32 * 4, dtype=torch.uint8, device="cuda")
    capi.check(capi.lib().xnor_b200_float_to_bit(xg.data_ptr(), out.data_ptr(), nbits, None), "float_to_bit")
    torch.cuda.synchronize()
    want = port.float_to_bit(x)
    assert_bits_equal(out.cpu().numpy()[:nbits // 8], want[:nbits // 8], "float_to_bit")
    packed = torch.zeros(2, 11 * 13, dtype=torch.int32, device="cuda")
    capi.check(capi.lib().xnor_b200_repack_input_bin(xg.data_ptr(), packed.data_ptr(), 13, 11, 64, None), "repack")
    torch.cuda.synchronize()
    assert_bits_equal(packed.cpu().numpy().view(np.uint32), port.repack_input_bin(x), "repack_input_bin")


def test_gemm_reference_signature_with_bias_leaky_and_shortcut(port):
    """The stand-alone GEMM entry point: ldc > N, fused shortcut add."""
    M, N, K = 40, 50, 675
    ld = new_lda(K)
    rng = np.random.default_rng(11)
    A = np.zeros((M, ld // 8), np.uint8)
    B = np.zeros((N, ld // 8), np.uint8)
    A[:, :K // 8] = rng.integers(0, 256, (M, K // 8), dtype=np.uint8)
    B[:, :K // 8] = rng.integers(0, 256, (N, K // 8), dtype=np.uint8)
    A[:, K // 8] = rng.integers(0, 8, M, dtype=np.uint8)   # K % 8 == 3 live bits in the last byte
    B[:, K // 8] = rng.integers(0, 8, N, dtype=np.uint8)
    mean = np.abs(synth.bell(1, (M,), 0.05)) + np.float32(0.01)
    bias = synth.bell(2, (M,), 0.01)
    sc_in = synth.bell(3, (M, 64), 1.0)
    want = port.gemm_bin_mean_transposed(M, N, K, A, ld, B, ld, mean)
    want = (want + bias[:, None]).astype(np.float32)
    want = np.where(np.signbit(want), (want * np.float32(0.1)).astype(np.float32), want)
    Cg = torch.zeros(M, 64, device="cuda")
    sc_out = torch.zeros(M, 64, device="cuda")
    L.gemm_nn_custom_bin_mean_transposed_gpu(M, N, K, dev(A), ld, dev(B), ld, Cg, 64, dev(mean), dev(bias), 1, dev(sc_in), sc_out)
    got = Cg.cpu().numpy()
    assert_bits_equal(got[:, :N], want, "gemm output")
    assert np.all(got[:, N:] == 0)
    assert_bits_equal(sc_out.cpu().numpy()[:, :N], (sc_in[:, :N] + want).astype(np.float32), "shortcut output")


def test_full_size_properties_without_oracle():
    """At a benchmark-sized batch the oracle is too slow; check size-independent properties instead:
    (1) every image of a batch made of one repeated image gives the same output as batch 1;
    (2) negating the input of a bias-free linear layer with no padded taps negates the output exactly
        (sign(-x) = not sign(x) when x != 0, so every popcount flips to K - count)."""
    c, h, w, n, ks = 128, 26, 26, 256, 3
    x1, wt, b = synth.conv_case(77, 1, c, h, w, n, ks)
    x1[x1 == 0] = np.float32(0.5)          # the negation property below needs x != 0
    l1 = make_layer(1, c, h, w, n, ks, 1, 1, 1, wt, b)
    y1 = L.forward_convolutional_layer_gpu(l1, dev(x1)).clone()
    batch = 64
    lb = make_layer(batch, c, h, w, n, ks, 1, 1, 1, wt, b)
    yb = L.forward_convolutional_layer_gpu(lb, dev(np.repeat(x1, batch, 0)))
    assert torch.equal(yb, y1.expand(batch, -1, -1, -1))
    l0 = make_layer(1, c, h, w, n, ks, 1, 0, 0, wt, np.zeros(n, np.float32))
    ya = L.forward_convolutional_layer_gpu(l0, dev(x1)).clone()
    yn = L.forward_convolutional_layer_gpu(l0, dev(-x1))
    assert torch.equal(yn, -ya)


def test_launch_errors_surface_as_codes():
    l = L.make_convolutional_layer(1, 8, 8, 32, 8, 3, 1, 1, capi.LINEAR)
    with pytest.raises(RuntimeError, match="binary_align_weights"):
        L.forward_convolutional_layer_gpu(l, torch.zeros(1, 32, 8, 8, device="cuda"))
    L.binary_align_weights(l)
    with pytest.raises(ValueError):
        L.forward_convolutional_layer_gpu(l, torch.zeros(1, 32, 8, 7, device="cuda"))
