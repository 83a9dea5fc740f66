"""CPU checks of the checker itself: the plain-C restatement (oracle/xnor_oracle.c) against the golden
vectors produced by the reference's own CPU code, against that code directly where it is built, and
against an independent closed form."""
import numpy as np
import pytest

import synth
from oracle.binding import new_lda, out_dim


def naive_sign_conv(x, w, b, stride, pad, leaky):
    """Closed form: out = act(fl(fl((2*cnt-K)*mean) + bias)), cnt = agreeing signs, padded taps = 'not > 0'."""
    c, h, wd = x.shape
    n, _, ks, _ = w.shape
    oh, ow = out_dim(h, ks, stride, pad), out_dim(wd, ks, stride, pad)
    sx = np.zeros((c, h + 2 * pad, wd + 2 * pad), bool)
    sx[:, pad:pad + h, pad:pad + wd] = x > 0
    sw = w > 0
    K = c * ks * ks
    mean = np.zeros(n, np.float32)
    for f in range(n):
        acc = np.float32(0)
        for v in np.abs(w[f].reshape(-1)):
            acc = np.float32(acc + v)
        mean[f] = np.float32(acc / np.float32(K))
    out = np.zeros((n, oh, ow), np.float32)
    for y in range(oh):
        for xx in range(ow):
            patch = sx[:, y * stride:y * stride + ks, xx * stride:xx * stride + ks]
            cnt = (patch[None] == sw).reshape(n, -1).sum(1).astype(np.int64)
            v = ((2 * cnt - K).astype(np.float32) * mean).astype(np.float32)
            out[:, y, xx] = (v + b).astype(np.float32)
    if leaky:
        out = np.where(np.signbit(out), (out * np.float32(0.1)).astype(np.float32), out)
    return out


def test_geometry_always_adds():
    assert new_lda(2304) == 2560 and new_lda(675) == 768 and new_lda(144) == 256 and new_lda(256) == 512
    from oracle.binding import bit_align
    assert bit_align(676) == 704 and bit_align(173056) == 173088 and bit_align(160) == 192


def test_port_matches_reference_golden(port, golden):
    cases, data = golden
    for i, (seed, c, h, w, n, ks, stride, pad, leaky) in enumerate(cases):
        x, wt, b = synth.conv_case(seed, 1, c, h, w, n, ks)
        out, tb, cnt = port.conv_forward(x, wt, b, stride, pad, leaky, dumps=True)
        A, mean = port.binary_align_weights(wt)
        K = c * ks * ks
        assert np.array_equal(A[:n * new_lda(K) // 8], data[f"c{i}_align_bit_weights"]), f"case {i}: packed weights"
        assert np.array_equal(mean.view(np.uint32), data[f"c{i}_mean_arr"].view(np.uint32)), f"case {i}: mean_arr"
        assert np.array_equal(tb[0], data[f"c{i}_t_bit_input"]), f"case {i}: t_bit_input"
        assert np.array_equal(out[0].view(np.uint32), data[f"c{i}_output"].view(np.uint32)), f"case {i}: output bits"


def test_port_inverted_weight_layout_matches_golden(port, golden):
    cases, data = golden
    seed, c, h, w, n, ks, stride, pad, leaky = cases[0]
    _, wt, _ = synth.conv_case(seed, 1, c, h, w, n, ks)
    A, _ = port.binary_align_weights(wt, invert=True)
    assert np.array_equal(A[:n * new_lda(c * ks * ks) // 8], data["c0_align_bit_weights_inverted"])


@pytest.mark.parametrize("shape", [
    (64, 13, 13, 48, 3, 1, 1, 1), (32, 9, 7, 16, 3, 1, 1, 0), (64, 8, 8, 32, 1, 1, 0, 1), (5, 10, 10, 8, 3, 1, 1, 1),
    (75, 26, 26, 64, 3, 1, 1, 1), (64, 16, 16, 32, 3, 2, 1, 1), (96, 7, 9, 17, 3, 1, 1, 1), (128, 6, 6, 9, 3, 2, 1, 0),
])
def test_port_matches_reference_live(port, ref, shape):
    c, h, w, n, ks, stride, pad, leaky = shape
    x, wt, b = synth.conv_case(100 + c + n, 1, c, h, w, n, ks)
    layer = ref.layer((c, h, w), wt, b, stride, pad, bool(leaky))
    ro = layer.forward(x[0])
    po, tb, _ = port.conv_forward(x, wt, b, stride, pad, leaky, dumps=True)
    A, mean = port.binary_align_weights(wt)
    assert np.array_equal(A, layer.align_bit_weights())
    assert np.array_equal(mean, layer.mean_arr())
    assert np.array_equal(tb[0], layer.t_bit_input())
    assert np.array_equal(ro.view(np.uint32), po[0].view(np.uint32))
    layer.close()


@pytest.mark.parametrize("shape", [
    (32, 6, 5, 7, 3, 1, 1, 1), (7, 6, 6, 5, 3, 1, 1, 0), (75, 5, 5, 6, 1, 1, 0, 1), (40, 9, 9, 4, 3, 2, 1, 1), (64, 4, 4, 3, 1, 1, 0, 0),
])
def test_port_matches_closed_form(port, shape):
    """Includes shapes the reference CPU code does not define (1x1 or strided with channels % 32 != 0)."""
    c, h, w, n, ks, stride, pad, leaky = shape
    x, wt, b = synth.conv_case(200 + c, 2, c, h, w, n, ks)
    po = port.conv_forward(x, wt, b, stride, pad, leaky)
    for img in range(2):
        want = naive_sign_conv(x[img], wt, b, stride, pad, leaky)
        assert np.array_equal(po[img].view(np.uint32), want.view(np.uint32))


def test_port_sign_edge_values(port):
    """0.0, -0.0, denormals and NaN are all 'not > 0'; +denormal and +inf are '> 0'."""
    vals = np.array([0.0, -0.0, 1e-45, -1e-45, np.inf, -np.inf, np.nan, 1.0] * 4, np.float32)
    bits = port.float_to_bit(vals)
    want = np.array([0, 0, 1, 0, 1, 0, 0, 1] * 4, np.uint8)
    got = np.unpackbits(bits[:4], bitorder="little")
    assert np.array_equal(got, want)


def test_port_stage_functions_against_reference(port, ref):
    """Each restated stage against the reference function it follows."""
    import ctypes as C
    rng_x = synth.bell(7, (64, 6, 5), 1.0)
    # float_to_bit
    flat = np.ascontiguousarray(rng_x.reshape(-1))
    got = port.float_to_bit(flat)
    want = np.zeros(flat.size // 8 + 1, np.uint8)
    ref.lib.ref_float_to_bit(flat, want, flat.size)
    assert np.array_equal(got, want)
    # repack_input + float_to_bit
    re = np.zeros(flat.size, np.float32)
    ref.lib.ref_repack_input(flat, re, 5, 6, 64)
    want = np.zeros(flat.size // 8 + 1, np.uint8)
    ref.lib.ref_float_to_bit(re, want, flat.size)
    got = port.repack_input_bin(rng_x)
    assert np.array_equal(got.reshape(-1).view(np.uint8), want[:flat.size // 8])
    # transpose_bin on a 64 x 96 bit matrix with zero slack around it
    n, m, lda, ldb = 64, 96, 128, 256
    rng = np.random.default_rng(3)
    A = np.zeros((n + 32) * lda // 8, np.uint8)
    rows = rng.integers(0, 256, (n, m // 8), dtype=np.uint8)
    A.reshape(n + 32, lda // 8)[:n, :m // 8] = rows
    Bp = np.zeros((m + 32) * ldb // 8, np.uint8)
    Br = np.zeros_like(Bp)
    port.lib.oracle_transpose_bin(A, Bp, n, m, lda, ldb)
    ref.lib.ref_transpose_bin(A.ctypes.data, Br.ctypes.data, n, m, lda, ldb, 8)
    assert np.array_equal(Bp, Br)
    # GEMM incl. odd M, N (scalar tails) and K not a multiple of 256
    M, N, K = 7, 5, 300
    ld = new_lda(K)
    Ab = np.zeros((M, ld // 8), np.uint8)
    Bb = np.zeros((N, ld // 8), np.uint8)
    Ab[:, :K // 8] = rng.integers(0, 256, (M, K // 8), dtype=np.uint8)
    Bb[:, :K // 8] = rng.integers(0, 256, (N, K // 8), dtype=np.uint8)
    Ab[:, K // 8] = rng.integers(0, 16, M, dtype=np.uint8)       # K % 8 == 4 live bits
    Bb[:, K // 8] = rng.integers(0, 16, N, dtype=np.uint8)
    mean = synth.bell(9, (M,), 0.05).astype(np.float32)
    got = port.gemm_bin_mean_transposed(M, N, K, Ab, ld, Bb, ld, mean)
    want = np.zeros((M, N), np.float32)
    ref.lib.ref_gemm_nn_custom_bin_mean_transposed(M, N, K, Ab.reshape(-1), ld, Bb.reshape(-1), ld, want.reshape(-1), N, mean)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
