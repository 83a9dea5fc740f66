"""The tcgen05 (tensor-core) variant of the XNOR GEMM against the oracle and against the integer-pipe kernel.

xnor_b200_set_tuning pins the route of every GEMM call -- "1" = the tensor-core kernel, "0" = the tiled integer-pipe
kernel, None = the library's own choice -- so both are exercised on identical operands.  Integer accumulators and fp32 outputs must be bit-identical to the oracle."""
import numpy as np
import pytest

import synth
from oracle.binding import new_lda

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, layer as L  # noqa: E402


@pytest.fixture
def force_tc():
    def set_mode(v, tc_kernel=0):
        """tc_kernel: 0 = the library picks the tcgen05 kernel, 1 = one tile per CTA, 2 = persistent."""
        capi.set_tuning(gemm_route={None: capi.ROUTE_AUTO, "0": capi.ROUTE_TILED, "1": capi.ROUTE_TENSOR}[v], tc_kernel=tc_kernel)
    yield set_mode
    capi.set_tuning()


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
    (128, 4097, 1152), (1, 1, 1), (257, 129, 9216), (64, 70000, 288), (32, 1000, 64), (100, 5000, 384), (128, 257, 129),
], ids=lambda s: "M%d_N%d_K%d" % s)
def test_tensor_core_counts_match_oracle(port, force_tc, shape):
    M, N, K = shape
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    A, ld = random_bits(rng, M, K)
    B, _ = random_bits(rng, N, K)
    want = port.gemm_counts(M, N, K, A, ld, B, ld)
    Ag, Bg = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    for variant in (1, 2):                      # both tcgen05 kernels, whatever the library would pick for this shape
        force_tc("1", variant)
        got_tc = L.gemm_counts(M, N, K, Ag, ld, Bg, ld).cpu().numpy()
        assert device_status() == 0
        assert np.array_equal(got_tc, want), f"tensor-core kernel {variant}: counts differ in {np.count_nonzero(got_tc != want)} of {want.size} entries"
    force_tc("0")
    got_int = L.gemm_counts(M, N, K, Ag, ld, Bg, ld).cpu().numpy()
    assert np.array_equal(got_int, want)


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
    """A batch-64 BASELINE-sized layer (eligible for the tensor-core kernel), 64 distinct images: every image equals the
    oracle bit for bit, and the integer kernel gives the same tensor."""
    batch, c, h, w, n, ks = 64, 256, 26, 26, 512, 3
    x, wt, b = synth.conv_case(777, batch, c, h, w, n, ks)
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
    want = port.conv_forward(x, wt, b, 1, 1, 1)
    assert np.array_equal(y_auto.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("shape", [(256, 640, 1152), (200, 300, 576), (96, 1000, 288), (48, 257, 300), (20, 129, 128), (512, 130, 2304)],
                         ids=lambda s: "M%d_N%d_K%d" % s)
def test_tensor_core_fused_shortcut_equals_integer_kernel(force_tc, shape):
    """fp32 output + fused shortcut add (the pipelined epilogue of the tensor-core kernel; every filter-tile width, ragged
    filter and pixel edges, ldc > N) against the integer-pipe kernel on the same operands, and without a shortcut."""
    M, N, K = shape
    rng = np.random.default_rng(M + 3 * N + 5 * K)
    A, ld = random_bits(rng, M, K)
    B, _ = random_bits(rng, N, K)
    Ag, Bg = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    ldc = N + 5
    mean = torch.from_numpy(rng.random(M, dtype=np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(M).astype(np.float32)).cuda()
    sc_in = torch.from_numpy(rng.standard_normal((M, ldc)).astype(np.float32)).cuda()
    outs = {}
    for mode in ("1", "1p", "0"):
        force_tc(mode[0], 2 if mode == "1p" else 1)
        for with_sc in (True, False):
            C_ = torch.full((M, ldc), float("nan"), device="cuda")
            sc_out = torch.full((M, ldc), float("nan"), device="cuda")
            capi.check(capi.lib().xnor_b200_gemm_bin_mean_transposed(
                M, N, K, Ag.data_ptr(), ld, Bg.data_ptr(), ld, C_.data_ptr(), ldc, mean.data_ptr(), bias.data_ptr(), 1,
                sc_in.data_ptr() if with_sc else None, sc_out.data_ptr() if with_sc else None,
                torch.cuda.current_stream().cuda_stream), "gemm")
            torch.cuda.synchronize()
            outs[(mode, with_sc)] = (C_[:, :N].clone(), sc_out[:, :N].clone())
            assert torch.isnan(C_[:, N:]).all() and torch.isnan(sc_out[:, N:]).all()        # nothing written past N
    assert device_status() == 0
    ref_c, ref_sc = outs[("0", True)]
    assert torch.equal(ref_sc, sc_in[:, :N] + ref_c)
    for key, (c_, s_) in outs.items():
        assert torch.equal(c_, ref_c), key
        if key[1]:
            assert torch.equal(s_, ref_sc), key


@pytest.mark.parametrize("mode", ["0", "1"], ids=["integer", "tensor-core"])
def test_shortcut_sum_without_the_layers_own_tensor(force_tc, mode):
    """xnor_b200_conv_forward_io with output = NULL and a fused shortcut: the sum equals the one of the full call, the
    layer's own tensor is not touched; NULL output together with sign outputs is refused."""
    batch, c, h, w, n = 2, 64, 20, 20, 96
    x, wt, b = synth.conv_case(999, batch, c, h, w, n, 3)
    l = L.make_convolutional_layer(batch, h, w, c, n, 3, 1, 1, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    xg = torch.from_numpy(x).cuda()
    l.bin_conv_shortcut_in_gpu = torch.randn(batch, n, h, w, device="cuda")
    l.bin_conv_shortcut_out_gpu = torch.empty(batch, n, h, w, device="cuda")
    force_tc(mode)
    y = L.forward_convolutional_layer_gpu(l, xg).clone()
    want = l.bin_conv_shortcut_out_gpu.clone()
    assert torch.equal(want, l.bin_conv_shortcut_in_gpu + y)
    l.output_gpu.fill_(float("nan"))
    l.bin_conv_shortcut_out_gpu.fill_(float("nan"))
    got = L.forward_convolutional_layer_io(l, x=xg, shortcut_only=True)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert torch.isnan(l.output_gpu).all()
    assert device_status() == 0
    import ctypes as C
    io = capi.ConvIO()
    io.input = xg.data_ptr()
    io.shortcut_in = l.bin_conv_shortcut_in_gpu.data_ptr()
    io.shortcut_out = l.bin_conv_shortcut_out_gpu.data_ptr()
    signs = torch.empty(batch, n // 32, h * w, dtype=torch.int32, device="cuda")
    io.output_signs = signs.data_ptr()
    rc = capi.lib().xnor_b200_conv_forward_io(C.byref(l.desc), C.byref(io), l.align_bit_weights_gpu.data_ptr(), l.mean_arr_gpu.data_ptr(),
                                              l.biases_gpu.data_ptr(), l.scratch.data_ptr(), l.scratch.numel(), None)
    assert rc != capi.OK


@pytest.mark.parametrize("case", [(2, 64, 20, 20, 96, 3), (1, 32, 16, 12, 256, 3), (3, 128, 9, 9, 64, 1)], ids=lambda c: "b%d_c%d_%dx%d_n%d_k%d" % c)
def test_sign_words_of_the_fused_shortcut_sum(case):
    """shortcut_signs: bit f%32 of word [image][f/32][pixel] = (shortcut_out of filter f > 0); the call runs on the tensor-core
    kernel by itself, the sum and the layer's own tensor stay what the plain call writes, and an xnor layer fed with the words
    gives the same output as from the fp32 sum."""
    batch, c, h, w, n, ks = case
    x, wt, b = synth.conv_case(4242 + n, batch, c, h, w, n, ks)
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, 1, ks // 2, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    xg = torch.from_numpy(x).cuda()
    l.bin_conv_shortcut_in_gpu = torch.from_numpy(synth.bell(7, (batch, n, h, w), 1.0)).cuda()
    l.bin_conv_shortcut_out_gpu = torch.empty(batch, n, h, w, device="cuda")
    y = L.forward_convolutional_layer_gpu(l, xg).clone()
    want_sum = l.bin_conv_shortcut_out_gpu.clone()
    l.output_gpu.fill_(float("nan"))
    l.bin_conv_shortcut_out_gpu.fill_(float("nan"))
    got = L.forward_convolutional_layer_io(l, x=xg, want_output=True, shortcut_signs=True)
    torch.cuda.synchronize()
    assert device_status() == 0
    assert torch.equal(got, y) and torch.equal(l.bin_conv_shortcut_out_gpu, want_sum)
    bits = (want_sum > 0).view(batch, n // 32, 32, h * w).to(torch.int64)
    words = (bits << torch.arange(32, device="cuda").view(1, 1, 32, 1)).sum(2)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    assert torch.equal(l.shortcut_signs_gpu, words)
    nxt = L.make_convolutional_layer(batch, h, w, n, 64, 1, 1, 0, capi.LINEAR)
    nxt.load_weights(torch.from_numpy(synth.bell(9, (64, n), 0.05)).cuda(), torch.from_numpy(synth.bell(10, (64,), 0.3)).cuda())
    L.binary_align_weights(nxt)
    ref = L.forward_convolutional_layer_gpu(nxt, want_sum).clone()
    assert torch.equal(L.forward_convolutional_layer_io(nxt, x_signs=l.shortcut_signs_gpu), ref)


@pytest.mark.parametrize("case", [(2, 64, 20, 20, 96), (1, 32, 16, 12, 256), (3, 128, 9, 9, 64)], ids=lambda c: "b%d_c%d_%dx%d_n%d" % c)
def test_shortcut_sum_signs_straight_into_a_1x1_readers_operand(case):
    """shortcut_sink: the 1x1 layer that reads the fused sum finds its packed operand filled by the producer's epilogue
    (equal to what its own pack kernel makes of the fp32 sum, padding words untouched) and gives the same output."""
    batch, c, h, w, n = case
    x, wt, b = synth.conv_case(777 + n, batch, c, h, w, n, 3)
    l = L.make_convolutional_layer(batch, h, w, c, n, 3, 1, 1, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    xg = torch.from_numpy(x).cuda()
    l.bin_conv_shortcut_in_gpu = torch.from_numpy(synth.bell(17, (batch, n, h, w), 1.0)).cuda()
    l.bin_conv_shortcut_out_gpu = torch.empty(batch, n, h, w, device="cuda")
    L.forward_convolutional_layer_gpu(l, xg)
    want_sum = l.bin_conv_shortcut_out_gpu.clone()
    nxt = L.make_convolutional_layer(batch, h, w, n, 40, 1, 1, 0, capi.LEAKY)
    nxt.load_weights(torch.from_numpy(synth.bell(19, (40, n), 0.05)).cuda(), torch.from_numpy(synth.bell(20, (40,), 0.3)).cuda())
    L.binary_align_weights(nxt)
    want_op = L.pack_input(nxt, want_sum).clone()
    ref = L.forward_convolutional_layer_gpu(nxt, want_sum).clone()
    nxt.scratch.zero_()
    l.bin_conv_shortcut_out_gpu.fill_(float("nan"))
    got_sum = L.forward_convolutional_layer_io(l, x=xg, shortcut_only=True, shortcut_sink=nxt)
    torch.cuda.synchronize()
    assert device_status() == 0
    assert torch.equal(got_sum, want_sum)
    assert torch.equal(nxt.scratch[:want_op.numel()].view(want_op.shape), want_op)
    assert torch.equal(L.forward_convolutional_layer_io(nxt, packed=True), ref)
    # a reader that is not 1x1 over these channels is refused
    bad = L.make_convolutional_layer(batch, h, w, n, 40, 3, 1, 1, capi.LEAKY)
    with pytest.raises(capi.XnorError, match="invalid"):
        L.forward_convolutional_layer_io(l, x=xg, shortcut_only=True, shortcut_sink=bad)


@pytest.mark.parametrize("variant", [1, 2], ids=["tile-per-cta", "persistent"])
def test_many_tiles_per_cta_repeatedly_equal_the_integer_kernel(force_tc, variant):
    """A GEMM with several tiles per SM (the persistent kernel walks five of them per CTA, re-using its operand rings, its two
    accumulator buffers and the per-row tables), launched five times on the same operands: every launch equals the integer
    kernel bit for bit.  A hand-over that is only right for some timings shows up here as a launch that differs."""
    M, N, K = 512, 148 * 128 * 5 + 77, 2304
    rng = np.random.default_rng(20241)
    A, ld = random_bits(rng, M, K)
    B, _ = random_bits(rng, N, K)
    Ag, Bg = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    mean = torch.from_numpy(rng.random(M, dtype=np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(M).astype(np.float32)).cuda()

    def run():
        out = torch.full((M, N), float("nan"), device="cuda")
        capi.check(capi.lib().xnor_b200_gemm_bin_mean_transposed(M, N, K, Ag.data_ptr(), ld, Bg.data_ptr(), ld, out.data_ptr(), N,
                                                                 mean.data_ptr(), bias.data_ptr(), 1, None, None,
                                                                 torch.cuda.current_stream().cuda_stream), "gemm")
        torch.cuda.synchronize()
        return out

    force_tc("0")
    want = run()
    force_tc("1", variant)
    for i in range(5):
        got = run()
        assert device_status() == 0
        assert torch.equal(got, want), f"launch {i}: {int((got != want).sum())} values differ"


@pytest.mark.parametrize("case", [(3, 128, 14, 14, 160, 3), (8, 64, 28, 28, 128, 3), (2, 256, 26, 26, 288, 1), (5, 64, 12, 20, 96, 3)],
                         ids=lambda c: "b%d_c%d_%dx%d_n%d_k%d" % c)
@pytest.mark.parametrize("variant", [1, 2], ids=["tile-per-cta", "persistent"])
def test_shortcut_sum_only_with_its_sign_words_on_both_kernels(force_tc, case, variant):
    """A layer of which only the fused shortcut sum is wanted, plus the sum's sign words or the 1x1 reader's operand: the persistent
    kernel brings the shortcut operand into shared memory with the copy engine, adds there and writes the sum with tensor stores
    (row copies where a 128-pixel tile runs over the end of an image, as it does in every case here).  Sum, words and operand
    equal what the integer kernel and the pack kernel produce."""
    batch, c, h, w, n, ks = case
    x, wt, b = synth.conv_case(515 + n, batch, c, h, w, n, ks)
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, 1, ks // 2, capi.LEAKY)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    xg = torch.from_numpy(x).cuda()
    l.bin_conv_shortcut_in_gpu = torch.from_numpy(synth.bell(27, (batch, n, h, w), 1.0)).cuda()
    l.bin_conv_shortcut_out_gpu = torch.empty(batch, n, h, w, device="cuda")
    force_tc("0")
    L.forward_convolutional_layer_gpu(l, xg)
    want_sum = l.bin_conv_shortcut_out_gpu.clone()
    bits = (want_sum > 0).view(batch, n // 32, 32, h * w).to(torch.int64)
    words = (bits << torch.arange(32, device="cuda").view(1, 1, 32, 1)).sum(2)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    nxt = L.make_convolutional_layer(batch, h, w, n, 40, 1, 1, 0, capi.LEAKY)
    nxt.load_weights(torch.from_numpy(synth.bell(19, (40, n), 0.05)).cuda(), torch.from_numpy(synth.bell(20, (40,), 0.3)).cuda())
    L.binary_align_weights(nxt)
    want_op = L.pack_input(nxt, want_sum).clone()
    force_tc("1", variant)
    for _ in range(3):
        l.bin_conv_shortcut_out_gpu.fill_(float("nan"))
        got = L.forward_convolutional_layer_io(l, x=xg, shortcut_only=True, shortcut_signs=True)
        torch.cuda.synchronize()
        assert device_status() == 0
        assert torch.equal(got, want_sum)
        assert torch.equal(l.shortcut_signs_gpu, words)
        nxt.scratch.zero_()
        l.bin_conv_shortcut_out_gpu.fill_(float("nan"))
        got = L.forward_convolutional_layer_io(l, x=xg, shortcut_only=True, shortcut_sink=nxt)
        torch.cuda.synchronize()
        assert device_status() == 0
        assert torch.equal(got, want_sum)
        assert torch.equal(nxt.scratch[:want_op.numel()].view(want_op.shape), want_op)


@pytest.mark.parametrize("shape", [(512, 676, 2304), (512, 64 * 676, 2304), (1024, 16 * 169, 4608), (256, 16 * 3136, 1152), (64, 8 * 50176, 288)],
                         ids=lambda s: "%dx%dx%d" % s)
def test_the_librarys_own_choice_is_close_to_the_fastest_kernel(shape):
    """The kernel choice rests on constants fitted on B200.  On layer shapes of the three benchmark networks (batch 1 to 64) the
    call the library routes by itself must not take more than 1.5x the time (+ 5 us) of the fastest of: integer kernels, tensor-core
    kernel with one tile per CTA, persistent tensor-core kernel (median of 5 timings of 10 calls each, CUDA events)."""
    M, N, K = shape
    rng = np.random.default_rng(99)
    A, ld = random_bits(rng, M, K)
    B, _ = random_bits(rng, N, K)
    Ag, Bg = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    mean = torch.from_numpy(rng.random(M, dtype=np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(M).astype(np.float32)).cuda()
    out = torch.empty((M, N), device="cuda")
    stream = torch.cuda.current_stream()

    def call():
        capi.check(capi.lib().xnor_b200_gemm_bin_mean_transposed(M, N, K, Ag.data_ptr(), ld, Bg.data_ptr(), ld, out.data_ptr(), N,
                                                                 mean.data_ptr(), bias.data_ptr(), 1, None, None, stream.cuda_stream), "gemm")

    def median_ms():
        for _ in range(3):
            call()
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(10):
                call()
            e1.record(stream)
            e1.synchronize()
            times.append(e0.elapsed_time(e1) / 10)
        return sorted(times)[2]

    routes = (("integer", dict(gemm_route=capi.ROUTE_INTEGER)), ("tile-per-cta", dict(gemm_route=capi.ROUTE_TENSOR, tc_kernel=1)),
              ("persistent", dict(gemm_route=capi.ROUTE_TENSOR, tc_kernel=2)))
    report = ""
    try:
        for attempt in range(3):                          # a timing on a shared machine: a second and third look before failing
            capi.set_tuning()
            own = median_ms()
            others = {}
            for name, kw in routes:
                capi.set_tuning(**kw)
                others[name] = median_ms()
            report = f"own choice {own * 1e3:.1f} us, others {({k: round(v * 1e3, 1) for k, v in others.items()})}"
            if own <= 1.5 * min(others.values()) + 0.005:
                break
        else:
            pytest.fail(report)
    finally:
        capi.set_tuning()
    assert device_status() == 0


def test_persistent_kernel_with_staged_output_is_the_same_on_every_launch(force_tc):
    """Short rows, 128-filter tiles and the fp32 results leaving through shared memory: the shape on which a raw operand stage was
    once handed back to the copy engine before every warp had read it (about one launch in thirty then differed in a few pixel
    columns of one tile).  200 launches, each equal to the tile-per-CTA kernel bit for bit."""
    M, N, K = 256, 64 * 676, 1152
    rng = np.random.default_rng(20251)
    A, ld = random_bits(rng, M, K)
    B, _ = random_bits(rng, N, K)
    Ag, Bg = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    mean = torch.from_numpy(rng.random(M, dtype=np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(M).astype(np.float32)).cuda()
    out = torch.empty((M, N), device="cuda")

    def run():
        out.fill_(float("nan"))
        capi.check(capi.lib().xnor_b200_gemm_bin_mean_transposed(M, N, K, Ag.data_ptr(), ld, Bg.data_ptr(), ld, out.data_ptr(), N,
                                                                 mean.data_ptr(), bias.data_ptr(), 1, None, None,
                                                                 torch.cuda.current_stream().cuda_stream), "gemm")
        return out

    force_tc("1", 1)
    want = run().clone()
    force_tc("1", 2)
    differing = [i for i in range(200) if not torch.equal(run(), want)]
    assert device_status() == 0
    assert differing == []


@pytest.mark.parametrize("variant", [1, 2], ids=["tile-per-cta", "persistent"])
def test_bounded_wait_runs_out_and_the_kernel_recovers(port, variant):
    """Failure detection without a fault: xnor_b200_set_tuning withholds one producer arrival of the first K block and gives
    every barrier wait a few thousand polls, so the issuer's wait runs out.  The kernel must come back by itself (every role
    leaves through the give-up path, tensor memory released), report it through xnor_b200_take_device_status once, and leave
    the device fit for the next launch, whose counts equal the oracle's."""
    M, N, K = 256, 1000, 1152
    rng = np.random.default_rng(99)
    A, ld = random_bits(rng, M, K)
    B, _ = random_bits(rng, N, K)
    Ag, Bg = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    want = port.gemm_counts(M, N, K, A, ld, B, ld)
    try:
        assert device_status() == 0
        capi.set_tuning(gemm_route=capi.ROUTE_TENSOR, tc_kernel=variant, tc_wait_polls=4000, tc_withhold_arrival=1)
        L.gemm_counts(M, N, K, Ag, ld, Bg, ld)
        assert device_status() == 1            # a wait ran out; the word is sticky until taken
        assert device_status() == 0            # ... and cleared by the call that took it
        capi.set_tuning(gemm_route=capi.ROUTE_TENSOR, tc_kernel=variant)
        for _ in range(2):
            got = L.gemm_counts(M, N, K, Ag, ld, Bg, ld).cpu().numpy()
            assert device_status() == 0
            assert np.array_equal(got, want)
    finally:
        capi.set_tuning()
