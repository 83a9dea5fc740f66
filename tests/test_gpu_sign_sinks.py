"""Direct sign sinks: an xnor layer's GEMM epilogue writes the packed activation operand of the next xnor layer
(through an optional 2x2 maxpool, x2 upsample or route concatenation).  Everything must equal, bit for bit, what the
unfused chain (fp32 tensor -> maxpool / upsample / cat -> pack kernel) produces."""
import ctypes as C

import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import torch.nn.functional as F  # noqa: E402

from darknet_b200 import capi, layer as L  # noqa: E402


@pytest.fixture(autouse=True, params=["auto", "tensor-core"])
def gemm_kernel(request):
    """Every test runs once with the library's own kernel choice (integer / short-K kernels at these sizes) and once
    with every GEMM forced onto the tcgen05 kernel, which has its own sink epilogue."""
    capi.set_tuning(gemm_route=capi.ROUTE_TENSOR if request.param == "tensor-core" else capi.ROUTE_AUTO)
    yield request.param
    capi.set_tuning()


def make(batch, c, h, w, n, ks, seed, act=capi.LINEAR):
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, 1, ks // 2, act)
    l.load_weights(torch.from_numpy(synth.bell(seed, (n, c * ks * ks), 0.05)).cuda(), torch.from_numpy(synth.bell(seed + 1, (n,), 0.3)).cuda())
    L.binary_align_weights(l)
    return l


def operand(l, x):
    """The consumer's packed operand as the pack kernel writes it (row-major rows)."""
    return L.pack_input(l, x.contiguous()).clone()


@pytest.mark.parametrize("case", [
    # batch, c1, h, w, n1 (= c2), n2, consumer kernel
    (1, 64, 26, 26, 128, 64, 3), (2, 32, 13, 13, 64, 40, 3), (1, 96, 13, 13, 256, 48, 1), (3, 32, 10, 14, 32, 33, 3),
    (1, 64, 26, 26, 256, 64, 3),            # 176 tiles of 32 filters: the one-shot kernel runs 16-filter tiles (half-word stores)
], ids=lambda c: "b%d_c%d_%dx%d_n%d_n%d_k%d" % c)
def test_plain_sink_fills_the_consumer_operand(case):
    batch, c1, h, w, n1, n2, ks2 = case
    a = make(batch, c1, h, w, n1, 3, 11)
    b = make(batch, n1, h, w, n2, ks2, 13, capi.LEAKY)
    x = torch.from_numpy(synth.bell(17, (batch, c1, h, w), 1.0)).cuda()
    y1 = L.forward_convolutional_layer_gpu(a, x).clone()
    want_op = operand(b, y1)
    want = L.forward_convolutional_layer_gpu(b, y1).clone()
    b.scratch.zero_()
    assert L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(b)]) is None
    torch.cuda.synchronize()
    got_op = b.scratch[:want_op.numel()].view(want_op.shape)
    assert torch.equal(got_op, want_op)
    got = L.forward_convolutional_layer_io(b, packed=True)
    assert torch.equal(got, want)


@pytest.mark.parametrize("case", [(1, 32, 16, 16, 64, 48), (2, 16, 24, 40, 32, 24), (1, 64, 52, 52, 128, 32), (1, 64, 26, 26, 256, 32)],
                         ids=lambda c: "b%d_c%d_%dx%d_n%d_n%d" % c)
def test_pooled_sink_and_window_major_order(case):
    """Layer A runs window-major (its own operand rows permuted), pools in the epilogue and still returns the right
    fp32 tensor when asked for both."""
    batch, c1, h, w, n1, n2 = case
    a = make(batch, c1, h, w, n1, 3, 21)
    b = make(batch, n1, h // 2, w // 2, n2, 3, 23)
    x = torch.from_numpy(synth.bell(27, (batch, c1, h, w), 1.0)).cuda()
    y1 = L.forward_convolutional_layer_gpu(a, x).clone()
    pooled = F.max_pool2d(y1, 2, 2)
    want_op = operand(b, pooled)
    want = L.forward_convolutional_layer_gpu(b, pooled).clone()
    b.scratch.zero_()
    a.window_major = True
    a.output_gpu.fill_(float("nan"))
    y1_again = L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(b, pool=2)], want_output=True)
    torch.cuda.synchronize()
    assert torch.equal(y1_again, y1)                      # fp32 output un-permuted correctly
    assert torch.equal(b.scratch[:want_op.numel()].view(want_op.shape), want_op)
    assert torch.equal(L.forward_convolutional_layer_io(b, packed=True), want)
    # sign words requested from a window-major layer come out in plain pixel order too
    signs = L.forward_convolutional_layer_io(a, x=x, want_signs=True)
    a.window_major = False
    assert torch.equal(signs, L.forward_convolutional_layer_io(a, x=x, want_signs=True))


def test_chain_of_window_major_layers():
    """A -> pool -> B -> pool -> C: B is fed through a sink AND pools itself, so its operand rows are window-major."""
    batch, h, w = 2, 32, 24
    a = make(batch, 32, h, w, 32, 3, 31)
    b = make(batch, 32, h // 2, w // 2, 64, 3, 33)
    c = make(batch, 64, h // 4, w // 4, 40, 3, 35, capi.LEAKY)
    x = torch.from_numpy(synth.bell(37, (batch, 32, h, w), 1.0)).cuda()
    y1 = L.forward_convolutional_layer_gpu(a, x).clone()
    y2 = L.forward_convolutional_layer_gpu(b, F.max_pool2d(y1, 2, 2)).clone()
    want = L.forward_convolutional_layer_gpu(c, F.max_pool2d(y2, 2, 2)).clone()
    for l in (b, c):
        l.scratch.zero_()
    a.window_major = b.window_major = True
    L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(b, pool=2)])
    L.forward_convolutional_layer_io(b, packed=True, sinks=[L.Sink(c, pool=2)])
    got = L.forward_convolutional_layer_io(c, packed=True)
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_upsample_and_route_sinks_build_a_concatenated_operand():
    """yolov3-tiny's second branch: cat(upsample(A1 @13x13, 128 filters), A2 @26x26, 256 filters) -> 3x3 conv over 384."""
    batch = 2
    a1 = make(batch, 64, 13, 13, 128, 1, 41)
    a2 = make(batch, 32, 26, 26, 256, 3, 43)
    b = make(batch, 384, 26, 26, 64, 3, 45, capi.LEAKY)
    x1 = torch.from_numpy(synth.bell(47, (batch, 64, 13, 13), 1.0)).cuda()
    x2 = torch.from_numpy(synth.bell(49, (batch, 32, 26, 26), 1.0)).cuda()
    y1 = L.forward_convolutional_layer_gpu(a1, x1).clone()
    y2 = L.forward_convolutional_layer_gpu(a2, x2).clone()
    cat = torch.cat([F.interpolate(y1, scale_factor=2, mode="nearest"), y2], 1).contiguous()
    want_op = operand(b, cat)
    want = L.forward_convolutional_layer_gpu(b, cat).clone()
    b.scratch.zero_()
    L.forward_convolutional_layer_io(a1, x=x1, sinks=[L.Sink(b, upsample=2)])
    y2_again = L.forward_convolutional_layer_io(a2, x=x2, sinks=[L.Sink(b, channel_offset=128)], want_output=True)
    torch.cuda.synchronize()
    assert torch.equal(y2_again, y2)
    assert torch.equal(b.scratch[:want_op.numel()].view(want_op.shape), want_op)
    assert torch.equal(L.forward_convolutional_layer_io(b, packed=True), want)


@pytest.mark.parametrize("variant", [1, 2], ids=["tile-per-cta", "persistent"])
@pytest.mark.parametrize("case", [(4, 64, 28, 28, 128, 2), (2, 32, 20, 24, 96, 1), (3, 128, 14, 14, 160, 1)], ids=lambda c: "b%d_c%d_%dx%d_n%d_s%d" % c)
def test_output_and_plain_sinks_from_both_tensor_core_kernels(case, variant):
    """darknet53's stride-2 layers: the fp32 tensor (the next block's shortcut operand) AND the operand of the 1x1 layer behind.
    The persistent kernel stages the values in shared memory, writes them with tensor stores and emits the sign words from the
    same registers; the other kernel stores both directly.  Tensor and operands equal the unfused chain, bit for bit; a second,
    upsampling sink rides along."""
    batch, c1, h, w, n1, stride = case
    a = L.make_convolutional_layer(batch, h, w, c1, n1, 3, stride, 1, capi.LEAKY)
    a.load_weights(torch.from_numpy(synth.bell(61, (n1, c1 * 9), 0.05)).cuda(), torch.from_numpy(synth.bell(62, (n1,), 0.3)).cuda())
    L.binary_align_weights(a)
    oh, ow = a.geom.out_h, a.geom.out_w
    near = make(batch, n1, oh, ow, 40, 1, 63, capi.LEAKY)
    far = make(batch, n1, 2 * oh, 2 * ow, 32, 3, 65)
    x = torch.from_numpy(synth.bell(67, (batch, c1, h, w), 1.0)).cuda()
    capi.set_tuning(gemm_route=capi.ROUTE_INTEGER)
    y = L.forward_convolutional_layer_gpu(a, x).clone()
    want_near = operand(near, y)
    want_far = operand(far, F.interpolate(y, scale_factor=2, mode="nearest").contiguous())
    capi.set_tuning(gemm_route=capi.ROUTE_TENSOR, tc_kernel=variant)
    for _ in range(3):
        near.scratch.zero_()
        far.scratch.zero_()
        a.output_gpu.fill_(float("nan"))
        got = L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(near), L.Sink(far, upsample=2)], want_output=True)
        torch.cuda.synchronize()
        assert torch.equal(got, y)
        assert torch.equal(near.scratch[:want_near.numel()].view(want_near.shape), want_near)
        assert torch.equal(far.scratch[:want_far.numel()].view(want_far.shape), want_far)


def test_two_sinks_from_one_layer():
    """yolov3-tiny's layer 8: fp32 for the route, a pooled sink for the next layer and a plain sink for the far one."""
    batch = 1
    a = make(batch, 32, 26, 26, 64, 3, 51)
    near = make(batch, 64, 13, 13, 32, 3, 53)
    far = make(batch, 96, 26, 26, 32, 3, 55)
    x = torch.from_numpy(synth.bell(57, (batch, 32, 26, 26), 1.0)).cuda()
    y = L.forward_convolutional_layer_gpu(a, x).clone()
    want_near = operand(near, F.max_pool2d(y, 2, 2))
    near.scratch.zero_()
    far.scratch.zero_()
    a.window_major = True
    L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(near, pool=2), L.Sink(far, channel_offset=32)], want_output=True)
    torch.cuda.synchronize()
    assert torch.equal(near.scratch[:want_near.numel()].view(want_near.shape), want_near)
    # the far consumer's channels 32..95 are this layer's signs, the rest still zero
    full = torch.cat([torch.full((batch, 32, 26, 26), -1.0, device="cuda"), y], 1).contiguous()
    want_far = operand(far, full)
    assert torch.equal(far.scratch[:want_far.numel()].view(want_far.shape), want_far)


def test_sink_argument_checks():
    a = make(1, 32, 8, 8, 32, 3, 61)
    ok = make(1, 32, 8, 8, 32, 3, 63)
    x = torch.zeros(1, 32, 8, 8, device="cuda")
    half = make(1, 32, 4, 4, 32, 3, 65)
    with pytest.raises(capi.XnorError, match="invalid"):       # pooled sink without window-major order
        L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(half, pool=2)])
    with pytest.raises(capi.XnorError, match="invalid"):       # consumer map does not match
        L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(half)])
    with pytest.raises(capi.XnorError, match="invalid"):       # channel range outside the consumer
        L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(ok, channel_offset=32)])
    strided = L.make_convolutional_layer(1, 8, 8, 32, 32, 3, 2, 1, capi.LINEAR)
    with pytest.raises(capi.XnorError, match="invalid"):       # consumer with stride 2
        L.forward_convolutional_layer_io(a, x=x, sinks=[L.Sink(strided)])
    with pytest.raises(capi.XnorError):                        # two kinds of input
        L.forward_convolutional_layer_io(ok, x=x, packed=True)
