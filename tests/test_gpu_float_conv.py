"""The fused few-channel float convolution (layer in front of the xnor path) against cuDNN fp32."""
import ctypes as C

import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, layer as L  # noqa: E402


@pytest.mark.parametrize("case", [
    (2, 3, 40, 56, 16, 3, 1, 1, 1), (1, 3, 33, 17, 32, 3, 1, 1, 0), (2, 3, 20, 20, 16, 3, 2, 1, 1),
    (1, 4, 12, 12, 8, 5, 1, 2, 1), (1, 1, 9, 9, 3, 1, 1, 0, 0), (1, 3, 416, 416, 16, 3, 1, 1, 1),
], ids=lambda c: "b%d_c%d_%dx%d_n%d_k%d_s%d_p%d_%d" % c)
def test_float_conv_small_matches_cudnn(case):
    torch.backends.cudnn.allow_tf32 = False
    batch, c, h, w, n, ks, stride, pad, leaky = case
    x = torch.from_numpy(synth.uniform01(sum(case), (batch, c, h, w))).cuda()
    wt = torch.from_numpy(synth.bell(sum(case) + 1, (n, c, ks, ks), 0.05)).cuda()
    b = torch.from_numpy(synth.bell(sum(case) + 2, (n,), 0.01)).cuda()
    want = torch.nn.functional.conv2d(x.double(), wt.double(), b.double(), stride, pad)
    if leaky:
        want = torch.where(want > 0, want, want * 0.1)
    desc = capi.ConvDesc(batch, c, h, w, n, ks, stride, pad, capi.LEAKY if leaky else capi.LINEAR)
    out = torch.full(want.shape, float("nan"), dtype=torch.float32, device="cuda")
    capi.check(capi.lib().xnor_b200_float_conv_small(C.byref(desc), x.data_ptr(), wt.data_ptr(), b.data_ptr(), out.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream), "xnor_b200_float_conv_small")
    torch.cuda.synchronize()
    # fp32 accumulation of <= 100 products of magnitude <= 0.2: absolute error far below 1e-5
    assert torch.isfinite(out).all()
    assert (out.double() - want).abs().max().item() <= 1e-5


def test_float_conv_small_rejects_wide_layers():
    desc = capi.ConvDesc(1, 64, 8, 8, 8, 3, 1, 1, capi.LINEAR)       # 576 taps
    z = torch.zeros(8, device="cuda")
    assert capi.lib().xnor_b200_float_conv_small(C.byref(desc), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None) == 6


def test_yolo_activate_matches_elementwise_definition():
    b, anchors, classes, hw = 2, 3, 80, 13 * 13
    x = torch.from_numpy(synth.bell(3, (b, anchors * (5 + classes), 13, 13), 3.0)).cuda()
    out = torch.empty_like(x)
    capi.check(capi.lib().xnor_b200_yolo_activate(x.data_ptr(), out.data_ptr(), b, anchors, classes, hw, None), "yolo")
    torch.cuda.synchronize()
    v = x.reshape(b, anchors, 5 + classes, hw).clone()
    v[:, :, 0:2] = torch.sigmoid(v[:, :, 0:2])
    v[:, :, 4:] = torch.sigmoid(v[:, :, 4:])
    assert torch.equal(out.reshape(v.shape)[:, :, 2:4], x.reshape(v.shape)[:, :, 2:4])
    assert (out.reshape(v.shape) - v).abs().max().item() <= 1e-6


@pytest.mark.parametrize("case", [
    # batch, c, h, w, n, size, leaky
    (1, 256, 13, 13, 512, 3, 1),        # the 3x3 float convolution of yolov3-tiny_xnor (8-way channel split)
    (1, 512, 13, 13, 255, 1, 0),        # yolo head, filter count not a multiple of 32
    (1, 256, 26, 26, 255, 1, 0),        # second head: 4 pixel tiles, the last one ragged
    (2, 64, 26, 26, 40, 3, 1),          # 3x3 on the largest map the kernel stages, two images
    (3, 32, 7, 5, 33, 1, 1),            # single pipeline stage, no split
    (2, 8, 9, 11, 64, 3, 0),            # one stage of 8 channels
    (5, 96, 13, 13, 96, 3, 1),          # channel count that only splits by 4
], ids=lambda c: "b%d_c%d_%dx%d_n%d_k%d_%d" % c)
def test_float_conv_map_matches_fp64_convolution(case):
    batch, c, h, w, n, ks, leaky = case
    pad = ks // 2
    x = torch.from_numpy(synth.bell(sum(case), (batch, c, h, w), 1.0)).cuda()
    wt = torch.from_numpy(synth.bell(sum(case) + 1, (n, c, ks, ks), 0.05)).cuda()
    b = torch.from_numpy(synth.bell(sum(case) + 2, (n,), 0.01)).cuda()
    want = torch.nn.functional.conv2d(x.double(), wt.double(), b.double(), 1, pad)
    if leaky:
        want = torch.where(want > 0, want, want * 0.1)
    desc = capi.ConvDesc(batch, c, h, w, n, ks, 1, pad, capi.LEAKY if leaky else capi.LINEAR)
    lib = capi.lib()
    nbytes = lib.xnor_b200_float_conv_map_weights_bytes(C.byref(desc))
    assert nbytes == ((n + 31) // 32) * 32 * c * ks * ks * 4
    blocked = torch.full((nbytes // 4,), float("nan"), dtype=torch.float32, device="cuda")
    capi.check(lib.xnor_b200_float_conv_map_prepare(C.byref(desc), wt.data_ptr(), blocked.data_ptr(), None), "prepare")
    out = torch.full(want.shape, float("nan"), dtype=torch.float32, device="cuda")
    capi.check(lib.xnor_b200_float_conv_map(C.byref(desc), x.data_ptr(), blocked.data_ptr(), b.data_ptr(), out.data_ptr(), None), "map conv")
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    # fp32 accumulation of c*k*k products of magnitude about 0.05: error grows like sqrt(K) * 2^-24 * |sum|
    tol = 2e-5 * max(1.0, want.abs().max().item())
    assert (out.double() - want).abs().max().item() <= tol
    # deterministic: the cluster reduction adds the partial sums in rank order
    out2 = torch.empty_like(out)
    capi.check(lib.xnor_b200_float_conv_map(C.byref(desc), x.data_ptr(), blocked.data_ptr(), b.data_ptr(), out2.data_ptr(), None), "map conv")
    assert torch.equal(out, out2)


def test_float_conv_map_rejects_other_shapes():
    lib = capi.lib()
    for bad in [capi.ConvDesc(1, 64, 13, 13, 32, 3, 2, 1, capi.LINEAR),      # stride 2
                capi.ConvDesc(1, 60, 13, 13, 32, 3, 1, 1, capi.LINEAR),      # channels not a multiple of 8
                capi.ConvDesc(1, 64, 40, 40, 32, 3, 1, 1, capi.LINEAR),      # map too large to stage
                capi.ConvDesc(1, 48, 13, 13, 32, 1, 1, 0, capi.LINEAR)]:     # 1x1 with channels not a multiple of 32
        assert lib.xnor_b200_float_conv_map_weights_bytes(C.byref(bad)) == 0
        z = torch.zeros(64, device="cuda")
        assert lib.xnor_b200_float_conv_map(C.byref(bad), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None) == 1


def _conv3(desc, pool, x, wt, b, planes=False, masks=False):
    n, h, w = desc.n, desc.h, desc.w
    oh, ow = (h // 2, w // 2) if pool else (h, w)
    if masks:
        out = torch.full((desc.batch, oh, ow, (n + 7) // 8), 0xAA, dtype=torch.uint8, device="cuda")
    elif planes:
        out = torch.full((desc.batch, n, oh, (ow + 31) // 32), -1, dtype=torch.int32, device="cuda")
    else:
        out = torch.full((desc.batch, n, oh, ow), float("nan"), dtype=torch.float32, device="cuda")
    fp32 = not (planes or masks)
    capi.check(capi.lib().xnor_b200_float_conv3_io(C.byref(desc), pool, x.data_ptr(), wt.data_ptr(), b.data_ptr(),
                                                  out.data_ptr() if fp32 else None, out.data_ptr() if planes else None,
                                                  out.data_ptr() if masks else None, None), "conv3_io")
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("case", [
    (2, 40, 56, 16, 1), (1, 34, 18, 32, 0), (1, 66, 130, 20, 1), (1, 416, 416, 16, 1), (3, 8, 70, 8, 1),
], ids=lambda c: "b%d_%dx%d_n%d_%d" % c)
def test_float_conv3_io_equals_small_kernel_and_its_pooled_sign(case):
    """Full-resolution output equals xnor_b200_float_conv_small bit for bit; the pooled output equals max_pool2d of it;
    the sign planes equal the sign of the pooled output, packed along x."""
    batch, h, w, n, leaky = case
    x = torch.from_numpy(synth.bell(sum(case), (batch, 3, h, w), 1.0)).cuda()
    wt = torch.from_numpy(synth.bell(sum(case) + 1, (n, 3, 3, 3), 0.3)).cuda()
    b = torch.from_numpy(synth.bell(sum(case) + 2, (n,), 0.1)).cuda()
    desc = capi.ConvDesc(batch, 3, h, w, n, 3, 1, 1, capi.LEAKY if leaky else capi.LINEAR)
    ref = torch.empty(batch, n, h, w, device="cuda")
    capi.check(capi.lib().xnor_b200_float_conv_small(C.byref(desc), x.data_ptr(), wt.data_ptr(), b.data_ptr(), ref.data_ptr(), None), "small")
    full = _conv3(desc, 0, x, wt, b)
    assert torch.equal(full, ref)
    pooled = _conv3(desc, 2, x, wt, b)
    want = torch.nn.functional.max_pool2d(ref, 2, 2)
    assert torch.equal(pooled, want)
    planes = _conv3(desc, 2, x, wt, b, planes=True).cpu().numpy().view(np.uint32)
    pos = (want > 0).cpu().numpy()
    ow = w // 2
    padded = np.zeros(pos.shape[:3] + (((ow + 31) // 32) * 32,), dtype=bool)
    padded[..., :ow] = pos
    bits = padded.reshape(pos.shape[:3] + (-1, 32))
    words = (bits.astype(np.uint64) << np.arange(32, dtype=np.uint64)).sum(-1).astype(np.uint32)
    assert np.array_equal(planes, words)
    masks = _conv3(desc, 2, x, wt, b, masks=True).cpu().numpy()                  # [batch][h/2][w/2][ceil(n/8)]
    nb = (n + 7) // 8
    chan = np.zeros((batch, h // 2, ow, nb * 8), dtype=np.uint8)
    chan[..., :n] = np.moveaxis(pos, 1, -1)
    want_masks = (chan.reshape(batch, h // 2, ow, nb, 8) << np.arange(8, dtype=np.uint8)).sum(-1).astype(np.uint8)
    assert np.array_equal(masks, want_masks)


def test_float_conv3_planes_feed_the_bit_path_xnor_layer():
    """conv 3->16 + maxpool + xnor conv 16->32: the xnor layer fed the sign planes gives the bits it gives on the fp32 tensor."""
    from darknet_b200 import layer as L
    batch, h, w = 2, 36, 76
    x = torch.from_numpy(synth.bell(5, (batch, 3, h, w), 1.0)).cuda()
    wt = torch.from_numpy(synth.bell(6, (16, 3, 3, 3), 0.3)).cuda()
    b = torch.from_numpy(synth.bell(7, (16,), 0.1)).cuda()
    desc = capi.ConvDesc(batch, 3, h, w, 16, 3, 1, 1, capi.LEAKY)
    pooled = _conv3(desc, 2, x, wt, b)
    planes = _conv3(desc, 2, x, wt, b, planes=True)
    masks = _conv3(desc, 2, x, wt, b, masks=True)
    for stride in (1, 2):
        l = L.make_convolutional_layer(batch, h // 2, w // 2, 16, 32, 3, stride, 1, capi.LEAKY)
        l.load_weights(torch.from_numpy(synth.bell(8, (32, 16 * 9), 0.05)).cuda(), torch.from_numpy(synth.bell(9, (32,), 0.01)).cuda())
        L.binary_align_weights(l)
        want = L.forward_convolutional_layer_gpu(l, pooled).clone()
        got = L.forward_convolutional_layer_io(l, x_signs=planes).clone()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        if stride == 1:
            assert L.conv_takes_masks(l)
            assert torch.equal(L.forward_convolutional_layer_io(l, x_masks=masks), want)
        else:
            assert not L.conv_takes_masks(l)


def test_float_conv3_io_argument_checks():
    lib = capi.lib()
    z = torch.zeros(4096, device="cuda")
    ok = capi.ConvDesc(1, 3, 8, 8, 8, 3, 1, 1, capi.LINEAR)
    odd = capi.ConvDesc(1, 3, 9, 8, 8, 3, 1, 1, capi.LINEAR)
    four = capi.ConvDesc(1, 4, 8, 8, 8, 3, 1, 1, capi.LINEAR)
    assert lib.xnor_b200_float_conv3_io(C.byref(ok), 0, z.data_ptr(), z.data_ptr(), z.data_ptr(), None, None, None, None) == 2        # no output
    assert lib.xnor_b200_float_conv3_io(C.byref(ok), 0, z.data_ptr(), z.data_ptr(), z.data_ptr(), None, z.data_ptr(), None, None) == 1  # planes need the pool
    assert lib.xnor_b200_float_conv3_io(C.byref(ok), 2, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None, None) == 2  # two outputs
    assert lib.xnor_b200_float_conv3_io(C.byref(odd), 2, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None, None, None) == 1  # odd height
    assert lib.xnor_b200_float_conv3_io(C.byref(four), 0, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None, None, None) == 1
    assert lib.xnor_b200_float_conv3_io(C.byref(ok), 3, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None, None, None) == 1


def test_float_conv_map_yolo_equals_conv_then_yolo_activate():
    batch, c, h, w, classes = 2, 64, 13, 13, 80
    n = 3 * (5 + classes)
    x = torch.from_numpy(synth.bell(71, (batch, c, h, w), 1.0)).cuda()
    wt = torch.from_numpy(synth.bell(72, (n, c, 1, 1), 0.2)).cuda()
    b = torch.from_numpy(synth.bell(73, (n,), 0.5)).cuda()
    desc = capi.ConvDesc(batch, c, h, w, n, 1, 1, 0, capi.LINEAR)
    lib = capi.lib()
    blocked = torch.empty(lib.xnor_b200_float_conv_map_weights_bytes(C.byref(desc)) // 4, device="cuda")
    capi.check(lib.xnor_b200_float_conv_map_prepare(C.byref(desc), wt.data_ptr(), blocked.data_ptr(), None), "prepare")
    raw = torch.empty(batch, n, h, w, device="cuda")
    capi.check(lib.xnor_b200_float_conv_map(C.byref(desc), x.data_ptr(), blocked.data_ptr(), b.data_ptr(), raw.data_ptr(), None), "map")
    want = torch.empty_like(raw)
    capi.check(lib.xnor_b200_yolo_activate(raw.data_ptr(), want.data_ptr(), batch, 3, classes, h * w, None), "yolo")
    got = torch.empty_like(raw)
    capi.check(lib.xnor_b200_float_conv_map_yolo(C.byref(desc), x.data_ptr(), blocked.data_ptr(), b.data_ptr(), got.data_ptr(), 5 + classes, None), "map yolo")
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert lib.xnor_b200_float_conv_map_yolo(C.byref(desc), x.data_ptr(), blocked.data_ptr(), b.data_ptr(), got.data_ptr(), 7, None) == 1


@pytest.mark.parametrize("case", [(2, 5, 4, 80, 1, 169), (3, 5, 4, 20, 1, 49), (1, 3, 4, 7, 0, 33), (2, 2, 6, 0, 1, 10)],
                         ids=lambda c: "b%d_a%d_coords%d_cls%d_sm%d_hw%d" % c)
def test_region_activate_matches_its_definition(case):
    """[region] head in one kernel against the same steps written with torch (logistic x, y, objectness; softmax over classes)."""
    batch, anchors, coords, classes, softmax, hw = case
    entries = coords + 1 + classes
    x = torch.from_numpy(synth.bell(91, (batch, anchors * entries, hw), 2.0)).cuda()
    out = torch.full_like(x, float("nan"))
    capi.check(capi.lib().xnor_b200_region_activate(x.data_ptr(), out.data_ptr(), batch, anchors, coords, classes, softmax, hw, None), "region")
    torch.cuda.synchronize()
    v = x.reshape(batch, anchors, entries, hw).double().clone()
    v[:, :, 0:2] = torch.sigmoid(v[:, :, 0:2])
    v[:, :, coords] = torch.sigmoid(v[:, :, coords])
    if softmax and classes > 0:
        v[:, :, coords + 1:] = torch.softmax(v[:, :, coords + 1:], dim=2)
    got = out.reshape(batch, anchors, entries, hw).double()
    assert torch.equal(got[:, :, 2:coords], v[:, :, 2:coords])                 # w, h (and further coords) untouched
    assert (got - v).abs().max().item() < 2e-6
    assert capi.lib().xnor_b200_region_activate(x.data_ptr(), x.data_ptr(), batch, anchors, coords, classes, softmax, hw, None) == 1   # in place: refused


@pytest.mark.parametrize("case", [(2, 33, 47, 32, 1), (1, 64, 64, 32, 0), (1, 20, 30, 20, 1)], ids=lambda c: "b%d_%dx%d_n%d_%d" % c)
def test_float_conv3_unpooled_masks_are_the_sign_words_of_the_output(case):
    """pool = 0 with output_sign_masks: byte f/8, bit f%8 of pixel (y, x) = (output of filter f > 0), odd sizes included;
    with 32 filters the tensor is the sign-word input of an xnor layer over those channels (here the stride-2 3x3 layer
    that follows darknet53's first convolution), which then gives the same output as from the fp32 tensor."""
    batch, h, w, n, leaky = case
    x = torch.from_numpy(synth.bell(sum(case) + 5, (batch, 3, h, w), 1.0)).cuda()
    wt = torch.from_numpy(synth.bell(sum(case) + 6, (n, 3, 3, 3), 0.3)).cuda()
    b = torch.from_numpy(synth.bell(sum(case) + 7, (n,), 0.1)).cuda()
    desc = capi.ConvDesc(batch, 3, h, w, n, 3, 1, 1, capi.LEAKY if leaky else capi.LINEAR)
    full = _conv3(desc, 0, x, wt, b)
    masks = _conv3(desc, 0, x, wt, b, masks=True)
    nb = (n + 7) // 8
    bits = torch.zeros(batch, nb * 8, h, w, dtype=torch.bool, device="cuda")
    bits[:, :n] = full > 0
    weights8 = (2 ** torch.arange(8, device="cuda")).view(1, 1, 8, 1, 1)
    want = (bits.view(batch, nb, 8, h, w) * weights8).sum(2).permute(0, 2, 3, 1).to(torch.uint8)
    assert torch.equal(masks, want)
    if n == 32:
        l = L.make_convolutional_layer(batch, h, w, 32, 64, 3, 2, 1, capi.LEAKY)
        l.load_weights(torch.from_numpy(synth.bell(3, (64, 32 * 9), 0.05)).cuda(), torch.from_numpy(synth.bell(4, (64,), 0.3)).cuda())
        L.binary_align_weights(l)
        ref = L.forward_convolutional_layer_gpu(l, full).clone()
        words = masks.view(torch.int32).reshape(batch, 1, h * w)
        assert torch.equal(L.forward_convolutional_layer_io(l, x_signs=words), ref)


@pytest.mark.parametrize("case", [
    (4, 256, 13, 13, 255, 0),      # yolo head shape, filters not a multiple of the tile, pixels not a multiple of 128
    (2, 1024, 13, 13, 425, 0),     # region head of tiny-yolo
    (3, 64, 10, 7, 130, 1),        # two K blocks, a tile that straddles three images, leaky
    (1, 50, 9, 9, 20, 1),          # channels neither a multiple of 32 nor of 4: scalar weight loads, zero-filled K tail
    (16, 512, 26, 26, 255, 0),     # 10816 pixels: many tiles per SM
], ids=lambda c: "b%d_c%d_%dx%d_n%d_%d" % c)
def test_float_conv_1x1_tc_matches_fp64_convolution(case):
    """The tensor-core 1x1 convolution (three tf32 products per operand pair) against an fp64 convolution."""
    batch, c, h, w, n, leaky = case
    x = torch.from_numpy(synth.bell(sum(case), (batch, c, h, w))).cuda()
    wt = torch.from_numpy(synth.bell(sum(case) + 1, (n, c, 1, 1), 0.05)).cuda()
    b = torch.from_numpy(synth.bell(sum(case) + 2, (n,), 0.01)).cuda()
    want = torch.nn.functional.conv2d(x.double(), wt.double(), b.double())
    if leaky:
        want = torch.where(want > 0, want, want * 0.1)
    desc = capi.ConvDesc(batch, c, h, w, n, 1, 1, 0, capi.LEAKY if leaky else capi.LINEAR)
    out = torch.full(want.shape, float("nan"), dtype=torch.float32, device="cuda")
    capi.check(capi.lib().xnor_b200_float_conv_1x1_tc(C.byref(desc), x.data_ptr(), wt.data_ptr(), b.data_ptr(), out.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream), "xnor_b200_float_conv_1x1_tc")
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    # sums of c products of magnitude ~0.05: |result| ~ 0.05 sqrt(c).  The tensor core's fp32 accumulation does not round to
    # nearest, so the error grows with the number of accumulating instructions (12 per 32 channels, spread over four
    # accumulators): 1e-5 + 4e-8 per channel covers it; a single tf32 product per pair would be off by ~1e-3.
    err = (out.double() - want).abs().max().item()
    assert err <= 1e-5 + 4e-8 * c, err
    st = C.c_int(-1)
    capi.check(capi.lib().xnor_b200_take_device_status(C.byref(st)), "xnor_b200_take_device_status")
    assert st.value == 0


def test_float_conv_1x1_tc_rejects_other_shapes():
    z = torch.zeros(64, device="cuda")
    desc = capi.ConvDesc(1, 32, 8, 8, 8, 3, 1, 1, capi.LINEAR)
    assert capi.lib().xnor_b200_float_conv_1x1_tc(C.byref(desc), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None) == 1
    desc = capi.ConvDesc(1, 32, 8, 8, 8, 1, 1, 0, capi.LINEAR)
    assert capi.lib().xnor_b200_float_conv_1x1_tc(C.byref(desc), None, z.data_ptr(), z.data_ptr(), z.data_ptr(), None) == 2
