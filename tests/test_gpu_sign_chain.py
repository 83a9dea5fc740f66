"""Chains of xnor layers that hand over sign bits instead of fp32 tensors (xnor_b200_conv_forward_io).

Layer 1 writes only the sign of its output (1 bit per value, 32 filters per word); layer 2 packs its operand from
those words, ORing them over a max-pool window when a [maxpool] sits in between.  Every result of layer 2 must be
bit-identical to the ordinary route (fp32 output -> maxpool -> pack), for both GEMM kernels."""
import os

import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import torch.nn.functional as F  # noqa: E402

from darknet_b200 import capi, layer as L  # noqa: E402


def build(batch, c, h, w, n, ks, leaky, seed):
    x, wt, b = synth.conv_case(seed, batch, c, h, w, n, ks)
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, 1, ks // 2, capi.LEAKY if leaky else capi.LINEAR)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    return l, torch.from_numpy(x).cuda()


@pytest.mark.parametrize("tc", ["0", "1"])
@pytest.mark.parametrize("case", [
    # batch, c1, h, w, n1 (= c2), n2, pool (size, stride, pad) or None
    (2, 32, 16, 16, 64, 48, (2, 2, 1)),
    (1, 64, 26, 26, 128, 40, None),
    (2, 16, 24, 24, 32, 24, (2, 2, 1)),          # layer 1 on the bit path (16 channels)
    (1, 96, 13, 13, 256, 64, (2, 1, 1)),         # stride-1 pool, window clipped at the edge
    (3, 64, 12, 10, 96, 33, (3, 2, 2)),
], ids=lambda c: "b%d_c%d_%dx%d_n%d_n%d_%s" % c)
def test_sign_chain_equals_fp32_chain(case, tc):
    batch, c1, h, w, n1, n2, pool = case
    capi.set_tuning(gemm_route=capi.ROUTE_TENSOR if tc == "1" else capi.ROUTE_TILED)
    try:
        l1, x = build(batch, c1, h, w, n1, 3, 0, 31 + c1)
        y1 = L.forward_convolutional_layer_gpu(l1, x).clone()
        signs = L.forward_convolutional_layer_io(l1, x=x, want_signs=True)
        # the sign words are the channel-packed signs of the fp32 output
        bits = (y1 > 0).reshape(batch, n1 // 32, 32, h * w).to(torch.int64)
        want_words = (bits << torch.arange(32, device="cuda").view(1, 1, 32, 1)).sum(2)
        assert torch.equal(signs.to(torch.int64) & 0xFFFFFFFF, want_words)

        if pool is None:
            h2, w2, pd, mid = h, w, None, y1
        else:
            ps, pst, pp = pool
            h2, w2 = (h + pp - ps) // pst + 1, (w + pp - ps) // pst + 1
            pd = capi.PoolDesc(ps, pst, pp, h, w)
            lo = pp // 2
            padded = F.pad(y1, (lo, max((w2 - 1) * pst + ps - lo - w, 0), lo, max((h2 - 1) * pst + ps - lo - h, 0)), value=float("-inf"))
            mid = F.max_pool2d(padded, ps, pst)[:, :, :h2, :w2].contiguous()
        l2, _ = build(batch, n1, h2, w2, n2, 3, 1, 77 + n1)
        want = L.forward_convolutional_layer_gpu(l2, mid).clone()
        got = L.forward_convolutional_layer_io(l2, x_signs=signs, pool=pd).clone()
        assert torch.equal(got, want)
    finally:
        capi.set_tuning()


def test_io_argument_checks():
    l, x = build(1, 32, 8, 8, 40, 3, 0, 5)               # 40 filters: not a multiple of 32
    with pytest.raises(capi.XnorError, match="invalid"):
        L.forward_convolutional_layer_io(l, x=x, want_signs=True)
    with pytest.raises(capi.XnorError, match="NULL"):
        L.forward_convolutional_layer_io(l)              # neither kind of input


@pytest.mark.parametrize("batch", [1, 4])
def test_network_with_sign_chains_equals_fp32_network(tmp_path, batch):
    """yolov3-tiny_xnor at a reduced input size: handing sign bits from one xnor layer to the next (with the
    maxpool between them turned into an OR) changes no bit of either head."""
    from darknet_b200 import cfgs, network
    cfg = tmp_path / "net.cfg"
    cfg.write_text(cfgs.yolov3_tiny_xnor_cfg(96, 96))
    net_cpu = network.parse_network_cfg(str(cfg), batch, "cpu")
    w = tmp_path / "net.weights"
    network.write_synthetic_weights(net_cpu, str(w), seed=5)
    x = torch.from_numpy(synth.uniform01(9, (batch, 3, 96, 96))).cuda()
    linked = network.load_network_custom(str(cfg), str(w), batch)
    plain = network.load_network_custom(str(cfg), str(w), batch, sign_chains=False, fuse_first_conv=False, side_branches=False)
    assert linked.layers[14].branch_start and linked.layers[16].branch_end and not plain.layers[14].branch_start
    assert plain.sign_links == 0 and plain.sink_links == 0
    if batch <= linked.sink_max_batch:
        # 2->4, 4->6, 6->8, 8->10 through maxpools, 12->13 directly, 13->18 through a route, 18->21 through upsample+route, 8->21 through the route
        assert linked.sink_links == 8 and linked.sign_links >= 2
        assert [l.index for l in linked.layers if l.skip] == [3, 5, 7, 9, 17, 19, 20]
        assert not linked.layers[8].need_fp32 and linked.layers[13].need_fp32
    else:
        assert linked.sink_links == 0 and linked.sign_links >= 4
    assert (linked.layers[0].emit_planes or linked.layers[0].emit_masks) and linked.layers[0].conv3_pool == 2
    got = network.forward_network_gpu(linked, x)
    want = network.forward_network_gpu(plain, x)
    assert len(got) == len(want) == 2
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_heads_written_to_pinned_host_memory(tmp_path):
    """forward_network_gpu(heads_host=...): the fused head convolutions store into the pinned host tensors themselves;
    what arrives there equals the device heads of a plain forward."""
    from darknet_b200 import cfgs, network
    cfg = tmp_path / "net.cfg"
    cfg.write_text(cfgs.yolov3_tiny_xnor_cfg(96, 96))
    net_cpu = network.parse_network_cfg(str(cfg), 1, "cpu")
    w = tmp_path / "net.weights"
    network.write_synthetic_weights(net_cpu, str(w), seed=5)
    x = torch.from_numpy(synth.uniform01(9, (1, 3, 96, 96))).cuda()
    net = network.load_network_custom(str(cfg), str(w), 1)
    want = [h.clone() for h in network.forward_network_gpu(net, x)]
    host = [torch.full(h.shape, float("nan")).pin_memory() for h in want]
    got = network.forward_network_gpu(net, x, host)
    torch.cuda.synchronize()
    assert all(g is h for g, h in zip(got, host))          # the returned heads are the host tensors
    for h, d in zip(host, want):
        assert torch.equal(h, d.cpu())
    net.heads_direct_to_host = False                        # the copy route gives the same
    host2 = [torch.full(h.shape, float("nan")).pin_memory() for h in want]
    network.forward_network_gpu(net, x, host2)
    torch.cuda.synchronize()
    for h, d in zip(host2, want):
        assert torch.equal(h, d.cpu())


@pytest.mark.parametrize("name,size,batch", [
    ("yolov3-tiny_xnor", 416, 1),          # the bench workload at its full size
    ("yolov3-tiny_xnor", 416, 8),          # tensor-core kernels with sinks
    ("tiny-yolo_xnor", 416, 2),
    ("darknet53_448_xnor", 224, 1),        # shortcuts, stride-2 xnor layers, softmax head
    ("darknet53_448_xnor", 128, 4),
    ("darknet53_448_xnor", 96, 8),         # from batch 4: the signs of the fused shortcut sums feed the next xnor layers
])
def test_linked_networks_equal_plain_networks_at_full_size(tmp_path, name, size, batch):
    """Every fusion the runner sets up (sinks, sign words, masks, folded pools, fused first conv, side branch, fused head
    activation) against the same network with all of them switched off: identical heads, bit for bit."""
    from darknet_b200 import cfgs, network
    cfg = tmp_path / "net.cfg"
    cfg.write_text(cfgs.CFGS[name](size, size))
    net_cpu = network.parse_network_cfg(str(cfg), batch, "cpu")
    w = tmp_path / "net.weights"
    network.write_synthetic_weights(net_cpu, str(w), seed=3)
    x = torch.from_numpy(synth.uniform01(13, (batch, 3, size, size))).cuda()
    linked = network.load_network_custom(str(cfg), str(w), batch)
    plain = network.load_network_custom(str(cfg), str(w), batch, sign_chains=False, fuse_first_conv=False, side_branches=False)
    assert linked.sink_links > 0 and plain.sink_links == 0
    if name.startswith("darknet53"):
        assert (linked.sum_sign_links > 0) == (batch >= 4) and plain.sum_sign_links == 0
    got = [h.clone() for h in network.forward_network_gpu(linked, x)]
    want = network.forward_network_gpu(plain, x)
    torch.cuda.synchronize()
    assert len(got) == len(want) > 0
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    # a second forward through the same buffers gives the same again (no state left behind by sinks or masks)
    again = network.forward_network_gpu(linked, x)
    torch.cuda.synchronize()
    for a, b in zip(again, want):
        assert torch.equal(a, b)
