"""[maxpool] folded into the next xnor layer's pack kernel: same bits and outputs as pooling first.

The oracle side pools with a plain restatement of Darknet's maxpool (window origin -pad/2, out-of-image elements
ignored, src-lib/maxpool_layer_kernels.cu:48-86) and then runs the ordinary xnor oracle on the pooled tensor."""
import numpy as np
import pytest

import synth
from oracle.binding import new_lda

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, layer as L  # noqa: E402


def darknet_maxpool(x, size, stride, pad):
    b, c, h, w = x.shape
    oh, ow = (h + pad - size) // stride + 1, (w + pad - size) // stride + 1
    out = np.full((b, c, oh, ow), -np.inf, np.float32)
    off = -(pad // 2)
    for i in range(oh):
        for j in range(ow):
            for l in range(size):
                for m in range(size):
                    yy, xx = off + i * stride + l, off + j * stride + m
                    if 0 <= yy < h and 0 <= xx < w:
                        out[:, :, i, j] = np.maximum(out[:, :, i, j], x[:, :, yy, xx])
    return out


CASES = [
    # batch, c, in_h, in_w, pool size, stride, pad, n, ks, conv stride, conv pad, leaky
    (2, 16, 24, 24, 2, 2, 1, 32, 3, 1, 1, 0),      # bit path behind a 2x2/2 pool (first xnor layer of the tiny nets)
    (2, 64, 20, 20, 2, 2, 1, 48, 3, 1, 1, 1),      # word path, 2x2/2
    (1, 512, 13, 13, 2, 1, 1, 64, 3, 1, 1, 0),     # the stride-1 pool of the tiny nets (window clipped at the right/bottom edge)
    (2, 32, 17, 15, 3, 2, 2, 16, 3, 1, 1, 1),      # odd sizes, 3x3/2 pool with padding 2 (window starts at -1)
    (1, 75, 14, 14, 2, 2, 1, 24, 3, 1, 1, 1),      # bit path, K = 675
    (1, 64, 16, 16, 2, 2, 1, 16, 1, 1, 0, 1),      # 1x1 convolution behind the pool
    (1, 40, 12, 12, 2, 2, 1, 8, 3, 2, 1, 0),       # bit path with a strided convolution (generic bit kernel)
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "b%d_c%d_%dx%d_pool%d_%d_%d_n%d_k%d_s%d_p%d_%d" % c)
def test_pooled_pack_and_forward_match_pool_then_oracle(port, case):
    batch, c, ih, iw, ps, pst, ppad, n, ks, stride, pad, leaky = case
    x, wt, b = synth.conv_case(sum(case), batch, c, ih, iw, n, ks)
    x[0, 0, 0, :4] = [0.0, -0.0, np.nan, -1.0]           # a window without any positive element
    pooled = darknet_maxpool(np.nan_to_num(x, nan=-1.0), ps, pst, ppad)
    h, w = pooled.shape[2:]
    want_out, want_tb, _ = port.conv_forward(pooled, wt, b, stride, pad, leaky, dumps=True)
    l = L.make_convolutional_layer(batch, h, w, c, n, ks, stride, pad, capi.LEAKY if leaky else capi.LINEAR)
    l.load_weights(torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda())
    L.binary_align_weights(l)
    pool = capi.PoolDesc(ps, pst, ppad, ih, iw)
    xg = torch.from_numpy(x).cuda()
    tb = L.pack_input_pooled(l, pool, xg).cpu().numpy()
    K = c * ks * ks
    assert np.array_equal(tb.reshape(batch, -1, new_lda(K) // 8), want_tb), "packed bits differ from pool-then-pack"
    y = L.forward_convolutional_layer_gpu(l, xg, pool).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), want_out.view(np.uint32))
    # and the unfused route through the same library gives the same bits
    tb2 = L.pack_input(l, torch.from_numpy(pooled).cuda()).cpu().numpy()
    assert np.array_equal(tb, tb2)


def test_pooled_descriptor_must_match_the_convolution_input():
    l = L.make_convolutional_layer(1, 10, 10, 32, 8, 3, 1, 1, capi.LINEAR)
    L.binary_align_weights(l)
    bad = capi.PoolDesc(2, 2, 1, 24, 24)                 # pools to 12x12, the layer expects 10x10
    x = torch.zeros(1, 32, 24, 24, device="cuda")
    with pytest.raises(capi.XnorError, match="invalid"):
        L.pack_input_pooled(l, bad, x)


def test_network_with_folded_maxpools_equals_unfolded(tmp_path):
    """yolov3-tiny_xnor at a reduced input size: folding the maxpools changes no output bit."""
    from darknet_b200 import cfgs, network
    cfg = tmp_path / "net.cfg"
    cfg.write_text(cfgs.yolov3_tiny_xnor_cfg(96, 96))
    net_cpu = network.parse_network_cfg(str(cfg), 2, "cpu")
    w = tmp_path / "net.weights"
    network.write_synthetic_weights(net_cpu, str(w), seed=5)
    x = torch.from_numpy(synth.uniform01(9, (2, 3, 96, 96))).cuda()
    net = network.load_network_custom(str(cfg), str(w), 2, sign_chains=False, fuse_first_conv=False)
    assert net.folded_maxpools == 0                     # below the batch threshold nothing is folded by default
    net.fold_maxpool_min_batch = 1
    network.fold_maxpools(net)
    assert net.folded_maxpools == 5                     # the five 2x2/stride-2 pools; the stride-1 pool stays a layer
    heads_folded = [h.clone() for h in network.forward_network_gpu(net, x)]
    for l in net.layers:
        l.folded = False
        l.pool_desc = None
    heads_plain = network.forward_network_gpu(net, x)
    assert len(heads_folded) == 2
    for a, b in zip(heads_folded, heads_plain):
        assert torch.equal(a, b)
