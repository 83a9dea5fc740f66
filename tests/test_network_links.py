"""The graph passes of the runner that decide which layers hand sign bits to which (no GPU needed: the passes only
look at the parsed layer list; the xnor layer objects are stand-ins)."""
import types

import pytest

torch = pytest.importorskip("torch")

from darknet_b200 import cfgs, network  # noqa: E402


def linked(name, batch, tmp_path):
    cfg = tmp_path / "net.cfg"
    cfg.write_text(cfgs.CFGS[name]())
    net = network.parse_network_cfg(str(cfg), batch, "cpu")
    for l in net.layers:
        if l.type == "convolutional" and l.xnor:
            l.xnor_layer = types.SimpleNamespace(window_major=False)
            if l.use_bin_output:
                l.activation = "linear"
    network.link_branches(net)
    network.link_sinks(net)
    network.link_sign_chains(net)
    return net


def test_readers_follow_routes_and_shortcuts(tmp_path):
    net = linked("yolov3-tiny_xnor", 1, tmp_path)
    readers = network._readers(net)
    assert readers[8] == [9, 20]            # maxpool behind it and the route that concatenates it
    assert readers[13] == [14, 17]          # the float conv and the single-input route
    assert readers[16] == [] and readers[23] == []
    assert readers[19] == [20] and readers[20] == [21]


def test_yolov3_tiny_links(tmp_path):
    net = linked("yolov3-tiny_xnor", 1, tmp_path)
    L = net.layers
    # 2->4, 4->6, 6->8, 8->10 through 2x2/2 maxpools; 12->13; 13->18 through a route; 18->21 through upsample + route; 8->21
    assert net.sink_links == 8
    assert [l.index for l in L if l.packed_input] == [4, 6, 8, 10, 13, 18, 21]
    assert [l.index for l in L if l.skip] == [3, 5, 7, 9, 17, 19, 20]
    assert [(s.pool, s.upsample, s.channel_offset) for s in L[8].sinks] == [(2, 0, 0), (0, 0, 128)]
    assert [(s.pool, s.upsample, s.channel_offset) for s in L[18].sinks] == [(0, 2, 0)]
    assert all(L[i].xnor_layer.window_major for i in (2, 4, 6, 8)) and not L[10].xnor_layer.window_major
    assert not L[8].need_fp32 and L[13].need_fp32 and not L[18].need_fp32 and L[21].need_fp32
    # the stride-1 maxpool between 10 and 12 is not a sink: that pair hands over sign words, pooled in the pack kernel
    assert L[10].emit_signs and L[12].sign_source == 10 and L[12].pool_desc is not None and L[11].folded
    assert not L[12].packed_input and [s.consumer for s in L[12].sinks] == [L[13].xnor_layer]
    # head branch 14..16 hangs off layer 13 only
    assert L[14].branch_start and L[16].branch_end
    assert sum(l.branch_start for l in L) == 1


def test_sink_threshold_and_switches(tmp_path):
    cfg = tmp_path / "net.cfg"
    cfg.write_text(cfgs.CFGS["yolov3-tiny_xnor"]())
    net = network.parse_network_cfg(str(cfg), 4, "cpu")
    for l in net.layers:
        if l.type == "convolutional" and l.xnor:
            l.xnor_layer = types.SimpleNamespace(window_major=False)
    net.sink_max_batch = 2
    net.side_branches = False
    network.link_branches(net)
    network.link_sinks(net)
    network.link_sign_chains(net)
    assert net.sink_links == 0 and not any(l.skip or l.packed_input or l.branch_start for l in net.layers)
    assert net.sign_links >= 4                      # the older hand-over (sign words + pooled pack) takes over


@pytest.mark.parametrize("name", ["tiny-yolo_xnor", "darknet53_448_xnor"])
def test_other_networks_link_consistently(name, tmp_path):
    net = linked(name, 1, tmp_path)
    L = net.layers
    assert net.sink_links > 0
    for l in L:
        if l.packed_input:
            assert l.type == "convolutional" and l.xnor and l.c % 32 == 0 and l.stride == 1
        for s in l.sinks:
            assert l.n % 32 == 0 and s.pool in (0, 2) and s.upsample in (0, 2)
            if s.pool == 2:
                assert l.xnor_layer.window_major and l.out_h % 2 == 0 and l.out_w % 2 == 0
        if l.skip:
            assert l.type in ("maxpool", "upsample", "route") and not l.need_fp32
        assert len(l.sinks) <= 2
    # every packed consumer gets all of its channels from sinks
    for c in L:
        if c.packed_input:
            got = sum(p.n for p in L for s in p.sinks if s.consumer is c.xnor_layer)
            assert got == c.c


def test_shortcut_sum_reader_that_pools_takes_words_not_rows(tmp_path):
    """conv + fused [shortcut] -> 1x1 xnor conv -> 2x2/2 maxpool -> xnor conv: link_sinks makes the 1x1 layer window-major
    (it feeds a pooled sink), so the sum's signs must reach it as words through its pack kernel; writing them straight
    into its operand would put row-major rows under a window-major GEMM."""
    text = "\n".join([
        "[net]\nbatch=1\nwidth=32\nheight=32\nchannels=3\n",
        cfgs._conv(32, 3),
        cfgs._conv(64, 3, xnor=1),
        cfgs._conv(64, 3, xnor=1),
        "[shortcut]\nfrom=-2\nactivation=linear\n",
        cfgs._conv(64, 1, xnor=1),
        cfgs._maxpool(2, 2),
        cfgs._conv(64, 3, xnor=1),
        # same block without the pool: the reader stays row-major and takes the signs straight into its operand
        cfgs._conv(64, 3, xnor=1),
        "[shortcut]\nfrom=-2\nactivation=linear\n",
        cfgs._conv(64, 1, xnor=1),
        cfgs._conv(32, 1, bn=0, activation="linear"),
    ])
    cfg = tmp_path / "net.cfg"
    cfg.write_text(text)
    net = network.parse_network_cfg(str(cfg), 4, "cpu")
    for l in net.layers:
        if l.type == "convolutional" and l.xnor:
            l.xnor_layer = types.SimpleNamespace(window_major=False)
    net.layers[3].blank = True
    net.layers[8].blank = True
    network.link_sinks(net)
    network.link_sign_chains(net)
    network.link_shortcut_sums(net)
    L = net.layers
    assert L[4].xnor_layer.window_major and L[6].packed_input            # 4 -> (maxpool 5) -> 6 is a pooled sink
    assert L[2].emit_sum_signs and L[2].sum_sink_to is None and L[4].sign_source == 3 and not L[4].packed_input
    assert L[7].sum_sink_to == 9 and L[9].packed_input and not L[9].xnor_layer.window_major
    assert net.sum_sign_links == 2
