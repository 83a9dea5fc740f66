"""The packed-weight cache beside a .weights file (the counterpart of Darknet's dormant bit-packed writer,
src-lib/weights.cpp:70-116): file format round trip and rejection rules on CPU; on the GPU a load from the cache holds
byte-identical packed weights and gives a bit-identical forward."""
import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")

from darknet_b200 import cfgs, network  # noqa: E402


def entry(index, c, n, size, seed):
    k = c * size * size
    new_lda = k + (256 - k % 256)
    rng = np.random.default_rng(seed)
    return dict(index=index, c=c, n=n, size=size, stride=1, pad=size // 2, new_lda=new_lda, crc=int(rng.integers(0, 2 ** 32)),
                bits=rng.integers(0, 256, n * new_lda // 8, dtype=np.uint8), mean=rng.random(n, dtype=np.float32))


def test_cache_file_round_trip_and_rejections(tmp_path):
    path = str(tmp_path / "net.weights.xnorpack")
    want = [entry(2, 16, 32, 3, 1), entry(4, 32, 64, 3, 2), entry(13, 1024, 256, 1, 3)]
    network.write_packed_cache(path, want)
    got = network.read_packed_cache(path)
    assert sorted(got) == [2, 4, 13]
    for e in want:
        g = got[e["index"]]
        assert all(g[k] == e[k] for k in ("c", "n", "size", "stride", "pad", "new_lda", "crc"))
        assert np.array_equal(g["bits"], e["bits"]) and np.array_equal(g["mean"].view(np.uint32), e["mean"].view(np.uint32))
    data = bytearray(open(path, "rb").read())
    # one flipped bit anywhere, a truncated file, a foreign file: all refused
    damaged = bytearray(data)
    damaged[len(damaged) // 2] ^= 0x10
    open(path, "wb").write(damaged)
    with pytest.raises(ValueError):
        network.read_packed_cache(path)
    open(path, "wb").write(data[:len(data) - 9])
    with pytest.raises(ValueError):
        network.read_packed_cache(path)
    open(path, "wb").write(b"not a cache file at all, just bytes")
    with pytest.raises(ValueError):
        network.read_packed_cache(path)
    with pytest.raises(ValueError):
        network.write_packed_cache(path, [dict(want[0], bits=want[0]["bits"][:-1])])


def test_entry_is_keyed_by_geometry_and_weights(tmp_path):
    cfg = tmp_path / "net.cfg"
    cfg.write_text(cfgs.yolov3_tiny_xnor_cfg(96, 96))
    net = network.parse_network_cfg(str(cfg), 1, "cpu")
    w = tmp_path / "net.weights"
    network.write_synthetic_weights(net, str(w), seed=4)
    network.load_weights(net, str(w))
    network.fuse_conv_batchnorm(net)
    l = net.layers[4]
    k = l.c * l.size * l.size
    new_lda = k + (256 - k % 256)
    e = dict(index=4, c=l.c, n=l.n, size=l.size, stride=l.stride, pad=l.pad, new_lda=new_lda, crc=network.weights_crc(l), bits=None, mean=None)
    assert network.cache_entry_matches(e, l, new_lda)
    assert not network.cache_entry_matches(None, l, new_lda)
    assert not network.cache_entry_matches(dict(e, n=l.n + 1), l, new_lda)
    assert not network.cache_entry_matches(dict(e, new_lda=new_lda + 256), l, new_lda)
    l.weights = l.weights.copy()
    l.weights[3, 1, 0, 2] = np.nextafter(l.weights[3, 1, 0, 2], np.float32(1))        # retrained by one ulp: stale
    assert not network.cache_entry_matches(e, l, new_lda)


@pytest.mark.gpu
@pytest.mark.parametrize("name,size", [("yolov3-tiny_xnor", 160), ("darknet53_448_xnor", 96)])
def test_load_from_cache_is_byte_identical(tmp_path, name, size):
    cfg, w = tmp_path / "net.cfg", tmp_path / "net.weights"
    cfg.write_text(cfgs.CFGS[name](size, size))
    network.write_synthetic_weights(network.parse_network_cfg(str(cfg), 1, "cpu"), str(w), seed=8)
    fresh = network.load_network_custom(str(cfg), str(w), 2, packed_cache=True)          # packs, writes the cache
    n_xnor = sum(1 for l in fresh.layers if l.type == "convolutional" and l.xnor)
    assert fresh.packed_from_cache == 0 and (tmp_path / "net.weights.xnorpack").exists()
    cached = network.load_network_custom(str(cfg), str(w), 2, packed_cache=True)
    assert cached.packed_from_cache == n_xnor > 0
    for a, b in zip(fresh.layers, cached.layers):
        if a.xnor_layer is not None:
            assert torch.equal(a.xnor_layer.align_bit_weights_gpu, b.xnor_layer.align_bit_weights_gpu)
            assert torch.equal(a.xnor_layer.mean_arr_gpu, b.xnor_layer.mean_arr_gpu)
    x = torch.from_numpy(synth.uniform01(3, (2, 3, size, size))).cuda()
    for ha, hb in zip(network.forward_network_gpu(fresh, x), network.forward_network_gpu(cached, x)):
        assert torch.equal(ha, hb)
    # other weights under the same name: nothing of the old cache is used, and the file is replaced
    network.write_synthetic_weights(network.parse_network_cfg(str(cfg), 1, "cpu"), str(w), seed=9)
    other = network.load_network_custom(str(cfg), str(w), 2, packed_cache=True)
    assert other.packed_from_cache == 0
    again = network.load_network_custom(str(cfg), str(w), 2, packed_cache=True)
    assert again.packed_from_cache == n_xnor
