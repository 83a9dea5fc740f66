"""Head decoding, suppression and row compaction on the device (xnor_b200_yolo_detections, _nms_sort, _detection_rows) against
the reference's own get_network_boxes / do_nms_sort: committed vectors made by tests/golden/make_refnet_golden.py and
make_nms_golden.py from the reference library, and the library itself where it is present."""
import ctypes as C
import os

import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from darknet_b200 import capi, cfgs, network  # noqa: E402
from oracle.binding import RefNet  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def canonical(rows: np.ndarray) -> np.ndarray:
    """Rows sorted by (class, probability descending, x, y): the reference's final order depends on its last sort."""
    rows = np.asarray(rows, np.float32).reshape(-1, 7)
    order = np.lexsort((rows[:, 1], rows[:, 0], -rows[:, 6], rows[:, 5]))
    return rows[order]


def assert_rows_equal(got: np.ndarray, want: np.ndarray) -> None:
    got, want = canonical(got), canonical(want)
    assert got.shape == want.shape, f"{len(got)} rows, the reference has {len(want)}"
    assert np.array_equal(got[:, 5], want[:, 5])                              # classes, exactly
    assert np.array_equal(got[:, 4].view(np.uint32), want[:, 4].view(np.uint32))   # objectness is copied, not computed
    assert np.array_equal(got[:, 6].view(np.uint32), want[:, 6].view(np.uint32))   # one fp32 product on both sides
    assert np.allclose(got[:, :4], want[:, :4], rtol=1e-5, atol=1e-7)         # boxes: expf differs in the last bits


def decode_heads(heads, size, thresh, nms):
    tmp_cfg = cfgs.yolov3_tiny_xnor_cfg(size, size)
    import tempfile
    with tempfile.TemporaryDirectory() as td:
        p = os.path.join(td, "net.cfg")
        open(p, "w").write(tmp_cfg)
        net = network.parse_network_cfg(p, 1, "cuda:0")
    dets = network.DetectionBuffers(1, 80, max_dets=1024, max_rows=4096)
    dev_heads = [torch.from_numpy(np.ascontiguousarray(h)).cuda() for h in heads]
    network.get_network_boxes(net, dev_heads, size, size, thresh, dets)
    if nms > 0:
        network.do_nms_sort(dets, nms)
    network.detection_rows(dets)
    torch.cuda.synchronize()
    return dets.rows_host()[0], int(dets.count.cpu()[0])


def test_decode_and_suppress_equal_the_reference_golden():
    g = np.load(os.path.join(GOLDEN, "refnet_golden.npz"))
    size, thresh, nms = int(g["size"]), float(g["thresh"]), float(g["nms"])
    rows_raw, count = decode_heads([g["head0"], g["head1"]], size, thresh, 0.0)
    assert_rows_equal(rows_raw, g["rows_raw"])
    rows_nms, _ = decode_heads([g["head0"], g["head1"]], size, thresh, nms)
    assert_rows_equal(rows_nms, g["rows_nms"])
    assert count > 0 and len(rows_nms) < len(rows_raw)


@pytest.mark.parametrize("tag", ["a", "b", "c"])
@pytest.mark.parametrize("thresh", [45, 20])
def test_suppression_of_crowded_boxes_equals_the_reference(tag, thresh):
    g = np.load(os.path.join(GOLDEN, "nms_golden.npz"))
    boxes, obj, probs, want = g[f"{tag}_boxes"], g[f"{tag}_obj"], g[f"{tag}_probs"], g[f"{tag}_after_{thresh}"]
    n, classes = probs.shape
    batch = 3                                        # the same list three times: every image is suppressed independently
    dets = network.DetectionBuffers(batch, classes, max_dets=2048, max_rows=16)
    for b in range(batch):
        dets.boxes[b, :n] = torch.from_numpy(boxes).cuda()
        dets.objectness[b, :n] = torch.from_numpy(obj).cuda()
        dets.probs[b, :n] = torch.from_numpy(probs).cuda()
    dets.count.fill_(n)
    network.do_nms_sort(dets, thresh / 100.0)
    torch.cuda.synchronize()
    got = dets.probs[:, :n].cpu().numpy()
    for b in range(batch):
        assert np.array_equal(got[b].view(np.uint32), want.view(np.uint32)), f"image {b}: {int((got[b] != want).sum())} probabilities differ"


def test_argument_checks_and_overflow():
    dets = network.DetectionBuffers(1, 80, max_dets=8, max_rows=4)
    head = torch.full((1, 3 * 85, 4, 4), 0.9, device="cuda")          # every candidate passes: 48 detections, 8 slots
    hd = capi.YoloHead()
    hd.output = head.data_ptr()
    hd.w, hd.h, hd.n, hd.classes = 4, 4, 3, 80
    for i in range(6):
        hd.anchors[i] = 10.0 + i
    lib = capi.lib()
    assert lib.xnor_b200_yolo_detections(C.byref(hd), 1, 64, 64, 64, 64, 0.5, 1, 0, 0, C.byref(dets.desc), None) == capi.OK
    network.detection_rows(dets)
    torch.cuda.synchronize()
    assert int(dets.count.cpu()[0]) == 48                  # found; only max_dets are stored
    assert int(dets.row_count.cpu()[0]) == 8 * 80          # pairs among the stored ones; only max_rows rows are written
    bad = capi.Detections(dets.boxes.data_ptr(), dets.objectness.data_ptr(), dets.probs.data_ptr(), dets.count.data_ptr(), 1 << 20, 80)
    assert lib.xnor_b200_nms_sort(C.byref(bad), 1, 0.45, None) != capi.OK
    hd.classes = 20
    assert lib.xnor_b200_yolo_detections(C.byref(hd), 1, 64, 64, 64, 64, 0.5, 1, 0, 0, C.byref(dets.desc), None) != capi.OK


@pytest.mark.skipif(not RefNet.available(), reason="oracle/_ref/liboracle_refnet.so not built")
@pytest.mark.parametrize("letter,img", [(0, (416, 416)), (1, (640, 480)), (0, (1280, 720))])
def test_decode_equals_the_reference_library(tmp_path, letter, img):
    """The same comparison against the library itself at the full 416x416 size, with the image-size / letterbox correction."""
    cfg, w = tmp_path / "net.cfg", tmp_path / "net.weights"
    cfg.write_text(cfgs.yolov3_tiny_xnor_cfg(416, 416))
    net_cpu = network.parse_network_cfg(str(cfg), 1, "cpu")
    network.write_synthetic_weights(net_cpu, str(w), seed=77)
    ref = RefNet(str(cfg), str(w), 1)
    ref.predict(synth.uniform01(5, (1, 3, 416, 416)))
    heads = [ref.layer_output(i) for i, l in enumerate(net_cpu.layers) if l.type == "yolo"]
    want = ref.detections(img[0], img[1], 0.5, 0.45, letter)
    ref.close()
    net = network.parse_network_cfg(str(cfg), 1, "cuda:0")
    dets = network.DetectionBuffers(1, 80, max_dets=4096, max_rows=1 << 16)
    network.get_network_boxes(net, [torch.from_numpy(h).cuda() for h in heads], img[0], img[1], 0.5, dets, letter=letter)
    network.do_nms_sort(dets, 0.45)
    network.detection_rows(dets)
    torch.cuda.synchronize()
    assert_rows_equal(dets.rows_host()[0], want)
