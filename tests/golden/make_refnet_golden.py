"""Generates tests/golden/refnet_golden.npz from the REFERENCE's own network code (oracle/_ref/liboracle_refnet.so, see
oracle/build_refnet.py): for a small yolov3-tiny_xnor the activated [yolo] head outputs of network_predict and the rows
that get_network_boxes + do_nms_sort leave.  The GPU tests feed these heads to the device decoder and compare its rows with
the reference's, also on machines where the reference library is absent.

    python tests/golden/make_refnet_golden.py
"""
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import synth  # noqa: E402
from darknet_b200 import cfgs, network  # noqa: E402
from oracle.binding import RefNet  # noqa: E402

SIZE, SEED, THRESH, NMS = 96, 41, 0.6, 0.45


def main() -> None:
    with tempfile.TemporaryDirectory() as td:
        cfg, w = os.path.join(td, "net.cfg"), os.path.join(td, "net.weights")
        open(cfg, "w").write(cfgs.yolov3_tiny_xnor_cfg(SIZE, SIZE))
        net = network.parse_network_cfg(cfg, 1, "cpu")
        network.write_synthetic_weights(net, w, seed=SEED)
        ref = RefNet(cfg, w, 1)
        x = synth.uniform01(SEED, (1, 3, SIZE, SIZE))
        ref.predict(x)
        heads = [ref.layer_output(i) for i, l in enumerate(net.layers) if l.type == "yolo"]
        rows_nms = ref.detections(SIZE, SIZE, THRESH, NMS)
        rows_raw = ref.detections(SIZE, SIZE, THRESH, 0.0)
        ref.close()
    out = os.path.join(HERE, "refnet_golden.npz")
    np.savez_compressed(out, size=SIZE, seed=SEED, thresh=THRESH, nms=NMS, head0=heads[0], head1=heads[1], rows_nms=rows_nms, rows_raw=rows_raw)
    print(out, os.path.getsize(out), "bytes;", len(rows_raw), "pairs before and", len(rows_nms), "after suppression")


if __name__ == "__main__":
    main()
