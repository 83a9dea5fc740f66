"""Generates tests/golden/nms_golden.npz with the REFERENCE's own do_nms_sort (src-lib/box.cpp:951, through
oracle/_ref/liboracle_refnet.so): crowded synthetic detections (many overlapping boxes, several classes) and the
probabilities the reference leaves after suppression at two thresholds.

    python tests/golden/make_nms_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.binding import RefNet  # noqa: E402


def crowd(seed: int, n: int, classes: int):
    """n boxes clustered around a few centres so that most of them overlap some other box; distinct scores."""
    rng = np.random.default_rng(seed)
    centres = rng.random((6, 2)).astype(np.float32)
    c = centres[rng.integers(0, 6, n)]
    boxes = np.concatenate([c + rng.normal(0, 0.03, (n, 2)), 0.1 + 0.15 * rng.random((n, 2))], 1).astype(np.float32)
    obj = (0.3 + 0.7 * rng.random(n)).astype(np.float32)
    probs = (obj[:, None] * rng.random((n, classes))).astype(np.float32)
    probs[probs < 0.25] = 0.0
    return boxes, obj, probs


def main() -> None:
    out = {}
    for tag, (seed, n, classes) in {"a": (1, 300, 5), "b": (2, 1500, 3), "c": (3, 40, 80)}.items():
        boxes, obj, probs = crowd(seed, n, classes)
        out[f"{tag}_boxes"], out[f"{tag}_obj"], out[f"{tag}_probs"] = boxes, obj, probs
        for t in (0.45, 0.2):
            out[f"{tag}_after_{int(t * 100)}"] = RefNet.nms_sort(boxes, obj, probs, t)
    path = os.path.join(HERE, "nms_golden.npz")
    np.savez_compressed(path, **out)
    kept = {k: int((v > 0).sum()) for k, v in out.items() if "after" in k or k.endswith("probs")}
    print(path, os.path.getsize(path), "bytes", kept)


if __name__ == "__main__":
    main()
