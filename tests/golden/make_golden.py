"""Generates tests/golden/xnor_ref_golden.npz from the reference's OWN CPU code.

Run where the reference tree is mounted, after ``make -C oracle ref``:

    python tests/golden/make_golden.py

Every case builds a batch-1 xnor layer with the reference constructor, runs the reference's
binary_align_weights and forward_convolutional_layer (through oracle/_ref/liboracle_ref.so) and
stores what they produced: packed weights, mean_arr, the packed transposed input (t_bit_input)
and the fp32 layer output.  Inputs are NOT stored; tests regenerate them from tests/synth.py with
the seed recorded here.  Only shapes on which the reference CPU path is defined are listed
(3x3/stride 1/pad 1 for any channel count; any kernel and stride when channels % 32 == 0).
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import synth  # noqa: E402
from oracle.binding import Ref  # noqa: E402

# seed, c, h, w, n, ks, stride, pad, leaky
CASES = [
    (11, 32, 9, 7, 16, 3, 1, 1, 0),      # word path, odd spatial size
    (12, 64, 8, 8, 32, 1, 1, 0, 1),      # word path, 1x1
    (13, 64, 16, 16, 32, 3, 2, 1, 1),    # word path, stride 2 (generic im2col branch)
    (14, 5, 10, 10, 8, 3, 1, 1, 1),      # bit path, K = 45
    (15, 75, 13, 13, 24, 3, 1, 1, 1),    # bit path, K = 675 (not word aligned)
    (16, 16, 20, 20, 32, 3, 1, 1, 0),    # bit path, C = 16 as in the first xnor layer of the tiny nets
    (17, 256, 13, 13, 64, 3, 1, 1, 1),   # word path, K = 2304 (a multiple of 256: a full block of padding)
    (18, 96, 7, 9, 17, 3, 1, 1, 1),      # word path, odd M and N (scalar tails of the reference GEMM)
    (19, 1024, 5, 5, 8, 1, 1, 0, 1),     # word path, 1x1 with K = 1024
]


def main() -> None:
    ref = Ref()
    ref.set_gpu_index(-1)
    out = {"cases": np.frombuffer(json.dumps(CASES).encode(), dtype=np.uint8)}
    for i, (seed, c, h, w, n, ks, stride, pad, leaky) in enumerate(CASES):
        x, wt, b = synth.conv_case(seed, 1, c, h, w, n, ks)
        layer = ref.layer((c, h, w), wt, b, stride, pad, bool(leaky))
        y = layer.forward(x[0])
        out[f"c{i}_align_bit_weights"] = layer.align_bit_weights()[: n * layer.new_lda // 8]
        out[f"c{i}_mean_arr"] = layer.mean_arr()
        out[f"c{i}_t_bit_input"] = layer.t_bit_input()
        out[f"c{i}_output"] = y
        layer.close()
    # GPU-build weight layout (complemented bytes) of one word-path case
    seed, c, h, w, n, ks, stride, pad, leaky = CASES[0]
    x, wt, b = synth.conv_case(seed, 1, c, h, w, n, ks)
    ref.set_gpu_index(0)
    layer = ref.layer((c, h, w), wt, b, stride, pad, bool(leaky))
    out["c0_align_bit_weights_inverted"] = layer.align_bit_weights()[: n * layer.new_lda // 8]
    layer.close()
    ref.set_gpu_index(-1)
    path = os.path.join(HERE, "xnor_ref_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
