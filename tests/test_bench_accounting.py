"""The byte accounting behind bench.py's roofline figures (no GPU): algorithmic bytes per decode step."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_weight_elements_of_the_named_shapes():
    # embeddings are not read by a product; every Linear and the vocabulary head are, once per step
    assert bench.weight_elements(bench.WORKLOADS["c5"]) == 32 * (6144 * 4096 + 4096 * 4096 + 28672 * 4096 + 4096 * 14336) + 128256 * 4096
    assert bench.weight_elements(bench.WORKLOADS["c1"]) == 30 * (960 * 576 + 576 * 576 + 3072 * 576 + 576 * 1536) + 49152 * 576


def test_step_bytes_are_weights_once_plus_every_visible_kv_row():
    w = bench.WORKLOADS["c5"]
    lengths = np.array([128, 4096, 1000])
    total, weights, kv = bench.step_bytes(w, lengths)
    assert weights == bench.weight_elements(w) * 18 // 32          # Q4_0: 18 bytes per 32 elements
    assert kv == int(sum(2 * 32 * 8 * 128 * 4 * (n + 1) for n in lengths))   # K and V, 32 layers, 8 kv heads of 128 floats
    assert total == weights + kv


def test_ragged_lengths_are_the_configured_range_and_reproducible():
    w = bench.WORKLOADS["c5"]
    a, b = bench.draw_lengths(w, 0), bench.draw_lengths(w, 0)
    assert a.tolist() == b.tolist() and len(a) == 64
    assert a.min() >= 128 and a.max() <= 4096


def test_rotating_weight_copies_put_twice_l2_between_two_uses_of_a_copy():
    """The sweep's launches read copies of the weights in turn (bench.rotating_weights); between two uses of one copy the
    others must bring at least 256 MB, twice the 126 MB L2, through the cache, whatever the matrix's size."""
    for n, k, block in [(576, 1536, 18), (2048, 8192, 34), (4096, 14336, 20), (14336, 4096, 18), (128256, 4096, 34), (128256, 4096, 18)]:
        size = n * (k // 32) * block
        copies = bench.weight_copies(size)
        assert copies >= 2 and (copies - 1) * size >= 256 << 20
        assert (copies - 2) * size < 256 << 20          # and no more copies than that takes
