"""The headline configuration's own shapes (Llama-3-8B-shaped Q4_0, 64 streams, ragged caches of up to 4096
positions) through the C ABI (needs a B200).

The CPU oracle cannot finish these sizes whole, so each case checks a sample of outputs against the oracle bit for
bit and a property that does not depend on size: a row's (a token's) bits are the same alone as in the batch of 64,
which also sets two different kernels against each other (the streamed matvec against the tensor-core pipeline;
the three-launch attention against the single launch).
"""
import numpy as np
import pytest

from helpers import bits, oracle, pkg

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = pkg.B200(0)
    yield d
    d.close()


def random_q4_0(rng, n, k):
    """n rows of k/32 ggml Q4_0 blocks: random nibbles under F16 scales of the size N(0, 0.02) weights give."""
    blocks = rng.integers(0, 256, size=(n * (k // 32), 18), dtype=np.uint8)
    scales = rng.uniform(0.004, 0.012, n * (k // 32)).astype(np.float16)
    blocks[:, 0:2] = scales.view(np.uint8).reshape(-1, 2)
    return blocks.reshape(n, (k // 32) * 18)


@pytest.mark.parametrize("n,k", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096)])
def test_products_of_the_headline_model(dev, n, k):
    rng = np.random.default_rng(n + k)
    w = random_q4_0(rng, n, k)
    x = rng.normal(0, 1, (64, k)).astype(np.float32)
    wb = dev.tensor(w)
    got = dev.block_matmul(x, wb, oracle.Q4_0, n)
    sample = np.unique(np.concatenate([[0, 1, 15, 16, n - 17, n - 16, n - 1], rng.integers(0, n, 57)]))
    want = oracle.matmul_reference(oracle.Q4_0, x, np.ascontiguousarray(w[sample]), len(sample))
    assert np.array_equal(bits(got[:, sample]), bits(want))
    for row in (0, 37, 63):
        alone = dev.block_matmul(x[row:row + 1], wb, oracle.Q4_0, n)
        assert np.array_equal(bits(alone[0]), bits(got[row])), row
    few = dev.block_matmul(x[10:13], wb, oracle.Q4_0, n)
    assert np.array_equal(bits(few), bits(got[10:13]))
    wb.free()


def uniform_fill(rng, shape):
    values = rng.random(shape, dtype=np.float32)
    values *= 2.0
    values -= 1.0
    return values


def test_attention_of_the_headline_step(dev):
    """64 streams, 32 query heads over 8 key/value heads of width 128, a cache of 4224 positions per stream holding 128..4096."""
    rng = np.random.default_rng(11)
    streams, kv_heads, group, width, capacity = 64, 8, 4, 128, 4224
    heads = kv_heads * group
    lengths = rng.integers(128, 4097, streams)
    lengths[3], lengths[40] = 4096, 128
    k = uniform_fill(rng, (streams, kv_heads, capacity, width))
    v = uniform_fill(rng, (streams, kv_heads, capacity, width))
    q = rng.normal(0, 1, (streams, heads, width)).astype(np.float32)
    table = np.array([[row, length - 1, length] for row, length in enumerate(lengths)], dtype=np.int32)
    scale = np.float32(1.0 / np.sqrt(width))
    got = dev.ragged_attention(q, k, v, table, scale)
    pairs = [(3, 0), (3, 31), (40, 5), (63, 17), (0, 12)] + [(int(t), int(h)) for t, h in zip(rng.integers(0, streams, 27), rng.integers(0, heads, 27))]
    for t, h in pairs:
        held = int(lengths[t])
        want = oracle.attend(q[t, h], k[t, h // group, :held], v[t, h // group, :held], scale)
        assert np.array_equal(bits(got[t, h]), bits(want)), (t, h, held)
    for t in (3, 40):  # one token alone is cut into position ranges and quarters of the width: the same bits
        alone = dev.ragged_attention(q[t:t + 1], k, v, table[t:t + 1], scale)
        assert np.array_equal(bits(alone[0]), bits(got[t])), t
