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


def random_blocks(rng, kind, n, k):
    """n rows of k/32 ggml blocks of `kind` with random payload bytes (every int8 and nibble value occurs) under F16 scales
    (and, for Q4_1, minima) of the size N(0, 0.02) weights give."""
    count = n * (k // 32)
    size = oracle.BLOCK_BYTES[kind]
    blocks = rng.integers(0, 256, size=(count, size), dtype=np.uint8)
    scales = rng.uniform(0.0002 if kind == oracle.Q8_0 else 0.004, 0.0006 if kind == oracle.Q8_0 else 0.012, count).astype(np.float16)
    blocks[:, 0:2] = scales.view(np.uint8).reshape(-1, 2)
    if kind == oracle.Q4_1:
        minima = rng.uniform(-0.08, -0.02, count).astype(np.float16)
        blocks[:, 2:4] = minima.view(np.uint8).reshape(-1, 2)
    return blocks.reshape(n, (k // 32) * size)


# The products of the baseline's other configurations, with the rows they run at: 135M-shaped Q8_0 and GPT-2-XL-shaped Q8_0
# (with biases) at one row, 1.7B-shaped Q4_1 at sixteen.
OTHER_PRODUCTS = [("Q8_0", 1, 960, 576, False), ("Q8_0", 1, 576, 576, False), ("Q8_0", 1, 3072, 576, False), ("Q8_0", 1, 576, 1536, False),
                  ("Q8_0", 1, 49152, 576, False),
                  ("Q4_1", 16, 6144, 2048, False), ("Q4_1", 16, 2048, 2048, False), ("Q4_1", 16, 16384, 2048, False),
                  ("Q4_1", 16, 2048, 8192, False), ("Q4_1", 16, 49152, 2048, False),
                  ("Q8_0", 1, 4800, 1600, True), ("Q8_0", 1, 1600, 1600, True), ("Q8_0", 1, 6400, 1600, True), ("Q8_0", 1, 1600, 6400, True),
                  ("Q8_0", 1, 50257, 1600, False)]


@pytest.mark.parametrize("name,rows,n,k,with_bias", OTHER_PRODUCTS)
def test_products_of_the_other_configurations(dev, name, rows, n, k, with_bias):
    kind = oracle.KIND_NAMES[name]
    rng = np.random.default_rng(n * 7 + k)
    w = random_blocks(rng, kind, n, k)
    x = rng.normal(0, 1, (rows, k)).astype(np.float32)
    bias = rng.normal(0, 0.1, n).astype(np.float32) if with_bias else None
    wb = dev.tensor(w)
    got = dev.block_matmul(x, wb, kind, n, bias)
    sample = np.unique(np.concatenate([[0, 1, n - 2, n - 1], rng.integers(0, n, 124)]))
    want = oracle.matmul_reference(kind, x, np.ascontiguousarray(w[sample]), len(sample), bias=bias[sample] if with_bias else None)
    assert np.array_equal(bits(got[:, sample]), bits(want))
    if rows > 1:
        alone = dev.block_matmul(x[rows - 1:rows], wb, kind, n, bias)
        assert np.array_equal(bits(alone[0]), bits(got[rows - 1]))
    wb.free()


# The baseline's standalone sweep: every format x shape x column count, "bit-exact comparison against the reference"
# (spec/block_matmul_spec.cr:103-123, 139-195 at these sizes).
SWEEP_SHAPES = [(576, 1536), (2048, 8192), (4096, 14336), (14336, 4096), (128256, 4096)]


@pytest.mark.parametrize("n,k", SWEEP_SHAPES)
@pytest.mark.parametrize("name", ["Q4_0", "Q4_1", "Q8_0"])
def test_sweep_of_formats_shapes_and_columns(dev, name, n, k):
    """Activations of 1, 8, 64 and 256 columns (rows of x) over the same weights: a sample of 64 weight rows against the
    oracle bit for bit at every column count, and each smaller product against the rows it shares with the 256-column
    one, output for output (a row alone has the bits it has in the batch), which sets the streamed kernel (1 column), the
    tensor-core kernels (8, 64) and their slabs of 64 activation rows (256) against one another."""
    kind = oracle.KIND_NAMES[name]
    rng = np.random.default_rng(n * 3 + k + kind)
    w = random_blocks(rng, kind, n, k)
    x = rng.normal(0, 1, (256, k)).astype(np.float32)
    wb = dev.tensor(w)
    sample = np.unique(np.concatenate([[0, 1, 15, 16, n - 17, n - 16, n - 1], rng.integers(0, n, 57)]))
    want = oracle.matmul_reference(kind, x, np.ascontiguousarray(w[sample]), len(sample))
    whole = dev.block_matmul(x, wb, kind, n)
    assert np.array_equal(bits(whole[:, sample]), bits(want)), 256
    for columns in (64, 8, 1):
        got = dev.block_matmul(x[:columns], wb, kind, n)
        assert np.array_equal(bits(got[:, sample]), bits(want[:columns])), columns
        assert np.array_equal(bits(got), bits(whole[:columns])), columns
    alone = dev.block_matmul(x[255:256], wb, kind, n)
    assert np.array_equal(bits(alone[0]), bits(whole[255]))
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


@pytest.mark.parametrize("streams,heads,kv_heads,capacity,low,high", [(1, 25, 25, 1024, 576, 576),    # GPT-2-XL-shaped, one stream
                                                                      (16, 32, 32, 512, 128, 384),   # 1.7B-shaped, sixteen streams
                                                                      (1, 9, 3, 256, 160, 160)])     # 135M-shaped, one stream
def test_attention_of_the_other_configurations(dev, streams, heads, kv_heads, capacity, low, high):
    """Heads of width 64 at the baseline's other shapes: every output against the oracle."""
    rng = np.random.default_rng(streams * 100 + heads)
    width, group = 64, heads // kv_heads
    lengths = rng.integers(low, high + 1, streams)
    k = uniform_fill(rng, (streams, kv_heads, capacity, width))
    v = uniform_fill(rng, (streams, kv_heads, capacity, width))
    q = rng.normal(0, 1, (streams, heads, width)).astype(np.float32)
    table = np.array([[row, length - 1, length] for row, length in enumerate(lengths)], dtype=np.int32)
    scale = np.float32(1.0 / np.sqrt(width))
    got = dev.ragged_attention(q, k, v, table, scale)
    for t in range(streams):
        held = int(lengths[t])
        for h in range(heads):
            want = oracle.attend(q[t, h], k[t, h // group, :held], v[t, h // group, :held], scale)
            assert np.array_equal(bits(got[t, h]), bits(want)), (t, h, held)
