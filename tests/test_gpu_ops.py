"""CUDA operators against the CPU oracle, through the C ABI (needs a B200).

Mirrors spec/quant_spec.cr, spec/block_matmul_spec.cr, spec/fused_llama_spec.cr, spec/llama_ops_spec.cr,
spec/attention_spec.cr, spec/batched_decode_spec.cr, spec/sampler_spec.cr and spec/buffer_pool_spec.cr.
Block products, gathers, RoPE, activations and cache writes are held to the oracle's bits; norms and
attention to 1e-5 relative in the fast mode and to the oracle's bits in the exact mode.
"""
import numpy as np
import pytest

import helpers
from helpers import bits, golden, oracle, pkg, rel_max

pytestmark = pytest.mark.gpu
KINDS = {"Q8_0": oracle.Q8_0, "Q4_0": oracle.Q4_0, "Q4_1": oracle.Q4_1}


@pytest.fixture(scope="module")
def dev():
    d = pkg.B200(0)
    yield d
    d.close()


@pytest.mark.parametrize("name", list(KINDS))
def test_weight_quantiser_gives_ggmls_bytes(dev, name):
    g = golden()
    for i in range(7):
        row = g[f"quant/rows/{i}"]
        buf = dev.quantize(row, KINDS[name])
        assert buf.numpy(np.uint8).tobytes() == g[f"quant/{name}/bytes/{i}"].tobytes(), (name, i)
        back = dev.dequantize(buf, row.size, KINDS[name])
        assert np.array_equal(bits(back.numpy(np.float32)), bits(g[f"quant/{name}/values/{i}"]))
    rng = np.random.default_rng(1)
    x = rng.normal(0, 0.02, 64 * 1024).astype(np.float32)
    x[:32] = 0
    assert dev.quantize(x, KINDS[name]).numpy(np.uint8).tobytes() == oracle.quantize(KINDS[name], x).tobytes()


def test_activation_quantiser_has_the_hosts_bits(dev):
    rng = np.random.default_rng(2)
    x = rng.uniform(-3, 3, (5, 1280)).astype(np.float32)
    x[1, :32] = 0
    x[2, :32] = [127.0 if j == 0 else j - 15.5 for j in range(32)]
    x[3, 64:96] *= 1e-20
    scales, sums, qs = dev.quantize_rows(x)
    ws, wm, wq = oracle.quantize_activations(x)
    assert np.array_equal(bits(scales), bits(ws)) and np.array_equal(bits(sums), bits(wm)) and np.array_equal(qs, wq)


def product_case(rng, count, n, k):
    values = rng.uniform(-2, 2, n * k).astype(np.float32)
    values[:32] = 0
    values[96] = 50
    x = rng.uniform(-3, 3, (count, k)).astype(np.float32)
    if count > 1:
        x[1, :32] = 0
    if count > 2:
        x[2, :32] = [127.0 if j == 0 else j - 15.5 for j in range(32)]
    return values, x


SHAPES = [(1, 37, 64), (3, 5, 1280), (2, 9, 4096),            # the reference's spec shapes (generic kernel)
          (1, 64, 576), (1, 960, 576), (4, 576, 1536),        # rows of 18 and 48 blocks (SmolLM2-135M's)
          (1, 1600, 1600), (2, 200, 6400),                    # 50 and 200 blocks (GPT-2 XL's)
          (1, 2048, 2048), (3, 1024, 4096), (1, 256, 14336),  # aligned rows, long rows
          (1, 4096, 14336), (3, 300, 14336), (4, 77, 28672), (2, 130, 16384), (1, 50, 10240), (4, 33, 12288),  # long rows in pieces: row tiles of up to 32 rows, a last tile that is short
          (8, 128, 2048), (16, 64, 576), (1, 7, 4096), (1, 4097, 256),
          (1, 2051, 1600), (1, 1027, 576), (1, 1025, 96),     # one row, not a whole number of groups: the streamed kernel and the generic one share the rows
          (5, 40, 1536), (33, 48, 4096), (64, 200, 1600), (100, 96, 576), (64, 1024, 2048), (17, 72, 14336),  # tensor-core kernels
          (64, 304, 4096), (70, 100, 1024), (12, 2400, 512), (24, 48, 2048), (64, 5000, 256), (40, 2500, 1024),  # odd group counts, two slabs of activation rows, several groups per CTA
          (64, 19008, 256), (9, 20000, 512), (70, 19200, 256),  # many rows: 16-row groups, one warp per group
          (9, 40000, 256), (33, 44, 2048), (64, 1000, 512)]  # more groups than one wave of CTAs holds; a last group of 4 rows


@pytest.mark.parametrize("name", list(KINDS))
def test_block_product_is_bit_exact(dev, name):
    rng = np.random.default_rng(11)
    kind = KINDS[name]
    for count, n, k in SHAPES:
        values, x = product_case(rng, count, n, k)
        bias = rng.normal(0, 1, n).astype(np.float32) if n % 2 else None
        w = oracle.quantize(kind, values)
        wb = dev.tensor(w)
        got = dev.block_matmul(x, wb, kind, n, bias=bias)
        want = oracle.matmul_reference(kind, x, w, n, bias=bias)
        wb.free()
        assert np.array_equal(bits(got), bits(want)), (name, count, n, k)


@pytest.mark.parametrize("name", list(KINDS))
def test_one_row_with_its_activations_kept_in_registers(dev, name):
    """One row of activations whose length divides a sweep of the streamed kernel's compute threads (8 .. 256 blocks; for
    Q4_0 and Q4_1 up to 512 blocks' worth of a sweep) keeps each thread's activation blocks in registers.  Row counts that
    leave a last tile short or a single row, a bias, a block of zero activations, one whose largest value is the first and a
    tiny one: the oracle's product (Quant.block_matmul over quantize_activations' blocks, quant.cr:45-60, 428-442), bit
    for bit."""
    rng = np.random.default_rng(31)
    kind = KINDS[name]
    for n, k in [(1, 256), (129, 512), (1000, 1024), (515, 4096), (300, 8192), (2501, 256), (64, 2048)]:
        values = rng.uniform(-2, 2, n * k).astype(np.float32)
        values[:32] = 0
        x = rng.uniform(-3, 3, (1, k)).astype(np.float32)
        x[0, 32:64] = 0
        x[0, 64:96] = [127.0 if j == 0 else j - 15.5 for j in range(32)]
        x[0, k - 32:] *= 1e-20
        bias = rng.normal(0, 1, n).astype(np.float32) if n % 2 else None
        w = oracle.quantize(kind, values)
        wb = dev.tensor(w)
        got = dev.block_matmul(x, wb, kind, n, bias=bias)
        want = oracle.matmul_reference(kind, x, w, n, bias=bias)
        wb.free()
        assert np.array_equal(bits(got), bits(want)), (name, n, k)


@pytest.mark.parametrize("name", list(KINDS))
def test_a_few_rows_quantised_inside_the_product_have_the_quantisers_bits(dev, name):
    """tsm_block_matmul of at most four rows quantises them inside the streamed kernel (one thread per block) instead of
    launching the quantiser first.  Rows that are views (a stride that is no multiple of four floats, so the 16-byte loads
    are off), blocks of zeros, a block whose largest value is negative, values that round half away from zero and a tiny
    block must give the oracle's product over Quant.quantize_activations' blocks (quant.cr:428-442), bit for bit."""
    import ctypes as C
    rng = np.random.default_rng(21)
    kind = KINDS[name]
    n, k = 1000, 2048
    w = oracle.quantize(kind, rng.normal(0, 0.02, n * k).astype(np.float32))
    wb = dev.tensor(w)
    for rows, stride in ((1, k), (3, k + 5), (4, k + 8), (2, 3 * k)):
        x = rng.normal(0, 1, (rows, stride)).astype(np.float32)
        x[0, 0:32] = 0.0                                     # a block of zeros: scale 0, inverse 0
        x[0, 32:64] = -np.abs(x[0, 32:64]) - 1.0             # the largest magnitude is negative
        x[0, 64:96] = np.arange(32, dtype=np.float32) * (127.0 / 62.0) - 63.5   # multiples of half a step
        x[rows - 1, 96:128] = 1e-20                          # a tiny block
        xb = dev.tensor(x)
        out = dev.alloc(rows * n * 4)
        dev.check(dev.lib.tsm_block_matmul(dev.ctx, C.c_uint64(xb.ptr), rows, k, C.c_int64(stride), C.c_uint64(wb.ptr), kind, n,
                                           C.c_uint64(0), C.c_uint64(out.ptr)), "tsm_block_matmul")
        dev.sync()
        got = out.numpy(np.float32)[:rows * n].reshape(rows, n)
        want = oracle.matmul_reference(kind, np.ascontiguousarray(x[:, :k]), w, n)
        xb.free(), out.free()
        assert np.array_equal(bits(got), bits(want)), (name, rows, stride)
    wb.free()


def test_block_product_with_a_scale_that_is_not_finite(dev):
    """A Q4_0 block whose scale is infinite: the outputs it reaches are the reference's infinities and NaNs."""
    rng = np.random.default_rng(12)
    n, k, count = 64, 1024, 16
    w = oracle.quantize(oracle.Q4_0, rng.normal(0, 0.02, n * k).astype(np.float32)).copy()
    blocks = w.reshape(n, k // 32, 18)
    blocks[3, 5, 0:2] = np.frombuffer(np.float16(np.inf).tobytes(), dtype=np.uint8)
    blocks[40, 0, 0:2] = np.frombuffer(np.float16(-np.inf).tobytes(), dtype=np.uint8)
    x = rng.uniform(-3, 3, (count, k)).astype(np.float32)
    wb = dev.tensor(w)
    got = dev.block_matmul(x, wb, oracle.Q4_0, n)
    want = oracle.matmul_reference(oracle.Q4_0, x, w, n)
    wb.free()
    assert np.isinf(want[:, 3]).any() or np.isnan(want[:, 3]).any()
    finite = np.isfinite(want)
    assert np.array_equal(finite, np.isfinite(got))
    assert np.array_equal(bits(got[finite]), bits(want[finite]))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[np.isinf(want)], want[np.isinf(want)])


def host_matmul_f32(x, w, bias=None):
    """devices/host.cr:700-734: every output adds its k products in index order, product and sum rounded separately."""
    acc = np.zeros((x.shape[0], w.shape[0]), dtype=np.float32)
    for s in range(x.shape[1]):
        acc = acc + x[:, s, None] * w[None, :, s]
    return acc + bias[None, :] if bias is not None else acc


@pytest.mark.parametrize("rows,k,n", [(1, 576, 300), (5, 100, 129), (9, 33, 64), (8, 32, 128), (64, 256, 1000), (3, 1, 7)])
def test_f32_product_has_the_hosts_bits(dev, rows, k, n):
    """A Linear whose weight stayed F32 (spec/llama_spec.cr and spec/gpt2_spec.cr run whole F32 models through it)."""
    rng = np.random.default_rng(rows * 1000 + k)
    x = rng.normal(0, 1, (rows, k)).astype(np.float32)
    w = rng.normal(0, 0.05, (n, k)).astype(np.float32)
    bias = rng.normal(0, 1, n).astype(np.float32)
    assert np.array_equal(bits(dev.matmul_f32(x, w)), bits(host_matmul_f32(x, w)))
    assert np.array_equal(bits(dev.matmul_f32(x, w, bias)), bits(host_matmul_f32(x, w, bias)))


def test_a_row_alone_equals_the_row_in_a_batch(dev):
    rng = np.random.default_rng(4)
    n, k = 512, 2048
    w = oracle.quantize(oracle.Q4_0, rng.normal(0, 0.02, n * k).astype(np.float32))
    wb = dev.tensor(w)
    x = rng.normal(0, 1, (9, k)).astype(np.float32)
    batch = dev.block_matmul(x, wb, oracle.Q4_0, n)
    for r in (0, 4, 8):
        assert np.array_equal(bits(dev.block_matmul(x[r:r + 1], wb, oracle.Q4_0, n)[0]), bits(batch[r]))


@pytest.mark.parametrize("name", list(KINDS))
def test_block_gather(dev, name):
    rng = np.random.default_rng(5)
    kind = KINDS[name]
    table = oracle.quantize(kind, rng.normal(0, 1, (50, 96)).astype(np.float32))
    tb = dev.tensor(table)
    ids = np.array([3, 0, 49, 7, 7], dtype=np.int32)
    assert np.array_equal(bits(dev.gather_blocks(tb, kind, 50, 96, ids)), bits(oracle.gather_blocks(kind, table, 50, 96, ids)))
    with pytest.raises(pkg.ExecutionError, match="index 50 out of range for 50 rows"):
        dev.gather_blocks(tb, kind, 50, 96, np.array([1, 50], dtype=np.int32))
    # the record is cleared: the next call succeeds
    dev.gather_blocks(tb, kind, 50, 96, ids)


@pytest.mark.parametrize("n", [32, 576, 1600, 2048, 4096])
def test_norms(dev, n):
    rng = np.random.default_rng(6)
    x = rng.normal(0, 2, (3, n)).astype(np.float32)
    w = rng.normal(1, 0.2, n).astype(np.float32)
    b = rng.normal(0, 0.2, n).astype(np.float32)
    dev.set_mode(pkg.FAST)
    assert rel_max(dev.rmsnorm(x, w), oracle.rmsnorm(x, w)) <= 1e-5
    assert rel_max(dev.layernorm(x, w, b), oracle.layernorm(x, w, b)) <= 1e-5
    dev.set_mode(pkg.EXACT)
    assert np.array_equal(bits(dev.rmsnorm(x, w)), bits(oracle.rmsnorm(x, w)))
    assert np.array_equal(bits(dev.rmsnorm(x, None)), bits(oracle.rmsnorm(x, None)))
    assert np.array_equal(bits(dev.layernorm(x, w, b)), bits(oracle.layernorm(x, w, b)))


@pytest.mark.parametrize("n", [512, 2048, 4096, 8192])
def test_the_chunked_sum_of_squares_is_the_sequential_sum(dev, n):
    """The norms add their squares chunk by chunk with integer arithmetic wherever the running sum stays in one binade, and
    term by term elsewhere; the result must be the host's sequential sum (rmsnorm_row, devices/host.cr:391-403) for rows built
    to defeat the shortcut: terms that are exact ties (powers of two, small integers), outliers a thousand times the rest,
    zeros, subnormal squares, a sum that overflows to infinity, and ordinary rows at several scales."""
    rng = np.random.default_rng(31)
    rows = []
    for scale in (1e-3, 0.02, 1.0, 30.0, 1e4):
        rows.append(rng.normal(0, scale, n))
    outliers = rng.normal(0, 1, n)
    outliers[rng.integers(0, n, 5)] *= 1000
    rows.append(outliers)
    holes = rng.normal(0, 1, n)
    holes[rng.integers(0, n, n // 2)] = 0
    rows.append(holes)
    rows.append(np.ones(n))                                              # every add a tie candidate
    rows.append(2.0 ** rng.integers(-12, 4, n))                          # powers of two: ties whenever the sum is large
    rows.append(rng.integers(0, 8, n) * 2.0 ** -3)                       # small integers
    rows.append(np.tile([1024.0, 2.0 ** -7, 2.0 ** -6.5, 0.75 * 2.0 ** -6], n // 4))
    rows.append(np.full(n, 1e-20))                                       # squares are subnormal or zero
    rows.append(np.concatenate([np.full(n // 2, 3e-20), rng.normal(0, 1, n - n // 2)]))
    rows.append(np.full(n, 1.5e19))                                      # the sum of squares overflows
    rows.append(np.concatenate([np.zeros(n - 1), [5.0]]))
    x = np.stack(rows).astype(np.float32)
    w = rng.normal(1, 0.2, n).astype(np.float32)
    b = rng.normal(0, 0.2, n).astype(np.float32)
    with np.errstate(all="ignore"):
        want = oracle.rmsnorm(x, w)
        want_layer = oracle.layernorm(x, w, b)
    got = dev.rmsnorm(x, w)
    assert np.array_equal(bits(got), bits(want)), [i for i in range(len(rows)) if not np.array_equal(bits(got[i]), bits(want[i]))]
    finite = np.isfinite(want_layer).all(axis=1)
    got_layer = dev.layernorm(x, w, b)
    assert np.array_equal(bits(got_layer[finite]), bits(want_layer[finite]))
    for seed in range(40):                                               # many ordinary rows: every chunk pattern
        y = np.random.default_rng(seed).normal(0, 2.0 ** (seed % 9 - 4), (8, n)).astype(np.float32)
        assert np.array_equal(bits(dev.rmsnorm(y, w)), bits(oracle.rmsnorm(y, w))), seed


def test_rope_is_bit_exact(dev):
    rng = np.random.default_rng(7)
    cos, sin = oracle.rope_tables(64, 300, 10000.0)
    x = rng.normal(0, 1, (6, 5, 64)).astype(np.float32)
    positions = np.array([0, 1, 17, 299, 128, 5], dtype=np.int32)
    got = dev.rope(x, cos, sin, positions)
    for t in range(6):
        want = oracle.rope(x[t], np.repeat(cos[positions[t]][None], 5, 0), np.repeat(sin[positions[t]][None], 5, 0))
        assert np.array_equal(bits(got[t]), bits(want))


def test_write_rows_places_tokens(dev):
    rng = np.random.default_rng(8)
    cache = rng.normal(0, 1, (3, 2, 10, 8)).astype(np.float32)
    values = rng.normal(0, 1, (4, 2, 8)).astype(np.float32)
    slots = np.array([0 * 10 + 3, 2 * 10 + 0, 2 * 10 + 1, 1 * 10 + 9], dtype=np.int32)
    got = dev.write_rows(cache, values, slots)
    want = cache.copy()
    for t, slot in enumerate(slots):
        want[slot // 10, :, slot % 10, :] = values[t]
    assert np.array_equal(got, want)


def test_activations_are_bit_exact(dev):
    rng = np.random.default_rng(9)
    gate = np.concatenate([rng.normal(0, 3, 4000), [0.0, -0.0, 100.0, -100.0, 88.8, -88.0]]).astype(np.float32).reshape(2, -1)
    up = rng.normal(0, 1, gate.shape).astype(np.float32)
    assert np.array_equal(bits(dev.swiglu(gate, up)), bits(oracle.swiglu(gate, up)))
    assert np.array_equal(bits(dev.gelu(gate)), bits(oracle.gelu(gate)))
    assert np.array_equal(bits(dev.silu(gate)), bits(oracle.silu(gate)))
    assert np.array_equal(bits(dev.add(gate, up)), bits(gate + up))


def attention_case(rng, rows, kv_heads, group, capacity, width, lengths):
    heads = kv_heads * group
    k = rng.normal(0, 1, (rows, kv_heads, capacity, width)).astype(np.float32)
    v = rng.normal(0, 1, (rows, kv_heads, capacity, width)).astype(np.float32)
    q = rng.normal(0, 1, (len(lengths), heads, width)).astype(np.float32)
    table = np.array([[row, length - 1, length] for row, length in lengths], dtype=np.int32)
    return q, k, v, table, heads


def oracle_attention(q, k, v, table, scale):
    tokens, heads, width = q.shape
    group = heads // k.shape[1]
    out = np.empty_like(q)
    for t in range(tokens):
        row, limit = table[t, 0], table[t, 1]
        for h in range(heads):
            out[t, h] = oracle.attend(q[t, h], k[row, h // group, :limit + 1], v[row, h // group, :limit + 1], scale)
    return out


@pytest.mark.parametrize("width,group", [(64, 1), (64, 3), (128, 4), (64, 2), (8, 2), (128, 8)])
def test_ragged_attention(dev, width, group):
    rng = np.random.default_rng(10)
    lengths = [(0, 1), (1, 300), (2, 256), (3, 257), (1, 77), (0, 700)]
    q, k, v, table, heads = attention_case(rng, 4, 2, group, 700, width, lengths)
    scale = np.float32(1.0 / np.sqrt(width))
    want = oracle_attention(q, k, v, table, scale)
    dev.set_mode(pkg.FAST)
    fast = dev.ragged_attention(q, k, v, table, scale)
    assert rel_max(fast, want) <= 1e-5
    # each token's bits do not depend on its neighbours in the batch
    alone = dev.ragged_attention(q[1:2], k, v, table[1:2], scale)
    assert np.array_equal(bits(alone[0]), bits(fast[1]))
    dev.set_mode(pkg.EXACT)
    exact = dev.ragged_attention(q, k, v, table, scale)
    assert np.array_equal(bits(exact), bits(want))
    assert np.array_equal(bits(dev.ragged_attention(q[1:2], k, v, table[1:2], scale)[0]), bits(exact[1]))


def test_long_caches_with_few_streams_take_the_three_launch_path(dev):
    """Few (token, kv head) pairs and a long cache: the score pass is cut by positions and the value pass by quarters of the
    width; the bits stay those of the oracle (and of the single launch, which the case above exercises)."""
    rng = np.random.default_rng(12)
    lengths = [(0, 1500), (1, 33), (2, 1024), (0, 1), (1, 1279)]
    q, k, v, table, heads = attention_case(rng, 3, 2, 4, 1536, 128, lengths)
    scale = np.float32(1.0 / np.sqrt(128))
    want = oracle_attention(q, k, v, table, scale)
    got = dev.ragged_attention(q, k, v, table, scale)
    assert np.array_equal(bits(got), bits(want))
    assert np.array_equal(bits(dev.ragged_attention(q[2:3], k, v, table[2:3], scale)[0]), bits(got[2]))


def test_softmax_denominators_of_degenerate_streams(dev):
    """Long streams through the three-launch path whose keys repeat (every score equal, every exp value 1: each add of the
    denominator a rounding tie), whose scores take a few values only, whose last key dominates, and whose scores are all near
    zero: the oracle's bits."""
    rng = np.random.default_rng(13)
    lengths = [(0, 2000), (1, 1536), (2, 1900), (3, 1100)]
    q, k, v, table, heads = attention_case(rng, 4, 1, 4, 2048, 128, lengths)
    k[0, :, :, :] = k[0, :, 0:1, :]                                  # one key repeated: all weights equal
    k[1, 0] = k[1, 0][rng.integers(0, 3, 2048)]                     # three distinct keys
    k[2, :, 1899, :] = 40.0 * q[2, 0]                               # one position takes nearly all the weight
    k[3] *= 1e-3                                                     # scores near zero: exp values near 1
    scale = np.float32(1.0 / np.sqrt(128))
    want = oracle_attention(q, k, v, table, scale)
    got = dev.ragged_attention(q, k, v, table, scale)
    assert np.array_equal(bits(got), bits(want))


def test_sampler_picks(dev):
    logits = np.array([[0.5, 2.0, 2.0, -1.0, 2.0, 1.5], [3.0, 1.0, 3.0, 0.0, 0.0, 0.0]], dtype=np.float32)
    assert dev.argmax(logits).tolist() == [1, 0]
    ids, values = dev.topk(logits, 4)
    assert ids.tolist() == [[1, 2, 4, 5], [0, 2, 1, 3]]
    assert values[0].tolist() == [2.0, 2.0, 2.0, 1.5]
    rng = np.random.default_rng(3)
    big = rng.normal(0, 1, (3, 50257)).astype(np.float32)
    assert dev.argmax(big).tolist() == [oracle.argmax_first(r) for r in big]
    assert dev.topk(big, 40)[0].tolist() == [oracle.topk(r, 40).tolist() for r in big]


def test_pool_reuses_exact_sizes(dev):
    dev.sync()
    a = dev.alloc(123456)
    ptr = a.ptr
    a.free()
    before = dev.counters()
    b = dev.alloc(123456)
    after = dev.counters()
    assert b.ptr == ptr and after["pool_hits"] == before["pool_hits"] + 1 and after["pool_misses"] == before["pool_misses"]
    c = dev.alloc(123457)
    assert c.ptr != ptr
    b.free(), c.free()
    assert dev.counters()["host_ops"] == 0
