"""The CPU oracle against the reference's golden vectors and its own kernel sources (no GPU).

Mirrors spec/quant_spec.cr, spec/f16_spec.cr, spec/maths_spec.cr, spec/llama_spec.cr,
spec/gpt2_spec.cr and spec/block_matmul_spec.cr of the reference.
"""
import numpy as np
import pytest

import helpers
from helpers import bits, golden, oracle

KINDS = {"Q8_0": oracle.Q8_0, "Q4_0": oracle.Q4_0, "Q4_1": oracle.Q4_1}


@pytest.mark.parametrize("name", list(KINDS))
def test_quantise_matches_ggml_byte_for_byte(name):
    g = golden()
    for i in range(7):
        row = g[f"quant/rows/{i}"]
        assert oracle.quantize(KINDS[name], row).tobytes() == g[f"quant/{name}/bytes/{i}"].tobytes(), (name, i)


@pytest.mark.parametrize("name", list(KINDS))
def test_dequantise_matches_ggml(name):
    g = golden()
    for i in range(7):
        raw = g[f"quant/{name}/bytes/{i}"]
        want = g[f"quant/{name}/values/{i}"]
        got = oracle.dequantize(KINDS[name], raw, want.size)
        assert np.array_equal(bits(got), bits(want)), (name, i)
    table = g["quant/table"]
    got = oracle.dequantize(KINDS[name], oracle.quantize(KINDS[name], table), table.size).reshape(table.shape)
    assert np.array_equal(bits(got), bits(g[f"quant/{name}/table"]))


def test_blocks_gguf_fixture_reads_back(tmp_path):
    g = golden()
    path = tmp_path / "blocks.gguf"
    path.write_bytes(g["quant/blocks_gguf"].tobytes())
    f = helpers.gguf.File(str(path))
    for name, kind in KINDS.items():
        gk, shape, raw = f.raw(name.lower())
        assert shape == [3, 64] and helpers.KIND_OF_GGUF[gk] == kind
        got = oracle.dequantize(kind, raw, 192).reshape(3, 64)
        assert np.array_equal(bits(got), bits(g[f"quant/{name}/table"]))


def test_f16_conversions_match_ieee():
    every = np.arange(65536, dtype=np.uint16)
    want = every.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_bits_to_f32(int(b)) for b in every[::7]], dtype=np.float32)
    assert np.array_equal(bits(got)[~np.isnan(want[::7])], bits(want[::7])[~np.isnan(want[::7])])
    rng = np.random.default_rng(3)
    values = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-6, 500), rng.normal(0, 3e4, 500),
                             [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, 2.0 ** -24, 2.0 ** -25, 6.1e-5]]).astype(np.float32)
    with np.errstate(over="ignore"):
        want16 = values.astype(np.float16).view(np.uint16)
    got16 = np.array([oracle.f32_to_f16_bits(float(v)) for v in values], dtype=np.uint16)
    assert np.array_equal(got16, want16)


def test_own_exp_and_tanh_stay_within_two_ulp():
    xs = np.concatenate([np.linspace(-87, 88, 4001), np.linspace(-1, 1, 1001)]).astype(np.float32)
    got = oracle.exp(xs).astype(np.float64)
    want = np.exp(xs.astype(np.float64))
    ulp = np.spacing(want.astype(np.float32)).astype(np.float64)
    assert np.max(np.abs(got - want) / ulp) <= 2.0
    assert oracle.exp(np.array([-np.inf], dtype=np.float32))[0] == 0.0
    ts = np.linspace(-10, 10, 4001).astype(np.float32)
    got = oracle.tanh(ts).astype(np.float64)
    want = np.tanh(ts.astype(np.float64))
    ulp = np.spacing(np.maximum(np.abs(want), 1e-30).astype(np.float32)).astype(np.float64)
    assert np.max(np.abs(got - want) / ulp) <= 2.5


def spec_case(rng, count, n, k):
    """The edge cases of spec/quant_spec.cr:31-47: a zero weight block, an outlier, a zero activation
    block, and activations that quantise to exactly 127."""
    values = rng.uniform(-2, 2, n * k).astype(np.float32)
    values[:32] = 0
    values[96] = 50
    x = rng.uniform(-3, 3, (count, k)).astype(np.float32)
    if count > 1:
        x[1, :32] = 0
    if count > 2:
        x[2, :32] = [127.0 if j == 0 else j - 15.5 for j in range(32)]
    return values, x


@pytest.mark.parametrize("name", list(KINDS))
def test_fast_product_has_the_reference_products_bits(name):
    rng = np.random.default_rng(11)
    for count, n, k in [(1, 37, 64), (3, 5, 1280), (2, 9, 4096)]:
        values, x = spec_case(rng, count, n, k)
        w = oracle.quantize(KINDS[name], values)
        ref = oracle.matmul_reference(KINDS[name], x, w, n)
        fast = oracle.matmul_fast(KINDS[name], x, w, n, threads=1)
        assert np.array_equal(bits(fast), bits(ref)), (name, count, n, k)


def test_fast_product_gives_the_same_bits_on_any_number_of_threads():
    rng = np.random.default_rng(12)
    n, k = 301, 2048
    values = rng.uniform(-2, 2, n * k).astype(np.float32)
    x = rng.uniform(-3, 3, (1, k)).astype(np.float32)
    bias = rng.normal(0, 1, n).astype(np.float32)
    for name, kind in KINDS.items():
        w = oracle.quantize(kind, values)
        ref = oracle.matmul_reference(kind, x, w, n, bias=bias)
        for threads in (1, 8, 3):
            got = oracle.matmul_fast(kind, x, w, n, bias=bias, threads=threads)
            assert np.array_equal(bits(got), bits(ref)), (name, threads)
    # many alternating products against stale span claims (spec/quant_spec.cr:74-98)
    small = oracle.quantize(oracle.Q8_0, values[:64 * 2048])
    big = oracle.quantize(oracle.Q8_0, values)
    want_small = oracle.matmul_reference(oracle.Q8_0, x, small, 64)
    want_big = oracle.matmul_reference(oracle.Q8_0, x, big, n)
    for i in range(200):
        assert np.array_equal(bits(oracle.matmul_fast(oracle.Q8_0, x, big, n, threads=4)), bits(want_big))
        assert np.array_equal(bits(oracle.matmul_fast(oracle.Q8_0, x, small, 64, threads=4)), bits(want_small))


@pytest.mark.skipif(not oracle.Ref.available(), reason="the reference's kernels were not compiled here")
@pytest.mark.parametrize("name", list(KINDS))
def test_oracle_equals_the_references_own_kernels(name):
    """quantize_rows_q8_f32 + block_matmul_f32 + gather_blocks_f32 of the reference, run on the host
    through its own emulation header, give the restated oracle's bits (spec/block_matmul_spec.cr:103-115)."""
    ref = oracle.Ref()
    rng = np.random.default_rng(5)
    kind = KINDS[name]
    for count, n, k in [(3, 37, 1280), (1, 64, 576), (2, 9, 4096)]:
        values, x = spec_case(rng, count, n, k)
        bias = rng.normal(0, 1, n).astype(np.float32)
        w = oracle.quantize(kind, values)
        scales, sums, qs = oracle.quantize_activations(x)
        rs, rm, rq = ref.quantize_rows(x)
        assert np.array_equal(bits(scales), bits(rs)) and np.array_equal(bits(sums), bits(rm)) and np.array_equal(qs, rq)
        got = oracle.matmul_reference(kind, x, w, n, bias=bias)
        want = ref.block_matmul(kind, x, w, n, bias=bias)
        assert np.array_equal(bits(got), bits(want)), (name, count, n, k)
    table = oracle.quantize(kind, rng.normal(0, 1, (20, 96)).astype(np.float32))
    ids = np.array([3, 0, 19, 7, 7], dtype=np.int32)
    want, errors = ref.gather_blocks(kind, table, 20, 96, ids)
    assert np.array_equal(bits(oracle.gather_blocks(kind, table, 20, 96, ids)), bits(want)) and errors[0] == 0
    with pytest.raises(IndexError):
        oracle.gather_blocks(kind, table, 20, 96, np.array([1, 20], dtype=np.int32))


def write_golden(tmp_path, key, name):
    path = tmp_path / name
    path.write_bytes(golden()[key].tobytes())
    return str(path)


def test_tiny_llama_f32_matches_pytorch_logits(tmp_path):
    """spec/llama_spec.cr:50-87: logits within 1e-4 of PyTorch's, greedy tokens equal, prefill == decode."""
    g = golden()
    model = helpers.oracle_llama(write_golden(tmp_path, "tiny_llama/f32_gguf", "model.gguf"))
    prompt = g["tiny_llama/prompt_ids"].tolist()
    cache = model.new_cache(1, 64)
    logits = model.forward(cache, [prompt], last=False)
    assert np.max(np.abs(logits - g["tiny_llama/logits"])) < 1e-4
    assert model.generate(prompt, 20) == g["tiny_llama/greedy"].tolist()
    # prefill == decode bit for bit (the host device is shape-invariant)
    cache2 = model.new_cache(1, 64)
    rows = [model.forward(cache2, [[t]])[0] for t in prompt]
    assert np.array_equal(bits(np.stack(rows)), bits(logits))


def test_tiny_llama_quantised_files_equal_quantising_here(tmp_path):
    """spec/block_matmul_spec.cr:244-284: the GGUF-quantised model has the bits of quantising the F32
    one with the restated quantiser; Q8_0's error is under a quarter of Q4_0's."""
    g = golden()
    f32 = helpers.gguf.File(write_golden(tmp_path, "tiny_llama/f32_gguf", "model.gguf"))
    errors = {}
    for name, kind in (("q8_0", oracle.Q8_0), ("q4_0", oracle.Q4_0)):
        path = write_golden(tmp_path, f"tiny_llama/{name}_gguf", f"model-{name}.gguf")
        qf = helpers.gguf.File(path)
        for tensor, (gk, shape, _) in qf.entries.items():
            if gk in helpers.KIND_OF_GGUF:
                want = qf.raw(tensor)[2]
                got = oracle.quantize(kind, f32.f32(tensor))
                assert want.tobytes() == got.tobytes(), tensor
        model = helpers.oracle_llama(path)
        prompt = g["tiny_llama/prompt_ids"].tolist()
        logits = model.forward(model.new_cache(1, 64), [prompt], last=False)
        errors[name] = float(np.max(np.abs(logits - g["tiny_llama/logits"])))
        # prefill == decode bitwise, and the reference product == the fast product
        cache = model.new_cache(1, 64)
        rows = np.stack([model.forward(cache, [[t]])[0] for t in prompt])
        assert np.array_equal(bits(rows), bits(logits))
        slow = helpers.oracle_llama(path, reference_products=True)
        assert np.array_equal(bits(slow.forward(slow.new_cache(1, 64), [prompt], last=False)), bits(logits))
    assert errors["q8_0"] < errors["q4_0"] / 4


def test_tiny_gpt2_f32_matches_pytorch_logits():
    """spec/gpt2_spec.cr:54-102."""
    g = golden()
    st = helpers.read_safetensors(g["tiny_gpt2/safetensors"])
    config = dict(arch="gpt2", layers=2, heads=4, kv_heads=4, width=32, head_width=8, hidden=128, context=64, vocab=400, eps=1e-5)
    model = oracle.Model(config, helpers.gpt2_tensors_from_hf(st, 2))
    prompt = g["tiny_gpt2/prompt_ids"].tolist()
    logits = model.forward(model.new_cache(1, 64), [prompt], last=False)
    assert np.max(np.abs(logits - g["tiny_gpt2/logits"])) < 1e-4
    assert model.generate(prompt, 20) == g["tiny_gpt2/greedy"].tolist()


def test_batched_rows_have_the_bits_of_each_row_alone(tmp_path):
    """spec/batched_decode_spec.cr:110-143: ragged appends with an idle row, then a reset."""
    path = write_golden(tmp_path, "tiny_llama/q8_0_gguf", "model-q8_0.gguf")
    model = helpers.oracle_llama(path)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 400, size=n).tolist() for n in (5, 9, 0, 3)]
    cache = model.new_cache(4, 32)
    batch = model.forward(cache, prompts)
    alone = []
    for p in prompts:
        if p:
            alone.append(model.forward(model.new_cache(1, 32), [p])[0])
    assert np.array_equal(bits(batch), bits(np.stack(alone)))
    step = model.forward(cache, [[1], [], [2], [3]])
    c = model.new_cache(1, 32)
    model.forward(c, [prompts[0]])
    assert np.array_equal(bits(step[0]), bits(model.forward(c, [[1]])[0]))
    cache.reset(1)
    again = model.forward(cache, [[], prompts[1], [], []])
    assert np.array_equal(bits(again[0]), bits(alone[1]))


def test_greedy_and_topk_ties_go_to_the_lower_index():
    """spec/sampler_spec.cr:27-29, 56-59."""
    logits = np.array([0.5, 2.0, 2.0, -1.0, 2.0, 1.5], dtype=np.float32)
    assert oracle.argmax_first(logits) == 1
    assert oracle.topk(logits, 4).tolist() == [1, 2, 4, 5]
