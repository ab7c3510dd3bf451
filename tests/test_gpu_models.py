"""Whole models through the C ABI against the CPU oracle (needs a B200).

Mirrors spec/block_matmul_spec.cr:244-297, spec/llama_spec.cr, spec/gpt2_spec.cr and
spec/batched_decode_spec.cr.  In the exact mode (the default) every logit has the oracle's bits, so
greedy sequences are identical by construction.  The fast mode adds in another order, and a sum that
differs in its last bit can move an activation across a rounding boundary of the 8-bit quantiser that
feeds the next product; one such flip alone moves a logit of these small models by about 3e-3 of the
largest.  So the fast mode is held to the budget the reference holds its own GPU to against its CPU
(spec/block_matmul_spec.cr:262-273): at most 0.001 nats of KL divergence per token, and logits within
5e-2 relative of the largest.
"""
import numpy as np
import pytest

import helpers
from helpers import bits, golden, oracle, pkg, rel_max

pytestmark = pytest.mark.gpu
FAST_REL = 5e-2
FAST_KL = 1e-3


def kl_per_token(want, got):
    """Mean KL(softmax(want) || softmax(got)) in nats, as the reference's budget is stated."""
    def log_softmax(x):
        x = x.astype(np.float64)
        x = x - x.max(axis=-1, keepdims=True)
        return x - np.log(np.exp(x).sum(axis=-1, keepdims=True))
    lw, lg = log_softmax(want), log_softmax(got)
    return float((np.exp(lw) * (lw - lg)).sum(axis=-1).mean())


def check(mode, got, want, what=None):
    if mode == pkg.EXACT:
        assert np.array_equal(bits(got), bits(want)), what
    else:
        assert rel_max(got, want) <= FAST_REL and kl_per_token(want, got) <= FAST_KL, (what, rel_max(got, want), kl_per_token(want, got))


@pytest.fixture(scope="module")
def dev():
    d = pkg.B200(0)
    yield d
    d.close()


def write_golden(tmp_path, key, name):
    path = tmp_path / name
    path.write_bytes(golden()[key].tobytes())
    return str(path)


@pytest.mark.parametrize("name", ["q8_0", "q4_0"])
def test_tiny_llama_gguf(dev, tmp_path, name):
    g = golden()
    path = write_golden(tmp_path, f"tiny_llama/{name}_gguf", f"model-{name}.gguf")
    ref = helpers.oracle_llama(path)
    model = pkg.Llama.load(path, dev)
    assert model.config["layers"] == 2 and model.config["kv_heads"] == 2 and model.config["head_width"] == 8
    prompt = g["tiny_llama/prompt_ids"].tolist()
    want = ref.forward(ref.new_cache(1, 64), [prompt], last=False)
    for mode in (pkg.EXACT, pkg.FAST):
        dev.set_mode(mode)
        cache = model.new_batch_cache(1, 64)
        check(mode, model.forward([prompt], cache), want, "prefill")
        # prefill == decode (spec/block_matmul_spec.cr:253-260)
        cache2 = model.new_batch_cache(1, 64)
        rows = np.stack([model.forward_last([[t]], cache2)[0] for t in prompt])
        check(mode, rows, want, "decode")
        if mode == pkg.EXACT:
            assert model.generate(prompt, 20) == ref.generate(prompt, 20)
        cache.free(), cache2.free()
    dev.set_mode(pkg.EXACT)
    assert dev.counters()["host_ops"] == 0
    model.free()


def test_tiny_llama_f32_gguf_matches_pytorch_logits(dev, tmp_path):
    """spec/llama_spec.cr:50-87 on the device: the reference's F32 fixture through the unquantised product.  Logits within
    1e-4 of PyTorch's and greedy tokens equal (the fixture), the oracle's bits, prefill == decode."""
    g = golden()
    path = write_golden(tmp_path, "tiny_llama/f32_gguf", "model.gguf")
    ref = helpers.oracle_llama(path)
    model = pkg.Llama.load(path, dev)
    assert model.tensor("0.qkv")[1] == pkg.F32 and model.tensor("embed")[1] == pkg.F32
    prompt = g["tiny_llama/prompt_ids"].tolist()
    cache = model.new_batch_cache(1, 64)
    got = model.forward([prompt], cache)
    assert np.max(np.abs(got - g["tiny_llama/logits"])) < 1e-4
    check(pkg.EXACT, got, ref.forward(ref.new_cache(1, 64), [prompt], last=False), "prefill")
    cache2 = model.new_batch_cache(1, 64)
    rows = np.stack([model.forward_last([[t]], cache2)[0] for t in prompt])
    assert np.array_equal(bits(rows), bits(got))
    assert model.generate(prompt, 20) == g["tiny_llama/greedy"].tolist()
    assert dev.counters()["host_ops"] == 0
    cache.free(), cache2.free()
    model.free()


@pytest.mark.parametrize("name", ["q4_0", "f32"])
def test_a_saved_llama_is_the_file_it_was_loaded_from(dev, tmp_path, name):
    """Module#save("model.gguf"): the tensors go out under llama.cpp's names with q and k rows back in llama.cpp's order, so
    every tensor of the reference's fixture comes back byte for byte, the metadata the loader reads is kept, and the saved
    file loads to the same logits."""
    g = golden()
    path = write_golden(tmp_path, f"tiny_llama/{name}_gguf", f"model-{name}.gguf")
    model = pkg.Llama.load(path, dev)
    saved = str(tmp_path / "saved.gguf")
    model.save(saved)
    a, b = helpers.gguf.File(path), helpers.gguf.File(saved)
    assert sorted(a.entries) == sorted(b.entries)
    for tensor in a.entries:
        ka, sa, ra = a.raw(tensor)
        kb, sb, rb = b.raw(tensor)
        assert ka == kb and list(sa) == list(sb) and ra.tobytes() == rb.tobytes(), tensor
    for key, value in b.metadata.items():
        assert a.metadata[key] == pytest.approx(value), key
    again = pkg.Llama.load(saved, dev)
    assert again.config == model.config
    prompt = g["tiny_llama/prompt_ids"].tolist()
    want = model.forward([prompt], model.new_batch_cache(1, 64))
    assert np.array_equal(bits(again.forward([prompt], again.new_batch_cache(1, 64))), bits(want))
    model.free(), again.free()


def test_a_gpt2_quantised_on_the_device_saves_ggmls_bytes(dev, tmp_path):
    """model.quantize(Q8_0, embeddings: true).save("model.gguf") (module.cr:154-156): the file holds the bytes of the
    oracle's quantiser under tensomite's names and loads to the same logits."""
    g = golden()
    path = tmp_path / "model.safetensors"
    path.write_bytes(g["tiny_gpt2/safetensors"].tobytes())
    st = helpers.read_safetensors(g["tiny_gpt2/safetensors"])
    model = pkg.GPT2.load_safetensors(path, dev, dict(arch="gpt2", heads=4), pkg.Q8_0)
    saved = str(tmp_path / "saved.gguf")
    model.save(saved)
    want_path = str(tmp_path / "want.gguf")
    helpers.write_gpt2_gguf(want_path, st, 2, 4, oracle.Q8_0)
    a, b = helpers.gguf.File(want_path), helpers.gguf.File(saved)
    assert sorted(a.entries) == sorted(b.entries)
    for tensor in a.entries:
        ka, sa, ra = a.raw(tensor)
        kb, sb, rb = b.raw(tensor)
        assert ka == kb and list(sa) == list(sb) and ra.tobytes() == rb.tobytes(), tensor
    assert b.metadata["gpt2.heads"] == "4"
    again = pkg.GPT2.load(saved, dev)
    prompt = g["tiny_gpt2/prompt_ids"].tolist()
    want = model.forward([prompt], model.new_batch_cache(1, 64))
    assert np.array_equal(bits(again.forward([prompt], again.new_batch_cache(1, 64))), bits(want))
    model.free(), again.free()


@pytest.mark.parametrize("half", ["F16", "BF16"])
def test_tiny_llama_gguf_with_half_matrices_is_widened(dev, tmp_path, half):
    """gguf.cr:112-136: F16 / BF16 tensors widen to F32 at load; the model then runs as the F32 one over the widened values."""
    g = golden()
    gg = helpers.gguf
    src = gg.File(write_golden(tmp_path, "tiny_llama/f32_gguf", "model.gguf"))
    tensors = []
    for name, (kind, shape, _) in src.entries.items():
        values = src.f32(name)
        if len(shape) == 2:
            if half == "F16":
                tensors.append((name, gg.F16, list(shape), values.astype(np.float16)))
            else:
                tensors.append((name, gg.BF16, list(shape), (values.view(np.uint32) >> 16).astype(np.uint16)))
        else:
            tensors.append((name, gg.F32, list(shape), values))
    path = str(tmp_path / f"model-{half}.gguf")
    gg.write(path, {k: v for k, v in src.metadata.items() if not isinstance(v, list)}, tensors)  # the tokeniser's lists are not needed
    ref = helpers.oracle_llama(path)
    model = pkg.Llama.load(path, dev)
    assert model.tensor("0.down")[1] == pkg.F32
    prompt = g["tiny_llama/prompt_ids"].tolist()
    want = ref.forward(ref.new_cache(1, 64), [prompt], last=False)
    check(pkg.EXACT, model.forward([prompt], model.new_batch_cache(1, 64)), want)
    assert model.generate(prompt, 12) == ref.generate(prompt, 12)
    model.free()


def test_tiny_gpt2_f32_safetensors_matches_pytorch_logits(dev, tmp_path):
    """spec/gpt2_spec.cr:54-102 on the device: GPT2.load("model.safetensors") kept in F32."""
    g = golden()
    path = tmp_path / "model.safetensors"
    path.write_bytes(g["tiny_gpt2/safetensors"].tobytes())
    st = helpers.read_safetensors(g["tiny_gpt2/safetensors"])
    config = dict(arch="gpt2", layers=2, heads=4, kv_heads=4, width=32, head_width=8, hidden=128, context=64, vocab=400, eps=1e-5)
    ref = oracle.Model(config, helpers.gpt2_tensors_from_hf(st, 2))
    model = pkg.GPT2.load_safetensors(path, dev, dict(arch="gpt2", heads=4), pkg.F32)
    prompt = g["tiny_gpt2/prompt_ids"].tolist()
    got = model.forward([prompt], model.new_batch_cache(1, 64))
    assert np.max(np.abs(got - g["tiny_gpt2/logits"])) < 1e-4
    check(pkg.EXACT, got, ref.forward(ref.new_cache(1, 64), [prompt], last=False))
    assert model.generate(prompt, 20) == g["tiny_gpt2/greedy"].tolist()
    model.free()


def test_an_f32_gpt2_saves_its_linears_as_the_module_holds_them(dev, tmp_path):
    """GPT2.load("model.safetensors").save("model.gguf") without quantising: under tensomite's names an unquantised Linear
    weight is [inputs, outputs] (modules.cr:1-20; Module#load reverses the shape for block formats only,
    module.cr:217-228), so the file holds Hugging Face's Conv1D matrices as they are, and loads back to the same logits."""
    g = golden()
    path = tmp_path / "model.safetensors"
    path.write_bytes(g["tiny_gpt2/safetensors"].tobytes())
    st = helpers.read_safetensors(g["tiny_gpt2/safetensors"])
    model = pkg.GPT2.load_safetensors(path, dev, dict(arch="gpt2", heads=4), pkg.F32)
    saved = str(tmp_path / "saved.gguf")
    model.save(saved)
    f = helpers.gguf.File(saved)
    for i in range(2):
        for name in ("attn.c_attn", "attn.c_proj", "mlp.c_fc", "mlp.c_proj"):
            hf = st[f"transformer.h.{i}.{name}.weight"]          # Conv1D: [inputs, outputs]
            kind, shape, _ = f.raw(f"h.{i}.{name}.weight")
            assert kind == helpers.gguf.F32 and list(shape) == list(hf.shape), (name, shape)
            assert np.array_equal(bits(f.f32(f"h.{i}.{name}.weight").reshape(hf.shape)), bits(hf))
    assert list(f.raw("wte.weight")[1]) == list(st["transformer.wte.weight"].shape)
    again = pkg.GPT2.load(saved, dev)
    prompt = g["tiny_gpt2/prompt_ids"].tolist()
    want = model.forward([prompt], model.new_batch_cache(1, 64))
    got = again.forward([prompt], again.new_batch_cache(1, 64))
    assert np.array_equal(bits(got), bits(want))
    assert np.max(np.abs(got - g["tiny_gpt2/logits"])) < 1e-4
    model.free(), again.free()


def test_tiny_gpt2_q8_0_with_f32_embeddings(dev, tmp_path):
    """Module#quantize(Q8_0) without embeddings: the tables stay F32, so the tied head is an F32 product fed by F32 rows
    while every layer reads quantised ones."""
    g = golden()
    st = helpers.read_safetensors(g["tiny_gpt2/safetensors"])
    path = str(tmp_path / "gpt2-q8_0-f32-tables.gguf")
    tensors = helpers.write_gpt2_gguf(path, st, 2, 4, oracle.Q8_0, embeddings=False)
    config = dict(arch="gpt2", layers=2, heads=4, kv_heads=4, width=32, head_width=8, hidden=128, context=64, vocab=400, eps=1e-5)
    ref = oracle.Model(config, tensors)
    model = pkg.GPT2.load(path, dev)
    assert model.tensor("embed")[1] == pkg.F32 and model.tensor("0.qkv")[1] == pkg.Q8_0
    prompt = g["tiny_gpt2/prompt_ids"].tolist()
    want = ref.forward(ref.new_cache(1, 64), [prompt], last=False)
    check(pkg.EXACT, model.forward([prompt], model.new_batch_cache(1, 64)), want)
    assert model.generate(prompt, 20) == ref.generate(prompt, 20)
    model.free()


def test_tiny_gpt2_q8_0_with_quantised_embeddings(dev, tmp_path):
    g = golden()
    st = helpers.read_safetensors(g["tiny_gpt2/safetensors"])
    path = str(tmp_path / "gpt2-q8_0.gguf")
    tensors = helpers.write_gpt2_gguf(path, st, 2, 4, oracle.Q8_0)
    config = dict(arch="gpt2", layers=2, heads=4, kv_heads=4, width=32, head_width=8, hidden=128, context=64, vocab=400, eps=1e-5)
    ref = oracle.Model(config, tensors)
    model = pkg.GPT2.load(path, dev)
    assert model.config["arch"] == "gpt2" and model.config["layers"] == 2 and model.config["context"] == 64
    prompt = g["tiny_gpt2/prompt_ids"].tolist()
    want = ref.forward(ref.new_cache(1, 64), [prompt], last=False)
    got = model.forward([prompt], model.new_batch_cache(1, 64))
    check(pkg.EXACT, got, want)
    assert model.generate(prompt, 20) == ref.generate(prompt, 20)
    dev.set_mode(pkg.FAST)
    try:
        check(pkg.FAST, model.forward([prompt], model.new_batch_cache(1, 64)), want)
    finally:
        dev.set_mode(pkg.EXACT)
    model.free()


def test_gpt2_from_safetensors_quantised_on_the_device(dev, tmp_path):
    """GPT2.load("model.safetensors").quantize(Q8_0, embeddings: true): Hugging Face names, Conv1D weights transposed, the
    device's quantiser; logits against the oracle over the oracle-quantised tensors, bit for bit."""
    g = golden()
    path = tmp_path / "model.safetensors"
    path.write_bytes(g["tiny_gpt2/safetensors"].tobytes())
    st = helpers.read_safetensors(g["tiny_gpt2/safetensors"])
    config = dict(arch="gpt2", layers=2, heads=4, kv_heads=4, width=32, head_width=8, hidden=128, context=64, vocab=400, eps=1e-5)
    ref = oracle.Model(config, helpers.gpt2_tensors_from_hf(st, 2, quantize_kind=oracle.Q8_0, embeddings=True))
    model = pkg.GPT2.load_safetensors(path, dev, dict(arch="gpt2", heads=4), pkg.Q8_0)
    assert {k: model.config[k] for k in ("layers", "width", "hidden", "context", "vocab")} == dict(layers=2, width=32, hidden=128, context=64, vocab=400)
    prompt = g["tiny_gpt2/prompt_ids"].tolist()
    want = ref.forward(ref.new_cache(1, 64), [prompt], last=False)
    check(pkg.EXACT, model.forward([prompt], model.new_batch_cache(1, 64)), want)
    assert model.generate(prompt, 20) == ref.generate(prompt, 20)
    model.free()
    with pytest.raises(pkg.Error):
        pkg.GPT2.load_safetensors(tmp_path / "absent.safetensors", dev, dict(arch="gpt2", heads=4), pkg.Q8_0)


@pytest.mark.parametrize("kind,tied", [(pkg.Q4_0, True), (pkg.Q4_1, False)])
def test_llama_from_safetensors_quantised_on_the_device(dev, tmp_path, kind, tied):
    rng = np.random.default_rng(21)
    layers, width, heads, kv_heads, hw, hidden, vocab = 2, 128, 4, 2, 32, 256, 512
    st = {"model.embed_tokens.weight": rng.normal(0, 0.02, (vocab, width)), "model.norm.weight": rng.normal(1, 0.1, width)}
    if not tied:
        st["lm_head.weight"] = rng.normal(0, 0.02, (vocab, width))
    for i in range(layers):
        p = f"model.layers.{i}."
        st[p + "input_layernorm.weight"] = rng.normal(1, 0.1, width)
        st[p + "post_attention_layernorm.weight"] = rng.normal(1, 0.1, width)
        st[p + "self_attn.q_proj.weight"] = rng.normal(0, 0.02, (heads * hw, width))
        st[p + "self_attn.k_proj.weight"] = rng.normal(0, 0.02, (kv_heads * hw, width))
        st[p + "self_attn.v_proj.weight"] = rng.normal(0, 0.02, (kv_heads * hw, width))
        st[p + "self_attn.o_proj.weight"] = rng.normal(0, 0.02, (width, heads * hw))
        st[p + "mlp.gate_proj.weight"] = rng.normal(0, 0.02, (hidden, width))
        st[p + "mlp.up_proj.weight"] = rng.normal(0, 0.02, (hidden, width))
        st[p + "mlp.down_proj.weight"] = rng.normal(0, 0.02, (width, hidden))
    st = {k: np.asarray(v, dtype=np.float32) for k, v in st.items()}
    path = tmp_path / "model.safetensors"
    helpers.write_safetensors(path, st)
    config = dict(arch="llama", layers=layers, width=width, heads=heads, kv_heads=kv_heads, head_width=hw, hidden=hidden, vocab=vocab,
                  context=128, eps=1e-5, rope_theta=10000.0, tied=tied)
    ref = oracle.Model(config, helpers.llama_tensors_from_hf(st, layers, kind))
    model = pkg.Llama.load_safetensors(path, dev, dict(arch="llama", heads=heads, kv_heads=kv_heads, context=128, eps=1e-5, rope_theta=10000.0), kind)
    assert model.config["hidden"] == hidden and model.config["tied"] == (1 if tied else 0)
    prompt = rng.integers(0, vocab, size=24).tolist()
    want = ref.forward(ref.new_cache(1, 64), [prompt], last=False)
    check(pkg.EXACT, model.forward([prompt], model.new_batch_cache(1, 64)), want)
    assert model.generate(prompt, 16) == ref.generate(prompt, 16)
    model.free()


SMALL = dict(layers=2, width=256, heads=4, kv_heads=2, head_width=64, hidden=512, vocab=1024, context=256,
             eps=1e-5, rope_theta=10000.0, tied=True)


@pytest.mark.parametrize("arch,kind", [("llama", pkg.Q8_0), ("llama", pkg.Q4_0), ("llama", pkg.Q4_1), ("gpt2", pkg.Q8_0),
                                       ("gpt2", pkg.Q4_1)])
def test_random_model_batched_decode(dev, arch, kind):
    """A device-made random model against the oracle over the same (downloaded) weights: ragged
    prompts with an idle row, then graph-replayed decode steps, then a reset row
    (spec/batched_decode_spec.cr:110-143), then a device-resident run."""
    config = dict(SMALL, arch=arch)
    if arch == "gpt2":
        config.update(kv_heads=4, hidden=1024)
    model = pkg.Model.random(dev, config, kind, seed=7)
    ref = helpers.oracle_from_device_model(model)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 1024, size=n).tolist() for n in (5, 17, 0, 3)]
    for mode in (pkg.EXACT, pkg.FAST):
        dev.set_mode(mode)
        cache, rcache = model.new_batch_cache(4, 64), ref.new_cache(4, 64)
        check(mode, model.forward_last(prompts, cache), ref.forward(rcache, prompts), "prompts")
        # fill the idle row, then decode every row with the replayed step
        check(mode, model.forward_last([[], [], [9, 8], []], cache), ref.forward(rcache, [[], [], [9, 8], []]), "idle row")
        ids = [1, 2, 3, 4]
        for step in range(6):
            tokens, logits = model.decode(cache, ids, logits=True)
            want = ref.forward(rcache, [[t] for t in ids])
            check(mode, logits, want, ("decode", step))
            assert tokens.tolist() == [oracle.argmax_first(r) for r in logits]
            ids = [oracle.argmax_first(r) for r in want]
        assert [cache.length(r) for r in range(4)] == rcache.lengths
        cache.reset(1), rcache.reset(1)
        check(mode, model.forward_last([[], prompts[1], [], []], cache), ref.forward(rcache, [[], prompts[1], [], []]), "after reset")
        if mode == pkg.EXACT:
            run = model.decode_run(cache, [5, 6, 7, 8], 5)
            ids = [5, 6, 7, 8]
            for step in range(5):
                want = ref.forward(rcache, [[t] for t in ids])
                ids = [oracle.argmax_first(r) for r in want]
                assert run[step].tolist() == ids, step
        cache.free()
    dev.set_mode(pkg.EXACT)
    assert dev.counters()["host_ops"] == 0
    model.free()


@pytest.mark.parametrize("capacity", [64, 1100])
def test_heads_of_width_128_in_groups_of_four(dev, capacity):
    """The streaming attention kernels (one launch for short caches, three for a long cache with few streams), which also
    write the quantised rows the next product reads: whole-model logits against the oracle, bit for bit."""
    config = dict(arch="llama", layers=2, width=512, heads=8, kv_heads=2, head_width=128, hidden=512, vocab=1024, context=2048,
                  eps=1e-5, rope_theta=10000.0, tied=True)
    model = pkg.Model.random(dev, config, pkg.Q4_0, seed=11)
    ref = helpers.oracle_from_device_model(model)
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, 1024, size=n).tolist() for n in (9, 40, 3)]
    cache, rcache = model.new_batch_cache(3, capacity), ref.new_cache(3, capacity)
    check(pkg.EXACT, model.forward_last(prompts, cache), ref.forward(rcache, prompts), "prompts")
    ids = [5, 6, 7]
    for step in range(4):
        tokens, logits = model.decode(cache, ids, logits=True)
        want = ref.forward(rcache, [[t] for t in ids])
        check(pkg.EXACT, logits, want, ("decode", step))
        ids = [oracle.argmax_first(r) for r in want]
        assert tokens.tolist() == ids
    cache.free()
    model.free()


def test_generate_matches_the_oracle_token_for_token(dev):
    config = dict(SMALL, arch="llama", layers=3, vocab=2048)
    model = pkg.Model.random(dev, config, pkg.Q8_0, seed=3)
    ref = helpers.oracle_from_device_model(model)
    prompt = np.random.default_rng(7).integers(0, 2048, size=32).tolist()
    want = ref.generate(prompt, 48)
    assert model.generate(prompt, 48) == want
    model.free()


def test_errors_are_raised_not_trapped(dev, tmp_path):
    config = dict(SMALL, arch="llama")
    model = pkg.Model.random(dev, config, pkg.Q8_0, seed=1)
    cache = model.new_batch_cache(2, 8)
    with pytest.raises(pkg.ExecutionError):
        model.forward_last([[5000], [1]], cache)          # a token id beyond the vocabulary
    cache.reset(0), cache.reset(1)
    with pytest.raises(pkg.ShapeError, match="positions exceed"):
        model.forward_last([list(range(9)), []], cache)   # more positions than a row holds
    with pytest.raises(pkg.ShapeError, match="forward of no tokens"):
        model.forward_last([[], []], cache)
    assert model.forward_last([[1, 2], [3]], cache).shape == (2, 1024)
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"not a gguf file at all, just text")
    with pytest.raises(pkg.Error):
        pkg.Llama.load(str(bad), dev)
    model.free()


def test_prompts_through_the_prefill_attention_kernel_have_the_decode_bits(dev):
    """spec/block_matmul_spec.cr:253-260 at a shape the prefill attention kernel takes (heads of width 128, four query heads
    per key/value head, eight layers): prompts of 150 and 37 tokens in one packed step (tiles of 16 tokens, a last tile
    that is not full, a row that stays idle), then a second chunk of 40 tokens on top of the first row's cache, give every
    position the logits it has when the tokens are fed one by one, bit for bit, and the oracle's."""
    config = dict(arch="llama", layers=8, width=1024, heads=8, kv_heads=2, head_width=128, hidden=2048, vocab=2048, context=512,
                  eps=1e-5, rope_theta=500000.0, tied=False)
    model = pkg.Model.random(dev, config, pkg.Q4_0, seed=77)
    rng = np.random.default_rng(8)
    first = rng.integers(0, config["vocab"], size=150).tolist()
    other = rng.integers(0, config["vocab"], size=37).tolist()
    more = rng.integers(0, config["vocab"], size=40).tolist()
    cache = model.new_batch_cache(3, 256)
    got = model.forward([first, [], other], cache)                 # 187 tokens, one step
    got_more = model.forward([more, [], []], cache)                # 40 more on a cache that already holds 150
    step = model.new_batch_cache(3, 256)
    rows = []
    for t in first:
        rows.append(model.forward_last([[t], [], []], step)[0])
    for t in other:
        rows.append(model.forward_last([[], [], [t]], step)[0])
    assert np.array_equal(bits(got), bits(np.stack(rows)))
    rows = [model.forward_last([[t], [], []], step)[0] for t in more]
    assert np.array_equal(bits(got_more), bits(np.stack(rows)))
    ref = oracle.model_from_device(model, threads=8)
    rcache = ref.new_cache(1, 256)
    want = ref.forward(rcache, [first], last=False)
    assert np.array_equal(bits(got[:150]), bits(want))
    cache.free(), step.free(), model.free()


@pytest.mark.gpu
@pytest.mark.parametrize("arch", ["llama", "gpt2"])
def test_decode_steps_that_rotate_and_append_inside_attention_have_the_prompt_bits(dev, arch):
    """A step of at most four rows with one token each leaves RoPE and the cache append (modules.cr:434-452, 194-217) to the
    attention kernel: every CTA rotates its query heads and its key as it loads them, one CTA per key/value head writes the
    cache, the others (here two groups of four query heads share the one key/value head) use their own copy.  Tokens fed that
    way, three rows at a time, must give the logits of the same tokens fed as packed prompts (separate rope + append launch),
    bit for bit, and the oracle's; and the cache they leave must serve a later packed step."""
    config = dict(arch=arch, layers=3, width=512, heads=8, kv_heads=1 if arch == "llama" else 8, head_width=64, hidden=1024, vocab=512,
                  context=128, eps=1e-5, rope_theta=10000.0, tied=True)
    model = pkg.Model.random(dev, config, pkg.Q8_0, seed=5)
    rng = np.random.default_rng(12)
    prompts = [rng.integers(0, config["vocab"], size=n).tolist() for n in (9, 1, 6)]
    steps = [rng.integers(0, config["vocab"], size=3).tolist() for _ in range(5)]
    tail = [rng.integers(0, config["vocab"], size=7).tolist() for _ in range(3)]
    packed = model.new_batch_cache(5, 64)                                      # two more rows: steps of 5 tokens take the separate launch
    model.forward_last(prompts + [[1], [2]], packed)
    want = [model.forward_last([[t] for t in step] + [[3], [4]], packed)[:3] for step in steps]
    want_tail = model.forward(tail + [[], []], packed)
    fed = model.new_batch_cache(3, 64)
    model.forward_last(prompts, fed)
    got = [model.forward_last([[t] for t in step], fed) for step in steps]     # one token per row: the fused path
    for a, b in zip(got, want):
        assert np.array_equal(bits(a), bits(b))
    assert np.array_equal(bits(model.forward(tail, fed)), bits(want_tail))     # 21 tokens over the cache the fused steps wrote
    ref = oracle.model_from_device(model, threads=4)
    rcache = ref.new_cache(1, 64)
    row0 = prompts[0] + [step[0] for step in steps]
    logits = ref.forward(rcache, [row0], last=False)
    assert np.array_equal(bits(got[-1][0]), bits(logits[-1]))
    packed.free(), fed.free(), model.free()
