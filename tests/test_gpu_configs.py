"""The baseline's own configurations, whole and at full size, against the CPU oracle (needs a B200).

Each model is drawn on the device from a seed (normal(0, 0.02), quantised on the device), downloaded through the C ABI
and rebuilt over the very same block bytes on the host, so that both sides hold the same weights; prompts are seeded
uniform token ids.  The device decodes in its default (exact) mode, so the greedy sequence has to be the oracle's token
for token over the whole generation, and the logits of the last step bit for bit
(spec/llama_spec.cr:122-159, spec/block_matmul_spec.cr:253-297 on small models; these are the sizes the baseline names).
"""
import os

import numpy as np
import pytest

from helpers import bits, oracle, pkg

pytestmark = pytest.mark.gpu
THREADS = os.cpu_count() or 1

C1 = dict(arch="llama", layers=30, width=576, heads=9, kv_heads=3, head_width=64, hidden=1536, vocab=49152, context=8192, eps=1e-5,
          rope_theta=10000.0, tied=True)
C3 = dict(arch="llama", layers=24, width=2048, heads=32, kv_heads=32, head_width=64, hidden=8192, vocab=49152, context=8192, eps=1e-5,
          rope_theta=130000.0, tied=True)
C4 = dict(arch="gpt2", layers=48, width=1600, heads=25, kv_heads=25, head_width=64, hidden=6400, vocab=50257, context=1024, eps=1e-5,
          rope_theta=0.0, tied=True)
C5 = dict(arch="llama", layers=32, width=4096, heads=32, kv_heads=8, head_width=128, hidden=14336, vocab=128256, context=8192, eps=1e-5,
          rope_theta=500000.0, tied=False)


@pytest.fixture(scope="module")
def dev():
    d = pkg.B200(0)
    yield d
    d.close()


def oracle_greedy(ref, prompt, count):
    """Generative#generate with Sampler.greedy on the oracle; also the logits the last token was picked from."""
    cache = ref.new_cache(1, len(prompt) + count)
    logits = ref.forward(cache, [list(prompt)])
    tokens = []
    for i in range(count):
        tokens.append(oracle.argmax_first(logits[0]))
        if i < count - 1:
            logits = ref.forward(cache, [[tokens[-1]]])
    return tokens, logits[0]


def device_greedy_with_last_logits(model, prompt, count):
    """The same loop through tsm_forward and the graph-replayed tsm_decode; the last step also returns its logits."""
    cache = model.new_batch_cache(1, len(prompt) + count)
    logits = model.forward_last([list(prompt)], cache)
    tokens = [int(np.argmax(logits[0]))]
    last = logits[0]
    for i in range(1, count):
        if i < count - 1:
            picked = model.decode(cache, [tokens[-1]])
        else:
            picked, out = model.decode(cache, [tokens[-1]], logits=True)
            last = out[0]
        tokens.append(int(picked[0]))
    cache.free()
    return tokens, last


def test_c1_the_135m_shaped_q8_0_model_generates_the_oracles_128_tokens(dev):
    """Configuration 1 exactly: 30 layers, 576 wide, 9 / 3 heads, vocabulary 49152, tied, Q8_0, a 32-token prompt of
    uniform ids, 128 greedy tokens."""
    model = pkg.Model.random(dev, C1, pkg.Q8_0, seed=20260102)
    ref = oracle.model_from_device(model, threads=THREADS)
    prompt = np.random.default_rng(7).integers(0, C1["vocab"], size=32).tolist()
    want, want_last = oracle_greedy(ref, prompt, 128)
    assert model.generate(prompt, 128) == want                       # prefill + the device-resident run
    got, got_last = device_greedy_with_last_logits(model, prompt, 128)  # prefill + 127 graph replays
    assert got == want
    assert np.array_equal(bits(got_last), bits(want_last))
    assert dev.counters()["host_ops"] == 0
    model.free()


def test_c4_the_gpt2_xl_shaped_q8_0_model_generates_the_oracles_tokens(dev):
    """Configuration 4's model (48 layers, 1600 wide, 25 heads, GELU MLP of 6400, learned positions, vocabulary 50257, Q8_0
    with F32 LayerNorms), a 64-token prompt and the first 96 of its greedy tokens."""
    model = pkg.Model.random(dev, C4, pkg.Q8_0, seed=20260104)
    ref = oracle.model_from_device(model, threads=THREADS)
    prompt = np.random.default_rng(7).integers(0, C4["vocab"], size=64).tolist()
    count = 96
    want, want_last = oracle_greedy(ref, prompt, count)
    assert model.generate(prompt, count) == want
    got, got_last = device_greedy_with_last_logits(model, prompt, count)
    assert got == want
    assert np.array_equal(bits(got_last), bits(want_last))
    model.free()


def test_c3_two_streams_of_the_1_7b_shaped_q4_1_model_through_a_real_prefill(dev):
    """Configuration 3's model (24 layers, 2048 wide, 32 heads, SwiGLU 8192, Q4_1), two of its sixteen streams in a
    batch cache of sixteen rows: 128-token prompts through the packed prefill, then 24 greedy steps of the whole batch."""
    model = pkg.Model.random(dev, C3, pkg.Q4_1, seed=20260103)
    ref = oracle.model_from_device(model, threads=THREADS)
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, C3["vocab"], size=128).tolist() for _ in range(16)]
    sampled, steps = [0, 15], 24
    cache = model.new_batch_cache(16, 128 + steps + 1)
    logits = model.forward_last(prompts, cache)                  # 2048 prompt tokens in one packed step
    rcache = ref.new_cache(2, 128 + steps + 1)
    want = ref.forward(rcache, [prompts[r] for r in sampled])
    assert np.array_equal(bits(logits[sampled]), bits(want))
    ids = np.argmax(logits, axis=1).astype(np.int32)
    want_ids = [oracle.argmax_first(row) for row in want]
    for step in range(steps):
        assert [int(ids[r]) for r in sampled] == want_ids, step
        if step < steps - 1:
            ids = model.decode(cache, ids)
        else:
            ids, logits = model.decode(cache, ids, logits=True)
        want = ref.forward(rcache, [[t] for t in want_ids])
        want_ids = [oracle.argmax_first(row) for row in want]
    assert [int(ids[r]) for r in sampled] == want_ids
    assert np.array_equal(bits(logits[sampled]), bits(want))
    cache.free(), model.free()


def test_c5_the_streams_at_the_length_extremes_decode_the_oracles_128_tokens(dev):
    """Configuration 5's model (Llama-3-8B-shaped, Q4_0) decoding a batch whose caches hold seeded values at ragged
    lengths; the streams holding 128 and 4096 positions, the extremes of the workload, are followed on the oracle from
    the same cache contents for all 128 greedy steps."""
    model = pkg.Model.random(dev, C5, pkg.Q4_0, seed=20260101)
    ref = oracle.model_from_device(model, threads=THREADS)
    steps = 128
    lengths = [128, 4096] + np.random.default_rng(11).integers(128, 4097, size=6).tolist()
    cache = model.new_batch_cache(len(lengths), 4096 + steps + 2)
    for row, n in enumerate(lengths):
        cache.fill(row, int(n), seed=1000 + row)
    dev.sync()
    rcache = oracle.cache_from_device(ref, model, cache, [0, 1], lengths[:2], 4096 + steps + 2)
    first = np.random.default_rng(7).integers(0, C5["vocab"], size=len(lengths)).astype(np.int32)
    got = model.decode_run(cache, first, steps)                  # [steps, rows], the loop resident on the device
    ids = [int(first[0]), int(first[1])]
    for step in range(steps):
        logits = ref.forward(rcache, [[ids[0]], [ids[1]]])
        ids = [oracle.argmax_first(logits[0]), oracle.argmax_first(logits[1])]
        assert got[step, :2].tolist() == ids, step
    cache.free(), model.free()
