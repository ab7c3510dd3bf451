"""One small decode through the C ABI on cuda:0, checked against the oracle (used by smoke())."""
import numpy as np


def run(pkg):
    from tests import helpers
    from tests.helpers import oracle
    dev = pkg.B200(0)
    config = dict(arch="llama", layers=2, width=256, heads=4, kv_heads=2, head_width=64, hidden=512, vocab=1024,
                  context=128, eps=1e-5, rope_theta=10000.0, tied=True)
    model = pkg.Model.random(dev, config, pkg.Q4_0, seed=11)
    ref = helpers.oracle_from_device_model(model)
    rng = np.random.default_rng(0)
    # the quantised product alone, bit for bit
    buf, kind, n, k = model.tensor("0.up")
    x = rng.normal(0, 1, (1, k)).astype(np.float32)
    got = dev.block_matmul(x, buf, kind, n)
    want = oracle.matmul_reference(kind, x, buf.numpy(np.uint8), n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "block product differs from the oracle"
    # a prompt and a few greedy tokens
    prompt = rng.integers(0, 1024, size=12).tolist()
    tokens = model.generate(prompt, 8)
    expect = ref.generate(prompt, 8)
    assert tokens == expect, (tokens, expect)
    counters = dev.counters()
    assert counters["launches"] > 0 and counters["host_ops"] == 0
    model.free()
    dev.close()
    print(f"smoke ok: tokens {tokens}, {counters['launches']} kernel launches, {counters['graph_replays']} graph replays")
