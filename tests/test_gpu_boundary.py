"""The rest of the boundary through the C ABI (needs a B200): the region write, generation with a stop list and a host-side
sampler, the per-operator profile, a bounded device wait that runs out, and the failure surface of the tensor-parallel
exchanges.  None of these faults, traps or hangs the GPU: the wait that runs out is a wait for a copy that was never issued,
with the limit lowered to about a millisecond, after which the kernel returns."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import bits, oracle, pkg

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = dict(arch="llama", layers=2, width=256, heads=4, kv_heads=2, head_width=64, hidden=512, vocab=1024, context=128, eps=1e-5,
             rope_theta=10000.0, tied=True)


@pytest.fixture(scope="module")
def dev():
    d = pkg.B200(0)
    yield d
    d.close()


def test_region_write_is_the_single_stream_caches_append(dev):
    """Tensor#write (tensor/structural.cr:64-74): a cache [1, heads, capacity, width] takes new keys at `start` along axis 2;
    other axes and a last-axis write too."""
    rng = np.random.default_rng(31)
    cache = rng.normal(0, 1, (1, 3, 16, 8)).astype(np.float32)
    new = rng.normal(0, 1, (1, 3, 5, 8)).astype(np.float32)
    want = cache.copy()
    want[:, :, 7:12, :] = new
    assert np.array_equal(bits(dev.write(cache, new, 2, 7)), bits(want))
    table = rng.normal(0, 1, (4, 2)).astype(np.float32)
    want = table.copy()
    want[1] = [1, 2]
    assert np.array_equal(dev.write(table, np.array([[1, 2]], dtype=np.float32), 0, 1), want)   # the reference's own example
    wide = rng.normal(0, 1, (3, 4, 10)).astype(np.float32)
    part = rng.normal(0, 1, (3, 4, 3)).astype(np.float32)
    want = wide.copy()
    want[:, :, 7:] = part
    assert np.array_equal(bits(dev.write(wide, part, -1, 7)), bits(want))
    with pytest.raises(pkg.ShapeError):
        dev.write(wide, part, 2, 8)


def test_generate_stops_at_a_stop_token_and_hands_the_samplers_candidates_over(dev):
    """Generative#generate(prompt, count, sampler, stop) (generative.cr:177-190): greedy with a stop list ends after the stop
    token; with a sampler the host's pick sees, at every step, the top_k candidates in Sampler#top's order (highest first,
    equal logits by lower index; sampler.cr:77-96) with the oracle's logits, and its choice is what the model is fed."""
    model = pkg.Model.random(dev, SMALL, pkg.Q8_0, seed=5)
    ref = oracle.model_from_device(model)
    prompt = np.random.default_rng(3).integers(0, SMALL["vocab"], size=9).tolist()
    greedy = ref.generate(prompt, 24)
    assert model.generate_sampled(prompt, 24) == greedy
    stop_at = greedy[6]
    first = greedy.index(stop_at)
    assert model.generate_sampled(prompt, 24, stop=[stop_at, 99999]) == greedy[:first + 1]
    # a sampler that always takes its third candidate: the oracle follows the same rule
    seen = []

    def third(step, ids, logits):
        seen.append((ids.tolist(), logits.copy()))
        return int(ids[2])

    got = model.generate_sampled(prompt, 10, pick=third, top_k=5)
    cache = ref.new_cache(1, 64)
    logits = ref.forward(cache, [prompt])
    want = []
    for step in range(10):
        order = oracle.topk(logits[0], 5)
        assert seen[step][0] == order.tolist(), step
        assert np.array_equal(bits(seen[step][1]), bits(logits[0][order])), step
        want.append(int(order[2]))
        logits = ref.forward(cache, [[want[-1]]])
    assert got == want
    # top_k = 0: the whole row in index order, and the greedy rule applied on the host gives the greedy tokens
    rows = []

    def first_max(step, ids, logits):
        assert ids is None and logits.size == SMALL["vocab"]
        rows.append(logits.copy())
        return int(np.argmax(logits))

    assert model.generate_sampled(prompt, 6, pick=first_max) == greedy[:6]
    model.free()


def test_profile_gives_gpu_time_per_operator(dev):
    """CUDA::Profile with per_kernel and shapes (cuda.cr:256-303): launches and GPU seconds per operator and shape."""
    model = pkg.Model.random(dev, SMALL, pkg.Q4_0, seed=6)
    cache = model.new_batch_cache(2, 32)
    model.forward_last([[1, 2, 3], [4]], cache)
    want = model.decode(cache, [5, 6])
    cache.reset(0), cache.reset(1)
    model.forward_last([[1, 2, 3], [4]], cache)
    dev.profile(shapes=True)
    got = model.decode(cache, [5, 6])              # launched kernel by kernel under the profile: the same tokens
    table = dev.profile_read(end=True)
    assert got.tolist() == want.tolist()
    labels = {label: (count, seconds) for label, count, seconds in table}
    # a decode step of a few rows: the attention kernel rotates q and k and appends to the cache itself
    assert labels["Rope+WriteRows+RaggedAttention [2,4,64]"][0] == SMALL["layers"]
    assert labels["BlockMatMul q4_0 [2,256,1024]"][0] == SMALL["layers"] + 1   # gate/up of every layer, and the head: 1024 rows each
    assert labels["RMSNorm [2,256]"][0] == 2 * SMALL["layers"] + 1
    assert all(seconds > 0 for _, seconds in labels.values())
    assert [s for _, _, s in table] == sorted((s for _, _, s in table), reverse=True)
    dev.profile(shapes=False)
    model.decode(cache, got)
    plain = dict((label, count) for label, count, _ in dev.profile_read(end=True))
    assert plain["BlockMatMul q4_0"] == 4 * SMALL["layers"] + 1 and "Rope+WriteRows+RaggedAttention" in plain
    assert model.decode(cache, got).size == 2      # and the graph replay is back afterwards
    cache.free(), model.free()


def test_a_device_wait_that_runs_out_returns_a_timeout_and_the_context_lives_on(dev):
    """Every wait of the kernels on an asynchronous copy is bounded.  Here the copy thread of a batched product leaves out its
    last stage and the limit is lowered: the warps waiting for that stage give up, the kernel returns, tsm_sync reports
    TSM_ERR_TIMEOUT and clears the record, and the next product has the oracle's bits again."""
    rng = np.random.default_rng(41)
    kind, rows, n, k = oracle.Q4_0, 16, 512, 2048
    w = oracle.quantize(kind, rng.normal(0, 0.02, n * k).astype(np.float32))
    x = rng.normal(0, 1, (rows, k)).astype(np.float32)
    wb = dev.tensor(w)
    want = oracle.matmul_reference(kind, x, w, n)
    assert np.array_equal(bits(dev.block_matmul(x, wb, kind, n)), bits(want))
    dev.debug_wait_limit(20000, 1)
    try:
        with pytest.raises(pkg.TimeoutError_, match="wait"):
            dev.block_matmul(x, wb, kind, n)
    finally:
        dev.debug_wait_limit(0, 0)
    dev.sync()                                      # the record was cleared with the report
    assert np.array_equal(bits(dev.block_matmul(x, wb, kind, n)), bits(want))
    wb.free()


def test_a_failing_exchange_is_a_comm_error(tmp_path):
    """The tensor-parallel exchanges against a stand-in NCCL whose collectives report a remote error (a peer that died):
    the step returns TSM_ERR_COMM at once, later exchanges are refused, and tsm_tp_abort leaves the context usable."""
    stub = str(tmp_path / "libnccl_stub.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", stub, os.path.join(ROOT, "tests", "nccl_stub.c")], check=True)
    script = r'''
import sys
sys.path.insert(0, %r); sys.path.insert(0, %r)
from helpers import pkg
dev = pkg.B200(0)
dev.tp_init(0, 2, pkg.tp_unique_id())
config = dict(arch="llama", layers=2, width=256, heads=4, kv_heads=2, head_width=64, hidden=512, vocab=1024, context=128, eps=1e-5, rope_theta=10000.0, tied=True)
model = pkg.Model.random(dev, config, pkg.Q8_0, seed=5)
cache = model.new_batch_cache(1, 32)
for attempt in range(2):
    try:
        model.forward_last([[1, 2, 3]], cache)
        print("no error")
    except pkg.CommError as problem:
        print("CommError", attempt, problem)
print("collectives", dev.counters()["collectives"])
dev.tp_abort()
dev.sync()
print("alive", dev.tp_info())
''' % (ROOT, os.path.join(ROOT, "tests"))
    env = dict(os.environ, TSM_NCCL_LIBRARY=stub)
    done = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
    assert "CommError 0" in done.stdout and "ncclAllGather" in done.stdout and "remote process exited" in done.stdout
    assert "CommError 1" in done.stdout and "no error" not in done.stdout
    assert "collectives 0" in done.stdout and "alive (0, 2)" in done.stdout
