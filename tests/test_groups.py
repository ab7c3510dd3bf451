"""Host-side logic of the multi-GPU paths, run as two gloo ranks on the CPU."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from tests import helpers  # noqa: E402

pkg = helpers.load_package()
groups = pkg.groups

LLAMA8B = dict(arch="llama", heads=32, kv_heads=8, head_width=128, width=4096, hidden=14336, vocab=128256)


def test_stream_shares_cover_every_row_once():
    for streams in (1, 16, 63, 64):
        for world in (1, 2, 4, 8):
            seen = []
            for rank in range(world):
                first, count = groups.stream_share(streams, world, rank)
                seen += list(range(first, first + count))
            assert seen == list(range(streams))
            sizes = [groups.stream_share(streams, world, r)[1] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def test_shards_tile_every_projection_and_keep_heads_whole():
    for world in (1, 2, 4, 8):
        rows = {}
        for rank in range(world):
            for name, ranges in groups.shard_rows(LLAMA8B, world, rank).items():
                rows.setdefault(name, []).extend(r for a, b in ranges for r in range(a, b))
        qn, kvn = 32 * 128, 8 * 128
        assert sorted(rows["qkv"]) == list(range(qn + 2 * kvn))
        assert sorted(rows["up"]) == list(range(2 * 14336))
        assert sorted(rows["o"]) == sorted(rows["down"]) == list(range(4096))
        assert sorted(rows["head"]) == list(range(128256))
        for rank in range(world):
            for a, b in groups.shard_rows(LLAMA8B, world, rank)["qkv"]:
                assert a % 128 == 0 and b % 128 == 0
    with pytest.raises(ValueError):
        groups.shard_rows(dict(LLAMA8B, kv_heads=3), 2, 0)


def test_combined_pick_is_the_first_maximum():
    rng = np.random.default_rng(3)
    logits = rng.integers(-5, 5, size=(7, 64)).astype(np.float32)  # many ties
    for world in (2, 4, 8):
        width = 64 // world
        parts = logits.reshape(7, world, width)
        values = parts.max(axis=2).T
        indices = parts.argmax(axis=2).T
        got = groups.combine_picks(values, indices, width)
        assert got.tolist() == [int(np.argmax(r)) for r in logits]


def _rank(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    payload = bytes(range(128)) if rank == 0 else b""
    got = groups.broadcast_bytes(dist, payload, 128)
    slowest = groups.max_over_ranks(dist, 1.0 + rank)

    class FakeDevice:
        def tp_init(self, r, w, group_id):
            self.joined = (r, w, group_id)
    dev = FakeDevice()
    groups.join_tensor_parallel(dev, dist, make_id=lambda: b"\x07" * 128)
    out.put((rank, got == bytes(range(128)), slowest, dev.joined == (rank, world, b"\x07" * 128)))
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_the_group_id_and_the_slowest_time():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True, 2.0, True), (1, True, 2.0, True)]


def _guarded_rank(rank, world, port, out):
    """Two ranks step together; rank 1 leaves after step 2, between steps; rank 0 must learn of it on the host, before it
    launches step 3, as a CommError, and not by waiting inside an exchange."""
    import datetime
    import torch.distributed as dist
    store = dist.TCPStore("127.0.0.1", port, world, is_master=rank == 0, timeout=datetime.timedelta(seconds=60))
    guard = groups.StepGuard(store, rank, world, patience=20.0)
    launched = []
    try:
        for step in range(5):
            if rank == 1 and step == 3:
                guard.leave()
                break
            guard.before_step(step)
            launched.append(step)   # here the rank would call tsm_decode
        out.put((rank, launched, None))
    except pkg.CommError as problem:
        out.put((rank, launched, str(problem)))
    if rank == 0:
        import time
        time.sleep(0.5)  # the store lives in rank 0: let the peer finish talking to it


def test_a_rank_that_leaves_between_steps_is_seen_on_the_host():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_guarded_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[1] == (1, [0, 1, 2], None)
    rank0, launched, problem = results[0]
    assert launched == [0, 1, 2] and problem is not None and "rank 1 left the group before step 3" in problem


def test_a_rank_that_never_arrives_runs_the_patience_out():
    class DictStore:
        def __init__(self):
            self.d = {}

        def set(self, k, v):
            self.d[k] = v

        def get(self, k):
            return self.d[k]

        def check(self, keys):
            return all(k in self.d for k in keys)

    guard = groups.StepGuard(DictStore(), 0, 2, patience=0.05)
    with pytest.raises(pkg.CommError, match="did not reach step 0"):
        guard.before_step(0)
