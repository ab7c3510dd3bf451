"""Host-side plumbing for several GPUs, one process per GPU (torch.distributed carries the few bytes the ranks
must agree on; the data path itself is NCCL inside the library, or nothing at all for independent streams).

Two ways to use N GPUs for the decode loop:
  * independent streams: every rank holds the whole model and `stream_share` of the rows; no exchange on the data path;
  * tensor parallelism: `join_tensor_parallel` makes the ranks one group; a model then built on the device holds the
    rank's rows of every projection (`shard_rows` mirrors the library's split) and all ranks decode the same rows.
"""
import numpy as np


def stream_share(streams, world, rank):
    """(first, count) of the rows rank `rank` of `world` decodes: contiguous, sizes differing by at most one."""
    first = streams * rank // world
    return first, streams * (rank + 1) // world - first


def shard_rows(config, world, rank):
    """The [start, stop) row ranges of each projection a tensor-parallel rank holds: every projection is split by
    output rows, joined projections part by part (a rank's heads of q, of k and of v; its slice of gate and of up)."""
    for name in ("heads", "kv_heads", "width", "hidden", "vocab"):
        if config[name] % world:
            raise ValueError(f"{name} = {config[name]} does not divide by {world} ranks")
    hw = config["head_width"]
    qn, kvn = config["heads"] * hw, config["kv_heads"] * hw

    def part(offset, size):
        return (offset + rank * size // world, offset + (rank + 1) * size // world)

    up = [part(0, config["hidden"])]
    if config.get("arch", "llama") == "llama":
        up.append(part(config["hidden"], config["hidden"]))
    return dict(qkv=[part(0, qn), part(qn, kvn), part(qn + kvn, kvn)], o=[part(0, config["width"])], up=up,
                down=[part(0, config["width"])], head=[part(0, config["vocab"])])


def combine_picks(best_values, best_indices, slice_size):
    """The greedy pick across ranks, as the library's combine kernel takes it: best_values / best_indices are
    [world, rows] (each rank's best logit of its vocabulary slice and its index in the slice); the highest value wins,
    equal values go to the lower rank (the lower index)."""
    best_values, best_indices = np.asarray(best_values), np.asarray(best_indices)
    who = np.zeros(best_values.shape[1], dtype=np.int64)
    top = best_values[0].copy()
    for r in range(1, best_values.shape[0]):
        better = best_values[r] > top
        who[better], top[better] = r, best_values[r][better]
    return who * slice_size + best_indices[who, np.arange(best_values.shape[1])]


def broadcast_bytes(dist, payload, size, device=None):
    """`payload` (bytes, on rank 0; ignored elsewhere) to every rank, over whatever backend the group has."""
    import torch
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    buf = torch.zeros(size, dtype=torch.uint8, device=device)
    if dist.get_rank() == 0:
        buf.copy_(torch.frombuffer(bytearray(payload), dtype=torch.uint8))
    dist.broadcast(buf, src=0)
    return bytes(buf.cpu().numpy().tobytes())


def join_tensor_parallel(device, dist, make_id=None):
    """Makes the ranks of the default process group one tensor-parallel group of `device`s."""
    from . import binding
    world, rank = dist.get_world_size(), dist.get_rank()
    if world == 1:
        return
    group_id = broadcast_bytes(dist, (make_id or binding.tp_unique_id)() if rank == 0 else b"", 128)
    device.tp_init(rank, world, group_id)


class StepGuard:
    """Failure detection between steps, on the host.

    A tensor-parallel step is a chain of kernels and exchanges that every rank must enter; a rank that has gone would leave
    the others waiting inside a collective.  So the ranks talk on the host first: each one publishes the step it is about to
    launch in a key-value store they share (a `torch.distributed` store, or anything with set / get / check), a rank that
    leaves says so, and `before_step` refuses to launch, with `CommError`, once a peer has left or has not reached the step
    within `patience` seconds.  The caller then drops its communicator (`device.tp_abort()`) and rebuilds the group; nothing
    was in flight on the GPU, so nothing hangs there.  Ranks only ever leave between steps."""

    def __init__(self, store, rank, world, patience=30.0, prefix="tsm/guard"):
        self.store, self.rank, self.world, self.patience, self.prefix = store, rank, world, patience, prefix

    def _key(self, what, rank):
        return f"{self.prefix}/{what}/{rank}"

    def leave(self):
        """Tells the others that this rank will launch no more steps."""
        self.store.set(self._key("gone", self.rank), b"1")

    def gone(self):
        """The ranks that have left."""
        return [r for r in range(self.world) if r != self.rank and self.store.check([self._key("gone", r)])]

    def before_step(self, step):
        """Call on every rank before launching step `step`: returns once every peer is about to launch it too."""
        import time
        from . import binding
        self.store.set(self._key("step", self.rank), str(step).encode())
        deadline = time.monotonic() + self.patience
        waiting = [r for r in range(self.world) if r != self.rank]
        while waiting:
            left = self.gone()
            if left:
                raise binding.CommError(f"rank {left[0]} left the group before step {step}")
            still = []
            for r in waiting:
                key = self._key("step", r)
                if not self.store.check([key]) or int(self.store.get(key)) < step:
                    still.append(r)
            waiting = still
            if waiting:
                if time.monotonic() > deadline:
                    raise binding.CommError(f"rank {waiting[0]} did not reach step {step} within {self.patience:g} s")
                time.sleep(0.002)


def max_over_ranks(dist, seconds, device=None):
    """The slowest rank's time: what a multi-GPU number is quoted on."""
    import torch
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return seconds
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    t = torch.tensor([seconds], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
