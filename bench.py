"""Benchmark of the quantised decode path:  python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (default `c5`): the Llama-3-8B-shaped model of the baseline's last configuration — 32 layers,
hidden 4096, 32 query / 8 key-value heads of width 128, SwiGLU 14336, vocabulary 128256, RoPE theta
500000, untied head, Q4_0 weights drawn N(0, 0.02) from a seed on the device — decoding 64 independent
streams whose F32 KV caches hold ragged lengths drawn uniformly from 128..4096 (seed 11) and filled with
seeded N(0,1) values.  A step is one greedy decode step of all 64 streams.  `value` is tokens/s with the
step loop resident on the device (`tsm_decode_run`: each step's picks feed the next on the device);
`e2e` is tokens/s through `tsm_decode` with host token buffers, the host->device copy of ids and
positions and the device->host copy of the picked tokens inside every step.  With N > 1 every rank runs
its own 64 streams on a full replica (no collective), so the job is 64*N streams ("weak").

Also on the line: `roofline` of the dominant kernel timed alone with CUDA events on the same buffers,
`cpu_baseline` (rank 0, N = 1: the CPU oracle's threaded decode on a bounded sample), `parity` (the same sampled streams
decoded on the device from the same caches and first tokens: are their greedy tokens the CPU's), `extra` with the
batch-1 numbers (135M-shaped Q8_0 model; matvec GB/s per shape and format), clocks, launch counts.

`--impl reference` times the CPU restatement of the reference's threaded decode (oracle/) on the host
cores for the same workload; Crystal is not installed, so the reference's own binary cannot be built.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402

WORKLOADS = {
    "c5": dict(name="llama-3-8b-shaped Q4_0, 64 ragged streams (KV 128..4096), greedy decode", arch="llama", kind="Q4_0",
               layers=32, width=4096, heads=32, kv_heads=8, head_width=128, hidden=14336, vocab=128256, context=8192,
               eps=1e-5, rope_theta=500000.0, tied=False, rows=64, len_lo=128, len_hi=4096),
    "c3": dict(name="smollm2-1.7b-shaped Q4_1, 16 streams, 128-token prompts, greedy decode", arch="llama", kind="Q4_1",
               layers=24, width=2048, heads=32, kv_heads=32, head_width=64, hidden=8192, vocab=49152, context=8192,
               eps=1e-5, rope_theta=130000.0, tied=True, rows=16, len_lo=128, len_hi=128),
    "c1": dict(name="smollm2-135m-shaped Q8_0, 1 stream, 32-token prompt, greedy decode", arch="llama", kind="Q8_0",
               layers=30, width=576, heads=9, kv_heads=3, head_width=64, hidden=1536, vocab=49152, context=8192,
               eps=1e-5, rope_theta=10000.0, tied=True, rows=1, len_lo=32, len_hi=32),
    "c4": dict(name="gpt2-xl-shaped Q8_0, 1 stream, 64-token prompt, greedy decode", arch="gpt2", kind="Q8_0",
               layers=48, width=1600, heads=25, kv_heads=25, head_width=64, hidden=6400, vocab=50257, context=1024,
               eps=1e-5, rope_theta=0.0, tied=True, rows=1, len_lo=64, len_hi=64),
}
KIND = {"Q8_0": 0, "Q4_0": 1, "Q4_1": 2}
BLOCK = {0: 34, 1: 18, 2: 20}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def ready(self, timeout=8.0):
        """Waits until the sampler has written its first line (nvidia-smi can take a second to start, longer when eight
        ranks start one each), so that a short timed region still sees samples."""
        deadline = time.time() + timeout
        while self.proc and time.time() < deadline and os.path.getsize(self.path) == 0:
            time.sleep(0.05)

    def begin(self):
        self.lo = os.path.getsize(self.path) if self.path else 0

    def end(self):
        self.hi = os.path.getsize(self.path) if self.path else 0

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        text = open(self.path).read()
        lo, hi = getattr(self, "lo", 0), getattr(self, "hi", len(text))
        inside = text[lo:hi]
        if inside.count("\n") < 1:  # a region shorter than the sampling period: the samples on either side of it
            inside = text[max(0, text.rfind("\n", 0, max(lo - 1, 0)) + 1):text.find("\n", hi) + 1 or len(text)]
        for line in inside.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])), mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


def model_config(w):
    return {k: w[k] for k in ("arch", "layers", "width", "heads", "kv_heads", "head_width", "hidden", "vocab", "context", "eps",
                              "rope_theta", "tied")}


def weight_elements(w):
    d, hw = w["width"], w["head_width"]
    qn, kvn = w["heads"] * hw, w["kv_heads"] * hw
    per_layer = (qn + 2 * kvn) * d + d * qn + (2 if w["arch"] == "llama" else 1) * w["hidden"] * d + d * w["hidden"]
    return w["layers"] * per_layer + w["vocab"] * d  # the head (the token table is read by rows only)


def step_bytes(w, lengths):
    """Algorithmic bytes of one decode step: every product weight once, plus each stream's keys and values."""
    weights = weight_elements(w) // 32 * BLOCK[KIND[w["kind"]]]
    kv = sum(2 * w["layers"] * w["kv_heads"] * w["head_width"] * 4 * (int(n) + 1) for n in lengths)
    return weights + kv, weights, kv


def draw_lengths(w, rank):
    rng = np.random.default_rng(11 + rank)
    return rng.integers(w["len_lo"], w["len_hi"] + 1, size=w["rows"])


def make_streams(pkg, dev, model, w, lengths, steps_budget, rank):
    capacity = int(max(lengths)) + steps_budget
    cache = model.new_batch_cache(w["rows"], capacity)
    for row, n in enumerate(lengths):
        cache.fill(row, int(n), seed=1000 * (rank + 1) + row)
    ids = np.random.default_rng(7 + rank).integers(0, w["vocab"], size=w["rows"]).astype(np.int32)
    return cache, ids


def refill(cache, lengths, rank):
    for row, n in enumerate(lengths):
        cache.fill(row, int(n), seed=1000 * (rank + 1) + row)


def time_kernel(torch, stream, fn, repeats):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()
    start.record(stream)
    for _ in range(repeats):
        fn()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop) / repeats / 1e3


def matvec_sweep(pkg, dev, torch, stream, peak):
    """Batch-1 quantised products of the baseline's shapes: GB/s of algorithmic bytes, timed alone.
    Between launches a 512 MB buffer is rewritten so that no weight is served from L2."""
    import ctypes as C
    shapes = [(576, 1536), (2048, 8192), (4096, 14336), (14336, 4096), (128256, 4096)]
    flush = dev.alloc(512 << 20)
    out = []
    for name, kind in KIND.items():
        for n, k in shapes:
            blocks = n * (k // 32)
            wbuf = dev.alloc(blocks * BLOCK[kind])
            src = dev.alloc(min(n, 4096) * k * 4)
            # weights: normal(0, 0.02) quantised on the device, in slabs of at most 4096 rows
            for r0 in range(0, n, 4096):
                rows = min(4096, n - r0)
                dev.check(dev.lib.tsm_fill_normal(dev.ctx, C.c_uint64(src.ptr), C.c_int64(rows * k), C.c_float(0.0), C.c_float(0.02),
                                                  C.c_uint64(n * 31 + r0)), "tsm_fill_normal")
                dev.check(dev.lib.tsm_quantize_blocks(dev.ctx, C.c_uint64(src.ptr), C.c_int64(rows * k), C.c_int(kind),
                                                      C.c_uint64(wbuf.ptr + r0 * (k // 32) * BLOCK[kind])), "tsm_quantize_blocks")
            x = dev.tensor(np.random.default_rng(5).normal(0, 1, (1, k)).astype(np.float32))
            scales, sums, qs, y = dev.alloc(k // 32 * 4), dev.alloc(k // 32 * 4), dev.alloc(k), dev.alloc(n * 4)
            dev.check(dev.lib.tsm_quantize_rows_q8(dev.ctx, C.c_uint64(x.ptr), 1, k, C.c_int64(k), C.c_uint64(scales.ptr),
                                                   C.c_uint64(sums.ptr), C.c_uint64(qs.ptr)), "tsm_quantize_rows_q8")

            def run():
                dev.lib.tsm_block_matmul_quantized(dev.ctx, C.c_uint64(scales.ptr), C.c_uint64(sums.ptr), C.c_uint64(qs.ptr), 1, k,
                                                   C.c_uint64(wbuf.ptr), kind, n, C.c_uint64(0), C.c_uint64(y.ptr))

            def flush_l2():
                dev.lib.tsm_fill_normal(dev.ctx, C.c_uint64(flush.ptr), C.c_int64((512 << 20) // 4), C.c_float(0.0), C.c_float(1.0),
                                        C.c_uint64(1))

            # time (flush + product) and (flush) alone, so the flush is taken out of the figure
            both = time_kernel(torch, stream, lambda: (flush_l2(), run()), 5)
            only = time_kernel(torch, stream, flush_l2, 5)
            seconds = max(both - only, 1e-9)
            algorithmic = blocks * BLOCK[kind] + k * 4 + n * 4
            out.append(dict(kind=name, n=n, k=k, us=round(seconds * 1e6, 2), gbs=round(algorithmic / seconds / 1e9, 1),
                            frac=round(algorithmic / seconds / 1e9 / peak, 3)))
            for b in (wbuf, src, x, scales, sums, qs, y):
                b.free()
    flush.free()
    dev.sync()
    return out


def kernel_case(pkg, dev, torch, stream, spec, repeats, peak):
    """One kernel on a small case, a few launches, for a profiler capture or a timing alone:
         matvec,<kind>,<n>,<k>             batch-1 product over already-quantised activations
         product,<kind>,<n>,<k>,<rows>     quantiser + batched product
         attention,<tokens>,<heads>,<kv_heads>,<width>,<capacity>[,<length>[,shared]]   ragged lengths 128..capacity-128 (seed 11),
                                                                          or every stream at <length> (0 = ragged); `shared`: all read one cache
       Returns the JSON record (microseconds per launch, GB/s of algorithmic bytes)."""
    import ctypes as C
    parts = spec.split(",")
    what = parts[0]
    if what in ("matvec", "product"):
        kind = KIND[parts[1].upper()]
        n, k = int(parts[2]), int(parts[3])
        rows = int(parts[4]) if what == "product" else 1
        blocks = n * (k // 32)
        wbuf = dev.alloc(blocks * BLOCK[kind])
        src = dev.alloc(min(n, 4096) * k * 4)
        for r0 in range(0, n, 4096):
            r = min(4096, n - r0)
            dev.check(dev.lib.tsm_fill_normal(dev.ctx, C.c_uint64(src.ptr), C.c_int64(r * k), C.c_float(0.0), C.c_float(0.02),
                                              C.c_uint64(n * 31 + r0)), "tsm_fill_normal")
            dev.check(dev.lib.tsm_quantize_blocks(dev.ctx, C.c_uint64(src.ptr), C.c_int64(r * k), C.c_int(kind),
                                                  C.c_uint64(wbuf.ptr + r0 * (k // 32) * BLOCK[kind])), "tsm_quantize_blocks")
        x = dev.tensor(np.random.default_rng(5).normal(0, 1, (rows, k)).astype(np.float32))
        y = dev.alloc(rows * n * 4)
        algorithmic = blocks * BLOCK[kind] + rows * k * 4 + rows * n * 4
        if what == "matvec":
            scales, sums, qs = dev.alloc(k // 32 * 4), dev.alloc(k // 32 * 4), dev.alloc(k)
            dev.check(dev.lib.tsm_quantize_rows_q8(dev.ctx, C.c_uint64(x.ptr), 1, k, C.c_int64(k), C.c_uint64(scales.ptr),
                                                   C.c_uint64(sums.ptr), C.c_uint64(qs.ptr)), "tsm_quantize_rows_q8")

            def run():
                dev.lib.tsm_block_matmul_quantized(dev.ctx, C.c_uint64(scales.ptr), C.c_uint64(sums.ptr), C.c_uint64(qs.ptr), 1, k,
                                                   C.c_uint64(wbuf.ptr), kind, n, C.c_uint64(0), C.c_uint64(y.ptr))
        else:
            def run():
                dev.lib.tsm_block_matmul(dev.ctx, C.c_uint64(x.ptr), rows, k, C.c_int64(k), C.c_uint64(wbuf.ptr), kind, n,
                                         C.c_uint64(0), C.c_uint64(y.ptr))
    elif what == "attention":
        tokens, H, KV, W, cap = (int(v) for v in parts[1:6])
        count = tokens * KV * cap * W
        kb, vb = dev.alloc(count * 4), dev.alloc(count * 4)
        for b, seed in ((kb, 1), (vb, 2)):
            dev.check(dev.lib.tsm_fill_normal(dev.ctx, C.c_uint64(b.ptr), C.c_int64(count), C.c_float(0.0), C.c_float(1.0),
                                              C.c_uint64(seed)), "tsm_fill_normal")
        lengths = np.random.default_rng(11).integers(128, cap - 127, size=tokens)
        if len(parts) > 6 and int(parts[6]) > 0:
            lengths = np.full(tokens, int(parts[6]))
        shared = len(parts) > 7 and parts[7] == "shared"   # every stream reads stream 0's cache (it stays in L2): the compute-bound time
        table = dev.tensor(np.stack([np.zeros(tokens, dtype=np.int64) if shared else np.arange(tokens), lengths, lengths + 1], 1).astype(np.int32))
        q = dev.tensor(np.random.default_rng(3).normal(0, 1, (tokens, H * W)).astype(np.float32))
        o = dev.alloc(tokens * H * W * 4)
        algorithmic = int(sum(2 * KV * W * 4 * (int(n) + 1) for n in lengths)) + 2 * tokens * H * W * 4

        def run():
            dev.lib.tsm_ragged_attention(dev.ctx, C.c_uint64(q.ptr), C.c_int64(H * W), tokens, H, W, C.c_uint64(kb.ptr),
                                         C.c_uint64(vb.ptr), tokens, KV, cap, C.c_uint64(table.ptr), C.c_float(1.0 / np.sqrt(W)),
                                         C.c_uint64(o.ptr))
    else:
        raise SystemExit(f"unknown case {spec!r}")
    dev.sync()
    if what == "matvec" and algorithmic < (256 << 20):
        # weights smaller than L2: a 512 MB buffer is rewritten before every launch and its time taken out, as in the sweep
        flush = dev.alloc(512 << 20)

        def flush_l2():
            dev.lib.tsm_fill_normal(dev.ctx, C.c_uint64(flush.ptr), C.c_int64((512 << 20) // 4), C.c_float(0.0), C.c_float(1.0), C.c_uint64(1))

        both = time_kernel(torch, stream, lambda: (flush_l2(), run()), repeats)
        only = time_kernel(torch, stream, flush_l2, repeats)
        seconds = max(both - only, 1e-9)
        flush.free()
    else:
        seconds = time_kernel(torch, stream, run, repeats)
    dev.sync()
    return dict(case=spec, launches=repeats + 1, us=seconds * 1e6, algorithmic_bytes=algorithmic, gbs=algorithmic / seconds / 1e9,
                frac=algorithmic / seconds / 1e9 / peak)


def oracle_model_from_device(model, threads):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from tests import helpers
    return helpers.oracle_from_device_model(model, threads=threads)


class CpuArm:
    """The CPU oracle's threaded decode over the first `sample_rows` streams of the device workload: same
    weights (downloaded once through the C ABI), same KV contents, same first tokens."""

    def __init__(self, pkg, model, cache, lengths, ids, threads, sample_rows, budget_steps):
        self.ref = oracle_model_from_device(model, threads)
        self.rows = sample_rows
        self.rcache = self.ref.new_cache(sample_rows, int(max(lengths[:sample_rows])) + budget_steps + 2)
        c = model.config
        row_floats = c["kv_heads"] * cache.capacity * c["head_width"]
        for layer in range(c["layers"]):
            kb, vb = cache.layer(layer)
            for row in range(sample_rows):
                n = int(lengths[row])
                for src, dst in ((kb, self.rcache.keys[layer]), (vb, self.rcache.values[layer])):
                    part = pkg.Buffer(model.device, src.ptr + row * row_floats * 4, row_floats * 4).numpy(np.float32)
                    dst[row, :, :n, :] = part.reshape(c["kv_heads"], cache.capacity, c["head_width"])[:, :n, :]
        for row in range(sample_rows):
            self.rcache.lengths[row] = int(lengths[row])
        self.tokens = [int(t) for t in ids[:sample_rows]]

    def step(self):
        """One greedy decode step of the sample's streams; returns seconds."""
        start = time.perf_counter()
        logits = self.ref.forward(self.rcache, [[t] for t in self.tokens])
        self.tokens = [int(np.argmax(r)) for r in logits]
        return time.perf_counter() - start


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extra", action="store_true", help="skip the batch-1 model and the matvec sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--parallelism", default="dp", choices=["dp", "tp", "tp_reduce"],
                    help="with --gpus N > 1: dp = every rank decodes its own streams on a whole replica (no collective); "
                         "tp = the ranks share one model split by tensor parallelism (NCCL all-gathers, the bits of one GPU) and decode "
                         "the same streams; tp_reduce = the same with o and down split by input columns and all-reduced (not bit-exact)")
    ap.add_argument("--mode", default="exact", choices=["exact", "fast"],
                    help="exact (default): the CPU path's bits; fast: tree sums and split-K attention, held to the reference's GPU budget "
                         "of 0.001 nats KL per token, not to its bits")
    ap.add_argument("--case", default=None, help="time one kernel on a small case instead (see kernel_case), e.g. matvec,q4_0,128256,4096")
    ap.add_argument("--repeats", type=int, default=3, help="timed launches of --case")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = dict(WORKLOADS[args.workload])
    K, W = args.steps, max(args.warmup, 0)
    threads = os.cpu_count() or 1

    if args.impl == "reference" and rank != 0:
        return
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    if world > 1 and args.impl == "ours":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    dev = pkg.B200(local)
    stream = torch.cuda.ExternalStream(dev.stream, device=local)
    peak, peak_kind = peaks()
    if args.mode == "fast":
        dev.set_mode(pkg.FAST)
    if args.case:
        print(json.dumps(kernel_case(pkg, dev, torch, stream, args.case, args.repeats, peak["hbm_gbs"])))
        dev.close()
        return
    tp = world if (args.parallelism != "dp" and args.impl == "ours") else 1
    if tp > 1:
        pkg.groups.join_tensor_parallel(dev, dist)
        if args.parallelism == "tp_reduce":
            dev.tp_variant(pkg.TP_REDUCE)
    data_rank = 0 if tp > 1 else rank          # tensor-parallel ranks decode the same streams
    jobs = 1 if tp > 1 else world              # independent sets of streams in the job
    lengths = draw_lengths(w, data_rank)
    model = pkg.Model.random(dev, model_config(w), KIND[w["kind"]], seed=20260101)
    dev.sync()
    rows = w["rows"]
    config = dict(workload=w["name"], streams_per_gpu=rows, kv_lengths=f"uniform {w['len_lo']}..{w['len_hi']} (seed 11)",
                  kv_dtype="f32", weights=w["kind"], mode=args.mode, l2="per-step working set (weights + KV) far exceeds the 126 MB L2",
                  parallelism=((f"tp{world}: projections split by output rows, 4 NCCL all-gathers per layer" if args.parallelism == "tp" else
                                f"tp{world}: o and down split by input columns, 2 NCCL all-reduces per layer (not bit-exact)") if tp > 1 else
                               f"dp{world}: a replica and {rows} streams per GPU, no collective") if world > 1 else "single gpu")

    if args.impl == "reference":
        sample_rows, sample_steps = min(rows, 2), 1
        cache, ids = make_streams(pkg, dev, model, w, lengths, 8 + K + W, rank)
        dev.sync()
        arm = CpuArm(pkg, model, cache, lengths, ids, threads, sample_rows, W + K)
        times = [arm.step() for _ in range(W + K)][W:]
        value = sample_rows * len(times) / float(np.sum(times))
        ms = float(np.mean(times)) * 1e3
        sample = f"{sample_rows} of {rows} streams x {sample_steps} decode step per bench step, all {threads} host threads"
        print(json.dumps(dict(metric="decode_tokens_per_second", value=value, unit="tokens/s", n_gpus=args.gpus, steps=K, warmup=W,
                              ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="int8 x int8 -> int32 blocks, f32 accumulate",
                              data="synthetic", config=config, impl="reference",
                              cpu_baseline=dict(value=value, unit="tokens/s", cores=threads, kind="port", sample=sample),
                              e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))))
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(seconds):
        if world == 1:
            return seconds
        t = torch.tensor([seconds], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cache, ids = make_streams(pkg, dev, model, w, lengths, W + K + 2, data_rank)
    dev.sync()
    # ---- value: the step loop resident on the device ----------------------------------------------
    with ClockSampler(local) as clocks:
        clocks.ready()
        if W:
            model.decode_run(cache, ids, W)
        dev.reset_counters()
        barrier()
        clocks.begin()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        tokens = model.decode_run(cache, ids, K)
        stop.record(stream)
        stop.synchronize()
        clocks.end()
        barrier()
    seconds = max_over_ranks(start.elapsed_time(stop) / 1e3)
    counters = dev.counters()
    value = rows * K * jobs / seconds
    clock_summary = clocks.summary()
    mid_lengths = lengths + W + K // 2
    total_bytes, weight_bytes, kv_bytes = step_bytes(w, mid_lengths)

    # ---- e2e: one C-ABI call per step with host buffers ---------------------------------------------
    refill(cache, lengths, data_rank)
    dev.sync()
    step_ids = ids.copy()
    for _ in range(W):
        step_ids = model.decode(cache, step_ids)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        step_ids = model.decode(cache, step_ids)
    torch.cuda.synchronize()
    e2e_seconds = max_over_ranks(time.perf_counter() - t0)
    barrier()
    e2e = dict(value=rows * K * jobs / e2e_seconds, unit="tokens/s", h2d_bytes_per_step=rows * 16, d2h_bytes_per_step=rows * 4 + 16,
               ms_per_step=e2e_seconds / K * 1e3)

    line = dict(metric="decode_tokens_per_second", value=value, unit="tokens/s", n_gpus=world, steps=K, warmup=W,
                ms_per_step=seconds / K * 1e3, higher_is_better=True, scaling="strong" if tp > 1 else "weak", vs_baseline=None,
                dtype="int8 x int8 -> int32 blocks, f32 accumulate", data="synthetic", config=config, e2e=e2e,
                gpu_launches=int(counters["launches"]), clocks=clock_summary,
                step_roofline=dict(bytes_per_step=total_bytes, weight_bytes=weight_bytes, kv_bytes=kv_bytes,
                                   achieved_gbs=total_bytes / (seconds / K) / 1e9, peak_gbs=peak["hbm_gbs"] * tp, peak_kind=peak_kind,
                                   frac=total_bytes / (seconds / K) / 1e9 / (peak["hbm_gbs"] * tp)))

    if rank == 0:
        # ---- roofline of the dominant kernels, timed alone on the same buffers -------------------------
        import ctypes as C
        c = model.config
        hw, H, KV = c["head_width"], c["heads"] // tp, c["kv_heads"] // tp   # a tensor-parallel rank attends over its own heads
        table = np.stack([np.arange(rows), lengths, lengths + 1], axis=1).astype(np.int32)
        tb = dev.tensor(table)
        q = dev.tensor(np.random.default_rng(3).normal(0, 1, (rows, H * hw)).astype(np.float32))
        o = dev.alloc(rows * H * hw * 4)
        kb, vb = cache.layer(0)
        scale = float(1.0 / np.sqrt(hw))

        def attn():
            dev.lib.tsm_ragged_attention(dev.ctx, C.c_uint64(q.ptr), C.c_int64(H * hw), rows, H, hw, C.c_uint64(kb.ptr), C.c_uint64(vb.ptr),
                                         rows, KV, cache.capacity, C.c_uint64(tb.ptr), C.c_float(scale), C.c_uint64(o.ptr))

        attn_s = time_kernel(torch, stream, attn, 10)
        attn_bytes = int(sum(2 * KV * hw * 4 * (int(n) + 1) for n in lengths)) + 2 * rows * H * hw * 4
        buf, kind, n, k = model.tensor("0.up")
        x = dev.tensor(np.random.default_rng(4).normal(0, 1, (rows, k)).astype(np.float32))
        y = dev.alloc(rows * n * 4)

        def up():
            dev.lib.tsm_block_matmul(dev.ctx, C.c_uint64(x.ptr), rows, k, C.c_int64(k), C.c_uint64(buf.ptr), kind, n, C.c_uint64(0),
                                     C.c_uint64(y.ptr))

        up_s = time_kernel(torch, stream, up, 10)
        up_bytes = n * (k // 32) * BLOCK[kind] + rows * k * 4 + rows * n * 4
        L = c["layers"]
        attn_share, up_share = attn_s * L, up_s * L
        kernels = [dict(kernel=f"ordered ragged attention (one layer, {rows} streams)", bytes=attn_bytes, us=attn_s * 1e6, gbs=attn_bytes / attn_s / 1e9,
                        share_of_step=attn_share / (seconds / K)),
                   dict(kernel=f"block product {n}x{k} {w['kind']} rows={rows} (+quantiser)", bytes=up_bytes, us=up_s * 1e6,
                        gbs=up_bytes / up_s / 1e9, share_of_step=up_share / (seconds / K))]
        top = max(kernels, key=lambda e: e["share_of_step"])
        # DRAM bytes (read + written) of one launch from the profiler captures summarised under profiles/, taken on exactly
        # these shapes and lengths; none for other workloads
        traffic = None
        if args.workload == "c5":
            traffic = 1310231256 if top is kernels[0] else 67894272
        line["roofline"] = dict(bound="hbm", kernel=top["kernel"], achieved=top["gbs"], peak=peak["hbm_gbs"], unit="GB/s",
                                frac=top["gbs"] / peak["hbm_gbs"], traffic=traffic, algorithmic_bytes=top["bytes"], peak_kind=peak_kind)
        line["kernels"] = kernels
        for b in (tb, q, o, x, y):
            b.free()

        # ---- CPU baseline on a bounded sample (N = 1 only) -----------------------------------------------
        if world == 1 and not args.no_cpu:
            refill(cache, lengths, rank)
            dev.sync()
            sample_rows, sample_steps = min(rows, 4), 5   # about 10 s of host work at the headline shape
            arm = CpuArm(pkg, model, cache, lengths, ids, threads, sample_rows, sample_steps + 1)
            cpu_tokens = []
            arm.step()  # warm-up: threads start, pages are touched
            cpu_tokens.append(list(arm.tokens))
            cpu_seconds = 0.0
            for _ in range(sample_steps):
                cpu_seconds += arm.step()
                cpu_tokens.append(list(arm.tokens))
            rate = sample_rows * sample_steps / cpu_seconds
            # The same steps on the device from the same caches and first tokens: the sampled streams' greedy tokens must be the
            # CPU path's, step for step (rows are independent, so the other 60 streams do not matter).
            try:
                refill(cache, lengths, rank)
                dev.sync()
                step_ids, gpu_tokens = ids.copy(), []
                for _ in range(sample_steps + 1):
                    step_ids = model.decode(cache, step_ids)
                    gpu_tokens.append([int(t) for t in step_ids[:sample_rows]])
                line["parity"] = dict(streams=sample_rows, steps=sample_steps + 1, identical_tokens=gpu_tokens == cpu_tokens,
                                      against="the CPU oracle's greedy tokens for the sampled streams at this workload's full size")
            except Exception as problem:  # the check must never cost the bench its line
                line["parity"] = dict(error=str(problem))
            line["cpu_baseline"] = dict(value=rate, unit="tokens/s", cores=threads, kind="port",
                                        sample=f"{sample_rows} of {rows} streams x {sample_steps} decode steps, {cpu_seconds:.1f} s, "
                                               f"oracle's threaded product on {threads} threads, other host ops on one thread")
        else:
            line["cpu_baseline"] = None
    cache.free()
    model.free()

    # ---- batch 1: the 135M-shaped model and the matvec sweep (rank 0, N = 1) ----------------------------
    if rank == 0 and world == 1 and not args.no_extra:
        extra = {}
        w1 = WORKLOADS["c1"]
        m1 = pkg.Model.random(dev, model_config(w1), KIND[w1["kind"]], seed=20260102)
        prompt = np.random.default_rng(7).integers(0, w1["vocab"], size=32).astype(np.int32)
        c1 = m1.new_batch_cache(1, 32 + 128 + 8)
        m1.forward_last([prompt.tolist()], c1)
        first = np.array([1], dtype=np.int32)
        m1.decode_run(c1, first, 4)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        m1.decode_run(c1, first, 120)
        stop.record(stream)
        stop.synchronize()
        s1 = start.elapsed_time(stop) / 1e3 / 120
        b1, _, _ = step_bytes(w1, np.array([32 + 64]))
        extra["c1_batch1"] = dict(workload=w1["name"], tokens_per_second=1 / s1, us_per_token=s1 * 1e6,
                                  bytes_per_token=b1, frac_of_hbm=b1 / s1 / 1e9 / peak["hbm_gbs"])
        c1.free(), m1.free()
        extra["matvec_batch1"] = matvec_sweep(pkg, dev, torch, stream, peak["hbm_gbs"])
        line["extra"] = extra
    if rank == 0:
        print(json.dumps(line))
    dev.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
