"""Benchmark of the quantised decode path:  python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (default `c5`): the Llama-3-8B-shaped model of the baseline's last configuration — 32 layers,
hidden 4096, 32 query / 8 key-value heads of width 128, SwiGLU 14336, vocabulary 128256, RoPE theta
500000, untied head, Q4_0 weights drawn N(0, 0.02) from a seed on the device — decoding 64 independent
streams whose F32 KV caches hold ragged lengths drawn uniformly from 128..4096 (seed 11) and filled with
seeded N(0,1) values.  A step is one greedy decode step of all 64 streams.  `value` is tokens/s with the
step loop resident on the device (`tsm_decode_run`: each step's picks feed the next on the device);
`e2e` is tokens/s through `tsm_decode` with host token buffers, the host->device copy of ids and
positions and the device->host copy of the picked tokens inside every step.

With N > 1 the N ranks share ONE model, split by tensor parallelism, and decode the same 64 streams: the job's work is
fixed ("strong"), which is the scaling the baseline asks of this configuration.  `--parallelism dp` runs a replica and its
own 64 streams per rank instead (no collective, "weak").  At N > 1 `extra.c3_dp` also times the baseline's data-parallel
configuration (the 1.7B-shaped Q4_1 model, its 16 streams split over the ranks) and `parity.tp_tokens_identical` compares
the group's greedy tokens with those of the whole model on one GPU.

Also on the line: `roofline` of the dominant kernel timed alone with CUDA events on the same buffers,
`cpu_baseline` (rank 0, N = 1: the CPU oracle's threaded decode on a bounded sample), `parity` (the same sampled streams
decoded on the device from the same caches and first tokens: are their greedy tokens the CPU's), `extra` with the
batch-1 models, the format x shape x columns sweep of the products (GB/s per kernel), prefill and load figures, the fast
mode's cost and error, clocks, launch counts.

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


L2_TURNOVER = 256 << 20   # bytes of other weights read between two uses of one copy: twice the 126 MB L2


def weight_copies(size):
    """Copies of a weight matrix of `size` bytes that time_rotating cycles through: between two uses of one copy the others
    bring at least L2_TURNOVER bytes through L2."""
    return 1 + -(-L2_TURNOVER // size)


def rotating_weights(dev, kind, n, k):
    """Copies of one quantised n x k weight matrix (normal(0, 0.02), quantised on the device in slabs of at most 4096 rows),
    enough of them that a launch reading the copies in turn never finds its weights in L2: L2_TURNOVER bytes of other copies
    pass through between two uses of the same one.  Returns (buffer, bytes from copy to copy, copies).  Rewriting a large buffer
    between launches instead left L2 full of modified lines, and the timed kernel then waited for their write-back."""
    import ctypes as C
    size = n * (k // 32) * BLOCK[kind]
    stride = (size + 255) & ~255
    copies = weight_copies(size)
    wbuf = dev.alloc(stride * copies)
    src = dev.alloc(min(n, 4096) * k * 4)
    for r0 in range(0, n, 4096):
        rows = min(4096, n - r0)
        dev.check(dev.lib.tsm_fill_normal(dev.ctx, C.c_uint64(src.ptr), C.c_int64(rows * k), C.c_float(0.0), C.c_float(0.02),
                                          C.c_uint64(n * 31 + r0)), "tsm_fill_normal")
        for c in range(copies):
            dev.check(dev.lib.tsm_quantize_blocks(dev.ctx, C.c_uint64(src.ptr), C.c_int64(rows * k), C.c_int(kind),
                                                  C.c_uint64(wbuf.ptr + c * stride + r0 * (k // 32) * BLOCK[kind])), "tsm_quantize_blocks")
    src.free()
    return wbuf, stride, copies


def time_rotating(torch, stream, run_on, wbuf, stride, copies, repeats):
    """Seconds per launch of run_on(weights pointer), each launch on the copy used longest ago.  Before the timed launches one
    untimed pass reads L2_TURNOVER bytes of copies, which also writes back whatever the set-up left modified in L2."""
    turn = [0]

    def run():
        run_on(wbuf.ptr + (turn[0] % copies) * stride)
        turn[0] += 1

    for _ in range(min(copies, 1 + -(-L2_TURNOVER // stride))):
        run()
    return time_kernel(torch, stream, run, repeats)


def product_sweep(pkg, dev, torch, stream, peak):
    """The baseline's standalone sweep: Q4_0 / Q4_1 / Q8_0 x five shapes x 1, 8, 64 and 256 activation columns (rows of x),
    each product timed alone on already-quantised activations: GB/s of algorithmic bytes per kernel.  Successive launches read
    different copies of the weights (rotating_weights), so that no weight is served from L2."""
    import ctypes as C
    shapes = [(576, 1536), (2048, 8192), (4096, 14336), (14336, 4096), (128256, 4096)]
    out = []
    for name, kind in KIND.items():
        for n, k in shapes:
            blocks = n * (k // 32)
            wbuf, stride, copies = rotating_weights(dev, kind, n, k)
            for columns in (1, 8, 64, 256):
                x = dev.tensor(np.random.default_rng(5).normal(0, 1, (columns, k)).astype(np.float32))
                scales, sums, qs, y = (dev.alloc(columns * (k // 32) * 4), dev.alloc(columns * (k // 32) * 4), dev.alloc(columns * k),
                                       dev.alloc(columns * n * 4))
                dev.check(dev.lib.tsm_quantize_rows_q8(dev.ctx, C.c_uint64(x.ptr), columns, k, C.c_int64(k), C.c_uint64(scales.ptr),
                                                       C.c_uint64(sums.ptr), C.c_uint64(qs.ptr)), "tsm_quantize_rows_q8")

                def run_on(weights):
                    dev.lib.tsm_block_matmul_quantized(dev.ctx, C.c_uint64(scales.ptr), C.c_uint64(sums.ptr), C.c_uint64(qs.ptr), columns, k,
                                                       C.c_uint64(weights), kind, n, C.c_uint64(0), C.c_uint64(y.ptr))

                seconds = max(time_rotating(torch, stream, run_on, wbuf, stride, copies, 5), 1e-9)
                algorithmic = blocks * BLOCK[kind] + columns * k * 4 + columns * n * 4
                out.append(dict(kind=name, n=n, k=k, columns=columns, us=round(seconds * 1e6, 2), gbs=round(algorithmic / seconds / 1e9, 1),
                                frac=round(algorithmic / seconds / 1e9 / peak, 3)))
                for b in (x, scales, sums, qs, y):
                    b.free()
            wbuf.free()
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
        rotate = rows <= 4   # a few rows: every launch on another copy of the weights, as in the sweep (none served from L2)
        wbuf, stride, copies = rotating_weights(dev, kind, n, k) if rotate else (None, 0, 1)
        if not rotate:
            wbuf = dev.alloc(blocks * BLOCK[kind])
            src = dev.alloc(min(n, 4096) * k * 4)
            for r0 in range(0, n, 4096):
                r = min(4096, n - r0)
                dev.check(dev.lib.tsm_fill_normal(dev.ctx, C.c_uint64(src.ptr), C.c_int64(r * k), C.c_float(0.0), C.c_float(0.02),
                                                  C.c_uint64(n * 31 + r0)), "tsm_fill_normal")
                dev.check(dev.lib.tsm_quantize_blocks(dev.ctx, C.c_uint64(src.ptr), C.c_int64(r * k), C.c_int(kind),
                                                      C.c_uint64(wbuf.ptr + r0 * (k // 32) * BLOCK[kind])), "tsm_quantize_blocks")
            src.free()
        x = dev.tensor(np.random.default_rng(5).normal(0, 1, (rows, k)).astype(np.float32))
        y = dev.alloc(rows * n * 4)
        algorithmic = blocks * BLOCK[kind] + rows * k * 4 + rows * n * 4
        if what == "matvec":
            scales, sums, qs = dev.alloc(k // 32 * 4), dev.alloc(k // 32 * 4), dev.alloc(k)
            dev.check(dev.lib.tsm_quantize_rows_q8(dev.ctx, C.c_uint64(x.ptr), 1, k, C.c_int64(k), C.c_uint64(scales.ptr),
                                                   C.c_uint64(sums.ptr), C.c_uint64(qs.ptr)), "tsm_quantize_rows_q8")

            def run_on(weights):
                dev.lib.tsm_block_matmul_quantized(dev.ctx, C.c_uint64(scales.ptr), C.c_uint64(sums.ptr), C.c_uint64(qs.ptr), 1, k,
                                                   C.c_uint64(weights), kind, n, C.c_uint64(0), C.c_uint64(y.ptr))
        else:
            def run_on(weights):
                dev.lib.tsm_block_matmul(dev.ctx, C.c_uint64(x.ptr), rows, k, C.c_int64(k), C.c_uint64(weights), kind, n,
                                         C.c_uint64(0), C.c_uint64(y.ptr))

        def run():
            run_on(wbuf.ptr)
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
    launches = repeats + 1
    if what in ("matvec", "product") and rotate:
        seconds = time_rotating(torch, stream, run_on, wbuf, stride, copies, repeats)
        launches += min(copies, 1 + -(-L2_TURNOVER // stride))
    else:
        seconds = time_kernel(torch, stream, run, repeats)
    dev.sync()
    return dict(case=spec, launches=launches, us=seconds * 1e6, algorithmic_bytes=algorithmic, gbs=algorithmic / seconds / 1e9,
                frac=algorithmic / seconds / 1e9 / peak)


def pick_sample(lengths, count=2):
    """The streams whose cached lengths bracket the workload's mean: the nearest below it and the nearest above (then the
    next nearest, alternately).  The CPU legs decode these, so that their tokens/s is that of a stream of average length."""
    lengths = np.asarray(lengths)
    mean = float(lengths.mean())
    below = sorted((i for i in range(len(lengths)) if lengths[i] <= mean), key=lambda i: mean - lengths[i])
    above = sorted((i for i in range(len(lengths)) if lengths[i] > mean), key=lambda i: lengths[i] - mean)
    order = [i for pair in zip(below, above) for i in pair] + below[len(above):] + above[len(below):]
    return sorted(order[:min(count, len(order))])


class CpuArm:
    """The CPU oracle's threaded decode over the streams `rows` of the device workload: same weights (downloaded once
    through the C ABI), same KV contents, same first tokens."""

    def __init__(self, pkg, model, cache, lengths, ids, threads, rows, budget_steps):
        from oracle import oracle   # the checker and the CPU baseline: the only use of oracle/ in this file
        self.oracle = oracle
        self.ref = oracle.model_from_device(model, threads=threads)
        self.rows = list(rows)
        held = [int(lengths[r]) for r in self.rows]
        self.rcache = oracle.cache_from_device(self.ref, model, cache, self.rows, held, max(held) + budget_steps + 2)
        self.tokens = [int(ids[r]) for r in self.rows]
        self.logits = None

    def step(self):
        """One greedy decode step of the sample's streams; returns seconds."""
        start = time.perf_counter()
        self.logits = self.ref.forward(self.rcache, [[t] for t in self.tokens])
        self.tokens = [self.oracle.argmax_first(r) for r in self.logits]
        return time.perf_counter() - start


def kl_per_token(want, got):
    """Mean KL(softmax(want) || softmax(got)) in nats per row."""
    def log_softmax(x):
        x = x.astype(np.float64)
        x = x - x.max(axis=-1, keepdims=True)
        return x - np.log(np.exp(x).sum(axis=-1, keepdims=True))
    lw, lg = log_softmax(want), log_softmax(got)
    return float((np.exp(lw) * (lw - lg)).sum(axis=-1).mean())


def load_traffic():
    """DRAM bytes (read + written) of one launch of the dominant kernels, from the profiler captures summarised under
    profiles/ (profiles/traffic.json names the commit, the case and the command of each)."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        return json.load(open(path))
    except Exception:
        return {}


def batch1_model(pkg, dev, torch, stream, w, seed, tokens, peak):
    """A batch-1 configuration: prompt through the packed step, then `tokens` greedy steps resident on the device."""
    m = pkg.Model.random(dev, model_config(w), KIND[w["kind"]], seed=seed)
    prompt = np.random.default_rng(7).integers(0, w["vocab"], size=w["len_lo"]).astype(np.int32)
    cache = m.new_batch_cache(1, w["len_lo"] + tokens + 16)
    first = np.argmax(m.forward_last([prompt.tolist()], cache), axis=1).astype(np.int32)
    first = m.decode_run(cache, first, 4)[-1]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    m.decode_run(cache, first, tokens)
    stop.record(stream)
    stop.synchronize()
    seconds = start.elapsed_time(stop) / 1e3 / tokens
    nbytes, _, _ = step_bytes(w, np.array([w["len_lo"] + 4 + tokens // 2]))
    cache.free(), m.free()
    return dict(workload=w["name"], tokens_per_second=1 / seconds, us_per_token=seconds * 1e6, bytes_per_token=nbytes,
                frac_of_hbm=nbytes / seconds / 1e9 / peak)


def prefill_rate(pkg, dev, torch, stream, model, rows, prompt_tokens, vocab):
    """Tokens/s of a packed prefill: `rows` streams of `prompt_tokens` seeded tokens each through one tsm_forward."""
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, vocab, size=prompt_tokens).tolist() for _ in range(rows)]
    cache = model.new_batch_cache(rows, prompt_tokens + 8)
    model.forward_last(prompts, cache)   # warm-up: sizes the workspace
    best = None
    for _ in range(2):
        for row in range(rows):
            cache.reset(row)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        model.forward_last(prompts, cache)
        stop.record(stream)
        stop.synchronize()
        seconds = start.elapsed_time(stop) / 1e3
        best = seconds if best is None else min(best, seconds)
    cache.free()
    return dict(streams=rows, prompt_tokens=prompt_tokens, ms=best * 1e3, tokens_per_second=rows * prompt_tokens / best)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extra", action="store_true", help="skip the batch-1 models, the product sweep, prefill, load and fast-mode figures")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--parallelism", default="auto", choices=["auto", "dp", "tp", "tp_reduce"],
                    help="with --gpus N > 1: tp_reduce (auto) = the ranks share one model split by tensor parallelism with o and down over "
                         "input columns and their partial sums exchanged (the split the baseline names; not bit-exact) and decode the "
                         "same streams; tp = every projection split by output rows with all-gathers (the bits of one GPU); "
                         "dp = every rank decodes its own streams on a whole replica (no collective)")
    ap.add_argument("--mode", default="exact", choices=["exact", "fast"],
                    help="exact (default): the CPU path's bits; fast: tree sums and split-K attention, held to the reference's GPU budget "
                         "of 0.001 nats KL per token, not to its bits")
    ap.add_argument("--case", default=None, help="time one kernel on a small case instead (see kernel_case), e.g. matvec,q4_0,128256,4096")
    ap.add_argument("--repeats", type=int, default=3, help="timed launches of --case")
    ap.add_argument("--parity-steps", type=int, default=6,
                    help="greedy steps over which the sampled streams are compared with the CPU oracle (N = 1); 128 is the whole generation")
    ap.add_argument("--profile", action="store_true", help="also print (to stderr) the per-operator GPU time of one decode step")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = dict(WORKLOADS[args.workload])
    K, W = max(args.steps, 1), max(args.warmup, 0)
    threads = os.cpu_count() or 1
    parallelism = args.parallelism if args.parallelism != "auto" else "tp_reduce"

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
    tp = world if (parallelism != "dp" and args.impl == "ours") else 1
    if tp > 1:
        pkg.groups.join_tensor_parallel(dev, dist)
        if parallelism == "tp_reduce":
            dev.tp_variant(pkg.TP_REDUCE)
    data_rank = 0 if tp > 1 else rank          # tensor-parallel ranks decode the same streams
    jobs = 1 if tp > 1 else world              # independent sets of streams in the job
    lengths = draw_lengths(w, data_rank)
    load_start = time.perf_counter()
    model = pkg.Model.random(dev, model_config(w), KIND[w["kind"]], seed=20260101)
    dev.sync()
    draw_seconds = time.perf_counter() - load_start
    rows = w["rows"]
    tp_named = world if parallelism != "dp" else 1   # what the job's own arm runs at this N: the reference arm names the same configuration
    config = dict(workload=w["name"], streams_per_gpu=rows if tp_named == 1 else f"{rows} shared by the {world} ranks",
                  kv_lengths=f"uniform {w['len_lo']}..{w['len_hi']} (seed 11)",
                  kv_dtype="f32", weights=w["kind"], mode=args.mode, l2="per-step working set (weights + KV) far exceeds the 126 MB L2",
                  parallelism=((f"tp{world}: projections split by output rows, NCCL all-gathers between them (the bits of one GPU)" if parallelism == "tp" else
                                f"tp{world}: q/k/v, gate/up and the head split by output rows, o and down by input columns with their partial "
                                f"sums exchanged over NVLink (not bit-exact)") if tp_named > 1 else
                               f"dp{world}: a replica and {rows} streams per GPU, no collective") if world > 1 else "single gpu")
    sample = pick_sample(lengths, 2)
    sample_note = f"streams {sample} of {rows} (cached lengths {[int(lengths[r]) for r in sample]}, workload mean {float(np.mean(lengths)):.0f})"

    if args.impl == "reference":
        cache, ids = make_streams(pkg, dev, model, w, lengths, 8 + K + W, rank)
        dev.sync()
        arm = CpuArm(pkg, model, cache, lengths, ids, threads, sample, W + K)
        times = [arm.step() for _ in range(W + K)][W:]
        value = len(sample) * len(times) / float(np.sum(times))
        ms = float(np.mean(times)) * 1e3
        note = (f"{sample_note} x 1 decode step per bench step, all {threads} host threads; weights and cache contents are drawn on the "
                f"device (set-up only) and copied to the host before the timed region")
        print(json.dumps(dict(metric="decode_tokens_per_second", value=value, unit="tokens/s", n_gpus=args.gpus, steps=K, warmup=W,
                              ms_per_step=ms, higher_is_better=True, scaling="strong" if (world > 1 and parallelism != "dp") else "weak",
                              vs_baseline=None, dtype="int8 x int8 -> int32 blocks, f32 accumulate",
                              data="synthetic", config=config, impl="reference",
                              cpu_baseline=dict(value=value, unit="tokens/s", cores=threads, kind="port", sample=note),
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

    cache, ids = make_streams(pkg, dev, model, w, lengths, max(W + K, args.parity_steps + 1, 24) + 2, data_rank)
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
                gpu_launches=int(counters["launches"]), collectives=int(counters["collectives"]), clocks=clock_summary,
                step_roofline=dict(bytes_per_step=total_bytes, weight_bytes=weight_bytes, kv_bytes=kv_bytes,
                                   achieved_gbs=total_bytes / (seconds / K) / 1e9, peak_gbs=peak["hbm_gbs"] * tp, peak_kind=peak_kind,
                                   frac=total_bytes / (seconds / K) / 1e9 / (peak["hbm_gbs"] * tp)))

    # ---- per-operator GPU time of one step (the library's profile mode) ------------------------------
    if args.profile:
        refill(cache, lengths, data_rank)
        dev.sync()
        model.decode(cache, ids)
        dev.profile(shapes=True)
        model.decode(cache, ids)
        table = dev.profile_read(end=True)
        if rank == 0:
            print(f"per-operator GPU time of one decode step ({config['parallelism']}):", file=sys.stderr)
            for label, count, secs in table:
                print(f"  {count:5d}  {secs * 1e3:9.3f} ms  {secs / max(count, 1) * 1e6:9.1f} us/launch  {label}", file=sys.stderr)
        barrier()

    # ---- tensor parallel: the group's tokens against the whole model on one GPU -----------------------
    if tp > 1:
        check_steps = min(K, 32)
        refill(cache, lengths, data_rank)
        dev.sync()
        tp_tokens = model.decode_run(cache, ids, check_steps)
        barrier()
        if rank == 0:
            try:
                whole_dev = pkg.B200(local)
                whole = pkg.Model.random(whole_dev, model_config(w), KIND[w["kind"]], seed=20260101)
                wcache, _ = make_streams(pkg, whole_dev, whole, w, lengths, check_steps + 2, data_rank)
                want = whole.decode_run(wcache, ids, check_steps)
                same = tp_tokens == want
                first_off = int(np.argmax(~same.all(axis=1))) if not same.all() else None
                line["parity"] = dict(tp_tokens_identical=bool(same.all()), steps=check_steps, streams=rows,
                                      agreeing_tokens=float(same.mean()), first_step_that_differs=first_off,
                                      against="the whole model's greedy tokens on one GPU, same weights, caches and first tokens")
                wcache.free(), whole.free(), whole_dev.close()
            except Exception as problem:  # the check must never cost the bench its line
                line["parity"] = dict(error=str(problem))
        barrier()

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
        kernels = [dict(kernel=f"ordered ragged attention (one layer, {rows} streams)", key="attention", bytes=attn_bytes, us=attn_s * 1e6,
                        gbs=attn_bytes / attn_s / 1e9, share_of_step=attn_share / (seconds / K)),
                   dict(kernel=f"block product {n}x{k} {w['kind']} rows={rows} (+quantiser)", key="up_product", bytes=up_bytes, us=up_s * 1e6,
                        gbs=up_bytes / up_s / 1e9, share_of_step=up_share / (seconds / K))]
        top = max(kernels, key=lambda e: e["share_of_step"])
        # DRAM bytes (read + written) of one launch from the profiler captures summarised under profiles/: taken on exactly
        # this workload's shapes and lengths at one GPU; none for other workloads or shards
        traffic = load_traffic().get(args.workload, {}).get(top["key"], {}).get("dram_bytes") if tp == 1 else None
        line["roofline"] = dict(bound="hbm", kernel=top["kernel"], achieved=top["gbs"], peak=peak["hbm_gbs"], unit="GB/s",
                                frac=top["gbs"] / peak["hbm_gbs"], traffic=traffic, algorithmic_bytes=top["bytes"], peak_kind=peak_kind)
        line["kernels"] = kernels
        for b in (tb, q, o, x, y):
            b.free()

        # ---- CPU baseline on a bounded sample, and the same streams on the device (N = 1 only) ------------
        if world == 1 and not args.no_cpu:
            parity_steps = max(args.parity_steps, 2)
            timed_steps = 5                       # about 10 s of host work at the headline shape
            refill(cache, lengths, rank)
            dev.sync()
            arm = CpuArm(pkg, model, cache, lengths, ids, threads, sample, parity_steps + 1)
            cpu_tokens, cpu_seconds, first_logits = [], 0.0, None
            for step in range(parity_steps):
                took = arm.step()
                if step == 0:
                    first_logits = arm.logits.copy()   # warm-up step: threads start, pages are touched; its logits serve the fast mode's check
                elif step <= timed_steps:
                    cpu_seconds += took
                cpu_tokens.append(list(arm.tokens))
            timed = min(timed_steps, parity_steps - 1)
            rate = len(sample) * timed / cpu_seconds
            # The same steps on the device from the same caches and first tokens: the sampled streams' greedy tokens must be the
            # CPU path's, step for step (rows are independent, so the other streams do not matter).
            try:
                refill(cache, lengths, rank)
                dev.sync()
                run = model.decode_run(cache, ids, parity_steps)
                gpu_tokens = [[int(t) for t in run[step, sample]] for step in range(parity_steps)]
                line["parity"] = dict(streams=len(sample), sample=sample_note, steps=parity_steps, identical_tokens=gpu_tokens == cpu_tokens,
                                      against="the CPU oracle's greedy tokens for the sampled streams at this workload's full size")
            except Exception as problem:  # the check must never cost the bench its line
                line["parity"] = dict(error=str(problem))
            line["cpu_baseline"] = dict(value=rate, unit="tokens/s", cores=threads, kind="port",
                                        sample=f"{sample_note} x {timed} decode steps, {cpu_seconds:.1f} s, "
                                               f"oracle's threaded product on {threads} threads, other host ops on one thread")
            # ---- the fast mode (tree sums, split-K online softmax) on the same workload: its speed and its distance from the CPU ----
            if not args.no_extra and args.mode == "exact":
                try:
                    dev.set_mode(pkg.FAST)
                    refill(cache, lengths, rank)
                    dev.sync()
                    fast_tokens, fast_logits = model.decode(cache, ids, logits=True)
                    model.decode_run(cache, fast_tokens, 3)
                    refill(cache, lengths, rank)
                    dev.sync()
                    fs, fe = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    fs.record(stream)
                    fast_run = model.decode_run(cache, ids, min(K, 20))
                    fe.record(stream)
                    fe.synchronize()
                    fast_seconds = fs.elapsed_time(fe) / 1e3 / min(K, 20)
                    got = fast_logits[sample]
                    rel = float(np.max(np.abs(got - first_logits)) / np.max(np.abs(first_logits)))
                    steps_same = 0
                    for step in range(min(parity_steps, fast_run.shape[0])):
                        if [int(t) for t in fast_run[step, sample]] != cpu_tokens[step]:
                            break
                        steps_same += 1
                    line.setdefault("extra", {})["c5_fast"] = dict(
                        tokens_per_second=rows / fast_seconds, ms_per_step=fast_seconds * 1e3, speedup_over_exact=(seconds / K) / fast_seconds,
                        max_relative_logit_error=rel, kl_nats_per_token=kl_per_token(first_logits, got),
                        greedy_steps_identical_to_cpu=steps_same, of_steps=min(parity_steps, fast_run.shape[0]), sample=sample_note)
                except Exception as problem:
                    line.setdefault("extra", {})["c5_fast"] = dict(error=str(problem))
                finally:
                    dev.set_mode(pkg.EXACT)
        else:
            line["cpu_baseline"] = None
    # ---- prefill of one long stream of this model (rank 0, N = 1) -------------------------------------
    if rank == 0 and world == 1 and not args.no_extra:
        try:
            line.setdefault("extra", {})["prefill_c5_one_stream"] = prefill_rate(pkg, dev, torch, stream, model, 1, 2048, w["vocab"])
        except Exception as problem:
            line.setdefault("extra", {})["prefill_c5_one_stream"] = dict(error=str(problem))
    cache.free()
    # ---- load time: the model written to a GGUF file and read back (rank 0, N = 1) -------------------
    if rank == 0 and world == 1 and not args.no_extra:
        try:
            path = os.path.join(tempfile.gettempdir(), f"tsm_bench_{os.getpid()}.gguf")
            t0 = time.perf_counter()
            model.save(path)
            save_seconds = time.perf_counter() - t0
            size = os.path.getsize(path)
            t0 = time.perf_counter()
            again = pkg.Model.load(path, dev)
            dev.sync()
            load_seconds = time.perf_counter() - t0
            again.free()
            os.unlink(path)
            line.setdefault("extra", {})["load"] = dict(file_bytes=size, load_seconds=load_seconds, load_gbs=size / load_seconds / 1e9,
                                                        save_seconds=save_seconds, draw_and_quantise_on_device_seconds=draw_seconds,
                                                        note="page cache warm: the file was just written")
        except Exception as problem:
            line.setdefault("extra", {})["load"] = dict(error=str(problem))
    model.free()

    # ---- batch 1 (135M- and GPT-2-XL-shaped), the 1.7B-shaped batch, the product sweep (rank 0, N = 1) ----
    if rank == 0 and world == 1 and not args.no_extra:
        extra = line.setdefault("extra", {})
        extra["c1_batch1"] = batch1_model(pkg, dev, torch, stream, WORKLOADS["c1"], 20260102, 120, peak["hbm_gbs"])
        extra["c4_batch1"] = batch1_model(pkg, dev, torch, stream, WORKLOADS["c4"], 20260104, 120, peak["hbm_gbs"])
        w3 = WORKLOADS["c3"]
        m3 = pkg.Model.random(dev, model_config(w3), KIND[w3["kind"]], seed=20260103)
        extra["prefill_c3"] = prefill_rate(pkg, dev, torch, stream, m3, 16, 128, w3["vocab"])
        m3.free()
        extra["product_sweep"] = product_sweep(pkg, dev, torch, stream, peak["hbm_gbs"])
        extra["matvec_batch1"] = [e for e in extra["product_sweep"] if e["columns"] == 1]

    # ---- N > 1: the baseline's data-parallel configuration, its 16 streams split over the ranks --------
    if world > 1 and not args.no_extra:
        w3 = WORKLOADS["c3"]
        first, count = pkg.groups.stream_share(w3["rows"], world, rank)
        solo = pkg.B200(local)   # a context of its own, outside the tensor-parallel group: a whole replica
        m3 = pkg.Model.random(solo, model_config(w3), KIND[w3["kind"]], seed=20260103)
        dp_steps = min(K, 50)
        seconds3 = 0.0
        if count > 0:
            c3 = m3.new_batch_cache(count, w3["len_lo"] + dp_steps + 8)
            for row in range(count):
                c3.fill(row, w3["len_lo"], seed=3000 + first + row)
            ids3 = np.random.default_rng(7).integers(0, w3["vocab"], size=w3["rows"]).astype(np.int32)[first:first + count]
            m3.decode_run(c3, ids3, 3)
        barrier()
        if count > 0:
            solo_stream = torch.cuda.ExternalStream(solo.stream, device=local)
            s3, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s3.record(solo_stream)
            m3.decode_run(c3, ids3, dp_steps)
            e3.record(solo_stream)
            e3.synchronize()
            seconds3 = s3.elapsed_time(e3) / 1e3
            c3.free()
        seconds3 = max_over_ranks(seconds3)
        m3.free(), solo.close()
        if rank == 0:
            line.setdefault("extra", {})["c3_dp"] = dict(workload=w3["name"], parallelism=f"dp{world}: {w3['rows']} streams split over the ranks, a replica each, no collective",
                                                          tokens_per_second=w3["rows"] * dp_steps / seconds3, ms_per_step=seconds3 / dp_steps * 1e3, scaling="strong")
    if rank == 0:
        print(json.dumps(line))
    dev.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
