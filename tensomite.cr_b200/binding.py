"""ctypes binding of libtsm_b200.so, with tensomite's host-side names on top.

Everything here forwards to the C ABI declared in include/tsm_b200.h.  The classes mirror the
reference's: a device with alloc/upload/download/sync (src/tensomite/device.cr:39-68), `Quant`-style
operator calls on device buffers, `Llama` / `GPT2` with `forward`, `forward_last`, `generate` and a
batch cache (src/tensomite/models/generative.cr).  Errors carry the reference's class names.
"""
import ctypes as C
import os
import re

import numpy as np

from . import build as _build

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "include", "tsm_b200.h")

Q8_0, Q4_0, Q4_1, F32 = 0, 1, 2, -1
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18, Q4_1: 20}
FAST, EXACT = 0, 1
TP_GATHER, TP_REDUCE = 0, 1


class Error(Exception):
    """Tensomite::Error"""


class DeviceError(Error):
    pass


class ShapeError(Error):
    pass


class ExecutionError(Error):
    pass


class DTypeError(Error):
    pass


class CommError(DeviceError):
    """The tensor-parallel group failed (TSM_ERR_COMM)."""


class TimeoutError_(DeviceError):
    """A bounded wait ran out (TSM_ERR_TIMEOUT)."""


_STATUS = {1: DeviceError, 2: ShapeError, 3: ExecutionError, 4: DeviceError, 5: Error, 6: DTypeError, 7: TimeoutError_,
           8: CommError}

_lib = None


class ModelConfig(C.Structure):
    _fields_ = [("arch", C.c_int), ("layers", C.c_int), ("width", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int),
                ("head_width", C.c_int), ("hidden", C.c_int), ("vocab", C.c_int), ("context", C.c_int),
                ("eps", C.c_float), ("rope_theta", C.c_double), ("tied", C.c_int)]


class Counters(C.Structure):
    _fields_ = [(name, C.c_int64) for name in
                ("launches", "uploads", "downloads", "upload_bytes", "download_bytes", "allocs", "pool_hits",
                 "pool_misses", "pool_held_bytes", "frees", "host_ops", "graph_replays", "collectives")]


class ProfileEntry(C.Structure):
    _fields_ = [("label", C.c_char * 80), ("count", C.c_int64), ("seconds", C.c_double)]


PICK_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_float), C.c_int)


def declared_symbols():
    """Every function include/tsm_b200.h declares."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tsm_[a-z0-9_]+)\s*\(", text)))


def library():
    """Loads the CUDA library, building it first when a source is newer; never falls back to anything else."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIBRARY
    if _build.stale():
        path = _build.build()
    lib = C.CDLL(path)
    lib.tsm_status_name.restype = C.c_char_p
    lib.tsm_ctx_stream.restype = C.c_void_p
    lib.tsm_ctx_stream.argtypes = [C.c_void_p]
    _lib = lib
    return lib


def tp_unique_id():
    """128 bytes that name a new tensor-parallel group; made on one rank, carried to the others by the host."""
    raw = (C.c_uint8 * 128)()
    rc = library().tsm_tp_unique_id(raw)
    if rc != 0:
        raise DeviceError("tsm_tp_unique_id: " + library().tsm_status_name(rc).decode() + " (is NCCL loadable?)")
    return bytes(raw)


def check_exports():
    lib = library()
    missing = [name for name in declared_symbols() if not hasattr(lib, name)]
    if missing:
        raise Error("libtsm_b200.so lacks " + ", ".join(missing))
    return True


def _ptr(a, t=C.c_void_p):
    return a.ctypes.data_as(t)


class Buffer:
    """Device memory owned by one device (CUDABuffer, src/tensomite/cuda.cr:49-70)."""

    def __init__(self, device, ptr, nbytes):
        self.device, self.ptr, self.nbytes = device, ptr, nbytes

    def free(self):
        if self.ptr:
            self.device.lib.tsm_free(self.device.ctx, C.c_uint64(self.ptr))
            self.ptr = 0

    def numpy(self, dtype, shape=None):
        count = self.nbytes // np.dtype(dtype).itemsize
        out = np.empty(count, dtype=dtype)
        self.device.download(self, out)
        return out.reshape(shape) if shape is not None else out


class B200:
    """The device (a `Tensomite::Device`): one CUDA context, one in-order stream, a buffer pool."""

    def __init__(self, ordinal=0):
        self.lib = library()
        self.ctx = C.c_void_p()
        rc = self.lib.tsm_ctx_create(C.c_int(ordinal), C.byref(self.ctx))
        if rc != 0:
            raise DeviceError(f"tsm_ctx_create({ordinal}): {self.lib.tsm_status_name(rc).decode()} (no CUDA device, "
                              "and this library has no other way to compute)")
        self.ordinal = ordinal

    def check(self, rc, what=""):
        if rc == 0:
            return
        buf = C.create_string_buffer(1024)
        self.lib.tsm_last_error(self.ctx, buf, 1024)
        raise _STATUS.get(rc, Error)(f"{what}: {self.lib.tsm_status_name(rc).decode()} ({buf.value.decode()})")

    def close(self):
        if self.ctx:
            self.lib.tsm_ctx_destroy(self.ctx)
            self.ctx = C.c_void_p()

    @property
    def stream(self):
        return self.lib.tsm_ctx_stream(self.ctx)

    def set_mode(self, mode):
        self.check(self.lib.tsm_set_mode(self.ctx, C.c_int(mode)), "tsm_set_mode")

    def tp_init(self, rank, world, group_id):
        """Joins this device to a tensor-parallel group of `world` ranks; `group_id` is tp_unique_id() of one rank.
        Models loaded or drawn afterwards hold this rank's rows only."""
        if world > 1 and len(group_id) != 128:
            raise ShapeError("a group id is 128 bytes")
        raw = (C.c_uint8 * 128).from_buffer_copy(bytes(group_id)) if world > 1 else None
        self.check(self.lib.tsm_tp_init(self.ctx, C.c_int(rank), C.c_int(world), raw), "tsm_tp_init")

    def tp_variant(self, variant):
        """TP_GATHER (default: the bits of one GPU) or TP_REDUCE (o and down over input columns, all-reduced); set before
        the model is loaded."""
        self.check(self.lib.tsm_tp_variant(self.ctx, C.c_int(variant)), "tsm_tp_variant")

    def tp_abort(self):
        """Leaves the group without waiting for the other ranks; later exchanges raise CommError."""
        self.check(self.lib.tsm_tp_abort(self.ctx), "tsm_tp_abort")

    def profile(self, shapes=False):
        """cuda.profile = CUDA::Profile.new(per_kernel: true, shapes: shapes): starts timing every operator on the GPU."""
        self.check(self.lib.tsm_profile_begin(self.ctx, C.c_int(1 if shapes else 0)), "tsm_profile_begin")

    def profile_read(self, end=False):
        """[(label, launches, GPU seconds)], longest first; with `end` the profile stops."""
        count = C.c_int()
        self.check(self.lib.tsm_profile_read(self.ctx, None, C.c_int(0), C.byref(count)), "tsm_profile_read")
        entries = (ProfileEntry * max(count.value, 1))()
        self.check(self.lib.tsm_profile_read(self.ctx, entries, C.c_int(count.value), C.byref(count)), "tsm_profile_read")
        if end:
            self.check(self.lib.tsm_profile_end(self.ctx), "tsm_profile_end")
        return [(entries[i].label.decode(), int(entries[i].count), float(entries[i].seconds)) for i in range(count.value)]

    def debug_wait_limit(self, spins, starve_copies):
        self.check(self.lib.tsm_debug_wait_limit(self.ctx, C.c_uint(spins), C.c_int(starve_copies)), "tsm_debug_wait_limit")

    def tp_info(self):
        rank, world = C.c_int(), C.c_int()
        self.check(self.lib.tsm_tp_info(self.ctx, C.byref(rank), C.byref(world)), "tsm_tp_info")
        return rank.value, world.value

    def alloc(self, nbytes):
        ptr = C.c_uint64()
        self.check(self.lib.tsm_alloc(self.ctx, C.c_int64(nbytes), C.byref(ptr)), "tsm_alloc")
        return Buffer(self, ptr.value, nbytes)

    def upload(self, buffer, array):
        array = np.ascontiguousarray(array)
        if array.nbytes > buffer.nbytes:
            raise ShapeError(f"{array.nbytes} bytes do not fit a buffer of {buffer.nbytes}")
        self.check(self.lib.tsm_upload(self.ctx, C.c_uint64(buffer.ptr), _ptr(array), C.c_int64(array.nbytes)),
                   "tsm_upload")

    def download(self, buffer, array):
        assert array.flags["C_CONTIGUOUS"]
        self.check(self.lib.tsm_download(self.ctx, _ptr(array), C.c_uint64(buffer.ptr), C.c_int64(array.nbytes)),
                   "tsm_download")

    def tensor(self, array):
        """A buffer holding `array`'s bytes (Tensor.from + realize)."""
        array = np.ascontiguousarray(array)
        buf = self.alloc(max(array.nbytes, 1))
        if array.nbytes:
            self.upload(buf, array)
        return buf

    def sync(self):
        self.check(self.lib.tsm_sync(self.ctx), "tsm_sync")

    def counters(self):
        out = Counters()
        self.check(self.lib.tsm_counters_read(self.ctx, C.byref(out)), "tsm_counters_read")
        return {name: getattr(out, name) for name, _ in Counters._fields_}

    def reset_counters(self):
        self.lib.tsm_counters_reset(self.ctx)

    # ---- operators --------------------------------------------------------------------------

    def quantize(self, x, kind):
        """Tensor#quantize: float32 array -> device buffer of ggml blocks."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        src = self.tensor(x)
        out = self.alloc(max(x.size // 32 * BLOCK_BYTES.get(kind, 0), 1))
        self.check(self.lib.tsm_quantize_blocks(self.ctx, C.c_uint64(src.ptr), C.c_int64(x.size), C.c_int(kind),
                                                C.c_uint64(out.ptr)), "tsm_quantize_blocks")
        self.sync()
        src.free()
        out.nbytes = x.size // 32 * BLOCK_BYTES[kind]
        return out

    def dequantize(self, blocks, count, kind):
        out = self.alloc(count * 4)
        self.check(self.lib.tsm_dequantize_blocks(self.ctx, C.c_uint64(blocks.ptr), C.c_int64(count), C.c_int(kind),
                                                  C.c_uint64(out.ptr)), "tsm_dequantize_blocks")
        self.sync()
        return out

    def quantize_rows(self, x):
        """quantize_rows_q8_f32: float32 [rows,k] -> (scales, sums, qs) numpy arrays."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, k = x.shape
        src = self.tensor(x)
        blocks = rows * (k // 32)
        scales, sums, qs = self.alloc(blocks * 4), self.alloc(blocks * 4), self.alloc(rows * k)
        self.check(self.lib.tsm_quantize_rows_q8(self.ctx, C.c_uint64(src.ptr), C.c_int(rows), C.c_int(k), C.c_int64(k),
                                                 C.c_uint64(scales.ptr), C.c_uint64(sums.ptr), C.c_uint64(qs.ptr)),
                   "tsm_quantize_rows_q8")
        self.sync()
        out = (scales.numpy(np.float32, (rows, -1)), sums.numpy(np.float32, (rows, -1)), qs.numpy(np.int8, (rows, k)))
        for b in (src, scales, sums, qs):
            b.free()
        return out

    def block_matmul(self, x, w, kind, n, bias=None):
        """Tensor#linear on a block weight: x float32 [rows,k] (numpy or Buffer+shape), w Buffer -> numpy [rows,n]."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, k = x.shape
        xb = self.tensor(x)
        bb = self.tensor(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
        out = self.alloc(max(rows * n * 4, 1))
        self.check(self.lib.tsm_block_matmul(self.ctx, C.c_uint64(xb.ptr), C.c_int(rows), C.c_int(k), C.c_int64(k),
                                             C.c_uint64(w.ptr), C.c_int(kind), C.c_int(n),
                                             C.c_uint64(bb.ptr if bb else 0), C.c_uint64(out.ptr)), "tsm_block_matmul")
        self.sync()
        result = out.numpy(np.float32)[:rows * n].reshape(rows, n)
        for b in (xb, bb, out):
            if b:
                b.free()
        return result

    def matmul_f32(self, x, w, bias=None):
        """Tensor#linear on an F32 weight: x float32 [rows,k], w float32 [n,k] -> numpy [rows,n], sums in index order."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        rows, k = x.shape
        n = w.shape[0]
        xb, wb = self.tensor(x), self.tensor(w)
        bb = self.tensor(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
        out = self.alloc(max(rows * n * 4, 1))
        try:
            self.check(self.lib.tsm_matmul_f32(self.ctx, C.c_uint64(xb.ptr), C.c_int(rows), C.c_int(k), C.c_uint64(wb.ptr), C.c_int(n),
                                               C.c_uint64(bb.ptr if bb else 0), C.c_uint64(out.ptr)), "tsm_matmul_f32")
            self.sync()
            return out.numpy(np.float32)[:rows * n].reshape(rows, n)
        finally:
            for b in (xb, wb, bb, out):
                if b:
                    b.free()

    def block_matmul_static(self, x, w, kind, n, bias=None):
        """As block_matmul, through tsm_block_matmul_static: the product's scratch is a fixed array in the library."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, k = x.shape
        xb = self.tensor(x)
        bb = self.tensor(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
        out = self.alloc(max(rows * n * 4, 1))
        try:
            self.check(self.lib.tsm_block_matmul_static(self.ctx, C.c_uint64(xb.ptr), C.c_int(rows), C.c_int(k), C.c_int64(k),
                                                        C.c_uint64(w.ptr), C.c_int(kind), C.c_int(n),
                                                        C.c_uint64(bb.ptr if bb else 0), C.c_uint64(out.ptr)),
                       "tsm_block_matmul_static")
            self.sync()
            return out.numpy(np.float32)[:rows * n].reshape(rows, n)
        finally:
            for b in (xb, bb, out):
                if b:
                    b.free()

    def gather_blocks(self, table, kind, table_rows, width, ids):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        idb = self.tensor(ids)
        out = self.alloc(max(ids.size * width * 4, 1))
        try:
            self.check(self.lib.tsm_gather_blocks(self.ctx, C.c_uint64(table.ptr), C.c_int(kind), C.c_int(table_rows),
                                                  C.c_int(width), C.c_uint64(idb.ptr), C.c_int(ids.size),
                                                  C.c_uint64(out.ptr)), "tsm_gather_blocks")
            self.sync()
            return out.numpy(np.float32)[:ids.size * width].reshape(ids.size, width)
        finally:
            idb.free()
            out.free()

    def _unary_rows(self, fn, name, x, *extra):
        x = np.ascontiguousarray(x, dtype=np.float32)
        xb = self.tensor(x)
        out = self.alloc(max(x.nbytes, 1))
        try:
            self.check(fn(xb, out, *extra), name)
            self.sync()
            return out.numpy(np.float32)[:x.size].reshape(x.shape)
        finally:
            xb.free()
            out.free()

    def rmsnorm(self, x, w, eps=1e-5):
        rows, n = x.shape
        wb = self.tensor(np.ascontiguousarray(w, dtype=np.float32)) if w is not None else None
        try:
            return self._unary_rows(lambda xb, out: self.lib.tsm_rmsnorm(
                self.ctx, C.c_uint64(xb.ptr), C.c_uint64(wb.ptr if wb else 0), C.c_int(rows), C.c_int(n), C.c_float(eps),
                C.c_uint64(out.ptr)), "tsm_rmsnorm", x)
        finally:
            if wb:
                wb.free()

    def layernorm(self, x, w, b, eps=1e-5):
        rows, n = x.shape
        wb, bb = self.tensor(np.ascontiguousarray(w, dtype=np.float32)), self.tensor(np.ascontiguousarray(b, dtype=np.float32))
        try:
            return self._unary_rows(lambda xb, out: self.lib.tsm_layernorm(
                self.ctx, C.c_uint64(xb.ptr), C.c_uint64(wb.ptr), C.c_uint64(bb.ptr), C.c_int(rows), C.c_int(n),
                C.c_float(eps), C.c_uint64(out.ptr)), "tsm_layernorm", x)
        finally:
            wb.free()
            bb.free()

    def rope(self, x, cos_table, sin_table, positions):
        """x float32 [tokens, heads, width]; tables [context, width]; positions int32 [tokens]."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        tokens, heads, width = x.shape
        cb, sb = self.tensor(np.ascontiguousarray(cos_table, dtype=np.float32)), self.tensor(np.ascontiguousarray(sin_table, dtype=np.float32))
        pb = self.tensor(np.ascontiguousarray(positions, dtype=np.int32))
        try:
            return self._unary_rows(lambda xb, out: self.lib.tsm_rope(
                self.ctx, C.c_uint64(xb.ptr), C.c_int(tokens), C.c_int(heads), C.c_int(width), C.c_int64(heads * width),
                C.c_uint64(cb.ptr), C.c_uint64(sb.ptr), C.c_int(cos_table.shape[0]), C.c_uint64(pb.ptr), C.c_uint64(out.ptr)),
                "tsm_rope", x)
        finally:
            for b in (cb, sb, pb):
                b.free()

    def swiglu(self, gate, up):
        gate = np.ascontiguousarray(gate, dtype=np.float32)
        up = np.ascontiguousarray(up, dtype=np.float32)
        rows, n = gate.shape
        ub = self.tensor(up)
        try:
            return self._unary_rows(lambda gb, out: self.lib.tsm_swiglu(
                self.ctx, C.c_uint64(gb.ptr), C.c_uint64(ub.ptr), C.c_int(rows), C.c_int(n), C.c_int64(n), C.c_uint64(out.ptr)),
                "tsm_swiglu", gate)
        finally:
            ub.free()

    def gelu(self, x):
        return self._unary_rows(lambda xb, out: self.lib.tsm_gelu(self.ctx, C.c_uint64(xb.ptr), C.c_int64(x.size), C.c_uint64(out.ptr)),
                                "tsm_gelu", x)

    def silu(self, x):
        return self._unary_rows(lambda xb, out: self.lib.tsm_silu(self.ctx, C.c_uint64(xb.ptr), C.c_int64(x.size), C.c_uint64(out.ptr)),
                                "tsm_silu", x)

    def add(self, a, b):
        bb = self.tensor(np.ascontiguousarray(b, dtype=np.float32))
        try:
            return self._unary_rows(lambda ab, out: self.lib.tsm_add(self.ctx, C.c_uint64(ab.ptr), C.c_uint64(bb.ptr), C.c_int64(a.size),
                                                                     C.c_uint64(out.ptr)), "tsm_add", a)
        finally:
            bb.free()

    def write_rows(self, cache, values, slots):
        """cache float32 [rows, heads, capacity, width] (numpy, returned updated), values [tokens, heads, width]."""
        cache = np.ascontiguousarray(cache, dtype=np.float32)
        values = np.ascontiguousarray(values, dtype=np.float32)
        rows, heads, capacity, width = cache.shape
        cb, vb = self.tensor(cache), self.tensor(values)
        sb = self.tensor(np.ascontiguousarray(slots, dtype=np.int32))
        try:
            self.check(self.lib.tsm_write_rows(self.ctx, C.c_uint64(cb.ptr), C.c_int(rows), C.c_int(heads), C.c_int(capacity),
                                               C.c_int(width), C.c_uint64(vb.ptr), C.c_int64(heads * width),
                                               C.c_int(values.shape[0]), C.c_uint64(sb.ptr)), "tsm_write_rows")
            self.sync()
            return cb.numpy(np.float32, cache.shape)
        finally:
            for b in (cb, vb, sb):
                b.free()

    def write(self, dst, value, axis, start):
        """Tensor#write: dst (numpy, returned updated) with `value` written at `start` along `axis`, in place on the device."""
        dst = np.ascontiguousarray(dst, dtype=np.float32)
        value = np.ascontiguousarray(value, dtype=np.float32)
        db, vb = self.tensor(dst), self.tensor(value)
        shape = (C.c_int32 * dst.ndim)(*dst.shape)
        try:
            self.check(self.lib.tsm_write(self.ctx, C.c_uint64(db.ptr), shape, C.c_int(dst.ndim), C.c_uint64(vb.ptr),
                                          C.c_int(value.shape[axis]), C.c_int(axis), C.c_int(start)), "tsm_write")
            self.sync()
            return db.numpy(np.float32, dst.shape)
        finally:
            db.free()
            vb.free()

    def ragged_attention(self, q, k, v, table, scale):
        """q [tokens, heads, width]; k, v [rows, kv_heads, capacity, width]; table int32 [tokens, 3]."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        tokens, heads, width = q.shape
        rows, kv_heads, capacity, _ = k.shape
        kb, vb = self.tensor(k), self.tensor(v)
        tb = self.tensor(np.ascontiguousarray(table, dtype=np.int32))
        try:
            return self._unary_rows(lambda qb, out: self.lib.tsm_ragged_attention(
                self.ctx, C.c_uint64(qb.ptr), C.c_int64(heads * width), C.c_int(tokens), C.c_int(heads), C.c_int(width),
                C.c_uint64(kb.ptr), C.c_uint64(vb.ptr), C.c_int(rows), C.c_int(kv_heads), C.c_int(capacity), C.c_uint64(tb.ptr),
                C.c_float(scale), C.c_uint64(out.ptr)), "tsm_ragged_attention", q)
        finally:
            for b in (kb, vb, tb):
                b.free()

    def argmax(self, logits):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        rows, n = logits.shape
        lb = self.tensor(logits)
        out = self.alloc(rows * 4)
        try:
            self.check(self.lib.tsm_argmax(self.ctx, C.c_uint64(lb.ptr), C.c_int(rows), C.c_int(n), C.c_uint64(out.ptr)), "tsm_argmax")
            self.sync()
            return out.numpy(np.int32)
        finally:
            lb.free()
            out.free()

    def topk(self, logits, count):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        rows, n = logits.shape
        lb = self.tensor(logits)
        ids, vals = self.alloc(rows * count * 4), self.alloc(rows * count * 4)
        try:
            self.check(self.lib.tsm_topk(self.ctx, C.c_uint64(lb.ptr), C.c_int(rows), C.c_int(n), C.c_int(count),
                                         C.c_uint64(ids.ptr), C.c_uint64(vals.ptr)), "tsm_topk")
            self.sync()
            return ids.numpy(np.int32, (rows, count)), vals.numpy(np.float32, (rows, count))
        finally:
            for b in (lb, ids, vals):
                b.free()


class BatchCache:
    """Generative::BatchCache (models/generative.cr:54-79)."""

    def __init__(self, model, rows, capacity):
        self.model, self.size, self.capacity = model, rows, capacity
        self.handle = C.c_void_p()
        model.device.check(model.device.lib.tsm_cache_create(model.handle, C.c_int(rows), C.c_int(capacity), C.byref(self.handle)),
                           "tsm_cache_create")

    def length(self, row):
        out = C.c_int()
        self.model.device.check(self.model.device.lib.tsm_cache_length(self.handle, C.c_int(row), C.byref(out)), "tsm_cache_length")
        return out.value

    def reset(self, row):
        self.model.device.check(self.model.device.lib.tsm_cache_reset(self.handle, C.c_int(row)), "tsm_cache_reset")

    def fill(self, row, length, seed):
        self.model.device.check(self.model.device.lib.tsm_cache_fill(self.handle, C.c_int(row), C.c_int(length), C.c_uint64(seed)),
                                "tsm_cache_fill")

    def layer(self, index):
        """Device addresses of layer `index`'s keys and values, each [rows, kv_heads, capacity, head_width] float32."""
        k, v = C.c_uint64(), C.c_uint64()
        self.model.device.check(self.model.device.lib.tsm_cache_layer(self.handle, C.c_int(index), C.byref(k), C.byref(v)), "tsm_cache_layer")
        c = self.model.config
        nbytes = self.size * c["kv_heads"] * self.capacity * c["head_width"] * 4
        return Buffer(self.model.device, k.value, nbytes), Buffer(self.model.device, v.value, nbytes)

    def free(self):
        if self.handle:
            self.model.device.lib.tsm_cache_free(self.handle)
            self.handle = C.c_void_p()


class Model:
    """A decoder with `Generative`'s interface; `Llama` and `GPT2` below only differ in how they are made."""

    def __init__(self, device, handle):
        self.device, self.handle = device, handle
        cfg = ModelConfig()
        device.check(device.lib.tsm_model_config_get(handle, C.byref(cfg)), "tsm_model_config_get")
        self.config = {name: getattr(cfg, name) for name, _ in ModelConfig._fields_}
        self.config["arch"] = "llama" if cfg.arch == 0 else "gpt2"

    @classmethod
    def load(cls, path, device):
        """Llama.load / GPT2.load of a .gguf file (models/llama.cr:165-206, models/gpt2.cr:75-89)."""
        handle = C.c_void_p()
        device.check(device.lib.tsm_model_load_gguf(device.ctx, str(path).encode(), C.byref(handle)), "tsm_model_load_gguf")
        return cls(device, handle)

    @classmethod
    def load_safetensors(cls, path, device, config, kind):
        """GPT2.load / Llama.load of a Hugging Face safetensors file, then .quantize(kind, embeddings: true) on the device.
        `config` needs arch and heads (GPT-2), or arch, heads, kv_heads, eps, rope_theta, context (Llama)."""
        cfg = ModelConfig(0 if config["arch"] == "llama" else 1, 0, 0, config["heads"], config.get("kv_heads", config["heads"]),
                          config.get("head_width", 0), 0, 0, config.get("context", 0), config.get("eps", 1e-5),
                          config.get("rope_theta", 10000.0), 0)
        handle = C.c_void_p()
        device.check(device.lib.tsm_model_load_safetensors(device.ctx, str(path).encode(), C.byref(cfg), C.c_int(kind), C.byref(handle)),
                     "tsm_model_load_safetensors")
        return cls(device, handle)

    @classmethod
    def random(cls, device, config, kind, seed):
        """Llama.new(config) / GPT2.new(config) with normal(0.02) weights from `seed`, quantised to `kind`."""
        cfg = ModelConfig(0 if config["arch"] == "llama" else 1, config["layers"], config["width"], config["heads"],
                          config.get("kv_heads", config["heads"]), config["head_width"], config["hidden"], config["vocab"],
                          config["context"], config.get("eps", 1e-5), config.get("rope_theta", 10000.0),
                          1 if config.get("tied", True) else 0)
        handle = C.c_void_p()
        device.check(device.lib.tsm_model_random(device.ctx, C.byref(cfg), C.c_int(kind), C.c_uint64(seed), C.byref(handle)),
                     "tsm_model_random")
        return cls(device, handle)

    def save(self, path):
        """Module#save to a .gguf file: quantised weights as they are."""
        self.device.check(self.device.lib.tsm_model_save_gguf(self.handle, str(path).encode()), "tsm_model_save_gguf")

    def tensor(self, name):
        """(Buffer, kind, n, k) of a parameter."""
        ptr, kind, n, k = C.c_uint64(), C.c_int(), C.c_int(), C.c_int()
        self.device.check(self.device.lib.tsm_model_tensor(self.handle, name.encode(), C.byref(ptr), C.byref(kind), C.byref(n),
                                                           C.byref(k)), "tsm_model_tensor")
        nbytes = n.value * k.value * 4 if kind.value < 0 else n.value * (k.value // 32) * BLOCK_BYTES[kind.value]
        return Buffer(self.device, ptr.value, nbytes), kind.value, n.value, k.value

    def new_batch_cache(self, rows, capacity=None):
        return BatchCache(self, rows, capacity or self.config["context"])

    def _packed(self, appends, cache, last):
        counts = np.array([len(a) for a in appends], dtype=np.int32)
        if counts.size != cache.size:
            raise ShapeError(f"{counts.size} appends for {cache.size} rows")
        ids = np.array([t for a in appends for t in a], dtype=np.int32)
        outputs = int((counts > 0).sum()) if last else int(counts.sum())
        logits = np.empty((max(outputs, 1), self.config["vocab"]), dtype=np.float32)
        if ids.size == 0:
            ids = np.zeros(1, dtype=np.int32)
        self.device.check(self.device.lib.tsm_forward(self.handle, cache.handle, _ptr(counts), _ptr(ids), C.c_int(1 if last else 0),
                                                      _ptr(logits)), "tsm_forward")
        return logits[:outputs]

    def forward(self, appends, cache):
        """Generative#forward(appends, BatchCache): logits of every new position, rows one after another."""
        return self._packed(appends, cache, last=False)

    def forward_last(self, appends, cache):
        """Generative#forward_last(appends, BatchCache): logits of each row's last new position."""
        return self._packed(appends, cache, last=True)

    def decode(self, cache, ids, logits=False):
        """One greedy step for every row (a replayed CUDA graph); returns the picked tokens (and logits)."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if ids.size != cache.size:
            raise ShapeError(f"{ids.size} tokens for {cache.size} rows")
        tokens = np.empty(cache.size, dtype=np.int32)
        out = np.empty((cache.size, self.config["vocab"]), dtype=np.float32) if logits else None
        self.device.check(self.device.lib.tsm_decode(self.handle, cache.handle, _ptr(ids), _ptr(tokens),
                                                     _ptr(out) if logits else None), "tsm_decode")
        return (tokens, out) if logits else tokens

    def decode_run(self, cache, ids, steps):
        """`steps` greedy steps for every row, fed on the device; returns tokens [steps, rows]."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if ids.size != cache.size:
            raise ShapeError(f"{ids.size} tokens for {cache.size} rows")
        tokens = np.empty((steps, cache.size), dtype=np.int32)
        self.device.check(self.device.lib.tsm_decode_run(self.handle, cache.handle, _ptr(ids), C.c_int(steps), _ptr(tokens)),
                          "tsm_decode_run")
        return tokens

    def generate(self, prompt, count):
        """Generative#generate with Sampler.greedy."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        tokens = np.empty(max(count, 1), dtype=np.int32)
        self.device.check(self.device.lib.tsm_generate(self.handle, _ptr(prompt), C.c_int(prompt.size), C.c_int(count), _ptr(tokens)),
                          "tsm_generate")
        return tokens[:count].tolist()

    def generate_sampled(self, prompt, count, pick=None, top_k=0, stop=()):
        """Generative#generate(prompt, count, sampler, stop): `pick(step, ids, logits)` chooses among the `top_k` candidates the
        device kept (ids None and every logit in index order when top_k is 0); None is the greedy sampler on the device."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        stop = np.ascontiguousarray(list(stop), dtype=np.int32)
        tokens = np.empty(max(count, 1), dtype=np.int32)
        produced = C.c_int()

        def trampoline(user, step, ids, logits, n):
            values = np.ctypeslib.as_array(logits, shape=(n,)).copy()
            which = np.ctypeslib.as_array(ids, shape=(n,)).copy() if ids else None
            return int(pick(step, which, values))

        callback = PICK_FN(trampoline) if pick is not None else C.cast(None, PICK_FN)
        self.device.check(self.device.lib.tsm_generate_sampled(self.handle, _ptr(prompt), C.c_int(prompt.size), C.c_int(count),
                                                               _ptr(stop) if stop.size else None, C.c_int(stop.size), C.c_int(top_k),
                                                               callback, None, _ptr(tokens), C.byref(produced)), "tsm_generate_sampled")
        return tokens[:produced.value].tolist()

    def free(self):
        if self.handle:
            self.device.lib.tsm_model_free(self.handle)
            self.handle = C.c_void_p()


class Llama(Model):
    pass


class GPT2(Model):
    pass


__all__ = ["tp_unique_id", "Q8_0", "Q4_0", "Q4_1", "F32", "BLOCK_BYTES", "FAST", "EXACT", "TP_GATHER", "TP_REDUCE", "Error", "DeviceError", "ShapeError", "ExecutionError",
           "DTypeError", "CommError", "TimeoutError_", "ModelConfig", "Counters", "declared_symbols", "library", "check_exports", "Buffer", "B200", "BatchCache",
           "Model", "Llama", "GPT2"]
