"""ctypes access to the CPU oracle (TEST INFRASTRUCTURE — never imported by the product).

`liboracle.so` is the C restatement in `tsm_oracle.c`; `_ref/libkernels.so` is
the reference's own kernel sources compiled for the host (Makefile target
`ref`), driven here through the two entry points its emulation header exports
(`tensomite_kernel`, `tensomite_launch`; scripts/cuda_stub/emulate.h:103-141).
Only tests, the smoke check and the CPU-baseline leg of the benchmark use this
module, and only as the checker.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
Q8_0, Q4_0, Q4_1 = 0, 1, 2
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18, Q4_1: 20}
KIND_NAMES = {"Q8_0": Q8_0, "Q4_0": Q4_0, "Q4_1": Q4_1}

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int32)


def build(ref=True, reference=None):
    """Compiles liboracle.so and, when a checkout of the reference is at hand, _ref/libkernels.so from its sources.

    The checkout is `reference`, else $TENSOMITE_REFERENCE, else the Makefile's own default (`make ref REFERENCE=...`)."""
    subprocess.run(["make", "-s", "-C", HERE], check=True)
    if not ref:
        return
    where = reference or os.environ.get("TENSOMITE_REFERENCE")
    if where is None:
        shown = subprocess.run(["make", "-s", "-C", HERE, "print-reference"], capture_output=True, text=True)
        where = shown.stdout.strip() if shown.returncode == 0 else ""
    if where and os.path.isdir(os.path.join(where, "src", "tensomite", "cuda")):
        subprocess.run(["make", "-s", "-C", HERE, "ref", "REFERENCE=" + where], check=True)


def _load():
    path = os.path.join(HERE, "liboracle.so")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(os.path.join(HERE, "tsm_oracle.c")):
        build(ref=False)
    lib = C.CDLL(path)
    lib.orc_f32_to_f16.restype = C.c_uint16
    lib.orc_f32_to_f16.argtypes = [C.c_float]
    lib.orc_f16_to_f32.restype = C.c_float
    lib.orc_f16_to_f32.argtypes = [C.c_uint16]
    lib.orc_exp.restype = C.c_float
    lib.orc_exp.argtypes = [C.c_float]
    lib.orc_tanh.restype = C.c_float
    lib.orc_tanh.argtypes = [C.c_float]
    lib.orc_gather_blocks.restype = C.c_int64
    return lib


lib = _load()


def _p(a, t):
    return a.ctypes.data_as(t)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def f32_to_f16_bits(v):
    return int(lib.orc_f32_to_f16(C.c_float(v)))


def f16_bits_to_f32(bits):
    return float(lib.orc_f16_to_f32(C.c_uint16(bits)))


def exp(x):
    x = _f32(x)
    return np.array([lib.orc_exp(C.c_float(v)) for v in x.ravel()], dtype=np.float32).reshape(x.shape)


def tanh(x):
    x = _f32(x)
    return np.array([lib.orc_tanh(C.c_float(v)) for v in x.ravel()], dtype=np.float32).reshape(x.shape)


def quantize(kind, values):
    """quant.cr:77-90 — block bytes of `values` (size a multiple of 32) as a uint8 array."""
    x = _f32(values).ravel()
    assert x.size % 32 == 0
    out = np.empty(x.size // 32 * BLOCK_BYTES[kind], dtype=np.uint8)
    lib.orc_quantize(C.c_int(kind), _p(x, _f32p), C.c_int64(x.size), _p(out, _u8p))
    return out


def dequantize(kind, data, count):
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.empty(count, dtype=np.float32)
    lib.orc_dequantize(C.c_int(kind), _p(data, _u8p), C.c_int64(count), _p(out, _f32p))
    return out


def quantize_activations(x, with_sums=True):
    """quant.cr:428-442 for each row of x [rows,k] -> scales, sums [rows,k/32] f32 and qs [rows,k] i8."""
    x = _f32(x)
    rows, k = x.shape
    scales = np.zeros((rows, k // 32), dtype=np.float32)
    sums = np.zeros((rows, k // 32), dtype=np.float32)
    qs = np.zeros((rows, k), dtype=np.int8)
    for r in range(rows):
        lib.orc_quantize_activations(_p(x[r], _f32p), C.c_int(k), _p(scales[r], _f32p), _p(sums[r], _f32p),
                                     _p(qs[r], _i8p), C.c_int(1 if with_sums else 0))
    return scales, sums, qs


def matmul_reference(kind, x, w, n, bias=None):
    """quant.cr:122-142 (+ bias as devices/host.cr:725-734): x [rows,k] f32, w bytes of [n,k] -> [rows,n]."""
    x = _f32(x)
    rows, k = x.shape
    w = np.ascontiguousarray(w, dtype=np.uint8)
    assert w.size == n * (k // 32) * BLOCK_BYTES[kind]
    out = np.empty((rows, n), dtype=np.float32)
    b = _p(_f32(bias), _f32p) if bias is not None else None
    lib.orc_matmul_reference(C.c_int(kind), _p(x, _f32p), _p(w, _u8p), C.c_int(rows), C.c_int(n), C.c_int(k), b,
                             _p(out, _f32p))
    return out


def matmul_fast(kind, x, w, n, bias=None, threads=1):
    """quant.cr:155-182 on `threads` threads."""
    x = _f32(x)
    rows, k = x.shape
    w = np.ascontiguousarray(w, dtype=np.uint8)
    assert w.size == n * (k // 32) * BLOCK_BYTES[kind]
    out = np.empty((rows, n), dtype=np.float32)
    b = _p(_f32(bias), _f32p) if bias is not None else None
    lib.orc_matmul_fast(C.c_int(kind), _p(x, _f32p), _p(w, _u8p), C.c_int(rows), C.c_int(n), C.c_int(k), b,
                        _p(out, _f32p), C.c_int(threads))
    return out


def gather_blocks(kind, table, table_rows, width, ids):
    table = np.ascontiguousarray(table, dtype=np.uint8)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.zeros((ids.size, width), dtype=np.float32)
    bad = lib.orc_gather_blocks(C.c_int(kind), _p(table, _u8p), C.c_int64(table_rows), C.c_int(width), _p(ids, _i32p),
                                C.c_int64(ids.size), _p(out, _f32p))
    if bad >= 0:
        raise IndexError(f"index {ids[bad]} out of range for {table_rows} rows")
    return out


def rmsnorm(x, w, eps=1e-5):
    x = _f32(x)
    rows, n = x.shape
    out = np.empty_like(x)
    lib.orc_rmsnorm(_p(x, _f32p), _p(_f32(w), _f32p) if w is not None else None, C.c_int(rows), C.c_int(n),
                    C.c_float(eps), _p(out, _f32p))
    return out


def layernorm(x, w, b, eps=1e-5):
    x = _f32(x)
    rows, n = x.shape
    out = np.empty_like(x)
    lib.orc_layernorm(_p(x, _f32p), _p(_f32(w), _f32p), _p(_f32(b), _f32p), C.c_int(rows), C.c_int(n), C.c_float(eps),
                      _p(out, _f32p))
    return out


def rope_tables(width, context, theta):
    cos = np.empty((context, width), dtype=np.float32)
    sin = np.empty((context, width), dtype=np.float32)
    lib.orc_rope_tables(C.c_int(width), C.c_int(context), C.c_double(theta), _p(cos, _f32p), _p(sin, _f32p))
    return cos, sin


def rope(x, cos, sin):
    """x [rows, n] each rotated by its own cos/sin row (host.cr:448-466)."""
    x, cos, sin = _f32(x), _f32(cos), _f32(sin)
    out = np.empty_like(x)
    for r in range(x.shape[0]):
        lib.orc_rope_row(_p(x[r], _f32p), _p(cos[r], _f32p), _p(sin[r], _f32p), C.c_int(x.shape[1]), _p(out[r], _f32p))
    return out


def swiglu(gate, up):
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib.orc_swiglu(_p(gate, _f32p), _p(up, _f32p), C.c_int64(gate.size), _p(out, _f32p))
    return out


def silu(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib.orc_silu(_p(x, _f32p), C.c_int64(x.size), _p(out, _f32p))
    return out


def gelu(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib.orc_gelu(_p(x, _f32p), C.c_int64(x.size), _p(out, _f32p))
    return out


def attend(q, k, v, scale):
    """One query [width] over k, v [len, width] in the composite's order of arithmetic."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    length, width = k.shape
    scores = np.empty(length, dtype=np.float32)
    out = np.empty(width, dtype=np.float32)
    lib.orc_attend(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), C.c_int(length), C.c_int(width), C.c_int64(width),
                   C.c_float(scale), _p(scores, _f32p), _p(out, _f32p))
    return out


def argmax_first(logits):
    logits = _f32(logits)
    return int(lib.orc_argmax_first(_p(logits, _f32p), C.c_int(logits.size)))


def topk(logits, count):
    logits = _f32(logits)
    out = np.empty(count, dtype=np.int32)
    lib.orc_topk(_p(logits, _f32p), C.c_int(logits.size), C.c_int(count), _p(out, _i32p))
    return out


# ---- whole models ---------------------------------------------------------------------------


class _Linear(C.Structure):
    _fields_ = [("kind", C.c_int), ("n", C.c_int), ("k", C.c_int), ("w", C.c_void_p), ("bias", C.c_void_p)]


class _Layer(C.Structure):
    _fields_ = [("norm1_w", C.c_void_p), ("norm1_b", C.c_void_p), ("norm2_w", C.c_void_p), ("norm2_b", C.c_void_p),
                ("qkv", _Linear), ("o", _Linear), ("up", _Linear), ("down", _Linear)]


class _Model(C.Structure):
    _fields_ = [("arch", C.c_int), ("layers", C.c_int), ("width", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int),
                ("head_width", C.c_int), ("hidden", C.c_int), ("vocab", C.c_int), ("context", C.c_int),
                ("eps", C.c_float), ("rope_theta", C.c_double), ("embed", _Linear), ("wpe", _Linear), ("head", _Linear),
                ("final_w", C.c_void_p), ("final_b", C.c_void_p), ("blocks", C.POINTER(_Layer)),
                ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("threads", C.c_int),
                ("reference_products", C.c_int)]


class _Cache(C.Structure):
    _fields_ = [("rows", C.c_int), ("capacity", C.c_int), ("keys", C.POINTER(C.c_void_p)),
                ("values", C.POINTER(C.c_void_p)), ("lengths", C.POINTER(C.c_int))]


def _linear(weight, n, k, kind, bias=None):
    """weight: uint8 block bytes (kind >= 0) or float32 [n,k] (kind -1)."""
    return _Linear(kind, n, k, weight.ctypes.data, bias.ctypes.data if bias is not None else None)


class Model:
    """A Llama (arch 0) or GPT-2 (arch 1) over numpy-held weights, run by `orc_forward`.

    `tensors` maps names to (kind, array): kind -1 with a float32 array, or a
    block kind with the uint8 block bytes.  Names (already un-permuted and
    row-joined as models/llama.cr:206-235 leaves them):
      embed [vocab,width], head (optional, else tied), final_w (, final_b),
      wpe (GPT-2), and per layer i: i.norm1_w (,i.norm1_b), i.qkv (,i.qkv_b),
      i.o (,i.o_b), i.norm2_w (,i.norm2_b), i.up (,i.up_b), i.down (,i.down_b).
    """

    def __init__(self, config, tensors, threads=1, reference_products=False):
        self.config = dict(config)
        self.keep = tensors
        c = self.config
        arch = 0 if c["arch"] == "llama" else 1
        L, d, H, KV, hw, F, V = (c["layers"], c["width"], c["heads"], c["kv_heads"], c["head_width"], c["hidden"],
                                 c["vocab"])

        def lin(name, n, k):
            kind, w = tensors[name]
            b = tensors.get(name + "_b")
            return _linear(w, n, k, kind, b[1] if b is not None else None)

        def vec(name):
            t = tensors.get(name)
            return t[1].ctypes.data if t is not None else None

        self.layers = (_Layer * L)()
        qkvn = (H + 2 * KV) * hw
        for i in range(L):
            self.layers[i] = _Layer(vec(f"{i}.norm1_w"), vec(f"{i}.norm1_b"), vec(f"{i}.norm2_w"), vec(f"{i}.norm2_b"),
                                    lin(f"{i}.qkv", qkvn, d), lin(f"{i}.o", d, H * hw),
                                    lin(f"{i}.up", 2 * F if arch == 0 else F, d), lin(f"{i}.down", d, F))
        if arch == 0:
            self.cos, self.sin = rope_tables(hw, c["context"], c.get("rope_theta", 10000.0))
        else:
            self.cos = self.sin = np.zeros(1, dtype=np.float32)
        embed = lin("embed", V, d)
        head = lin("head", V, d) if "head" in tensors else embed
        wpe = lin("wpe", c["context"], d) if arch == 1 else _Linear(-1, 0, 0, None, None)
        self.m = _Model(arch, L, d, H, KV, hw, F, V, c["context"], c.get("eps", 1e-5), c.get("rope_theta", 10000.0),
                        embed, wpe, head, vec("final_w"), vec("final_b"), self.layers, self.cos.ctypes.data,
                        self.sin.ctypes.data, threads, 1 if reference_products else 0)

    def new_cache(self, rows, capacity):
        return Cache(self, rows, capacity)

    def forward(self, cache, appends, last=True):
        """models/generative.cr:112-125: appends[row] = list of new token ids (may be empty).

        Returns the logits of each row's last new token (last=True) or of every
        new token, in row order, and advances the cache."""
        ids, rows, positions, want = [], [], [], []
        for row, new in enumerate(appends):
            past = cache.lengths[row]
            if past + len(new) > min(cache.capacity, self.config["context"]):
                raise ValueError(f"{past + len(new)} positions exceed the {cache.capacity} a row holds")
            for j, token in enumerate(new):
                ids.append(token), rows.append(row), positions.append(past + j)
                want.append(1 if (not last or j == len(new) - 1) else 0)
        if not ids:
            raise ValueError("forward of no tokens")
        total = len(ids)
        ids_a, rows_a, pos_a = (np.array(v, dtype=np.int32) for v in (ids, rows, positions))
        want_a = np.array(want, dtype=np.uint8)
        logits = np.empty((int(want_a.sum()), self.config["vocab"]), dtype=np.float32)
        rc = lib.orc_forward(C.byref(self.m), C.byref(cache.c), _p(ids_a, _i32p), _p(rows_a, _i32p), _p(pos_a, _i32p),
                             C.c_int(total), _p(want_a, _u8p), _p(logits, _f32p))
        if rc != 0:
            raise IndexError("token id out of range")
        for row, new in enumerate(appends):
            cache.lengths[row] += len(new)
        return logits

    def generate(self, prompt, count):
        """models/generative.cr:177-190 with the greedy sampler (sampler.cr:36)."""
        cache = self.new_cache(1, min(self.config["context"], len(prompt) + count))
        logits = self.forward(cache, [list(prompt)])
        tokens = []
        for i in range(count):
            token = argmax_first(logits[0])
            tokens.append(token)
            if i < count - 1:
                logits = self.forward(cache, [[token]])
        return tokens


def model_from_device(model, threads=1):
    """An oracle Model over the very weights a device model holds, downloaded through the C ABI (`model` is the
    binding's Model: only its `config` and `tensor(name)` are used)."""
    c = dict(model.config)
    names = ["embed", "final_w"] + (["wpe", "final_b"] if c["arch"] == "gpt2" else [])
    if not c["tied"]:
        names.append("head")
    for i in range(c["layers"]):
        names += [f"{i}.{p}" for p in ("norm1_w", "norm2_w", "qkv", "o", "up", "down")]
        if c["arch"] == "gpt2":
            names += [f"{i}.{p}" for p in ("norm1_b", "norm2_b", "qkv_b", "o_b", "up_b", "down_b")]
    t = {}
    for name in names:
        buf, kind, n, k = model.tensor(name)
        if kind < 0:
            t[name] = (-1, buf.numpy(np.float32).reshape(-1) if n == 1 else buf.numpy(np.float32).reshape(n, k))
        else:
            t[name] = (kind, buf.numpy(np.uint8).reshape(n, -1))
    return Model(c, t, threads=threads)


def cache_from_device(ref, device_model, device_cache, rows, lengths, capacity):
    """An oracle Cache of `capacity` positions holding what rows `rows` of a device batch cache hold: lengths[i] positions
    of row rows[i], keys and values of every layer, read back through the C ABI."""
    c = device_model.config
    out = ref.new_cache(len(rows), capacity)
    row_floats = c["kv_heads"] * device_cache.capacity * c["head_width"]
    piece = type(device_cache.layer(0)[0])
    for layer in range(c["layers"]):
        kb, vb = device_cache.layer(layer)
        for i, (row, n) in enumerate(zip(rows, lengths)):
            n = int(n)
            for src, dst in ((kb, out.keys[layer]), (vb, out.values[layer])):
                part = piece(device_model.device, src.ptr + int(row) * row_floats * 4, row_floats * 4).numpy(np.float32)
                dst[i, :, :n, :] = part.reshape(c["kv_heads"], device_cache.capacity, c["head_width"])[:, :n, :]
    for i, n in enumerate(lengths):
        out.lengths[i] = int(n)
    return out


class Cache:
    def __init__(self, model, rows, capacity):
        c = model.config
        self.rows, self.capacity = rows, capacity
        shape = (rows, c["kv_heads"], capacity, c["head_width"])
        self.keys = [np.zeros(shape, dtype=np.float32) for _ in range(c["layers"])]
        self.values = [np.zeros(shape, dtype=np.float32) for _ in range(c["layers"])]
        self.lengths = [0] * rows
        self.kp = (C.c_void_p * c["layers"])(*[a.ctypes.data for a in self.keys])
        self.vp = (C.c_void_p * c["layers"])(*[a.ctypes.data for a in self.values])
        self.c = _Cache(rows, capacity, self.kp, self.vp, None)

    def reset(self, row):
        self.lengths[row] = 0


# ---- the reference's own kernels, compiled for the host -------------------------------------


class _View(C.Structure):
    """prelude.cu:8-14: ndim, offset, shape[8], strides[8], dense."""
    _fields_ = [("ndim", C.c_int), ("offset", C.c_int), ("shape", C.c_int * 8), ("strides", C.c_int * 8),
                ("dense", C.c_int)]


def _dense_view(shape):
    v = _View()
    v.ndim = len(shape)
    stride = 1
    for i in reversed(range(len(shape))):
        v.shape[i] = shape[i]
        v.strides[i] = stride
        stride *= shape[i]
    v.dense = 1
    return v


class Ref:
    """Runs kernels of the reference's src/tensomite/cuda/kernels.cu on the host."""

    def __init__(self):
        path = os.path.join(HERE, "_ref", "libkernels.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        self.lib.tensomite_kernel.restype = C.c_void_p
        self.lib.tensomite_kernel.argtypes = [C.c_char_p]

    @staticmethod
    def available():
        return os.path.exists(os.path.join(HERE, "_ref", "libkernels.so"))

    def launch(self, name, grid, block, args):
        handle = self.lib.tensomite_kernel(name.encode())
        assert handle, name
        boxes = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
        self.lib.tensomite_launch(C.c_void_p(handle), C.c_uint(grid), C.c_uint(1), C.c_uint(1), C.c_uint(block),
                                  C.c_uint(1), boxes)

    def quantize_rows(self, x):
        """kernels.cu:1190-1207, launched as cuda.cr:745-747 does."""
        x = _f32(x)
        rows, k = x.shape
        blocks = rows * k // 32
        scales = np.zeros(blocks, dtype=np.float32)
        sums = np.zeros(blocks, dtype=np.float32)
        qs = np.zeros(rows * k, dtype=np.int8)
        args = [C.c_void_p(x.ctypes.data), C.c_void_p(scales.ctypes.data), C.c_void_p(sums.ctypes.data),
                C.c_void_p(qs.ctypes.data), _dense_view([rows, k]), C.c_uint(blocks)]
        self.launch("quantize_rows_q8_f32", (blocks + 255) // 256, 256, args)
        return scales.reshape(rows, -1), sums.reshape(rows, -1), qs.reshape(rows, k)

    def block_matmul(self, kind, x, w, n, bias=None):
        """kernels.cu:1233-1246 after quantize_rows, as cuda.cr:736-769 launches them."""
        x = _f32(x)
        rows, k = x.shape
        scales, sums, qs = self.quantize_rows(x)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        out = np.zeros(rows * n, dtype=np.float32)
        b = _f32(bias) if bias is not None else None
        args = [C.c_void_p(w.ctypes.data), C.c_void_p(scales.ctypes.data), C.c_void_p(sums.ctypes.data),
                C.c_void_p(qs.ctypes.data), C.c_void_p(out.ctypes.data), C.c_void_p(b.ctypes.data if b is not None else None),
                C.c_uint(kind), C.c_uint(BLOCK_BYTES[kind]), C.c_uint(0), C.c_uint(n), C.c_uint(k), C.c_uint(rows * n)]
        self.launch("block_matmul_f32", (rows * n + 255) // 256, 256, args)
        return out.reshape(rows, n)

    def gather_blocks(self, kind, table, table_rows, width, ids):
        """kernels.cu:1172-1185."""
        table = np.ascontiguousarray(table, dtype=np.uint8)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        n = ids.size * width
        out = np.zeros(n, dtype=np.float32)
        errors = np.zeros(3, dtype=np.int32)
        args = [C.c_void_p(table.ctypes.data), C.c_void_p(ids.ctypes.data), C.c_void_p(out.ctypes.data),
                C.c_void_p(errors.ctypes.data), C.c_uint(kind), C.c_uint(BLOCK_BYTES[kind]), C.c_uint(0),
                _dense_view([ids.size]), C.c_uint(width), C.c_int(table_rows), C.c_uint(n)]
        self.launch("gather_blocks_f32", (n + 255) // 256, 256, args)
        return out.reshape(ids.size, width), errors
