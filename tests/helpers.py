"""Test helpers: build oracle models from model files, make seeded synthetic models."""
import json
import os
import struct
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402

pkg = load_package()
gguf = pkg.gguf

from oracle import oracle  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden", "reference_fixtures.npz")
KIND_OF_GGUF = {gguf.Q8_0: oracle.Q8_0, gguf.Q4_0: oracle.Q4_0, gguf.Q4_1: oracle.Q4_1}
GGUF_OF_KIND = {v: k for k, v in KIND_OF_GGUF.items()}


def golden():
    return np.load(GOLDEN)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _rows(kind, raw, shape):
    """A [n,k] tensor as n rows: float32 [n,k] for kind -1, else uint8 [n,row_bytes]."""
    n = shape[0]
    if kind < 0:
        return raw.reshape(n, -1)
    return raw.reshape(n, -1)


def _entry(f, name):
    kind, shape, raw = f.raw(name)
    if kind in KIND_OF_GGUF:
        return KIND_OF_GGUF[kind], shape, raw.reshape(shape[0], -1)
    return -1, shape, f.f32(name).reshape(shape[0], -1) if len(shape) > 1 else f.f32(name)


def unpermute_order(rows, heads):
    """models/llama.cr:226-235: loaded row head*hw + pair*(hw/2) + i = stored row head*hw + 2i + pair."""
    half = rows // heads // 2
    return [head * 2 * half + 2 * i + pair for head in range(heads) for pair in range(2) for i in range(half)]


def llama_config(f):
    m = f.metadata
    width, heads = m["llama.embedding_length"], m["llama.attention.head_count"]
    return dict(arch="llama", layers=m["llama.block_count"], heads=heads,
                kv_heads=m.get("llama.attention.head_count_kv", heads), width=width,
                hidden=m["llama.feed_forward_length"], head_width=m.get("llama.rope.dimension_count", width // heads),
                context=m["llama.context_length"],
                vocab=m.get("llama.vocab_size", f.entries["token_embd.weight"][1][0]),
                rope_theta=float(m.get("llama.rope.freq_base", 10000.0)),
                eps=float(m["llama.attention.layer_norm_rms_epsilon"]), tied="output.weight" not in f.entries)


def oracle_llama(path, threads=1, reference_products=False):
    """models/llama.cr:184-213: read by GGUF names, un-permute q/k rows, join [q;k;v] and [gate;up]."""
    f = gguf.File(path)
    c = llama_config(f)
    t = {}

    def put(name, kind, rows):
        t[name] = (kind, np.ascontiguousarray(rows))

    kind, _, rows = _entry(f, "token_embd.weight")
    put("embed", kind, rows)
    if not c["tied"]:
        kind, _, rows = _entry(f, "output.weight")
        put("head", kind, rows)
    t["final_w"] = (-1, np.ascontiguousarray(f.f32("output_norm.weight")))
    for i in range(c["layers"]):
        t[f"{i}.norm1_w"] = (-1, np.ascontiguousarray(f.f32(f"blk.{i}.attn_norm.weight")))
        t[f"{i}.norm2_w"] = (-1, np.ascontiguousarray(f.f32(f"blk.{i}.ffn_norm.weight")))
        kq, _, q = _entry(f, f"blk.{i}.attn_q.weight")
        kk, _, k = _entry(f, f"blk.{i}.attn_k.weight")
        kv, _, v = _entry(f, f"blk.{i}.attn_v.weight")
        assert kq == kk == kv
        q = q[unpermute_order(q.shape[0], c["heads"])]
        k = k[unpermute_order(k.shape[0], c["kv_heads"])]
        put(f"{i}.qkv", kq, np.concatenate([q, k, v], axis=0))
        ko, _, o = _entry(f, f"blk.{i}.attn_output.weight")
        put(f"{i}.o", ko, o)
        kg, _, g = _entry(f, f"blk.{i}.ffn_gate.weight")
        ku, _, u = _entry(f, f"blk.{i}.ffn_up.weight")
        assert kg == ku
        put(f"{i}.up", kg, np.concatenate([g, u], axis=0))
        kd, _, dn = _entry(f, f"blk.{i}.ffn_down.weight")
        put(f"{i}.down", kd, dn)
    return oracle.Model(c, t, threads=threads, reference_products=reference_products)


def read_safetensors(raw):
    raw = bytes(raw)
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        assert info["dtype"] == "F32"
        a, b = info["data_offsets"]
        out[name] = np.frombuffer(raw[8 + n + a:8 + n + b], dtype=np.float32).reshape(info["shape"]).copy()
    return out


def write_safetensors(path, tensors):
    """A safetensors file of F32 tensors (name -> array), as safetensors.cr reads them."""
    header, payload, at = {}, [], 0
    for name, array in tensors.items():
        array = np.ascontiguousarray(array, dtype=np.float32)
        header[name] = {"dtype": "F32", "shape": list(array.shape), "data_offsets": [at, at + array.nbytes]}
        payload.append(array.tobytes())
        at += array.nbytes
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(payload))


def llama_tensors_from_hf(st, layers, kind):
    """Hugging Face Llama names -> oracle tensors, every Linear and the embedding table quantised to `kind`."""
    def q(w):
        w = np.ascontiguousarray(w, dtype=np.float32)
        return (kind, oracle.quantize(kind, w).reshape(w.shape[0], -1))

    t = {"embed": q(st["model.embed_tokens.weight"]), "final_w": (-1, st["model.norm.weight"])}
    if "lm_head.weight" in st:
        t["head"] = q(st["lm_head.weight"])
    for i in range(layers):
        p = f"model.layers.{i}."
        t[f"{i}.norm1_w"] = (-1, st[p + "input_layernorm.weight"])
        t[f"{i}.norm2_w"] = (-1, st[p + "post_attention_layernorm.weight"])
        t[f"{i}.qkv"] = q(np.concatenate([st[p + f"self_attn.{n}_proj.weight"] for n in "qkv"]))
        t[f"{i}.o"] = q(st[p + "self_attn.o_proj.weight"])
        t[f"{i}.up"] = q(np.concatenate([st[p + "mlp.gate_proj.weight"], st[p + "mlp.up_proj.weight"]]))
        t[f"{i}.down"] = q(st[p + "mlp.down_proj.weight"])
    return t


def gpt2_tensors_from_hf(st, layers, quantize_kind=None, embeddings=False):
    """Hugging Face GPT-2 names ([in,out] Conv1D weights) -> oracle tensors ([out,in] rows).

    With quantize_kind, Linear weights (and with `embeddings` wte/wpe) are quantised as
    Module#quantize does (src/tensomite/module.cr), through the oracle's quantiser."""
    def lin(w):
        w = np.ascontiguousarray(w.T)  # [out, in]
        if quantize_kind is None:
            return (-1, w)
        return (quantize_kind, oracle.quantize(quantize_kind, w).reshape(w.shape[0], -1))

    def table(w):
        if quantize_kind is None or not embeddings:
            return (-1, np.ascontiguousarray(w))
        return (quantize_kind, oracle.quantize(quantize_kind, w).reshape(w.shape[0], -1))

    p = "transformer."
    t = {"embed": table(st[p + "wte.weight"]), "wpe": table(st[p + "wpe.weight"]),
         "final_w": (-1, st[p + "ln_f.weight"]), "final_b": (-1, st[p + "ln_f.bias"])}
    for i in range(layers):
        h = f"{p}h.{i}."
        t[f"{i}.norm1_w"] = (-1, st[h + "ln_1.weight"])
        t[f"{i}.norm1_b"] = (-1, st[h + "ln_1.bias"])
        t[f"{i}.norm2_w"] = (-1, st[h + "ln_2.weight"])
        t[f"{i}.norm2_b"] = (-1, st[h + "ln_2.bias"])
        for ours, theirs in (("qkv", "attn.c_attn"), ("o", "attn.c_proj"), ("up", "mlp.c_fc"), ("down", "mlp.c_proj")):
            t[f"{i}.{ours}"] = lin(st[h + theirs + ".weight"])
            t[f"{i}.{ours}_b"] = (-1, st[h + theirs + ".bias"])
    return t


def oracle_from_device_model(model, threads=1):
    """An oracle model over the very weights a device model holds (downloaded through the C ABI)."""
    return oracle.model_from_device(model, threads=threads)


def write_gpt2_gguf(path, st, layers, heads, kind, embeddings=True):
    """A GPT-2 in tensomite's own GGUF names (gpt2.cr:75-89), Linear weights quantised and, with `embeddings`, both
    tables too (Module#quantize(kind, embeddings: true)); without, the tables stay F32 and so does the tied head."""
    t = gpt2_tensors_from_hf(st, layers, quantize_kind=kind, embeddings=embeddings)
    gk = GGUF_OF_KIND[kind]
    tk = gk if embeddings else gguf.F32
    d = st["transformer.wte.weight"].shape[1]
    tensors = [("wte.weight", tk, list(st["transformer.wte.weight"].shape), t["embed"][1]),
               ("wpe.weight", tk, list(st["transformer.wpe.weight"].shape), t["wpe"][1]),
               ("ln_f.weight", gguf.F32, [d], t["final_w"][1]), ("ln_f.bias", gguf.F32, [d], t["final_b"][1])]
    for i in range(layers):
        for ours, theirs in (("norm1", "ln_1"), ("norm2", "ln_2")):
            tensors.append((f"h.{i}.{theirs}.weight", gguf.F32, [d], t[f"{i}.{ours}_w"][1]))
            tensors.append((f"h.{i}.{theirs}.bias", gguf.F32, [d], t[f"{i}.{ours}_b"][1]))
        for ours, theirs in (("qkv", "attn.c_attn"), ("o", "attn.c_proj"), ("up", "mlp.c_fc"), ("down", "mlp.c_proj")):
            w = st[f"transformer.h.{i}.{theirs}.weight"]
            tensors.append((f"h.{i}.{theirs}.weight", gk, [w.shape[1], w.shape[0]], t[f"{i}.{ours}"][1]))
            tensors.append((f"h.{i}.{theirs}.bias", gguf.F32, [w.shape[1]], t[f"{i}.{ours}_b"][1]))
    gguf.write(path, {"general.architecture": "gpt2", "gpt2.heads": str(heads)}, tensors)
    return t


def rel_max(a, b):
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-30))
