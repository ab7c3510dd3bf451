"""Builds tests/golden/reference_fixtures.npz from the reference's own test fixtures.

Run once where the reference tree is mounted:  python tests/golden/make_golden.py <reference tree>
The arrays are the golden vectors the reference's specs check against
(spec/quant_spec.cr:15-27,115-134; spec/llama_spec.cr:50-87; spec/gpt2_spec.cr:54-102;
spec/block_matmul_spec.cr:244-284), repacked as numpy arrays so that the tests can run
where the reference tree is absent:

  quant/rows/<i>, quant/<KIND>/bytes/<i>, quant/<KIND>/values/<i>   7 rows, ggml's bytes and values
  quant/table, quant/<KIND>/table                                  the 3x64 table and its round trips
  quant/blocks_gguf                                                the fixture's GGUF file, raw
  tiny_llama/{f32,q8_0,q4_0}_gguf                                  model files, raw
  tiny_llama/{prompt_ids,logits,greedy}                            PyTorch F32 expectations
  tiny_gpt2/safetensors, tiny_gpt2/{prompt_ids,logits,greedy}
"""
import json
import os
import sys

import numpy as np

ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
fx = os.path.join(ref, "spec", "fixtures")
out = {}


def raw(path):
    return np.fromfile(path, dtype=np.uint8)


q = json.load(open(os.path.join(fx, "quant", "expected.json")))
for i, row in enumerate(q["rows"]):
    out[f"quant/rows/{i}"] = np.array(row, dtype=np.float32)
out["quant/table"] = np.array(q["table"], dtype=np.float32)
for kind in ("Q8_0", "Q4_0", "Q4_1"):
    for i in range(len(q["rows"])):
        out[f"quant/{kind}/bytes/{i}"] = np.frombuffer(bytes.fromhex(q[kind]["bytes"][i]), dtype=np.uint8)
        out[f"quant/{kind}/values/{i}"] = np.array(q[kind]["values"][i], dtype=np.float32)
    out[f"quant/{kind}/table"] = np.array(q[kind]["table"], dtype=np.float32)
out["quant/blocks_gguf"] = raw(os.path.join(fx, "quant", "blocks.gguf"))

tl = os.path.join(fx, "tiny_llama")
out["tiny_llama/f32_gguf"] = raw(os.path.join(tl, "model.gguf"))
out["tiny_llama/q8_0_gguf"] = raw(os.path.join(tl, "model-q8_0.gguf"))
out["tiny_llama/q4_0_gguf"] = raw(os.path.join(tl, "model-q4_0.gguf"))
e = json.load(open(os.path.join(tl, "logits.json")))
out["tiny_llama/prompt_ids"] = np.array(e["prompt_ids"], dtype=np.int32)
out["tiny_llama/logits"] = np.array(e["logits"], dtype=np.float32)
out["tiny_llama/logit_rows"] = np.array(e["logit_rows"], dtype=np.int32)
out["tiny_llama/greedy"] = np.array(e["greedy"], dtype=np.int32)

tg = os.path.join(fx, "tiny_gpt2")
out["tiny_gpt2/safetensors"] = raw(os.path.join(tg, "model.safetensors"))
e = json.load(open(os.path.join(tg, "expected.json")))
out["tiny_gpt2/prompt_ids"] = np.array(e["prompt_ids"], dtype=np.int32)
out["tiny_gpt2/logits"] = np.array(e["logits"], dtype=np.float32)
out["tiny_gpt2/logit_rows"] = np.array(e["logit_rows"], dtype=np.int32)
out["tiny_gpt2/greedy"] = np.array(e["greedy"], dtype=np.int32)

target = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.npz")
np.savez_compressed(target, **out)
print(target, os.path.getsize(target), "bytes,", len(out), "arrays")
