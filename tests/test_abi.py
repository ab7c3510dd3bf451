"""The C ABI library on a machine without a GPU: it builds, loads, exports what the header declares,
and refuses to compute (there is no CPU path behind it).  Also the host-side GGUF code."""
import ctypes as C

import numpy as np
import pytest

import helpers
from helpers import pkg, oracle


def test_library_exports_every_declared_symbol():
    names = pkg.declared_symbols()
    assert len(names) >= 40 and "tsm_block_matmul" in names and "tsm_decode" in names
    assert pkg.check_exports()
    lib = pkg.library()
    assert lib.tsm_status_name(0) == b"TSM_OK" and lib.tsm_status_name(3) == b"TSM_ERR_EXECUTION"


def test_no_device_means_no_compute():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    lib = pkg.library()
    count = C.c_int(-1)
    rc = lib.tsm_device_count(C.byref(count))
    assert count.value == 0 and rc != 0
    with pytest.raises(pkg.DeviceError):
        pkg.B200(0)


def test_gguf_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, (8, 64)).astype(np.float32)
    blocks = oracle.quantize(oracle.Q4_1, w)
    path = str(tmp_path / "t.gguf")
    pkg.gguf.write(path, {"general.architecture": "llama", "llama.block_count": 3, "llama.rope.freq_base": 500000.0,
                          "name": "x"},
                   [("a.weight", pkg.gguf.Q4_1, [8, 64], blocks), ("b", pkg.gguf.F32, [5], np.arange(5, dtype=np.float32))])
    f = pkg.gguf.File(path)
    assert f.metadata["llama.block_count"] == 3 and f.metadata["name"] == "x" and f.metadata["llama.rope.freq_base"] == 500000.0
    kind, shape, raw = f.raw("a.weight")
    assert kind == pkg.gguf.Q4_1 and shape == [8, 64] and raw.tobytes() == blocks.tobytes()
    assert f.f32("b").tolist() == [0, 1, 2, 3, 4]
    assert all(off % 32 == 0 for _, _, off in f.entries.values())
    # the reference's own fixture parses too
    g = helpers.golden()
    fixture = tmp_path / "blocks.gguf"
    fixture.write_bytes(g["quant/blocks_gguf"].tobytes())
    assert sorted(pkg.gguf.File(str(fixture)).entries) == ["q4_0", "q4_1", "q8_0"]


def _gguf_bytes(tensors, metadata=None):
    """A little GGUF v3 image: tensors = [(name, dims innermost first, kind, offset)], no payload beyond `tail` zeros."""
    import struct

    def text(s):
        return struct.pack("<Q", len(s)) + s.encode()

    metadata = metadata or {"general.architecture": "llama"}
    out = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(metadata))
    for key, value in metadata.items():
        out += text(key) + struct.pack("<I", 8) + text(value)
    for name, dims, kind, offset in tensors:
        out += text(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d & (2 ** 64 - 1)) for d in dims)
        out += struct.pack("<I", kind) + struct.pack("<Q", offset & (2 ** 64 - 1))
    out += b"\0" * (-len(out) % 32)
    return out


def test_malformed_gguf_files_are_refused_not_read(tmp_path):
    """gguf.cr:297-325 raises on files it cannot trust; here the same cases come back as TSM_ERR_IO with a reason, and no byte
    outside the mapping is touched: a truncated file, an offset that is negative as a signed number, an offset past the end,
    an empty axis, a count that overflows, a token table with one axis."""
    lib = pkg.library()

    def check(image):
        path = tmp_path / "case.gguf"
        path.write_bytes(image)
        reason = C.create_string_buffer(512)
        return lib.tsm_gguf_check(str(path).encode(), reason, 512), reason.value.decode()

    good = _gguf_bytes([("token_embd.weight", [64, 4], 0, 0)]) + b"\0" * (64 * 4 * 4)
    assert check(good) == (0, "")
    rc, why = check(good[:-8])
    assert rc == 5 and "do not fit" in why                                   # truncated payload
    assert check(good[:40])[0] == 5                                          # truncated header
    assert check(_gguf_bytes([("token_embd.weight", [64, 4], 0, -32)]) + b"\0" * 1024)[0] == 5       # "negative" offset
    assert check(_gguf_bytes([("token_embd.weight", [64, 4], 0, 1 << 40)]) + b"\0" * 1024)[0] == 5   # far past the end
    assert check(_gguf_bytes([("token_embd.weight", [0, 4], 0, 0)]) + b"\0" * 1024)[0] == 5          # an empty axis
    assert check(_gguf_bytes([("token_embd.weight", [1 << 39, 1 << 39], 0, 0)]) + b"\0" * 1024)[0] == 5  # overflowing count
    rc, why = check(_gguf_bytes([("token_embd.weight", [64], 0, 0)]) + b"\0" * 1024)
    assert rc == 5 and "not a matrix" in why                                 # a 1-D token table
    rc, why = check(_gguf_bytes([("wte.weight", [64], 0, 0), ("wpe.weight", [64, 4], 0, 256)], {"gpt2.heads": "2"}) + b"\0" * 2048)
    assert rc == 5 and "wte.weight" in why
    assert check(b"GGUF" + b"\0" * 8)[0] == 5                                # shorter than a header
    assert lib.tsm_gguf_check(str(tmp_path / "absent.gguf").encode(), None, 0) == 5


def test_unpermute_order_inverts_llama_cpps_rotary_layout():
    # models/llama.cr:226-235: loaded row head*hw + pair*(hw/2) + i = stored row head*hw + 2i + pair
    order = helpers.unpermute_order(16, 2)
    assert order[:8] == [0, 2, 4, 6, 1, 3, 5, 7] and order[8:] == [8, 10, 12, 14, 9, 11, 13, 15]


def test_the_crystal_stub_binds_every_entry_point():
    """INTEGRATION.md's `lib LibTSM` is what a maintainer copies: every function the header declares has its `fun` line,
    with as many arguments as the C declaration."""
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "tsm_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    stub = open(os.path.join(root, "INTEGRATION.md")).read()
    declared = {name: args for name, args in re.findall(r"\b(tsm_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", header)}
    assert set(declared) == set(pkg.declared_symbols())
    for name, args in declared.items():
        found = re.search(r"fun \w+ = " + name + r"\(([^)]*)\)", stub)
        assert found, f"{name} has no fun line in the integration notes"
        want = 0 if args.strip() in ("", "void") else args.count(",") + 1
        got = 0 if not found.group(1).strip() else found.group(1).count(",") + 1
        assert want == got, (name, want, got)
