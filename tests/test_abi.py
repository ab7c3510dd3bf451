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
        assert found, f"{name} has no fun line in INTEGRATION.md"
        want = 0 if args.strip() in ("", "void") else args.count(",") + 1
        got = 0 if not found.group(1).strip() else found.group(1).count(",") + 1
        assert want == got, (name, want, got)
