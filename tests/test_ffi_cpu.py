"""Host-side checks that need no GPU: the library loads and exports every symbol the public header declares."""
import ctypes
import re

from conftest import ROOT, pkg


def header_symbols():
    text = (ROOT / "include" / "q4b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q4b_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    ffi = pkg("_ffi")
    pkg("build").build()
    lib = ffi.lib()
    names = header_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/q4b200.h but not exported"
    assert set(names) == set(ffi.SIGNATURES), "ctypes signatures out of step with the header"
    assert lib.q4b_version() >= 1000


def test_struct_layout_matches_header(tmp_path):
    """sizeof of the descriptor structs as gcc sees the header equals the ctypes mirror."""
    import subprocess
    ffi = pkg("_ffi")
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "q4b200.h"\nint main(){printf("%zu %zu %zu\\n",'
                   "sizeof(q4b_decode_desc),sizeof(q4b_layer),sizeof(q4b_linear));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), "-o", str(exe), str(src)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert got == [ctypes.sizeof(ffi.DecodeDesc), ctypes.sizeof(ffi.Layer), ctypes.sizeof(ffi.Linear)]


def test_host_side_validation_needs_no_gpu():
    """Bad shapes and null pointers are rejected before any CUDA call."""
    ffi = pkg("_ffi")
    lib = ffi.lib()
    assert lib.q4b_gemv_q4_0(16, 16, 16, 16, None, 4, 33, 0, 0, None) == ffi.E_SHAPE
    assert lib.q4b_gemv_q4_0(None, 16, 16, 16, None, 4, 32, 0, 0, None) == ffi.E_ALIGN
    assert lib.q4b_gemv_q4_0(16, 16, 16, 16, None, 4, 32, 9, 0, None) == ffi.E_ARG
    assert lib.q4b_gemv_q4_0(16, 16, 16, 16, None, 3, 32, ffi.EPI["swiglu"], 0, None) == ffi.E_SHAPE
    assert lib.q4b_attn_decode(16, 16, 16, 16, 16, 16, 16, 1, 12, 5, 128, 64, 1.0, 16, 1 << 20, None) == ffi.E_SHAPE
    assert lib.q4b_attn_decode(16, 16, 16, 16, 16, 16, 16, 1, 12, 2, 128, 64, 1.0, 16, 8, None) == ffi.E_WORKSPACE
    assert b"workspace" in lib.q4b_last_error()
    assert lib.q4b_attn_decode_workspace(1, 12, 128, 1024) > 0


def test_synth_model_shapes():
    s = pkg("synth")
    m = s.synth_model(s.TINY, seed=1)
    c = s.TINY
    assert m["embed"].shape == (c.vocab, c.hidden) and m["embed"].dtype.name == "float16"
    L = m["layers"][0]
    assert L["qkv"][0].shape == (c.qkv_rows, c.hidden // 8) and L["qkv"][1].shape == (c.qkv_rows, c.hidden // 32)
    assert L["gu"][0].shape == (2 * c.ffn, c.hidden // 8) and L["down"][0].shape == (c.hidden, c.ffn // 8)
    m2 = s.synth_model(s.TINY, seed=1)
    assert (m2["layers"][1]["o"][0] == m["layers"][1]["o"][0]).all()
    assert s.QWEN25_1P5B.q4_bytes_per_layer() * 28 == 736985088
    assert s.QWEN25_1P5B.head_bytes() == 466747392 and s.QWEN25_1P5B.kv_bytes_per_position() == 28672
    assert s.QWEN25_7B.q4_bytes_per_layer() == 131088384 and s.QWEN25_7B.kv_bytes_per_position() == 57344
