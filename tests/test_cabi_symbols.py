"""CPU: the C-ABI library loads and exports every symbol the headers declare (no compute)."""
import ctypes
import re
from pathlib import Path

import castforge_b200
from castforge_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    decl = castforge_b200.declared_functions()
    assert len(decl) >= 18
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    missing = [n for n in decl if not hasattr(lib, n)]
    assert not missing, missing


def test_header_parser_sees_every_prototype():
    # every `cfb200_` / `castforge_` identifier followed by '(' in the headers is bound
    names = set()
    for h in _lib.HEADERS:
        if h.exists():
            text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
            names |= set(re.findall(r"\b((?:cfb200|castforge)_\w+)\s*\(", text))
    assert names == set(castforge_b200.declared_functions())


def test_version_and_error_string_without_gpu():
    lib = castforge_b200.load()
    assert lib.cfb200_version().decode().count(".") == 2
    # argument validation happens before any CUDA call: NULL scale pointer -> INVALID (1)
    rc = lib.cfb200_quant_sym_tensor(None, 0, 0, 8, None, None, None)
    assert rc == 1 and b"scale_absmax" in lib.cfb200_last_error()
    rc = lib.cfb200_quant_int4_asym(ctypes.c_void_p(16), 0, 128, 100, ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), None)
    assert rc == 1 and b"group" in lib.cfb200_last_error()
    rc = lib.cfb200_quant_sym_tensor(ctypes.c_void_p(4), 0, 16, 8, ctypes.c_void_p(16), ctypes.c_void_p(16), None)
    assert rc == 2  # misaligned source
    # the bf16 product with row pitches: a pitch shorter than the row, an unknown triangle selector, C += into a bf16 result
    p = ctypes.c_void_p(256)
    assert lib.cfb200_gemm_bf16_nt_ex(p, 64, p, 64, 128, 128, 64, 1.0, p, 64, 1, 0, 0, None, None) == 1 and b"pitch" in lib.cfb200_last_error()
    assert lib.cfb200_gemm_bf16_nt_ex(p, 64, p, 64, 128, 128, 64, 1.0, p, 128, 1, 3, 0, None, None) == 1 and b"triangle" in lib.cfb200_last_error()
    assert lib.cfb200_gemm_bf16_nt_ex(p, 64, p, 64, 128, 128, 64, 1.0, p, 128, 0, 0, 1, None, None) == 1 and b"f32" in lib.cfb200_last_error()
    # knobs: known keys are accepted, unknown ones are not
    assert lib.cfb200_tune(b"gemm_pair", 1) == 0 and lib.cfb200_tune(b"colpar_p2p", 1) == 0 and lib.cfb200_tune(b"no_such_knob", 1) != 0


def test_product_does_not_reference_the_oracle():
    for p in (ROOT / "castforge_b200").rglob("*"):
        if p.suffix in {".py", ".cu", ".cuh", ".cpp", ".h"}:
            text = p.read_text()
            assert "cf_oracle" not in text and "oracle_lib" not in text, p
