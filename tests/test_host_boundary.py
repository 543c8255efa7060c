"""CPU: the host boundary -- C ABI rules of castforge.h, pipeline grammar and option validation,
SafeTensors layout.  Nothing here launches a kernel."""
import json
import struct

import numpy as np
import pytest

import castforge_b200 as cfb

MLIR = """module @m {
  func.func @main(%x: tensor<2x2xf32>) -> tensor<2x2xf32> {
    %w = stablehlo.constant dense<[[0.5, -0.25], [0.75, 0.5]]> : tensor<2x2xf32>
    %out = stablehlo.dot_general %x, %w, contracting_dims = [1] x [0]
      : (tensor<2x2xf32>, tensor<2x2xf32>) -> tensor<2x2xf32>
    func.return %out : tensor<2x2xf32>
  }
}
"""


def test_version_and_free_null():
    cf = cfb.CastForge()
    assert cf.version() == "1.0.0"
    cfb.load().castforge_free_string(None)   # NULL is accepted (src/ffi.rs:25-31)


def test_empty_pipeline_returns_module_and_empty_telemetry():
    text, tel = cfb.CastForge().optimize(MLIR, "")
    assert "stablehlo.dot_general" in text and tel == []


def test_unknown_pass_and_bad_specs_are_errors():
    cf = cfb.CastForge()
    with pytest.raises(cfb.CastForgeError, match="Unknown pass `dce`"):
        cf.optimize(MLIR, "dce")
    with pytest.raises(cfb.CastForgeError, match="unrecognized option `bogus`"):
        cf.optimize(MLIR, "quantize(bogus=1)")
    with pytest.raises(cfb.CastForgeError, match="Unclosed"):
        cf.optimize(MLIR, "quantize(bits=8")
    with pytest.raises(cfb.CastForgeError, match="key=value"):
        cf.optimize(MLIR, "quantize(bits)")
    with pytest.raises(cfb.CastForgeError, match="trailing characters"):
        cf.optimize(MLIR, "quantize(bits=8)x")
    with pytest.raises(cfb.CastForgeError, match="parse error"):
        cf.optimize("not mlir at all", "")


def test_null_arguments_follow_the_reference_rules():
    import ctypes
    lib = cfb.load()
    out, err = ctypes.c_void_p(1), ctypes.c_void_p(1)
    rc = lib.castforge_optimize_mlir(None, b"", ctypes.byref(out), None, ctypes.byref(err))
    assert rc == 1 and out.value is None and err.value           # out-pointers are NULLed first, message set
    lib.castforge_free_string(err)
    code, err2 = ctypes.c_void_p(), ctypes.c_void_p()
    assert lib.castforge_compile_mlir(MLIR.encode(), b"", b"fortran", ctypes.byref(code), ctypes.byref(err2)) == 1
    assert b"Unknown codegen target" in ctypes.cast(err2, ctypes.c_char_p).value
    lib.castforge_free_string(err2)
    with pytest.raises(cfb.CastForgeError, match="unsupported in this build"):
        cfb.CastForge().compile(MLIR, "cuda", "")


def test_graph_only_passes_need_no_gpu():
    text, tel = cfb.CastForge().optimize(MLIR, "quantize(dtype=bf16)")      # lower-mixed-precision (tests/loop_ir_tests.rs:495-505)
    assert text.count("stablehlo.convert") == 4 and 'castforge.compute_precision = "bf16"' in text
    assert tel[0]["pass_name"] == "quantize" and tel[0]["changed"] and tel[0]["ops_created"] == 4
    assert list(tel[0]) == ["iteration", "pass_name", "changed", "elapsed_us", "live_ops_before", "live_ops_after",
                            "ops_created", "ops_modified", "ops_removed"]
    q = MLIR.replace("dense<[[0.5, -0.25], [0.75, 0.5]]> : tensor<2x2xf32>",
                     "dense<[[85, -42], [127, 85]]> : tensor<2x2x!quant.uniform<i8:f32,0.005906:0>>")
    q = q.replace("%out = stablehlo.dot_general %x, %w,", "%w_deq = stablehlo.uniform_dequantize %w : (tensor<2x2x!quant.uniform<i8:f32,0.005906:0>>) -> tensor<2x2xf32>\n    %out = stablehlo.dot_general %x, %w_deq,")
    fused, tel = cfb.CastForge().optimize(q, "fuse-gemm(kind=dequant)")
    assert "castforge.fused_qmatmul" in fused and "stablehlo.uniform_dequantize" not in fused      # tests/ai_opt_tests.rs:758-760
    assert "scale = 0.005906" in fused and "zero_point = 0" in fused and "packed_rhs" not in fused
    assert tel[0]["ops_modified"] == 1 and tel[0]["ops_removed"] == 1


def test_store_pipeline_validation_without_gpu():
    st = cfb.TensorStore()
    st.insert("w", np.ones((4, 4), np.float32))
    with pytest.raises(cfb.CastForgeError, match="Unknown pass"):
        st.run_pipeline("cse")
    with pytest.raises(cfb.CastForgeError, match="unrecognized option"):
        st.run_pipeline("quantize(colour=red)")
    assert st.run_pipeline("") == []
    tel = st.run_pipeline("lower-mixed-precision(dtype=bf16)")     # graph-only: the store is untouched
    assert tel[0]["changed"] is False and len(st) == 1


def test_safetensors_layout_and_roundtrip(tmp_path):
    st = cfb.TensorStore()
    w = np.arange(6, dtype=np.float32).reshape(3, 2) - 2.5
    h = np.array([0x3C00, 0xC000, 0x0001], np.uint16)
    st.insert("w", w)
    st.insert("h", h, dtype="F16")
    st.insert("q", np.array([[1, -2], [3, -128]], np.int8))
    p = tmp_path / "s.safetensors"
    st.save_safetensors(p)
    raw = p.read_bytes()
    hl = struct.unpack("<Q", raw[:8])[0]
    assert hl % 8 == 0                                              # header padded with spaces to 8 bytes (tensor_store.rs:542-546)
    header = raw[8:8 + hl].decode()
    assert header.rstrip(" ").endswith("}") and header.startswith('{"w":{"dtype":"F32","shape":[3,2],"data_offsets":[0,24]}')
    meta = json.loads(header)
    assert meta["h"] == {"dtype": "F16", "shape": [3], "data_offsets": [24, 30]}
    assert raw[8 + hl:8 + hl + 24] == w.tobytes()
    st2 = cfb.TensorStore()
    st2.load_safetensors(p)
    e = st2.entries()
    assert np.array_equal(e["w"]["data"], w.ravel()) and e["w"]["shape"] == [3, 2]
    assert np.array_equal(e["h"]["data"], h) and np.array_equal(e["q"]["data"], [1, -2, 3, -128])
    # scale / zero_point header extension of quantized entries (tensor_store.rs:300-309, :478-497)
    ext = json.dumps({"q": {"dtype": "I8", "shape": [2], "data_offsets": [0, 2], "scale": 0.005905512, "zero_point": 0}}).encode()
    ext += b" " * (-len(ext) % 8)
    st3 = cfb.TensorStore()
    st3.load_safetensors_bytes(struct.pack("<Q", len(ext)) + ext + bytes([85, 214]))
    q = st3.entries()["q"]
    assert q["quantized"] and q["scale"] == np.float32(0.005905512) and q["data"].tolist() == [85, -42]
    p3 = tmp_path / "q.safetensors"
    st3.save_safetensors(p3)
    assert b'"scale":0.005905512,"zero_point":0' in p3.read_bytes()


def test_safetensors_hardening():
    st = cfb.TensorStore()
    def blob(meta, body=b""):
        h = json.dumps(meta).encode()
        return struct.pack("<Q", len(h)) + h + body
    for bad, msg in [(b"\x01\x02", "shorter than 8-byte"),
                     (struct.pack("<Q", 1 << 40) + b"{}", "exceeds 100 MiB"),
                     (struct.pack("<Q", 64) + b"{}", "truncated inside JSON header"),
                     (blob({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 16]}}, b"\0" * 8), "Invalid data_offsets"),
                     (blob({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}, "b": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, b"\0" * 8), "Overlapping"),
                     (blob({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8), "does not match shape"),
                     (blob({"a": {"dtype": "F32", "shape": [2], "data_offsets": [-8, 0]}}, b"\0" * 8), "non-negative integer"),
                     (blob({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0.5, 8]}}, b"\0" * 8), "non-negative integer"),
                     (blob({"a": {"dtype": "F32", "shape": [2], "data_offsets": ["0", 8]}}, b"\0" * 8), "non-negative integer")]:
        with pytest.raises(cfb.CastForgeError, match=msg):
            st.load_safetensors_bytes(bad)


def test_safetensors_unknown_dtype_is_kept_as_raw_bytes(tmp_path):
    """A dtype the store has no arithmetic for (I64 position ids, BOOL masks, F64 ...) loads as an opaque U8 entry holding
    the raw bytes of its slice, like the reference's reader (src/ir/tensor_store.rs:742-750), and the quantize passes
    leave it alone; the float tensor beside it is still quantized."""
    ids = np.arange(5, dtype=np.int64)
    w = (np.arange(8, dtype=np.float32) - 4) * np.float32(0.25)
    meta = {"position_ids": {"dtype": "I64", "shape": [5], "data_offsets": [0, 40]},
            "w": {"dtype": "F32", "shape": [2, 4], "data_offsets": [40, 72]}}
    h = json.dumps(meta).encode()
    st = cfb.TensorStore()
    st.load_safetensors_bytes(struct.pack("<Q", len(h)) + h + ids.tobytes() + w.tobytes())
    e = st.entries()
    assert e["position_ids"]["dtype"] == 4 and e["position_ids"]["shape"] == [5]
    assert e["position_ids"]["data"].tobytes() == ids.tobytes()
    assert np.array_equal(e["w"]["data"], w)


def test_safetensors_lazy_file(tmp_path):
    """load_safetensors_lazy_file (src/ir/tensor_store.rs:779-890): only the header is read, every tensor becomes a
    slice of the file that is fetched when its bytes are asked for; the same validation as the eager loader."""
    st = cfb.TensorStore()
    w = (np.arange(3000, dtype=np.float32).reshape(30, 100) - 1500) * np.float32(0.01)
    h = np.arange(64, dtype=np.uint16) + 0x3C00
    st.insert("w", w)
    st.insert("h", h, dtype="F16")
    p = tmp_path / "s.safetensors"
    st.save_safetensors(p)
    lazy = cfb.TensorStore()
    assert lazy.load_safetensors_lazy(p) == 2 and len(lazy) == 2
    e = lazy.entries()                                              # asking for the bytes reads the slices
    assert np.array_equal(e["w"]["data"], w.ravel()) and e["w"]["shape"] == [30, 100] and e["w"]["dtype"] == 0
    assert np.array_equal(e["h"]["data"], h)
    # saving a store whose entries are still on disk copies the slices through
    lazy2 = cfb.TensorStore()
    lazy2.load_safetensors_lazy(p)
    p2 = tmp_path / "copy.safetensors"
    lazy2.save_safetensors(p2)
    assert p2.read_bytes() == p.read_bytes()
    # hardening: short file, oversized / truncated header, out-of-bounds and overlapping slices
    def write(name, raw):
        q = tmp_path / name
        q.write_bytes(raw)
        return q
    def blob(meta, body=b""):
        hh = json.dumps(meta).encode()
        return struct.pack("<Q", len(hh)) + hh + body
    for raw, msg in [(b"\x01\x02", "shorter than 8-byte header"),
                     (struct.pack("<Q", 1 << 40) + b"{}", "Invalid or truncated Safetensors header length"),
                     (struct.pack("<Q", 64) + b"{}", "Invalid or truncated Safetensors header length"),
                     (blob({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 16]}}, b"\0" * 8), "Invalid data_offsets"),
                     (blob({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}, "b": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, b"\0" * 8), "Overlapping")]:
        with pytest.raises(cfb.CastForgeError, match=msg):
            cfb.TensorStore().load_safetensors_lazy(write("bad.safetensors", raw))
    with pytest.raises(cfb.CastForgeError, match="cannot open"):
        cfb.TensorStore().load_safetensors_lazy(tmp_path / "missing.safetensors")
    # a slice that disappears before it is read is reported, not ignored
    gone = cfb.TensorStore()
    gone.load_safetensors_lazy(p2)
    p2.unlink()
    with pytest.raises(cfb.CastForgeError, match="cannot open"):
        gone.entries()


def test_scale_string():
    assert cfb.format_scale(0.75 / 127) == "0.005906"
    assert cfb.format_scale(1.0) == "1.0" and cfb.format_scale(7.9e-8) == "0.0" and cfb.format_scale(2.5) == "2.5"
