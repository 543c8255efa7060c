"""GPU: the reference-facing boundary end to end -- MLIR text through castforge_optimize_mlir and
weight sets through the TensorStore pipeline, checked against the oracle and the reference tests' facts."""
import numpy as np
import pytest

import castforge_b200 as cfb

pytestmark = pytest.mark.gpu

QMATMUL = """module @qmatmul {
  func.func @forward(%x: tensor<2x2xf32>) -> tensor<2x2xf32> {
    %two = stablehlo.constant dense<2.0> : tensor<2xf32>
    %w = stablehlo.constant dense<[[0.5, -0.25], [0.75, 0.5]]> : tensor<2x2xf32>
    %out = stablehlo.dot_general %x, %w, contracting_dims = [1] x [0]
      : (tensor<2x2xf32>, tensor<2x2xf32>) -> tensor<2x2xf32>
    func.return %out : tensor<2x2xf32>
  }
}
"""


def f32(bits):
    return np.array(bits, dtype=np.uint32).view(np.float32)


def test_mlir_quantize_then_fuse(cuda_device):
    """tests/ai_opt_tests.rs:737-765 and tests/pipeline_tests.rs:127-146 on the 2x2 weight of :656."""
    cf = cfb.CastForge()
    text, tel = cf.optimize(QMATMUL, "quantize(bits=8,min_elements=4)")
    assert "%w = stablehlo.constant dense<[[85, -42], [127, 85]]> : tensor<2x2x!quant.uniform<i8:f32,0.005906:0>>" in text
    assert "%w_deq = stablehlo.uniform_dequantize %w : (tensor<2x2x!quant.uniform<i8:f32,0.005906:0>>) -> tensor<2x2xf32>" in text
    assert "stablehlo.dot_general %x, %w_deq," in text
    assert "dense<2.0> : tensor<2xf32>" in text                      # min_elements=4 leaves the 2-element constant alone
    assert tel[0]["ops_modified"] == 1 and tel[0]["ops_created"] == 1 and tel[0]["changed"]
    fused, tel = cf.optimize(QMATMUL, "quantize(bits=8,min_elements=4),fuse-gemm(kind=dequant)")
    assert "castforge.fused_qmatmul" in fused and "stablehlo.uniform_dequantize" not in fused
    assert [t["pass_name"] for t in tel] == ["quantize", "fuse-gemm"]
    # default min_elements = 2: the splat is quantized too and prints as a splat
    text, _ = cf.optimize(QMATMUL, "quantize(bits=8)")
    assert "%two = stablehlo.constant dense<127> : tensor<2x!quant.uniform<i8:f32,0.015748:0>>" in text
    # bits=4,group=128: `group` is only an alias, the scheme stays per-tensor INT4 (families.rs:103-137)
    text, _ = cf.optimize(QMATMUL, "quantize(bits=4,group=128,min_elements=4)")
    assert "!quant.uniform<i4:f32,0.107143:0>" in text and "dense<[[5, -2], [7, 5]]>" in text


def test_mlir_fake_quant_schemes(cuda_device, golden):
    cf = cfb.CastForge()
    awq = QMATMUL.replace("[[0.5, -0.25], [0.75, 0.5]]", "[[1.0, 2.0], [3.0, 4.0]]")
    text, _ = cf.optimize(awq, "quantize(scheme=awq,bits=4,group_size=2,salient_ratio=0.25)")   # tests/frontend_tests.rs:746-755
    assert 'castforge.quant_scheme = "awq_groupwise"' in text and "castforge.awq_salient_channels = 1" in text
    want = f32(golden["a2_awq_2x2"]["out_bits"])
    lit = text.split("%w = stablehlo.constant dense<")[1].split(">")[0]
    got = np.array([float(t) for t in lit.replace("[", " ").replace("]", " ").replace(",", " ").split()], np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    text, _ = cf.optimize(QMATMUL, "quantize(scheme=fp8)")
    assert 'castforge.fp8_format = "fp8_e4m3"' in text and "castforge.mxfp8 = true" in text                       # frontend_tests.rs:812-817
    text, _ = cf.optimize(QMATMUL, "quantize(scheme=nvfp4)")
    assert 'castforge.quant_scheme = "nvfp4"' in text
    text, _ = cf.optimize(QMATMUL, "quantize(scheme=hadamard,block_size=2)")
    assert "castforge.hadamard_rotated = true" in text and "castforge.hadamard_block = 2" in text
    text, _ = cf.optimize(QMATMUL, "quantize(scheme=qat_ste)")
    assert "castforge.qat_ste = true" in text


def _weights(shape, seed, scale=0.02):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale))


def test_store_quantize_bits8_matches_oracle_and_roundtrips(cuda_device, oracle, tmp_path):
    st = cfb.TensorStore()
    ws = {"q_proj": _weights((512, 512), 1), "gate": _weights((512, 1376), 2), "gamma": np.ones(512, np.float32), "tiny": np.float32([0.5])}
    for k, v in ws.items():
        st.insert(k, v)
    bf = (_weights((300, 257), 3).view(np.uint32) >> 16).astype(np.uint16)
    st.insert("bf", bf, dtype="BF16")
    tel = st.run_pipeline("quantize(bits=8)")
    assert tel[0]["ops_modified"] == 4 and tel[0]["ops_created"] == 4        # `tiny` has 1 element < min_elements
    e = st.entries()
    for k in ("q_proj", "gate", "gamma"):
        q, s, _ = oracle.quant_sym(ws[k], 8)
        assert e[k]["quantized"] and e[k]["scale"] == s and e[k]["zero_point"] == 0
        assert np.array_equal(e[k]["data"], q) and e[k]["shape"] == list(ws[k].shape)
    q, s, _ = oracle.quant_sym(oracle.to_f32(bf, 2), 8)
    assert np.array_equal(e["bf"]["data"], q) and e["bf"]["scale"] == s
    assert not e["tiny"]["quantized"]
    assert st.run_pipeline("quantize(bits=8)")[0]["changed"] is False       # already quantized: nothing left to do
    p = tmp_path / "q.safetensors"
    st.save_safetensors(p)                                                  # tests/pipeline_tests.rs:331-367
    st2 = cfb.TensorStore()
    st2.load_safetensors(p)
    e2 = st2.entries()
    assert e2["gate"]["quantized"] and e2["gate"]["scale"] == e["gate"]["scale"] and np.array_equal(e2["gate"]["data"], e["gate"]["data"])


def test_store_pipeline_streams_a_lazily_loaded_file(cuda_device, oracle, tmp_path):
    """Weights registered as file slices go file -> pinned staging -> device inside run_pipeline: same codes, scales and
    saved bytes as the eager store; entries the pass does not touch stay on disk until they are saved."""
    src = cfb.TensorStore()
    ws = {f"layers.{i}.w": _weights((700 + 13 * i, 512), 10 + i) for i in range(7)}      # more tensors than staging buffers
    ws["big"] = _weights((3000, 4096), 30)                                              # 49 MB: split over reader threads
    for k, v in ws.items():
        src.insert(k, v)
    bf = (_weights((300, 258), 3).view(np.uint32) >> 16).astype(np.uint16)
    src.insert("bf", bf, dtype="BF16")
    src.insert("ids", np.arange(10, dtype=np.int8))                                     # not a float tensor: left alone
    p = tmp_path / "w.safetensors"
    src.save_safetensors(p)
    eager, lazy = cfb.TensorStore(), cfb.TensorStore()
    eager.load_safetensors(p)
    assert lazy.load_safetensors_lazy(p) == len(ws) + 2
    te, tl = eager.run_pipeline("quantize(bits=8)"), lazy.run_pipeline("quantize(bits=8)")
    assert tl[0]["ops_modified"] == te[0]["ops_modified"] == len(ws) + 1
    pe, pl = tmp_path / "e.safetensors", tmp_path / "l.safetensors"
    eager.save_safetensors(pe)
    lazy.save_safetensors(pl)
    assert pe.read_bytes() == pl.read_bytes()
    e = lazy.entries()
    q, sc, _ = oracle.quant_sym(ws["big"], 8)
    assert np.array_equal(e["big"]["data"], q) and e["big"]["scale"] == sc and np.array_equal(e["ids"]["data"], np.arange(10))
    # a fake-quant pass (works on f32 values) over a lazily loaded bf16 tensor takes the widen-on-host path
    lz = cfb.TensorStore()
    lz.load_safetensors_lazy(p)
    eg = cfb.TensorStore()
    eg.load_safetensors(p)
    lz.run_pipeline("quantize(scheme=fp8)")
    eg.run_pipeline("quantize(scheme=fp8)")
    assert np.array_equal(lz.entries()["bf"]["data"], eg.entries()["bf"]["data"])


def test_store_fake_quant_and_extension_schemes(cuda_device, oracle):
    w = _weights((256, 384), 7)
    def run(spec):
        st = cfb.TensorStore()
        st.insert("w", w)
        st.insert("vec", np.linspace(-1, 1, 64, dtype=np.float32))
        st.run_pipeline(spec)
        return st.entries()
    e = run("quantize(bits=4,group_size=128)")                               # groupwise, awq_salient defaults to true
    want, thr, k = oracle.fakequant_group(w, 4, 128, 0.01, True)
    assert np.array_equal(e["w"]["data"].view(np.uint32), want.view(np.uint32)) and e["w"]["attrs"]["castforge.awq_salient_channels"] == str(k)
    assert np.array_equal(e["vec"]["data"], np.linspace(-1, 1, 64, dtype=np.float32))       # rank 1: skipped (schemes.rs:503)
    e = run("quantize-fp8(format=e5m2,block_size=64)")
    assert np.array_equal(e["w"]["data"].view(np.uint32), oracle.fakequant_fp8grid(w, 64, True, True).view(np.uint32))
    e = run("quantize-fp4")
    assert np.array_equal(e["w"]["data"].view(np.uint32), oracle.fakequant_e2m1(w, 16).view(np.uint32))
    e = run("smooth-quantize(alpha=0.5)")
    assert np.array_equal(e["w"]["data"].view(np.uint32), oracle.smoothquant(w, 8, 0.5)[0].view(np.uint32))
    e = run("insert-qat-ste(bits=4)")
    assert np.array_equal(e["w"]["data"].view(np.uint32), oracle.fakequant_tensor(w, 4)[0].view(np.uint32))
    e = run("rotate-hadamard(block_size=64)")
    assert np.array_equal(e["w"]["data"].view(np.uint32), oracle.fwht_cols(w, 256, 384, 64)[0].ravel().view(np.uint32))
    e = run("quantize(scheme=per_channel)")
    q, s = oracle.quant_per_channel(w, 256, 384, 8)
    assert np.array_equal(e["w"]["data"], q.ravel()) and np.array_equal(e["w.scales"]["data"], s)
    e = run("quantize(scheme=int4_asym,group_size=128)")
    c, sc, z = oracle.quant_int4_asym(w, 128)
    assert np.array_equal(e["w"]["data"], c) and np.array_equal(e["w.scales"]["data"], sc) and np.array_equal(e["w.zeros"]["data"], z)
    e = run("quantize(scheme=nf4)")
    c, a8, a2 = oracle.quant_nf4(w, 64, 256)
    assert np.array_equal(e["w"]["data"], c) and np.array_equal(e["w.absmax8"]["data"], a8) and np.array_equal(e["w.absmax2"]["data"], a2)
    e = run("quantize(scheme=nonsense_name)")                                 # unknown scheme strings mean per-tensor weights (schemes.rs:114-150)
    assert e["w"]["quantized"] and np.array_equal(e["w"]["data"], oracle.quant_sym(w, 8)[0])


def test_two_host_threads_share_one_device(cuda_device):
    """The C ABI is re-entrant like the reference's: two host threads run quantize pipelines on the same device at the
    same time (the per-device staging slots are handed from one call to the next under a lock) and each gets exactly
    what a serial run gives."""
    import threading
    rng = np.random.default_rng(3)
    sets = [[(rng.standard_normal((257, 130 + 7 * k + t)) * 0.02).astype(np.float32) for k in range(6)] for t in range(2)]

    def run(ws, spec):
        st = cfb.TensorStore()
        for i, w in enumerate(ws):
            st.insert(f"w{i}", w)
        st.run_pipeline(spec)
        out = {n: (e["data"].copy(), e["scale"]) for n, e in st.entries().items()}
        st.close()
        return out

    specs = ["quantize(bits=8)", "quantize(scheme=nf4)"]
    serial = [run(sets[t], specs[t]) for t in range(2)]
    for _ in range(3):
        got = [None, None]
        errs = []

        def work(t):
            try:
                got[t] = run(sets[t], specs[t])
            except Exception as e:  # noqa: BLE001
                errs.append(e)
        th = [threading.Thread(target=work, args=(t,)) for t in range(2)]
        for x in th:
            x.start()
        for x in th:
            x.join()
        assert not errs, errs
        for t in range(2):
            assert got[t].keys() == serial[t].keys()
            for n in serial[t]:
                assert np.array_equal(got[t][n][0], serial[t][n][0]) and got[t][n][1] == serial[t][n][1], (t, n)


def test_a1_status_word_reads_zero_after_normal_runs(cuda_device):
    """cfb200_quant_sym_status: the persistent kernel's bounded waits have not run out (nothing here makes one expire)."""
    import ctypes
    import torch
    from castforge_b200 import device as D
    w = (torch.randn(24 << 20, device=cuda_device) * 0.02).to(torch.bfloat16)   # 48 MB: takes the persistent kernel
    D.quant_sym_tensor(w, 8)
    D.quant_sym_tensors([w[: 1 << 20], w[1 << 20: 3 << 20]], 8)
    flag = ctypes.c_int32(-1)
    assert cfb.load().cfb200_quant_sym_status(ctypes.byref(flag)) == 0 and flag.value == 0


def test_bounded_waits_give_up_and_report(cuda_device):
    """A wait that can never complete runs out after its limit and the host sees it: through the sticky A1 status word
    (which the self-test clears again) and through a caller's error word as the tensor-core kernels use it.  The wait is
    on a barrier in the probe kernel's own shared memory that nothing arrives at; no fault, no hang, microseconds."""
    import ctypes
    lib = cfb.load()
    seen = ctypes.c_int32(-1)
    assert lib.cfb200_selftest_expired_wait(0, ctypes.byref(seen)) == 0 and seen.value == 1
    flag = ctypes.c_int32(-1)
    assert lib.cfb200_quant_sym_status(ctypes.byref(flag)) == 0 and flag.value == 0      # cleared: later runs start clean
    assert lib.cfb200_selftest_expired_wait(1, ctypes.byref(seen)) == 0 and seen.value == 7
    assert lib.cfb200_selftest_expired_wait(2, ctypes.byref(seen)) == 0 and seen.value == 8      # the pair kernel's sleeping wait
    assert lib.cfb200_selftest_expired_wait(3, ctypes.byref(seen)) == 0 and seen.value == 9      # ... and its cluster-scope wait
    assert lib.cfb200_selftest_expired_wait(9, ctypes.byref(seen)) == 1
