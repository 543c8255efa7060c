"""Run one entry point of the library on one shape, a few times, and print its device time.

    python bench_cases.py e3 --shape 14336x4096 --dtype bf16 --iters 3
    python bench_cases.py gemv_w4 --shape 4x4096x4096
    python bench_cases.py gemm_fp8 --shape 4096x4096x4096

Meant for timing a kernel in isolation and as the small, self-ending command a profiler wraps.
Inputs are seeded synthetic data; `--rotate R` cycles through R distinct input buffers so that a
timed launch does not find its input in L2 (default 3).  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys

from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
from castforge_b200 import device as D  # noqa: E402

HBM_CASES = ("a1", "a1list", "a1layer", "e4list", "gguf_q8_pack", "gguf_q8_unpack", "gguf_q4_unpack", "e1", "e2", "e3", "e4rows", "e4tensor", "a2", "a2awq", "a3", "a4", "a6", "fwht",
             "kv_page", "kv_head", "kv_tensor", "kv_decode", "e4m3_slice_enc", "e4m3_slice_dec",
             "merge_linear", "merge_slerp", "merge_ties", "task_merge", "prune_2to4", "prune_cols", "transpose", "lora_bake")
GEMM_CASES = ("gemm_fp8", "gemm_bf16", "gemm_w4", "gemv_w4", "gptq")
HOST_CASES = ("stream_file",)


def _weights(rows, cols, dt, n, dev, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    return [(torch.randn(rows * cols, device=dev, generator=g) * 0.02).to(dt).reshape(rows, cols) for _ in range(n)]


LLAMA3_8B_LAYER = ((4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (14336, 4096), (4096, 14336))


def hbm_case(name, rows, cols, dt, rotate, dev):
    if name == "a1layer":  # `rotate` decoder layers of Llama-3-8B shape (q, k, v, o, gate, up, down) as ONE list call
        ws = []
        for i in range(rotate):
            for (r, c) in LLAMA3_8B_LAYER:
                ws += _weights(r, c, dt, 1, dev, seed=len(ws))
        n = sum(w.numel() for w in ws)
        return [ws], (lambda lst: D.quant_sym_tensors([w.reshape(-1) for w in lst], 8)), n * (ws[0].element_size() + 1)
    if name.startswith("kv_"):  # ROWS pages of COLS tokens, 8 kv heads of 128: keys and values of one layer's cache
        g = torch.Generator(device=dev).manual_seed(3)
        caches = [(torch.randn((rows, cols, 8, 128), device=dev, generator=g).to(dt),
                   (torch.randn((rows, cols, 8, 128), device=dev, generator=g) * 3).to(dt)) for _ in range(rotate)]
        n = rows * cols * 8 * 128
        esz = caches[0][0].element_size()
        if name == "kv_decode":
            enc = [D.kv_encode_k16v8(k, v, "page_head") for k, v in caches]
            return enc, (lambda e: D.kv_decode_k16v8(e[0], e[1], e[2], "page_head")), n * (3 + 8) + 4 * rows * 8
        scope = {"kv_page": "page_head", "kv_head": "layer_head", "kv_tensor": "tensor"}[name]
        return caches, (lambda kv: D.kv_encode_k16v8(kv[0], kv[1], scope)), n * (2 * esz + 3)
    ws = _weights(rows, cols, dt, rotate, dev)
    esz = ws[0].element_size()
    n = rows * cols
    if name.startswith("merge_") or name == "task_merge":  # f32 tensor pairs: (a, a + small difference)
        g = torch.Generator(device=dev).manual_seed(5)
        pairs = [(w.float(), w.float() + torch.randn(w.shape, device=dev, generator=g) * 0.003) for w in ws]
        if name == "task_merge":  # one fine-tune, half of the deltas dropped: 12 bytes per element is the floor (base, ft, out)
            return pairs, (lambda p: D.task_vector_merge(p[0], [p[1]], 1.0, 0.5)), n * 12
        return pairs, (lambda p: D.merge_f32(p[0], p[1], name[6:], 0.5)), n * 12
    if name == "lora_bake":  # rank-16 adapters baked into a ROWS x COLS f32 weight
        g = torch.Generator(device=dev).manual_seed(6)
        f32 = [w.float() for w in ws]
        a = torch.randn(rows, 16, device=dev, generator=g) * 0.1
        b = torch.randn(16, cols, device=dev, generator=g) * 0.1
        return f32, (lambda w: D.lora_bake_(w, a, b, 0.5)), n * 8
    if name in ("prune_2to4", "prune_cols", "transpose"):
        f32 = [w.float() for w in ws]
        if name == "prune_2to4":
            return f32, (lambda w: D.prune_2to4_(w)), n * 8
        if name == "transpose":
            return f32, (lambda w: D.transpose_f32(w)), n * 8
        return f32, (lambda w: D.prune_columns_l1(w, sparsity=0.5)), n * 6  # read once, half of it written
    if name == "e4m3_slice_enc":
        f32 = [w.float().reshape(-1) * 50 for w in ws]
        return f32, (lambda w: D.e4m3_slice_encode(w)), n * 5
    if name == "e4m3_slice_dec":
        g = torch.Generator(device=dev).manual_seed(4)
        codes = [torch.randint(0, 256, (n,), device=dev, dtype=torch.uint8, generator=g) for _ in range(rotate)]
        return codes, (lambda c: D.e4m3_slice_decode(c)), n * 5
    if name == "a1":
        return ws, (lambda w: D.quant_sym_tensor(w.reshape(-1), 8)), n * (esz + 1)
    if name == "e4list":  # the per-tensor E4M3 cast of the whole rotation as ONE list call
        return [ws], (lambda lst: D.cast_e4m3_tensors([w.reshape(-1) for w in lst])), rotate * n * (esz + 1)
    if name == "a1list":  # the whole rotation as ONE list call
        return [ws], (lambda lst: D.quant_sym_tensors([w.reshape(-1) for w in lst], 8)), rotate * n * (esz + 1)
    if name == "gguf_q8_pack":
        codes = [D.quant_sym_tensor(w.reshape(-1), 8)[0] for w in ws]
        return codes, (lambda c: D.gguf_pack_q8_0(c, 0.0123)), n * (1 + 34 / 32)
    if name in ("gguf_q8_unpack", "gguf_q4_unpack"):
        bb = 34 if name == "gguf_q8_unpack" else 18
        g = torch.Generator(device=dev).manual_seed(2)
        blocks = [torch.randint(0, 255, ((n + 31) // 32 * bb,), device=dev, dtype=torch.uint8, generator=g) for _ in range(rotate)]
        for b in blocks:
            b.view(-1, bb)[:, 1] = 0x2E  # finite block scales
        kind = "q8_0" if bb == 34 else "q4_0"
        return blocks, (lambda b: D.gguf_unpack(b, n, kind)), n * (bb / 32 + 4)
    if name == "e1":
        return ws, (lambda w: D.quant_per_channel(w, 8)), n * (esz + 1) + 4 * rows
    if name == "e2":
        return ws, (lambda w: D.quant_int4_asym(w.reshape(-1), 128)), n * (esz + 0.5 + 2.5 / 128)
    if name == "e3":
        return ws, (lambda w: D.quant_nf4(w.reshape(-1), 64, 256)), n * (esz + 0.5 + 1 / 64 + 4 / 16384)
    if name == "e4rows":
        return ws, (lambda w: D.cast_e4m3_rows(w)), n * (esz + 1) + 4 * rows
    if name == "e4tensor":
        return ws, (lambda w: D.cast_e4m3_tensor(w)), n * (esz + 1)
    f32 = [w.float() for w in ws] if dt != torch.float32 else ws
    if name == "a2":
        return f32, (lambda w: D.fakequant_group(w.reshape(-1), 4, 128, 0.0, False)), n * 8
    if name == "a2awq":  # the pass as the reference runs it by default: exact salient threshold (radix select) + fake quant
        return f32, (lambda w: D.fakequant_group(w.reshape(-1), 4, 128, 0.01, True)), n * 8
    if name == "a3":
        return f32, (lambda w: D.fakequant_fp8grid(w.reshape(-1), 32, False, True)), n * 8
    if name == "a4":
        return f32, (lambda w: D.fakequant_e2m1(w.reshape(-1), 16)), n * 8
    if name == "a6":
        return f32, (lambda w: D.fakequant_tensor(w.reshape(-1), 8)), n * 8
    if name == "fwht":
        return f32, (lambda w: D.fwht_cols_(w, 128)), n * 8
    raise SystemExit(f"unknown case {name}")


def gemm_case(name, M, N, K, rotate, dev):
    g = torch.Generator(device=dev).manual_seed(1)
    flops = 2.0 * M * N * K
    if name == "gemm_fp8":
        a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        ws = _weights(N, K, torch.bfloat16, rotate, dev)
        ac, asc = D.cast_e4m3_rows(a)
        packed = [D.cast_e4m3_tensor(w) for w in ws]
        packed = [(c, sa, float(sa[0].item())) for c, sa in packed]
        return packed, (lambda p: D.gemm_fp8(ac, asc, p[0], p[2], out_f32=False, check=False)), flops, M * K + N * K + 2 * M * N
    if name == "gemm_bf16":
        a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        ws = _weights(N, K, torch.bfloat16, rotate, dev)
        return ws, (lambda w: D.gemm_bf16_nt(a, w, check=False)), flops, 2 * (M * K + N * K) + 4 * M * N
    if name in ("gemm_w4", "gemv_w4"):
        a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        ws = _weights(N, K, torch.bfloat16, rotate, dev)
        packed = [D.quant_int4_asym(w.reshape(-1), 128) for w in ws]
        nbytes = N * K / 2 + 2.5 * N * K / 128 + 2 * M * K + 2 * M * N
        if name == "gemv_w4":
            return packed, (lambda p: D.gemv_w4a16(a, p[0], p[1], p[2], N, 128)), flops, nbytes
        return packed, (lambda p: D.gemm_w4a16(a, p[0], p[1], p[2], N, 128, check=False)), flops, nbytes
    if name == "gptq":  # M = tokens, N = output rows, K = input channels
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        ws = _weights(N, K, torch.bfloat16, rotate, dev)
        u = D.gptq_prepare(D.gptq_hessian(x), 0.01)
        return ws, (lambda w: D.gptq_quantize(w, u, want_dequant=False)), 2.0 * N * K * K / 2, None
    raise SystemExit(f"unknown case {name}")


def stream_file_case(layers, iters):
    """Wall-clock time of `quantize(bits=8)` over a SafeTensors file, lazily loaded (file slices -> pinned staging ->
    device, several reader threads) against eagerly loaded (the whole file into host memory first).  The file is written
    to a temporary directory under /dev/shm when there is one (page-cache speed: the reader threads, not a disk, are what
    is measured), else under the system's temporary directory."""
    import os
    import tempfile
    import time

    import numpy as np

    from castforge_b200 import TensorStore
    root = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else None
    out = {"case": "stream_file", "layers": layers, "tmp_root": root or tempfile.gettempdir()}
    with tempfile.TemporaryDirectory(dir=root) as tmp:
        path = os.path.join(tmp, "layers.safetensors")
        st = TensorStore()
        rng = np.random.default_rng(0)
        blk = (rng.standard_normal(1 << 22, dtype=np.float32) * np.float32(0.02)).view(np.uint32) >> 16
        blk = blk.astype(np.uint16)
        nbytes = 0
        for li in range(layers):
            for ti, (r, c) in enumerate(LLAMA3_8B_LAYER):
                w = np.resize(blk, r * c).reshape(r, c)
                st.insert(f"layers.{li}.t{ti}", w, dtype="BF16")
                nbytes += w.nbytes
        st.save_safetensors(path)
        st.close()
        out["file_GB"] = round(nbytes / 1e9, 3)
        for mode in ("lazy", "eager"):
            best = None
            for _ in range(max(1, iters)):
                s2 = TensorStore()
                t0 = time.perf_counter()
                if mode == "lazy":
                    s2.load_safetensors_lazy(path)
                else:
                    s2.load_safetensors(path)
                t1 = time.perf_counter()
                tel = s2.run_pipeline("quantize(bits=8)")
                t2 = time.perf_counter()
                assert tel[0]["ops_modified"] == 7 * layers
                s2.close()
                tot = t2 - t0
                if best is None or tot < best[0]:
                    best = (tot, t1 - t0, t2 - t1)
            out[mode] = {"total_s": round(best[0], 4), "load_s": round(best[1], 4), "pipeline_s": round(best[2], 4),
                         "input_GBps": round(nbytes / best[0] / 1e9, 2)}
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=HBM_CASES + GEMM_CASES + HOST_CASES)
    ap.add_argument("--shape", default=None, help="ROWSxCOLS for quantizers, MxNxK for GEMMs")
    ap.add_argument("--dtype", default="bf16", choices=("bf16", "f16", "f32"))
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--rotate", type=int, default=3)
    ap.add_argument("--burst", type=int, default=1, help="launches per timed interval (back to back, rotating inputs); "
                    "the time printed is per launch.  Use it for launches of a few microseconds.")
    ap.add_argument("--graph", action="store_true", help="capture the burst in a CUDA graph and time its replay")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE", help="performance knob for cfb200_tune")
    args = ap.parse_args(argv)
    for kv in args.tune:
        from castforge_b200 import load
        key, _, val = kv.partition("=")
        if load().cfb200_tune(key.encode(), int(val)) != 0:
            raise SystemExit(f"unknown tunable {key!r}")
    if not torch.cuda.is_available():
        raise SystemExit("bench_cases.py needs a CUDA device")
    dev = torch.device("cuda:0")
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[args.dtype]
    if args.case == "stream_file":  # --shape LAYERSx1: a .safetensors file of LAYERS Llama-3-8B decoder layers (bf16)
        print(json.dumps(stream_file_case(int((args.shape or "2x1").split("x")[0]), args.iters)))
        return
    if args.case == "gptq":  # the three steps timed separately: --shape TOKENSxOUT_ROWSxIN_CHANNELS
        T, N, K = map(int, (args.shape or "8192x4096x4096").split("x"))
        g = torch.Generator(device=dev).manual_seed(1)
        chan = torch.exp(torch.empty(K, device=dev).uniform_(-2.3, 2.3, generator=g))  # log-uniform channel scales in [0.1, 10]
        x = (torch.randn(T, K, device=dev, generator=g) * chan).to(torch.bfloat16)
        w = _weights(N, K, torch.bfloat16, 1, dev)[0]

        def t3(fn):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn()
            e1.record()
            e1.synchronize()
            return r, e0.elapsed_time(e1)

        D.gptq_quantize(w[:128].contiguous(), D.gptq_prepare(D.gptq_hessian(x[:1024].contiguous()), 0.01), want_dequant=False)  # warm up
        h, ms_h = t3(lambda: D.gptq_hessian(x))
        u, ms_p = t3(lambda: D.gptq_prepare(h, 0.01))
        _, ms_q = t3(lambda: D.gptq_quantize(w, u, want_dequant=False))
        print(json.dumps({"case": "gptq", "tokens": T, "out_rows": N, "in_channels": K,
                          "hessian_ms": round(ms_h, 3), "hessian_TFLOPps_upper_only": round(T * K * K / ms_h / 1e9, 1),
                          "prepare_ms": round(ms_p, 3), "quantize_ms": round(ms_q, 3),
                          "quantize_update_TFLOPps": round(N * K * K / ms_q / 1e9, 2)}))
        return
    if args.case in HBM_CASES:
        rows, cols = map(int, (args.shape or "14336x4096").split("x"))
        inputs, fn, nbytes = hbm_case(args.case, rows, cols, dt, args.rotate, dev)
        flops = None
    else:
        M, N, K = map(int, (args.shape or "4096x4096x4096").split("x"))
        inputs, fn, flops, nbytes = gemm_case(args.case, M, N, K, args.rotate, dev)
    torch.cuda.synchronize()
    for i in range(args.warmup):
        fn(inputs[i % len(inputs)])
    torch.cuda.synchronize()
    times = []
    graph = None
    if args.graph:  # one CUDA graph of `burst` launches: takes the host's per-call cost out of the interval
        graph = torch.cuda.CUDAGraph()
        keep = []
        with torch.cuda.graph(graph):
            for b in range(args.burst):
                keep.append(fn(inputs[b % len(inputs)]))
        graph.replay()
        torch.cuda.synchronize()
    for i in range(args.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            for b in range(args.burst):
                fn(inputs[(i * args.burst + b) % len(inputs)])
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) / args.burst)
    ms = sorted(times)[len(times) // 2]
    out = {"case": args.case, "shape": args.shape, "dtype": args.dtype, "ms_median": round(ms, 4), "iters": args.iters, "burst": args.burst, "rotate": args.rotate}
    if nbytes:
        out["algorithmic_GBps"] = round(nbytes / ms / 1e6, 1)
    if flops:
        out["TFLOPps"] = round(flops / ms / 1e9, 1)
    print(json.dumps(out))


if __name__ == "__main__":
    main(sys.argv[1:])
