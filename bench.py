#!/usr/bin/env python
"""Headline benchmark: whole-model weight quantization throughput on B200.

Workload (metric: weight-quantize GB/s on an 8B-shaped set): a Llama-3-8B-shaped bf16 weight
set (32 x {q,o 4096x4096; k,v 1024x4096; gate,up 14336x4096; down 4096x14336} + embedding and
lm_head 128256x4096 = 8.03e9 elements, 16.06 GB), synthetic N(0, 0.02) values, run through
`quantize(bits=8)` -- the reference's per-tensor symmetric INT8 pass
(src/passes/quantize/formats.rs:664-698).  One step = one pass over every tensor of the set.
GB/s counts ALGORITHMIC bytes: 2 B read + 1 B written per element.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 is launched with torch.distributed.run (one rank per GPU).  `value` is weak scaling: every rank quantizes one
set's worth of tensors, no data-path collective, times are max over ranks.  The same line carries `strong`: ONE set
dealt over the N ranks (whole tensors largest first, the two vocabulary tensors cut into row blocks whose partial absmax
meet in one NCCL MAX all-reduce of one float each), `nf4_llama2_7b` (BASELINE config 3: one Llama-2-7B-shaped set dealt
per tensor over the ranks) and, for N > 1, `colpar` (column-parallel W4A16 / FP8 GEMM + NCCL all-gather).  At N = 1 the
`secondary` block times the GEMM / decode / GPTQ figures of BASELINE configs 2, 4 and 5.
`--impl reference` times the CPU restatement of the reference pass (the reference is Rust and
cannot be built here) on the host cores over a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = "llama3-8b-shaped bf16 weight set (8.03e9 elements per GPU), quantize(bits=8) per-tensor symmetric INT8"
METRIC = "weight_quantize_throughput"
UNIT = "GB/s"
ALG_BYTES_PER_ELEM = 3.0  # bf16 read once + int8 written (the second read is an implementation cost)


def llama3_8b_tensors() -> list[tuple[str, int, int]]:
    t = []
    for layer in range(32):
        for name, r, c in (("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
                           ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)):
            t.append((f"layers.{layer}.{name}", r, c))
    t.append(("embed_tokens", 128256, 4096))
    t.append(("lm_head", 128256, 4096))
    return t


def shard_greedy(tensors, world: int, rank: int):
    """N sets over N ranks: largest-first onto the least-loaded rank (no communication needed)."""
    items = []
    for rep in range(world):
        items += [(f"set{rep}.{n}", r, c) for (n, r, c) in tensors]
    items.sort(key=lambda x: -(x[1] * x[2]))
    load = [0] * world
    mine = []
    for it in items:
        j = min(range(world), key=lambda i: load[i])
        load[j] += it[1] * it[2]
        if j == rank:
            mine.append(it)
    return mine


def measured_peak_hbm():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        rows = [l.strip().split(", ") for l in open(self.f.name) if l.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for nm, v in zip(names, r[5:9]):
                    if v.strip().lower() == "active":
                        reasons.add(nm)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


_CPU_SAMPLE: dict = {}


def cpu_baseline_run(threads: int, seconds_budget: float = 20.0):
    """Oracle port of the reference pass on host cores over a bounded sample: one decoder layer of
    the workload (7 tensors, 218 M elements), bf16 -> f32 widening (resolve_f32_attr) + quantize."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_lib
    orc = oracle_lib.load()
    if threads <= 0:  # every core this process may run on (a launcher's OMP_NUM_THREADS=1 is not the host's core count)
        threads = max(orc.max_threads(), len(os.sched_getaffinity(0)))
    # one vocabulary-sized tensor first (the workload has two), then decoder-layer tensors until the time budget is spent
    layer = [("embed_tokens", 128256, 4096)] + [t for t in llama3_8b_tensors() if t[0].startswith("layers.0.")] * 64
    rng = np.random.default_rng(0)
    total_elems, total_t = 0, 0.0
    for (name, r, c) in layer:
        n = r * c
        if n not in _CPU_SAMPLE:   # one synthetic tensor per distinct size, generated once
            _CPU_SAMPLE[n] = ((rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).view(np.uint32) >> 16).astype(np.uint16)
        bf = _CPU_SAMPLE[n]
        t0 = time.perf_counter()
        f = orc.to_f32(bf, 2, threads=threads)
        orc.quant_sym(f, 8, threads=threads)
        total_t += time.perf_counter() - t0
        total_elems += n
        if total_t > seconds_budget:
            break
    gbs = total_elems * ALG_BYTES_PER_ELEM / total_t / 1e9
    return {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"one 128256x4096 tensor, then decoder-layer tensors of the workload until {seconds_budget:.0f} s of CPU time ({total_elems} elements), bf16->f32 widen + quantize_symmetric_f32, {total_t:.2f} s"}, total_t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_all = []
    cb = None
    for _ in range(max(args.warmup, 0)):
        cpu_baseline_run(0, 3.0)
    for _ in range(max(args.steps, 1)):
        cb, t = cpu_baseline_run(0, 15.0)
        t_all.append((cb["value"], t))
    val = sum(v for v, _ in t_all) / len(t_all)
    ms = sum(t for _, t in t_all) / len(t_all) * 1e3
    cb["value"] = val
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "reference_impl": "C++ restatement of the reference's Rust CPU pass (Rust toolchain absent), all host threads",
                       "step": cb["sample"]},
            "cpu_baseline": cb,
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def llama2_7b_tensors() -> list[tuple[str, int, int]]:
    t = []
    for layer in range(32):
        for name, r, c in (("q", 4096, 4096), ("k", 4096, 4096), ("v", 4096, 4096), ("o", 4096, 4096),
                           ("gate", 11008, 4096), ("up", 11008, 4096), ("down", 4096, 11008)):
            t.append((f"layers.{layer}.{name}", r, c))
    t.append(("embed_tokens", 32000, 4096))
    t.append(("lm_head", 32000, 4096))
    return t


def traffic_ratios():
    """DRAM bytes per algorithmic byte of the persistent A1 kernel, read from the ncu summary that sits under profiles/
    (lines `traffic_ratio_layers: x` / `traffic_ratio_vocab: x`); None when the summary is absent."""
    import re
    f = ROOT / "profiles" / "a1_persist_kernel_llama3-8b_layers.md"
    try:
        text = f.read_text()
        lay = float(re.search(r"traffic_ratio_layers:\s*([0-9.]+)", text).group(1))
        voc = float(re.search(r"traffic_ratio_vocab:\s*([0-9.]+)", text).group(1))
        return lay, voc
    except Exception:
        return None


def timed_steps(step, steps, stream, barrier, world, dev):
    """K steps between two events on `stream`, barrier + synchronize on both sides, max over ranks.  Returns ms per step
    and every rank's own ms per step."""
    import torch
    import torch.distributed as dist
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record(stream)
    for _ in range(steps):
        step()
    t1.record(stream)
    barrier()
    ms = t0.elapsed_time(t1) / steps
    per_rank = [ms]
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        gathered = [torch.zeros_like(tt) for _ in range(world)]
        dist.all_gather(gathered, tt)
        per_rank = [float(x.item()) for x in gathered]
    return max(per_rank), per_rank


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="castforge_b200")
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of the set (32 = full workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the GEMM / decode / GPTQ figures reported beside the headline metric")
    ap.add_argument("--no-strong", action="store_true", help="skip the one-set-over-N-ranks and column-parallel legs")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE", help="performance knob passed to cfb200_tune (never changes results)")
    ap.add_argument("--e2e-layers", type=int, default=-1,
                    help="decoder layers streamed from host per e2e step (-1: the whole set at one GPU when host memory allows, else 4)")
    args = ap.parse_args()
    if args.e2e_layers == 0:
        args.e2e_layers = 1  # the end-to-end leg is part of the output line: it always streams at least one layer
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import castforge_b200
    from castforge_b200._lib import check

    lib = castforge_b200.load()  # raises if the CUDA library is missing: no fallback
    persist = True
    for kv in args.tune:
        key, _, val = kv.partition("=")
        if key == "a1_persist":
            persist = int(val) != 0
        if lib.cfb200_tune(key.encode(), int(val)) != 0:
            raise SystemExit(f"unknown tunable {key!r}")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    torch.cuda.set_device(local_rank)
    dev = torch.device(f"cuda:{local_rank}")
    from castforge_b200 import multi_gpu, sharding
    all_cpus = os.sched_getaffinity(0)
    numa_cpus = sharding.bind_host_to_device_node(local_rank)  # host staging memory local to this GPU's PCIe root
    comm = multi_gpu.Comm.from_torch_distributed() if world > 1 else None   # the library's own NCCL communicator

    tensors = llama3_8b_tensors()
    if args.layers != 32:
        tensors = [t for t in tensors if not t[0].startswith("layers.") or int(t[0].split(".")[1]) < args.layers]
    mine = shard_greedy(tensors, world, rank)
    n_total = sum(r * c for _, r, c in mine)

    # ---- device-resident inputs: one flat bf16 arena, per-tensor views (256-byte aligned) ------
    offs, o = [], 0
    for _, r, c in mine:
        offs.append(o)
        o += (r * c + 127) // 128 * 128
    arena = torch.empty(o, dtype=torch.bfloat16, device=dev)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    CH = 1 << 27
    for s in range(0, o, CH):
        e = min(o, s + CH)
        arena[s:e] = (torch.randn(e - s, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    codes = torch.empty(o, dtype=torch.int8, device=dev)
    scales = torch.zeros(len(mine) * 2, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev)
    sp = ctypes.c_void_p(stream.cuda_stream)
    vp = ctypes.c_void_p
    views = [(arena.data_ptr() + 2 * off, r * c, codes.data_ptr() + off) for off, (_, r, c) in zip(offs, mine)]

    cnt = len(views)
    srcs = (vp * cnt)(*[v[0] for v in views])
    outs = (vp * cnt)(*[v[2] for v in views])
    ns = (ctypes.c_size_t * cnt)(*[v[1] for v in views])
    n_stages = ctypes.c_int32(0)
    check(lib.cfb200_quant_sym_tensors_plan(cnt, ns, 2, 0, ctypes.byref(n_stages)))
    n_stages = n_stages.value

    def new_events():
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_stages + 1)]
        for e in evs:
            e.record(stream)  # materialise the cudaEvent_t handles
        return evs, (vp * len(evs))(*[e.cuda_event for e in evs])

    def step(ev_handles=None):
        # one C-ABI call quantizes every tensor of this rank's store (n_stages kernel launches)
        check(lib.cfb200_quant_sym_tensors(cnt, srcs, 2, ns, 8, outs, vp(scales.data_ptr()), 0, ev_handles, sp))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    evs = [new_events() for _ in range(args.steps)]
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record(stream)
    for k in range(args.steps):
        step(evs[k][1])
    t1.record(stream)
    barrier()
    clocks = sampler.stop() if sampler else None
    ms_total = t0.elapsed_time(t1)
    if world > 1:
        tt = torch.tensor([ms_total], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total = float(tt.item())
    ms_step = ms_total / args.steps
    # the cooperative kernel reports an expired wait through a device flag, not a return code: a run that saw one
    # has no valid figure
    a1_flag = ctypes.c_int32(-1)
    check(lib.cfb200_quant_sym_status(ctypes.byref(a1_flag)))
    if a1_flag.value != 0:
        raise SystemExit("bench: the A1 kernel gave up a bounded wait on this device; its outputs are incomplete")
    # dominant kernel.  Default: a1_persist_kernel<bf16>, ONE cooperative launch per step that walks the
    # whole list (per tensor group: absmax pass, grid barrier, quantize pass).  With --tune a1_persist=0:
    # a1_stage_kernel<bf16>, one launch per tensor group.  Algorithmic bytes = 2 B read + 1 B written per
    # element; the second read of the weights is an implementation cost that is NOT counted.
    k_ms = [evl[i].elapsed_time(evl[i + 1]) for (evl, _) in evs for i in range(n_stages)]
    k_launches = len(k_ms)
    k_avg_ms = sum(k_ms) / k_launches
    k_alg_bytes = n_total * ALG_BYTES_PER_ELEM / n_stages   # average algorithmic bytes per launch
    achieved = k_alg_bytes / (k_avg_ms * 1e-3) / 1e9
    peak, peak_src = measured_peak_hbm()
    traffic, traffic_src = None, "no ncu summary of this kernel under profiles/"
    if persist:
        kernel_name = "a1_persist_kernel<bf16> (whole list in one cooperative launch: absmax pass, grid barrier, quantize pass per tensor group)"
        tr = traffic_ratios()
        if tr:
            big = sum(r * c for (_, r, c) in mine if r * c * 2 > (512 << 20))   # tensors far beyond L2 + shared memory
            traffic = (tr[0] * (n_total - big) + tr[1] * big) / n_total * k_alg_bytes
            traffic_src = (f"ncu dram__bytes_read+write of smaller captures of the same kernel, scaled by elements: {tr[0]} x algorithmic "
                           f"for decoder-layer tensors, {tr[1]} x for the 128256x4096 tensors")
    else:
        kernel_name = "a1_stage_kernel<bf16> (pass 2 of one tensor group + pass 1 of the next)"

    # ---- e2e: host buffers in, codes + scales back to the host, copies inside the timed region ---
    e2e = run_e2e(args, lib, dev, rank, world, mine)

    total_elems_all = n_total
    if world > 1:
        tt = torch.tensor([float(n_total)], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        total_elems_all = float(tt.item())
    value = total_elems_all * ALG_BYTES_PER_ELEM / (ms_step * 1e-3) / 1e9

    spot = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        # one tensor of the timed run against the CPU restatement (the checker of the CPU-baseline leg): k of layer 0
        i_k = next(i for i, (n, _, _) in enumerate(mine) if n.endswith("layers.0.k"))
        off, (_, r, c) = offs[i_k], mine[i_k]
        spot = (arena[off: off + r * c].view(torch.int16).cpu().numpy().view("uint16"), codes[off: off + r * c].cpu().numpy(),
                float(scales[2 * i_k].item()))

    extra = {}
    if not args.no_strong:
        extra["strong"] = strong_leg(args, lib, comm, dev, rank, world, arena, codes, tensors, barrier, stream)
        extra["nf4_llama2_7b"] = nf4_leg(args, lib, dev, rank, world, arena, codes, barrier, stream)
        if world > 1:
            extra["colpar"] = colpar_leg(args, comm, dev, rank, world, barrier, stream)

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": WORKLOAD,
                           "tensors_per_gpu": len(views), "elements_per_gpu": n_total,
                           "bytes_counted": "2 B read + 1 B written per element (algorithmic)",
                           "l2": "inputs (16 GB per GPU) are larger than L2; no flush needed"},
                "clocks": clocks, "e2e": e2e, "gpu_launches": n_stages * args.steps,
                "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": achieved,
                             "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": traffic, "traffic_source": traffic_src,
                             "launches": k_launches, "avg_ms": k_avg_ms,
                             "whole_step_frac": value / world / peak}}
        line.update(extra)
        del arena, codes
        torch.cuda.empty_cache()
        if not args.no_secondary and world == 1:
            line["secondary"] = secondary_metrics(dev)
        line["e2e"]["host_cpus_bound_to_gpu_numa_node"] = len(numa_cpus) if numa_cpus else None
        if not args.no_cpu_baseline and world == 1:  # the CPU leg runs at N = 1 only, on every host core
            os.sched_setaffinity(0, all_cpus)
            cb, _ = cpu_baseline_run(0, 12.0)
            cb1, _ = cpu_baseline_run(1, 8.0)
            cb["single_thread_value"] = cb1["value"]
            if spot is not None:
                import numpy as np
                import oracle_lib
                orc = oracle_lib.load()
                q, sc, _ = orc.quant_sym(orc.to_f32(spot[0], 2, threads=0), 8, threads=0)
                if not (np.array_equal(q, spot[1]) and float(sc) == spot[2]):
                    raise SystemExit("bench: codes / scale of the timed run differ from the CPU restatement on layers.0.k")
                cb["spot_check"] = "layers.0.k of the timed GPU run == the CPU restatement (codes and scale)"
            line["cpu_baseline"] = cb
        print(json.dumps(line))
    if comm is not None:
        comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def strong_leg(args, lib, comm, dev, rank, world, arena, codes, tensors, barrier, stream):
    """ONE 8B-shaped set over the N ranks: cfb200_shard_assign deals whole tensors (largest first) and marks the
    two 128256 x 4096 tensors for row blocks; every rank runs cfb200_quant_sym_tensors_sharded on its part (the row
    blocks' partial absmax meet in one grouped NCCL MAX all-reduce of one float each).  At N = 1 this is the weak leg."""
    import torch
    import torch.distributed as dist
    from castforge_b200 import multi_gpu
    from castforge_b200._lib import check
    vp = ctypes.c_void_p
    nbytes = [r * c * 2 for _, r, c in tensors]
    owner = multi_gpu.shard_assign(nbytes, world, 512 << 20)
    parts = []  # (elements, is_row_block)
    for (name, r, c), ow in zip(tensors, owner):
        if ow == -1:
            lo, hi = multi_gpu.shard_row_range(r, world, rank, 1)
            parts.append(((hi - lo) * c, 1))
        elif ow == rank:
            parts.append((r * c, 0))
    # whole tensors largest first (the order the weak leg uses: tensors of one size then share groups), row blocks last
    parts.sort(key=lambda p: (p[1], -p[0]))
    offs, o = [], 0
    for n, _ in parts:
        offs.append(o)
        o += (n + 127) // 128 * 128
    assert o <= arena.numel()
    cnt = len(parts)
    srcs = (vp * cnt)(*[arena.data_ptr() + 2 * off for off in offs])
    outs = (vp * cnt)(*[codes.data_ptr() + off for off in offs])
    ns = (ctypes.c_size_t * cnt)(*[n for n, _ in parts])
    flags = (ctypes.c_int32 * cnt)(*[f for _, f in parts])
    sa = torch.zeros(cnt * 2, dtype=torch.float32, device=dev)
    sp = vp(stream.cuda_stream)
    if comm is None:
        comm_h, own = multi_gpu.Comm.single(), True
    else:
        comm_h, own = comm, False

    def step():
        check(lib.cfb200_quant_sym_tensors_sharded(comm_h.handle, cnt, srcs, 2, ns, flags, 8, outs, vp(sa.data_ptr()), sp))

    for _ in range(3):
        step()
    ms, per_rank = timed_steps(step, args.steps, stream, barrier, world, dev)
    if own:
        comm_h.close()
    my_bytes = float(sum(n for n, _ in parts) * 2)
    tot = float(sum(nbytes))
    share = torch.tensor([my_bytes / tot], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(share, op=dist.ReduceOp.MAX)
    n_all = sum(r * c for _, r, c in tensors)
    peak, _ = measured_peak_hbm()
    val = n_all * ALG_BYTES_PER_ELEM / (ms * 1e-3) / 1e9
    return {"value": val, "unit": UNIT, "scaling": "strong", "ms_per_step": ms,
            "workload": "ONE llama3-8b-shaped bf16 set (8.03e9 elements) dealt over all ranks; 128256x4096 tensors cut into row blocks",
            "frac_of_aggregate_hbm_peak": val / (world * peak), "largest_rank_share_of_bytes": float(share.item()),
            "rank_ms": per_rank, "slowest_rank": int(max(range(world), key=lambda i: per_rank[i])),
            "collective": "one grouped ncclAllReduce(MAX) of 2 floats per step" if world > 1 else "none"}


def nf4_leg(args, lib, dev, rank, world, arena, codes, barrier, stream):
    """BASELINE config 3: NF4 block 64 + 8-bit double-quantised absmax (blocks of 256) over ONE Llama-2-7B-shaped bf16 set
    (6.74e9 elements), tensors dealt whole over the ranks (largest first), no communication.  Algorithmic bytes per
    element: 2 read + 0.5 + 1/64 + 4/16384 written."""
    import torch
    from castforge_b200 import multi_gpu
    from castforge_b200._lib import check
    vp = ctypes.c_void_p
    tensors = llama2_7b_tensors()
    owner = multi_gpu.shard_assign([r * c * 2 for _, r, c in tensors], world, 0)
    mine = [(r * c) for (_, r, c), ow in zip(tensors, owner) if ow == rank]
    offs, o = [], 0
    for n in mine:
        offs.append(o)
        o += (n + 16383) // 16384 * 16384
    if o > arena.numel():  # a shortened set (--layers) leaves an arena smaller than this rank's share of the 7B-shaped set
        return {"skipped": "the weight arena of this run is smaller than the NF4 set's share per rank"}
    nb_tot = o // 64
    a8 = torch.empty(max(nb_tot, 1), dtype=torch.uint8, device=dev)
    a2 = torch.empty(nb_tot // 256 + len(mine) + 1, dtype=torch.float32, device=dev)
    cnt = len(mine)
    ns = (ctypes.c_size_t * cnt)(*mine)
    srcs = (vp * cnt)(*[arena.data_ptr() + 2 * off for off in offs])
    outs = (vp * cnt)(*[codes.data_ptr() + off // 2 for off in offs])
    o8 = (vp * cnt)(*[a8.data_ptr() + off // 64 for off in offs])
    o2 = (vp * cnt)(*[a2.data_ptr() + 4 * (off // 16384) for off in offs])
    need = lib.cfb200_quant_nf4_tensors_workspace_bytes(cnt, ns, 64)
    ws = torch.empty(need + 256, dtype=torch.uint8, device=dev)
    wp = vp(ws.data_ptr() + (-ws.data_ptr()) % 256)
    sp = vp(stream.cuda_stream)

    def step():   # one C-ABI call, two launches, for this rank's whole share of the set
        check(lib.cfb200_quant_nf4_tensors(cnt, srcs, 2, ns, 64, 256, outs, o8, o2, wp, need, sp))

    for _ in range(3):
        step()
    ms, per_rank = timed_steps(step, args.steps, stream, barrier, world, dev)
    n_all = sum(r * c for _, r, c in tensors)
    alg = 2 + 0.5 + 1 / 64 + 4 / 16384
    peak, _ = measured_peak_hbm()
    val = n_all * alg / (ms * 1e-3) / 1e9
    return {"value": val, "unit": UNIT, "scaling": "strong", "ms_per_step": ms, "gpu_launches_per_step": 2, "tensors_per_rank": len(mine),
            "workload": "ONE llama2-7b-shaped bf16 set (6.74e9 elements), NF4 block 64 + double-quantised absmax, dealt per tensor over the ranks",
            "bytes_counted": f"{alg:.4f} B per element (algorithmic)", "frac_of_aggregate_hbm_peak": val / (world * peak), "rank_ms": per_rank}


def colpar_leg(args, comm, dev, rank, world, barrier, stream):
    """Column-parallel GEMMs (every rank owns N / world rows of the [N, K] weight and the whole activation matrix):
    local tensor-core kernel + the rejoin of the bf16 blocks (peer loads or ncclAllGather, as the library chooses by size),
    timed as one unit and with the rejoin's share measured by timing the local kernel alone."""
    import torch
    from castforge_b200 import device as D, multi_gpu as mg
    out = {}
    g = torch.Generator(device=dev).manual_seed(77)
    bf16_peak, _ = measured_peak_bf16()
    hbm, _ = measured_peak_hbm()

    def time_fn(fn, iters=20):
        for _ in range(3):
            fn()
        ms, _ = timed_steps(fn, iters, stream, barrier, world, dev)
        return ms

    for (M, N, K) in ((2048, 4096, 4096), (8192, 14336, 4096), (8, 128256, 4096)):
        nl = N // world // 8 * 8
        a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(nl, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        c4, s4, z4 = D.quant_int4_asym(w.reshape(-1), 128)
        t_all = time_fn(lambda: mg.gemm_w4a16_colpar(comm, a, c4, s4, z4, nl, 128, layout=0, check_flag=False))
        if M <= 16:
            t_loc = time_fn(lambda: D.gemv_w4a16(a, c4, s4, z4, nl, 128))
            nbytes = world * (nl * K / 2 + 2.5 * nl * K / 128) + 2 * M * K + 2 * M * nl * world
            out[f"w4a16_decode_M{M}_N{nl * world}_K{K}"] = {"ms": t_all, "local_kernel_ms": t_loc, "rejoin_ms": t_all - t_loc,
                                                            "aggregate_GBps": nbytes / t_all / 1e6, "frac_of_aggregate_hbm_peak": nbytes / t_all / 1e6 / (world * hbm)}
        else:
            t_loc = time_fn(lambda: D.gemm_w4a16(a, c4, s4, z4, nl, 128, check=False))
            tf = 2.0 * M * nl * world * K / t_all / 1e9
            out[f"w4a16_prefill_{M}x{nl * world}x{K}"] = {"ms": t_all, "local_kernel_ms": t_loc, "rejoin_ms": t_all - t_loc,
                                                          "aggregate_TFLOPps": tf, "frac_of_aggregate_bf16_peak": tf / (world * bf16_peak)}
            ac, asc = D.cast_e4m3_rows(a)
            wc, wsa = D.cast_e4m3_tensor(w)
            wsc = float(wsa[0].item())
            wc = wc.reshape(nl, K)
            t_all = time_fn(lambda: mg.gemm_fp8_colpar(comm, ac, asc, wc, wsc, layout=0, check_flag=False))
            t_loc = time_fn(lambda: D.gemm_fp8(ac, asc, wc, wsc, out_f32=False, check=False))
            tf = 2.0 * M * nl * world * K / t_all / 1e9
            out[f"fp8_gemm_{M}x{nl * world}x{K}"] = {"ms": t_all, "local_kernel_ms": t_loc, "rejoin_ms": t_all - t_loc,
                                                     "aggregate_TFLOPps": tf, "frac_of_aggregate_2x_bf16_peak": tf / (world * 2 * bf16_peak)}
        del a, w
    out["note"] = ("weights resident and reused between launches (one shape per figure): these are schedule + exchange figures, not cold-weight "
                   "figures; rejoin = products of 8 MB and more: one barrier all-reduce + the library's peer-load kernel over IPC-mapped "
                   "exchange buffers; smaller ones: ncclAllGather + interleave, on the kernel's stream")
    return out


def measured_peak_bf16():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured burst (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def secondary_metrics(dev):
    """The two companion figures of the headline metric (W4A16 decode against the HBM roofline; FP8 and W4A16 prefill
    against the tensor-pipe peak), each kernel timed alone (CUDA events around a CUDA graph of
    back-to-back launches that rotate through distinct weights, so no launch finds its weights in L2):
    W4A16 decode as a fraction of the measured HBM peak, FP8 and W4A16 prefill GEMMs in TFLOP/s."""
    import torch
    import bench_cases as run_case
    hbm, hbm_src = measured_peak_hbm()
    bf16, bf16_src = measured_peak_bf16()
    out = {}

    def timed(name, M, N, K, rotate, burst):
        inputs, fn, flops, nbytes = run_case.gemm_case(name, M, N, K, rotate, dev)
        torch.cuda.synchronize()
        for i in range(min(3, len(inputs))):
            fn(inputs[i])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        keep = []
        with torch.cuda.graph(graph):
            for b in range(burst):
                keep.append(fn(inputs[b % len(inputs)]))
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) / burst)
        ms = sorted(times)[len(times) // 2]
        del graph, keep, inputs
        torch.cuda.empty_cache()
        return ms, flops, nbytes

    # BASELINE config 2 (N = K = 4096, M in {1, 8, 16, 128, 2048}) plus the vocabulary- and MLP-sized decode shapes
    for (M, N, K) in ((1, 4096, 4096), (8, 4096, 4096), (16, 4096, 4096), (1, 128256, 4096), (8, 128256, 4096), (16, 128256, 4096),
                      (8, 14336, 4096)):
        rot = max(2, min(12, int(400e6 // (N * K / 2)) + 1))   # > 126 MB of distinct weights between reuses
        if N * K // 2 < (32 << 20):
            rot = 32                                           # small weights: 32 distinct sets (> 126 MB together)
        ms, _, nbytes = timed("gemv_w4", M, N, K, rot, rot)
        gbs = nbytes / ms / 1e6
        out[f"w4a16_decode_M{M}_N{N}_K{K}"] = {"ms": ms, "GBps": gbs, "frac_of_hbm_peak": gbs / hbm}
    for (M, N, K) in ((4096, 4096, 4096), (8192, 14336, 4096)):   # BASELINE config 4
        ms, flops, _ = timed("gemm_fp8", M, N, K, 3, 6)
        tf = flops / ms / 1e9
        out[f"fp8_gemm_{M}x{N}x{K}"] = {"ms": ms, "TFLOPps": tf, "frac_of_2x_bf16_peak": tf / (2 * bf16)}
    for (M, N, K) in ((128, 4096, 4096), (2048, 4096, 4096), (8192, 14336, 4096)):
        ms, flops, _ = timed("gemm_w4", M, N, K, 3, 6)
        tf = flops / ms / 1e9
        out[f"w4a16_prefill_{M}x{N}x{K}"] = {"ms": ms, "TFLOPps": tf, "frac_of_bf16_peak": tf / bf16}
    out["gptq_config5"] = gptq_config5(dev)
    out["peaks"] = {"hbm_GBps": hbm, "hbm_source": hbm_src, "bf16_TFLOPps": bf16, "bf16_source": bf16_src,
                    "fp8_note": "no measured FP8 peak exists; fractions are against 2 x the measured bf16 burst figure"}
    return out


def gptq_config5(dev):
    """BASELINE config 5 on one GPU: 128 x 2048 calibration tokens, bf16 N(0, 1) with a per-channel scale drawn
    log-uniformly from [0.1, 10]; Hessian (tensor cores, upper triangle), factor, column walk, each timed alone."""
    import torch
    from castforge_b200 import device as D
    out = {}
    T = 128 * 2048
    for name, N, K in (("gate_up_14336x4096", 14336, 4096), ("down_4096x14336", 4096, 14336)):
        g = torch.Generator(device=dev).manual_seed(K)
        ch = torch.exp((torch.rand(K, device=dev, generator=g) * 2 - 1) * 2.302585)
        x = torch.empty(T, K, dtype=torch.bfloat16, device=dev)
        for t0 in range(0, T, 16384):
            x[t0:t0 + 16384] = (torch.randn(16384, K, device=dev, generator=g) * ch).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)

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
        del x
        torch.cuda.empty_cache()
        u, ms_p = t3(lambda: D.gptq_prepare(h, 0.01))
        _, ms_q = t3(lambda: D.gptq_quantize(w, u, want_dequant=False))
        out[name] = {"tokens": T, "hessian_ms": ms_h, "hessian_TFLOPps_upper_triangle": T * K * K / ms_h / 1e9, "factor_ms": ms_p,
                     "quantize_ms": ms_q, "quantize_update_TFLOPps": N * K * K / ms_q / 1e9}
        del h, u, w
        torch.cuda.empty_cache()
    return out


def host_memory_available() -> float:
    """Bytes of host memory this process may still take: MemAvailable, capped by the cgroup limit where there is one."""
    avail = float("inf")
    try:
        for l in open("/proc/meminfo"):
            if l.startswith("MemAvailable:"):
                avail = float(l.split()[1]) * 1024
    except OSError:
        pass
    for lim, use in (("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory.current"),
                     ("/sys/fs/cgroup/memory/memory.limit_in_bytes", "/sys/fs/cgroup/memory/memory.usage_in_bytes")):
        try:
            l = open(lim).read().strip()
            if l != "max":
                avail = min(avail, float(l) - float(open(use).read().strip()))
        except (OSError, ValueError):
            pass
    return avail


def run_e2e(args, lib, dev, rank, world, mine):
    """Same metric through the reference-facing boundary with HOST buffers: a TensorStore of pinned
    bf16 host tensors goes through cfb200_store_run_pipeline("quantize(bits=8)") -- host -> device
    copies, both kernel passes and the copy of codes and scales back to host memory are all inside
    the timed region.  At one GPU the whole set is streamed (16 GB in, 8 GB out per step) when the host has the memory
    for it; with several ranks, or on a small host, four decoder layers per rank (the rate is PCIe-bound and does not
    depend on how many layers are streamed).  `copy_only` is the ceiling the figure is read against: the same host
    buffers copied to the device and the same number of result bytes copied back, on two streams, with no kernel."""
    import torch
    import torch.distributed as dist
    from castforge_b200 import TensorStore
    layers_req = args.e2e_layers
    if layers_req < 0:
        full_bytes = 3.2 * sum(r * c for _, r, c in mine) * 2   # inputs + results + staging, with margin
        layers_req = 32 if (world == 1 and host_memory_available() > full_bytes) else 4
    layers = [t for t in mine if ".layers." in t[0]]
    keep = {n for n, _, _ in layers[: 7 * layers_req]} if layers_req < 32 else None
    sub = sorted([t for t in mine if keep is None or t[0] in keep], key=lambda t: t[0])
    if not sub:
        sub = list(mine[:1])  # a rank whose share holds no decoder-layer tensor (short sets over many ranks) streams what it has
    n_sub = sum(r * c for _, r, c in sub)
    h_in = [torch.empty(r * c, dtype=torch.bfloat16).pin_memory() for _, r, c in sub]
    gcpu = torch.Generator().manual_seed(7 + rank)
    blk = (torch.randn(1 << 22, generator=gcpu) * 0.02).to(torch.bfloat16)
    for h in h_in:
        h.copy_(blk.repeat((h.numel() + blk.numel() - 1) // blk.numel())[: h.numel()])

    def one_pass():
        st = TensorStore()
        for (name, r, c), h in zip(sub, h_in):
            st.insert_pointer(name, h.data_ptr(), "BF16", (r, c))   # borrowed: no host copy
        tel = st.run_pipeline("quantize(bits=8)")                    # returns when codes + scales are in host memory
        assert tel[0]["ops_modified"] == len(sub)
        st.close()                                                   # result buffers go back to the pinned pool

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        for _ in range(2):
            fn()
        sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fn()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / args.steps
        if world > 1:
            tt = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt = float(tt.item())
        return dt

    dt = timed(one_pass)

    # copy-only ceiling: same inputs host -> device, as many result bytes device -> host, two streams, three device slots
    max_n = max(r * c for _, r, c in sub)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    d_in = [torch.empty(max_n, dtype=torch.bfloat16, device=dev) for _ in range(3)]
    d_out = [torch.zeros(max_n, dtype=torch.int8, device=dev) for _ in range(3)]
    h_out = [torch.empty(max_n, dtype=torch.int8).pin_memory() for _ in range(3)]

    def copy_pass():
        done = [None, None, None]
        for t, h in enumerate(h_in):
            sl, n = t % 3, h.numel()
            with torch.cuda.stream(s_in):
                if done[sl] is not None:
                    s_in.wait_event(done[sl])
                d_in[sl][:n].copy_(h, non_blocking=True)
                e = torch.cuda.Event()
                e.record(s_in)
            with torch.cuda.stream(s_out):
                s_out.wait_event(e)
                h_out[sl][:n].copy_(d_out[sl][:n], non_blocking=True)
                done[sl] = torch.cuda.Event()
                done[sl].record(s_out)
        s_in.synchronize()
        s_out.synchronize()

    dt_copy = timed(copy_pass)
    del d_in, d_out, h_out

    n_all = float(n_sub)
    if world > 1:
        tt = torch.tensor([n_all], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        n_all = float(tt.item())
    val = n_all * ALG_BYTES_PER_ELEM / dt / 1e9
    val_copy = n_all * ALG_BYTES_PER_ELEM / dt_copy / 1e9
    return {"value": val, "unit": UNIT, "h2d_bytes_per_step": int(2 * n_sub),
            "d2h_bytes_per_step": int(n_sub + 16 * len(sub)),
            "api": "cfb200_store_run_pipeline(store, \"quantize(bits=8)\") on pinned host tensors",
            "sample": f"{len(sub)} tensors ({n_sub} elements) per GPU streamed from pinned host memory per step", "ms_per_step": dt * 1e3,
            "copy_only_GBps": val_copy, "copy_only_ms_per_step": dt_copy * 1e3, "frac_of_copy_only": val / val_copy,
            "copy_only_note": "same host buffers copied in and as many result bytes copied out, two streams, no kernels: the host-link ceiling of this figure"}


if __name__ == "__main__":
    main()
