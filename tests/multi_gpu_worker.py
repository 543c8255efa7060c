"""One rank of the multi-GPU parity checks (launched by tests/test_multi_gpu.py through torch.distributed.run, one
process per GPU).  Every rank builds the same seeded inputs, computes the one-GPU answer on its own device and compares
its share of the sharded answer with it.  torch.distributed (gloo) only carries the 128-byte NCCL id and the final
barrier; all communication under test is the library's own NCCL calls.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def rel_err(got, ref):
    ref = ref.double()
    return float((got.double() - ref).abs().max() / ref.pow(2).mean().sqrt())


def shard_w4(codes, scales, zps, N, K, lo, hi, group=128):
    ng = K // group
    assert (lo * ng) % 2 == 0 and (hi * ng) % 2 == 0
    return (codes[lo * K // 2: hi * K // 2].contiguous(), scales[lo * ng: hi * ng].contiguous(),
            zps[lo * ng // 2: hi * ng // 2].contiguous())


def check_colpar(comm, dev, rank, world):
    """Both ways of rejoining the blocks: ncclAllGather + interleave (knob 0) and the peer-load kernel over the ranks'
    IPC-mapped exchange buffers (knob -1: for every size; the default takes it from 8 MB of product)."""
    import castforge_b200
    lib = castforge_b200.load()
    try:
        for knob in (0, -1):
            assert lib.cfb200_tune(b"colpar_p2p", knob) == 0
            check_colpar_once(comm, dev, rank, world)
            check_colpar_once(comm, dev, rank, world)      # again: the exchange buffer's other half
    finally:
        lib.cfb200_tune(b"colpar_p2p", 1)
    return True


def check_colpar_once(comm, dev, rank, world):
    import castforge_b200
    from castforge_b200 import device as cf, multi_gpu as mg
    lib = castforge_b200.load()
    g = torch.Generator(device=dev).manual_seed(11)
    N, K = 1024 * world, 1024
    w = torch.randn(N, K, device=dev, generator=g) * 0.02
    w.view(-1)[torch.randint(0, N * K, (N * K // 1000,), device=dev, generator=g)] *= 20
    codes, scales, zps = cf.quant_int4_asym(w.reshape(-1), 128)
    nl = N // world
    lo, hi = rank * nl, (rank + 1) * nl
    c_l, s_l, z_l = shard_w4(codes, scales, zps, N, K, lo, hi)
    for M in (1, 8, 16, 384):
        a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        got = mg.gemm_w4a16_colpar(comm, a, c_l, s_l, z_l, nl, 128, layout=0)
        assert got.shape == (M, N)
        # (a) every rank's block equals the one-GPU kernel run on that shard alone, bit for bit
        for r in range(world):
            cr, sr, zr = shard_w4(codes, scales, zps, N, K, r * nl, (r + 1) * nl)
            one = cf.gemv_w4a16(a, cr, sr, zr, nl, 128, out_f32=False) if M <= 16 else cf.gemm_w4a16(a, cr, sr, zr, nl, 128, out_f32=False)
            assert torch.equal(got[:, r * nl:(r + 1) * nl], one), f"W4A16 colpar block {r} differs at M={M}"
        # (b) and the one-GPU product of the whole weight: identical when the kernel schedule is the same (M > 256: no
        # split-K), within the GEMM tolerance of 1e-2 x RMS otherwise (decode kernels pick their K split by shape)
        full = cf.gemv_w4a16(a, codes, scales, zps, N, 128, out_f32=False) if M <= 16 else cf.gemm_w4a16(a, codes, scales, zps, N, 128, out_f32=False)
        if M > 256:
            assert torch.equal(got, full), f"W4A16 colpar differs from the one-GPU product at M={M}"
        else:
            assert rel_err(got.float(), full.float()) < 1e-2
        lay1 = mg.gemm_w4a16_colpar(comm, a, c_l, s_l, z_l, nl, 128, layout=1)
        assert torch.equal(lay1.permute(1, 0, 2).reshape(M, N), got)
    # FP8: per-token x per-tensor scales
    M = 256
    x = torch.randn(M, K, device=dev, generator=g)
    x[:, ::100] *= 50
    ac, asc = cf.cast_e4m3_rows(x.to(torch.bfloat16))
    wc, wsa = cf.cast_e4m3_tensor(w.to(torch.bfloat16))
    wc = wc.reshape(N, K)
    full = cf.gemm_fp8(ac, asc, wc, float(wsa[0]), out_f32=False)
    got = mg.gemm_fp8_colpar(comm, ac, asc, wc[lo:hi].contiguous(), float(wsa[0]), layout=0)
    assert torch.equal(got, full), "FP8 colpar differs from the one-GPU product"
    return True


def check_quant_sharded(comm, dev, rank, world):
    from castforge_b200 import device as cf, multi_gpu as mg
    g = torch.Generator(device=dev).manual_seed(5)
    shapes = [(512, 1024), (3000, 1024), (64, 64), (4096, 1024), (7, 33), (1024, 1024), (5001, 512)]
    ws = [(torch.randn(r, c, device=dev, generator=g) * 0.02).to(torch.bfloat16) for r, c in shapes]
    ws[3][17, 5] = 3.0          # the absmax of the split tensors sits in ONE rank's rows
    ws[6][5000, 1] = -7.0
    nbytes = [w.numel() * 2 for w in ws]
    owner = mg.shard_assign(nbytes, world, split_min_bytes=4096 * 1024 * 2 if world > 1 else 0)
    if world > 1:
        owner[6] = -1           # a second split tensor with a row count that does not divide evenly
    ref_codes, ref_sa = cf.quant_sym_tensors(ws, 8)
    mine, flags, idx = [], [], []
    for i, w in enumerate(ws):
        if owner[i] == -1:
            lo, hi = mg.shard_row_range(w.shape[0], world, rank, 1)
            mine.append(w[lo:hi].contiguous()); flags.append(True); idx.append((i, lo, hi))
        elif owner[i] == rank:
            mine.append(w); flags.append(False); idx.append((i, 0, w.shape[0]))
    codes, sa = mg.quant_sym_tensors_sharded(comm, mine, flags, 8)
    torch.cuda.synchronize()
    for (i, lo, hi), c, s in zip(idx, codes, sa):
        cols = ws[i].shape[1]
        assert torch.equal(c, ref_codes[i][lo * cols: hi * cols]), f"codes of tensor {i} rows {lo}:{hi} differ"
        assert float(s[0]) == float(ref_sa[i, 0]) and float(s[1]) == float(ref_sa[i, 1]), f"scale of tensor {i} differs"
    return True


def check_gptq(comm, dev, rank, world):
    from castforge_b200 import device as cf, multi_gpu as mg
    g = torch.Generator(device=dev).manual_seed(3)
    N, K, T = 256, 512, 2048
    w = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    ch = torch.exp(torch.rand(K, device=dev, generator=g) * 4.6 - 2.3)
    x = (torch.randn(T, K, device=dev, generator=g) * ch).to(torch.bfloat16)
    h = cf.gptq_hessian(x)
    u = cf.gptq_prepare(h, 0.01)
    codes, scales, zps, _ = cf.gptq_quantize(w, u, True)
    lo, hi = mg.shard_row_range(N, world, rank, 2)     # two rows per unit keeps the packed zero points byte aligned
    c_l, s_l, z_l, _ = cf.gptq_quantize(w[lo:hi].contiguous(), u, True)
    ng = K // 128
    assert torch.equal(c_l, codes[lo * K // 2: hi * K // 2]), "GPTQ codes of the row shard differ"
    assert torch.equal(s_l.view(torch.int16), scales.view(torch.int16)[lo * ng: hi * ng]) and torch.equal(z_l, zps[lo * ng // 2: hi * ng // 2])
    # token-parallel Hessian: the sum over ranks adds in another order, so equality is to rounding.  The error is
    # measured against the RMS of H while the largest entries (diagonal, channel scale up to 10) are ~100 x the RMS,
    # and the tensor cores' f32 accumulation is good to ~1e-5 of the VALUE: bound 1e-3 of the RMS.
    tl0, tl1 = mg.shard_row_range(T, world, rank, 8)
    h2 = mg.gptq_hessian_sharded(comm, x[tl0:tl1].contiguous(), T)
    torch.cuda.synchronize()
    assert rel_err(h2, h) < 1e-3, rel_err(h2, h)
    return True


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("gloo")
    from castforge_b200 import multi_gpu as mg
    comm = mg.Comm.from_torch_distributed()
    try:
        check_quant_sharded(comm, dev, rank, world)
        check_colpar(comm, dev, rank, world)
        check_gptq(comm, dev, rank, world)
        torch.cuda.synchronize()
        dist.barrier()
        print(f"multi-gpu parity ok: rank {rank} of {world}", flush=True)
    finally:
        comm.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
