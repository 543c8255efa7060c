"""Torch-tensor front end of the multi-GPU entry points (communicators, sharded A1, column-parallel GEMMs,
token-parallel GPTQ Hessian).

Everything that computes or communicates is in libcastforge_b200.so (NCCL opened by the library itself); torch supplies
device memory, streams and -- in `Comm.from_torch_distributed` -- a way to hand rank 0's 128-byte NCCL id to the other
ranks.  A host without torch.distributed passes the id some other way and calls `Comm(id, world, rank)`.
"""
from __future__ import annotations

import ctypes

import torch

from ._lib import check, load

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def unique_id() -> bytes:
    """A fresh NCCL id (cfb200_comm_unique_id): make it on one rank, give the same bytes to all."""
    buf = ctypes.create_string_buffer(128)
    check(load().cfb200_comm_unique_id(buf))
    return buf.raw


class Comm:
    """One rank's communicator on the current CUDA device (cfb200_comm_init)."""

    def __init__(self, nccl_id: bytes, world: int, rank: int):
        if len(nccl_id) != 128:
            raise ValueError("an NCCL id is 128 bytes")
        h = ctypes.c_void_p()
        check(load().cfb200_comm_init(nccl_id, world, rank, ctypes.byref(h)))
        self.handle, self.world, self.rank = h, world, rank

    @classmethod
    def from_torch_distributed(cls, group=None) -> "Comm":
        """Rank 0 of `group` makes the id, a broadcast of 128 bytes hands it round (any backend)."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        backend = dist.get_backend(group)
        dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
        t = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            t.copy_(torch.frombuffer(bytearray(unique_id()), dtype=torch.uint8))
        dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(bytes(t.cpu().numpy().tobytes()), world, rank)

    @classmethod
    def single(cls) -> "Comm":
        """A one-rank communicator: every sharded entry point then behaves like its one-GPU form."""
        return cls(unique_id(), 1, 0)

    def close(self):
        if self.handle:
            load().cfb200_comm_free(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def shard_assign(nbytes, world: int, split_min_bytes: int = 0) -> list[int]:
    """cfb200_shard_assign: owner rank per tensor, -1 = cut into row blocks over all ranks."""
    cnt = len(nbytes)
    arr = (ctypes.c_size_t * cnt)(*[int(b) for b in nbytes])
    owner = (ctypes.c_int32 * cnt)()
    check(load().cfb200_shard_assign(cnt, arr, world, split_min_bytes, owner))
    return list(owner)


def shard_row_range(rows: int, world: int, rank: int, align: int = 1) -> tuple[int, int]:
    lo, hi = ctypes.c_size_t(0), ctypes.c_size_t(0)
    check(load().cfb200_shard_row_range(rows, world, rank, align, ctypes.byref(lo), ctypes.byref(hi)))
    return lo.value, hi.value


def quant_sym_tensors_sharded(comm: Comm, ws: list[torch.Tensor], is_row_block: list[bool], bits: int = 8):
    """A1 over this rank's tensors; entries flagged in is_row_block are this rank's rows of a tensor split over all
    ranks.  Returns (codes list, scale_absmax f32[len, 2])."""
    if not ws:
        return [], None
    ws = [w.contiguous() for w in ws]
    dev, dt = ws[0].device, _DT[ws[0].dtype]
    cnt = len(ws)
    with torch.cuda.device(dev):
        codes = [torch.empty(w.numel(), dtype=torch.int8, device=dev) for w in ws]
        sa = torch.zeros((cnt, 2), dtype=torch.float32, device=dev)
        srcs = (ctypes.c_void_p * cnt)(*[w.data_ptr() for w in ws])
        outs = (ctypes.c_void_p * cnt)(*[c.data_ptr() for c in codes])
        ns = (ctypes.c_size_t * cnt)(*[w.numel() for w in ws])
        flags = (ctypes.c_int32 * cnt)(*[1 if f else 0 for f in is_row_block])
        check(load().cfb200_quant_sym_tensors_sharded(comm.handle, cnt, srcs, dt, ns, flags, bits, outs, _p(sa), _stream(dev)))
    return codes, sa


def _colpar_ws(M, n_local, K, world, w4, dev):
    need = load().cfb200_gemm_colpar_workspace_bytes(M, n_local, K, world, 1 if w4 else 0)
    return torch.empty(need + 256, dtype=torch.uint8, device=dev), need


def _aligned(ws: torch.Tensor):
    off = (-ws.data_ptr()) % 256
    return ctypes.c_void_p(ws.data_ptr() + off)


def gemm_w4a16_colpar(comm: Comm, a: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, zps: torch.Tensor, n_local: int,
                      group: int = 128, layout: int = 0, check_flag: bool = True) -> torch.Tensor:
    """Column-parallel W4A16 product: this rank's [n_local, K] weight shard in, the whole bf16 product out
    ([M, world * n_local] for layout 0, [world, M, n_local] for layout 1)."""
    a = a.contiguous()
    M, K = a.shape
    dev = a.device
    with torch.cuda.device(dev):
        ws, need = _colpar_ws(M, n_local, K, comm.world, True, dev)
        shape = (M, comm.world * n_local) if layout == 0 else (comm.world, M, n_local)
        c = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        check(load().cfb200_gemm_w4a16_colpar(comm.handle, _p(a), _p(codes), _p(scales), _p(zps), M, n_local, K, group, _p(c), layout,
                                              _aligned(ws), need, _p(flag), _stream(dev)))
        if check_flag and int(flag.item()) != 0:  # reading the flag synchronises: timing loops pass check_flag=False
            raise RuntimeError("gemm_w4a16_colpar: a bounded wait ran out inside the kernel")
    return c


def gemm_fp8_colpar(comm: Comm, a_codes: torch.Tensor, a_scales, w_codes_local: torch.Tensor, w_scale: float, layout: int = 0,
                    check_flag: bool = True) -> torch.Tensor:
    """Column-parallel FP8 product (per-token x per-tensor scales): [n_local, K] weight shard in, whole bf16 product out."""
    a_codes = a_codes.contiguous()
    M, K = a_codes.shape
    n_local = w_codes_local.shape[0]
    dev = a_codes.device
    with torch.cuda.device(dev):
        ws, need = _colpar_ws(M, n_local, K, comm.world, False, dev)
        shape = (M, comm.world * n_local) if layout == 0 else (comm.world, M, n_local)
        c = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        check(load().cfb200_gemm_fp8_colpar(comm.handle, _p(a_codes), _p(a_scales), _p(w_codes_local), float(w_scale), M, n_local, K,
                                            _p(c), layout, _aligned(ws), need, _p(flag), _stream(dev)))
        if check_flag and int(flag.item()) != 0:
            raise RuntimeError("gemm_fp8_colpar: a bounded wait ran out inside the kernel")
    return c


def gptq_hessian_sharded(comm: Comm, x_local: torch.Tensor, t_total: int) -> torch.Tensor:
    """H = X^T X / t_total summed over the ranks' token shards (x_local: [T_local, K] bf16)."""
    x_local = x_local.contiguous()
    T, K = x_local.shape
    dev = x_local.device
    lib = load()
    with torch.cuda.device(dev):
        h = torch.empty((K, K), dtype=torch.float32, device=dev)
        need = lib.cfb200_gptq_hessian_workspace_bytes(max(T, 8), K)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        check(lib.cfb200_gptq_hessian_sharded(comm.handle, _p(x_local), T, t_total, K, _p(h), _p(ws), need, _p(flag), _stream(dev)))
        if int(flag.item()) != 0:
            raise RuntimeError("gptq_hessian_sharded: a bounded wait ran out inside the kernel")
    return h
