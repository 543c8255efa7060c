"""Spreading the quantize passes over the GPUs of one node, one process per GPU.

The passes shard without a data-path collective: every tensor of a TensorStore is quantized
independently (QuantizeWeightsPass::run, src/passes/quantize/schemes.rs:324-452, walks the weights one at a time), so
each rank takes a subset of the tensors.  The only exchange a split can need is one f32 per
tensor: when a single tensor is cut into row blocks for per-tensor symmetric quantization, the
scale comes from the absmax of the WHOLE tensor, so the ranks combine their partial absmax with a
MAX all-reduce before the apply pass.  Per-channel, per-group, NF4 and FP8-per-row units lie
inside a row, so row blocks of those need no exchange at all.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist


def assign_tensors(sizes: Sequence[int], world: int, split_min_bytes: int = 0) -> list[int]:
    """Owner rank of each tensor: largest first onto the least-loaded rank (ties -> lowest rank,
    equal sizes keep their order), computed identically on every rank, so nothing is exchanged.
    With split_min_bytes > 0 and more than one rank, a tensor of that many bytes or more is marked -1: it is cut into
    row blocks and every rank takes one (its bytes count 1/world towards every rank's load).  This is the rule of
    cfb200_shard_assign, restated for the tests."""
    if world < 1:
        raise ValueError("world must be >= 1")
    load = [0] * world
    owner = [0] * len(sizes)
    whole = []
    for i, b in enumerate(sizes):
        if world > 1 and split_min_bytes > 0 and int(b) >= split_min_bytes:
            owner[i] = -1
            for r in range(world):
                load[r] += int(b) // world
        else:
            whole.append(i)
    order = sorted(whole, key=lambda i: (-int(sizes[i]), i))
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += int(sizes[i])
    return owner


def my_tensors(sizes: Sequence[int], world: int, rank: int) -> list[int]:
    """Indices of the tensors `rank` owns, in store order."""
    return [i for i, r in enumerate(assign_tensors(sizes, world)) if r == rank]


def row_range(rows: int, world: int, rank: int, align: int = 1) -> tuple[int, int]:
    """Contiguous row block [lo, hi) of `rank`: blocks differ by at most `align` rows, every row is
    owned exactly once, trailing ranks may be empty when rows < world * align."""
    if not (0 <= rank < world) or align < 1:
        raise ValueError("bad rank/world/align")
    units = -(-rows // align)
    base, extra = divmod(units, world)
    lo_u = rank * base + min(rank, extra)
    hi_u = lo_u + base + (1 if rank < extra else 0)
    return min(rows, lo_u * align), min(rows, hi_u * align)


def parse_cpulist(text: str) -> list[int]:
    """'0-3,8,10-11' -> [0, 1, 2, 3, 8, 10, 11] (the format of /sys/devices/system/node/nodeN/cpulist)."""
    cpus: list[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def numa_cpus_of_pci(bdf: str, sysfs: str = "/sys") -> list[int] | None:
    """CPUs of the NUMA node a PCI function (domain:bus:device.function) hangs off, or None when the node is unknown
    (single-node machine, virtualised PCI topology: numa_node reads -1 or the files are absent)."""
    try:
        node = int(open(f"{sysfs}/bus/pci/devices/{bdf.lower()}/numa_node").read())
        if node < 0:
            return None
        return parse_cpulist(open(f"{sysfs}/devices/system/node/node{node}/cpulist").read()) or None
    except (OSError, ValueError):
        return None


def bind_host_to_device_node(device_index: int, sysfs: str = "/sys") -> list[int] | None:
    """Pin this process to the CPUs of the NUMA node its GPU hangs off, so that the pinned staging buffers it allocates
    afterwards (first touch) and the reader threads it starts are local to that GPU's PCIe root.  With one process per
    GPU and no binding, the ranks' host buffers land on whichever socket the scheduler picked and the host -> device
    streams of the far socket's GPUs share the inter-socket link.  Returns the CPU list, or None when the node is
    unknown or the affinity call is refused -- nothing is changed then.  Only this process's own CPU affinity is
    touched."""
    import os
    try:
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        cpus = numa_cpus_of_pci(bdf, sysfs)
        if not cpus:
            return None
        allowed = sorted(set(cpus) & os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except (OSError, AttributeError, RuntimeError, AssertionError):
        return None


class _DeviceBackend:
    """The CUDA entry points; raises if the library or a GPU is missing."""

    def absmax(self, t: torch.Tensor) -> torch.Tensor:
        from . import device
        return device.absmax(t)

    def quant_sym_apply(self, t: torch.Tensor, absmax: torch.Tensor, bits: int):
        from . import device
        return device.quant_sym_apply(t, absmax, bits)


def quant_sym_row_sharded(block: torch.Tensor, bits: int = 8, group: dist.ProcessGroup | None = None, backend=None):
    """Per-tensor symmetric quantization of a tensor whose rows are spread over the ranks of
    `group`; `block` is this rank's row block (it may have zero rows).  Returns (codes, scale),
    bit-identical to quantizing the whole tensor on one GPU: the scale is a function of the absmax
    of the whole tensor (quantize_symmetric_f32, src/passes/quantize/formats.rs:664-677), and max is exact under any
    grouping.  One f32 crosses the ranks; the codes never do.
    """
    backend = backend or _DeviceBackend()
    if block.numel():
        amax = backend.absmax(block).reshape(1).to(torch.float32)
    else:
        amax = torch.zeros(1, dtype=torch.float32, device=block.device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    if block.numel():
        codes, scale_absmax = backend.quant_sym_apply(block, amax, bits)
        scale = float(scale_absmax[0].item())
    else:
        codes = torch.empty(0, dtype=torch.int8, device=block.device)
        qmax = 7.0 if bits == 4 else 127.0
        a = float(amax.item())
        scale = 1.0 if a < 1e-12 else float((amax / qmax).item())
    return codes, scale


def run_sharded(names: Sequence[str], sizes: Sequence[int], rank: int, world: int, fn: Callable[[str], object]) -> dict:
    """Calls fn(name) for the tensors this rank owns; returns {name: result}.  No communication."""
    return {names[i]: fn(names[i]) for i in my_tensors(sizes, world, rank)}
