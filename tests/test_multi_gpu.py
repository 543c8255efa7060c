"""Multi-GPU rows of the path: placement arithmetic (CPU), the sharded entry points with a one-rank communicator
(one GPU) and with one process per GPU (two or more GPUs; skipped on a single-GPU machine).

What is compared with what:
  * cfb200_shard_assign / cfb200_shard_row_range against the Python statement of the same rules (castforge_b200.sharding);
  * column-parallel W4A16 / FP8 GEMM + all-gather: every rank's column block == the one-GPU kernel on that shard,
    and == the one-GPU product of the whole weight where the kernel schedule does not depend on N (tests/multi_gpu_worker.py);
  * A1 over a store dealt across ranks, two tensors cut into row blocks: codes and scales == the one-GPU list call;
  * GPTQ: a rank's output rows with the replicated factor == the same rows of the one-GPU run; the token-parallel
    Hessian agrees with the one-GPU Hessian to 1e-3 of its RMS (another summation order; the largest entries are ~100 x the RMS).
"""
import os
import random
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_shard_assign_matches_python_rule():
    from castforge_b200 import multi_gpu as mg, sharding
    rnd = random.Random(0)
    for trial in range(40):
        cnt = rnd.randint(0, 40)
        sizes = [rnd.choice([8 << 20, 32 << 20, 117 << 20, 1 << 30, rnd.randint(1, 1 << 26)]) for _ in range(cnt)]
        for world in (1, 2, 3, 8):
            assert mg.shard_assign(sizes, world, 0) == sharding.assign_tensors(sizes, world)
            split = 512 << 20
            assert mg.shard_assign(sizes, world, split) == sharding.assign_tensors(sizes, world, split_min_bytes=split)


def test_shard_assign_balances_the_8b_set():
    """Llama-3-8B-shaped bf16 set over 8 ranks with the two vocabulary tensors cut into row blocks: no rank holds more
    than 1/8 + 5 % of the bytes."""
    from castforge_b200 import multi_gpu as mg
    sizes = []
    for _ in range(32):
        sizes += [4096 * 4096 * 2, 1024 * 4096 * 2, 1024 * 4096 * 2, 4096 * 4096 * 2, 14336 * 4096 * 2, 14336 * 4096 * 2, 4096 * 14336 * 2]
    sizes += [128256 * 4096 * 2] * 2
    for world in (2, 4, 8):
        owner = mg.shard_assign(sizes, world, 512 << 20)
        assert owner[-1] == -1 and owner[-2] == -1
        load = [0.0] * world
        for o, b in zip(owner, sizes):
            if o == -1:
                for r in range(world):
                    lo, hi = mg.shard_row_range(128256, world, r, 1)
                    load[r] += (hi - lo) * 4096 * 2
            else:
                load[o] += b
        assert abs(sum(load) - sum(sizes)) < 1
        assert max(load) <= sum(sizes) * (1.0 / world + 0.05)


def test_shard_row_range_matches_python_rule():
    from castforge_b200 import multi_gpu as mg, sharding
    for rows in (0, 1, 7, 128, 4096, 128256, 5001):
        for world in (1, 2, 3, 8):
            for align in (1, 2, 128, 16384):
                got = [mg.shard_row_range(rows, world, r, align) for r in range(world)]
                assert got == [sharding.row_range(rows, world, r, align) for r in range(world)]
                assert got[0][0] == 0 and got[-1][1] == rows and all(a[1] == b[0] for a, b in zip(got, got[1:]))


def test_sharded_calls_reject_a_null_communicator():
    import ctypes
    import castforge_b200
    lib = castforge_b200.load()
    assert lib.cfb200_quant_sym_tensors_sharded(None, 1, None, 2, None, None, 8, None, None, None) == 1
    assert lib.cfb200_gemm_fp8_colpar(None, None, None, None, ctypes.c_float(1.0), 1, 8, 16, None, 0, None, 0, None, None) == 1
    assert b"communicator" in lib.cfb200_last_error()


def _run_ranks(world: int):
    env = dict(os.environ)
    env.update({"NCCL_NVLS_ENABLE": "0", "OMP_NUM_THREADS": "4"})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29400 + world), str(ROOT / "tests" / "multi_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    assert r.stdout.count("multi-gpu parity ok") == world, r.stdout[-3000:]


@pytest.mark.gpu
def test_sharded_entry_points_with_one_rank(cuda_device):
    """The whole multi-GPU code path (communicator, NCCL all-gather / all-reduce of one rank, interleave) on one GPU."""
    _run_ranks(1)


@pytest.mark.gpu
def test_sharded_entry_points_with_two_ranks(cuda_device):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run_ranks(2)


@pytest.mark.gpu
def test_sharded_entry_points_with_four_ranks(cuda_device):
    import torch
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    _run_ranks(4)
