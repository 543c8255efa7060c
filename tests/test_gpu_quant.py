"""GPU parity: every memory-bound quantization kernel against the CPU oracle, bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def f32(bits):
    return np.array(bits, dtype=np.uint32).view(np.float32)


def u32(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def weights(n, seed, dtype, outliers=True, scale=0.02):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, generator=g) * scale
    if outliers and n > 100:
        idx = torch.randint(0, n, (max(1, n // 1000),), generator=g)
        w[idx] *= 20
    return w.to(dtype)


def host_f32(t):
    return t.detach().float().cpu().numpy()


def bits_equal(got: torch.Tensor, want: np.ndarray):
    g = got.detach().cpu().numpy()
    if g.dtype == np.float32:
        return np.array_equal(g.view(np.uint32).ravel(), np.ascontiguousarray(want, np.float32).view(np.uint32).ravel())
    return np.array_equal(g.ravel(), np.asarray(want).ravel())


# ------------------------------------------------------------------------------------------- A1
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("n", [1, 7, 8, 1000, 4099, 1 << 20, (1 << 20) + 13])
def test_a1_bit_exact(cuda_device, oracle, dtype, bits, n):
    from castforge_b200 import device as cf
    w = weights(n, n + bits, DT[dtype]).to(cuda_device)
    codes, sa = cf.quant_sym_tensor(w, bits)
    q, s, _ = oracle.quant_sym(host_f32(w), bits, threads=0)
    assert bits_equal(sa[:1], np.array([s], np.float32))
    assert bits_equal(codes, q)


def test_a1_golden_fixtures(cuda_device, golden):
    from castforge_b200 import device as cf
    for case in ("a1_2x2", "a1_ramp_b8", "a1_ramp_b4", "a1_tiny"):
        g = golden[case]
        w = torch.from_numpy(f32(g["w_bits"]).copy()).to(cuda_device)
        codes, sa = cf.quant_sym_tensor(w, g["bits"])
        assert codes.cpu().tolist() == g["codes"], case
        assert int(sa[:1].cpu().numpy().view(np.uint32)[0]) == g["scale_bits"], case


def test_a1_special_values(cuda_device, oracle):
    from castforge_b200 import device as cf
    base = weights(5000, 5, torch.float32)
    cases = {
        "nan": base.clone().index_fill_(0, torch.tensor([3, 777]), float("nan")),
        "inf": base.clone().index_fill_(0, torch.tensor([10]), float("inf")),
        "neg_inf_nan": base.clone().index_fill_(0, torch.tensor([10]), float("-inf")).index_fill_(0, torch.tensor([11]), float("nan")),
        "zeros": torch.zeros(4096),
        "tiny": torch.full((4096,), 1e-13),
        "denorm": torch.full((4096,), 1e-40),
        "ties": (torch.arange(-254, 255, dtype=torch.float32) * 0.5),   # quotients on exact .5 ties
        "huge": base * 1e36,
    }
    for name, w in cases.items():
        for bits in (8, 4):
            codes, sa = cf.quant_sym_tensor(w.to(cuda_device), bits)
            q, s, _ = oracle.quant_sym(w.numpy(), bits)
            assert bits_equal(sa[:1], np.array([s], np.float32)), (name, bits)
            assert bits_equal(codes, q), (name, bits)


def test_a1_every_bf16_pattern(cuda_device, oracle):
    """All 65536 bf16 bit patterns (incl. NaN payloads, infinities, subnormals) in one tensor, and
    the finite ones alone (so that the scale is finite)."""
    from castforge_b200 import device as cf
    pats = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    w_all = pats.view(torch.bfloat16)
    finite = w_all[torch.isfinite(w_all.float())]
    small = finite[finite.float().abs() < 3.0]
    for w in (w_all, finite, small):
        wd = w.contiguous().to(cuda_device)
        codes, sa = cf.quant_sym_tensor(wd, 8)
        q, s, _ = oracle.quant_sym(host_f32(w), 8)
        assert bits_equal(sa[:1], np.array([s], np.float32))
        assert bits_equal(codes, q)


def test_a1_back_to_back_calls_share_nothing(cuda_device, oracle):
    from castforge_b200 import device as cf
    a = weights(100_000, 1, torch.bfloat16).to(cuda_device)
    b = (weights(50_000, 2, torch.bfloat16) * 0.1).to(cuda_device)
    ca, sa = cf.quant_sym_tensor(a, 8)
    cb, sb = cf.quant_sym_tensor(b, 8)
    ca2, sa2 = cf.quant_sym_tensor(a, 8)
    assert torch.equal(ca, ca2) and torch.equal(sa, sa2)
    assert sb[1] < sa[1]


@pytest.fixture(params=[0, 1, 2])
def a1_merge_mode(request):
    """Every scheduling variant of the A1 stage kernel must give the same bits."""
    import castforge_b200
    lib = castforge_b200.load()
    assert lib.cfb200_tune(b"a1_persist", 0) == 0  # the launch-per-stage path (the persistent one is the default)
    assert lib.cfb200_tune(b"a1_merge", request.param) == 0
    yield request.param
    assert lib.cfb200_tune(b"a1_merge", 0) == 0
    assert lib.cfb200_tune(b"a1_persist", 1) == 0


@pytest.mark.parametrize("dtype", ["bf16", "f32", "f16"])
@pytest.mark.parametrize("group_bytes", [0, 1, 1 << 30])
def test_a1_tensor_list_matches_single_calls(cuda_device, oracle, dtype, group_bytes, a1_merge_mode):
    """The pipelined multi-tensor entry point: ragged sizes, empty tensors, more tensors than one
    launch takes, every grouping -- codes and scales identical to the oracle."""
    from castforge_b200 import device as cf
    sizes = [1000, 0, 4096 * 64, 7, 123457, 8, 1 << 20, 33, 5000, 77777, 1, 4096, 999999, 64, 2, 31]
    ws = [weights(max(n, 1), 100 + i, DT[dtype])[:n].contiguous().to(cuda_device) * (1 + i) for i, n in enumerate(sizes)]
    codes, sa, events = cf.quant_sym_tensors(ws, 8, group_bytes, time_stages=True)
    torch.cuda.synchronize()
    assert all(events[i].elapsed_time(events[i + 1]) >= 0 for i in range(len(events) - 1))
    for i, w in enumerate(ws):
        q, s, _ = oracle.quant_sym(host_f32(w), 8)
        assert bits_equal(sa[i, :1], np.array([s], np.float32)), i
        assert bits_equal(codes[i], q), i


@pytest.fixture
def a1_persist():
    """The list entry point as one cooperative launch (tensor heads kept in shared memory)."""
    import castforge_b200
    lib = castforge_b200.load()
    assert lib.cfb200_tune(b"a1_persist", 2) == 0  # 2 = every dtype (the default, 1, sends f32 sources the other way)
    yield
    assert lib.cfb200_tune(b"a1_persist", 1) == 0  # the default


@pytest.mark.parametrize("dtype", ["bf16", "f32", "f16"])
@pytest.mark.parametrize("group_bytes", [0, 1, 1 << 30])
def test_a1_persistent_list_matches_oracle(cuda_device, oracle, dtype, group_bytes, a1_persist):
    """group_bytes = 1 makes every tensor a group of its own that keeps its head on chip, including
    empty tensors and tensors shorter than one vector."""
    from castforge_b200 import device as cf
    sizes = [1000, 0, 4096 * 64, 7, 123457, 8, 1 << 20, 33, 5000, 77777, 1, 4096, 999999, 64, 2, 31, 3_000_001]
    ws = [weights(max(n, 1), 100 + i, DT[dtype])[:n].contiguous().to(cuda_device) * (1 + i) for i, n in enumerate(sizes)]
    codes, sa, events = cf.quant_sym_tensors(ws, 8, group_bytes, time_stages=True)
    torch.cuda.synchronize()
    assert len(events) == 2 and events[0].elapsed_time(events[1]) > 0
    for i, w in enumerate(ws):
        q, s, _ = oracle.quant_sym(host_f32(w), 8)
        assert bits_equal(sa[i, :1], np.array([s], np.float32)), i
        assert bits_equal(codes[i], q), i


@pytest.mark.parametrize("dtype", ["bf16", "f32", "f16"])
def test_a1_persistent_nan_and_inf(cuda_device, oracle, dtype, a1_persist):
    """Tensors holding NaN (dropped by the absmax, code 0) or infinities (absmax = inf) take the guarded
    path; their finite neighbours in the same call take the unguarded one."""
    from castforge_b200 import device as cf
    n = 700_001
    clean = weights(n, 1, DT[dtype])
    with_nan = weights(n, 2, DT[dtype]).clone()
    with_nan[[3, 65_536, n - 1]] = float("nan")
    with_inf = weights(n, 3, DT[dtype]).clone()
    with_inf[12_345] = float("inf")
    with_inf[n - 2] = float("-inf")
    tail_nan = weights(n, 4, DT[dtype]).clone()
    tail_nan[n - 1] = float("nan")  # in the elements past the last whole vector
    ws = [t.to(cuda_device) for t in (clean, with_nan, with_inf, tail_nan, clean * 3)]
    for group_bytes in (0, 1):
        codes, sa = cf.quant_sym_tensors(ws, 8, group_bytes)
        torch.cuda.synchronize()
        for i, w in enumerate(ws):
            q, s, _ = oracle.quant_sym(host_f32(w), 8)
            assert bits_equal(sa[i, :1], np.array([s], np.float32)), i
            assert bits_equal(codes[i], q), i


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_a1_persistent_large_tensor_head_and_tail(cuda_device, oracle, dtype, a1_persist):
    """A tensor larger than the L2 budget: head from shared memory, the rest re-read back to front;
    more tensors than one descriptor table takes."""
    from castforge_b200 import device as cf
    n = 40_000_003 if dtype == "bf16" else 20_000_003
    big = weights(n, 7, DT[dtype]).to(cuda_device)
    small = [weights(300 + i, 1000 + i, DT[dtype]).to(cuda_device) for i in range(1100)]
    ws = small[:5] + [big] + small[5:]
    codes, sa = cf.quant_sym_tensors(ws, 8)
    torch.cuda.synchronize()
    for i in (0, 5, 6, 700, 1100):
        q, s, _ = oracle.quant_sym(host_f32(ws[i]), 8, threads=0)
        assert bits_equal(sa[i, :1], np.array([s], np.float32)), i
        assert bits_equal(codes[i], q), i
    ref_codes, ref_sa = cf.quant_sym_tensor(big, 8)
    assert torch.equal(ref_codes, codes[5]) and torch.equal(ref_sa, sa[5])


def test_a1_apply_with_foreign_absmax_clamps(cuda_device, oracle):
    """Row-block sharding: pass 2 with an absmax that is not this shard's own (larger: the global
    one; smaller: a caller's mistake) must still clamp like the reference."""
    import ctypes
    import castforge_b200
    from castforge_b200._lib import check
    lib = castforge_b200.load()
    w = weights(50_000, 3, torch.bfloat16).to(cuda_device)
    for factor in (4.0, 0.05):
        am = torch.tensor([float(w.float().abs().max()) * factor], dtype=torch.float32, device=cuda_device)
        codes = torch.empty(w.numel(), dtype=torch.int8, device=cuda_device)
        sa = torch.empty(2, dtype=torch.float32, device=cuda_device)
        check(lib.cfb200_quant_sym_apply(ctypes.c_void_p(w.data_ptr()), 2, w.numel(), 8, ctypes.c_void_p(am.data_ptr()),
                                         ctypes.c_void_p(codes.data_ptr()), ctypes.c_void_p(sa.data_ptr()), None))
        scale = np.float32(am.cpu().numpy()[0]) / np.float32(127)
        x = (host_f32(w) / scale).astype(np.float32)          # IEEE f32 division
        t = np.trunc(x)
        want = np.clip(t + (np.abs(x - t) >= np.float32(0.5)) * np.sign(x), -128, 127).astype(np.int8)
        assert np.array_equal(codes.cpu().numpy(), want), factor
        assert bits_equal(sa[:1], np.array([scale], np.float32))


# ------------------------------------------------------------------------------------------- A6
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("n", [5, 4096, 100_003])
def test_a6_fakequant_tensor(cuda_device, oracle, bits, n):
    from castforge_b200 import device as cf
    w = weights(n, 11 + n, torch.float32).to(cuda_device)
    out, sa = cf.fakequant_tensor(w, bits)
    want, s = oracle.fakequant_tensor(host_f32(w), bits)
    assert bits_equal(sa[:1], np.array([s], np.float32))
    assert bits_equal(out, want)  # includes the sign of zero


@pytest.mark.parametrize("alpha", [0.5, 0.05, 0.99])
def test_a6_smoothquant(cuda_device, oracle, alpha):
    from castforge_b200 import device as cf
    w = weights(70_001, 12, torch.float32).to(cuda_device)
    want, params = oracle.smoothquant(host_f32(w), 8, alpha)
    # the two scalars need powf and stay on the host (here taken from the oracle's host math)
    got = cf.smoothquant_apply(w, 8, float(params[0]), float(params[1]))
    assert bits_equal(got, want)
    assert float(cf.absmax(w).cpu()) == float(np.abs(host_f32(w)).max())


# ------------------------------------------------------------------------------------------- E1
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(3, 5), (64, 4096), (17, 1000), (5, 9000), (300, 14336), (2, 40000)])
def test_e1_per_channel(cuda_device, oracle, dtype, shape):
    from castforge_b200 import device as cf
    rows, cols = shape
    w = weights(rows * cols, rows, DT[dtype]).reshape(rows, cols).to(cuda_device)
    codes, scales = cf.quant_per_channel(w, 8)
    q, s = oracle.quant_per_channel(host_f32(w), rows, cols, 8, threads=0)
    assert bits_equal(scales, s)
    assert bits_equal(codes, q)


# ------------------------------------------------------------------------------------------- A2
@pytest.mark.parametrize("n", [4, 1000, 1 << 18, (1 << 18) + 5])
@pytest.mark.parametrize("ratio", [0.01, 0.25, 0.5, 1e-9])
def test_a2_select_kth(cuda_device, oracle, n, ratio):
    from castforge_b200 import device as cf
    w = weights(n, n, torch.float32)
    if n > 10:
        w[3] = float("nan")
    thr, k = cf.select_kth_abs(w.to(cuda_device), ratio)
    want_thr, want_k = oracle.salient_threshold(w.numpy(), ratio)
    assert k == want_k
    assert bits_equal(thr, np.array([want_thr], np.float32))


@pytest.mark.parametrize("kind", ["gauss", "outliers", "ties", "two_values", "nan_inf", "sorted", "tiny_range"])
@pytest.mark.parametrize("ratio", [0.001, 0.01, 0.05, 0.2])
def test_a2_select_single_pass_path_is_exact(cuda_device, kind, ratio):
    """Tensors large enough for the single-pass path (sample, bracket, one full pass, exact rank among the candidates;
    ranks in the top 5 %) on distributions chosen to break a bracket: heavy ties, two distinct values, NaN / inf,
    values sorted in memory, a range a sample cannot resolve.  The result must equal the k-th largest |v| under the
    total order (torch.sort of the bit patterns) exactly, whichever path ran, and equal the three-pass path."""
    from castforge_b200 import device as cf
    n = (1 << 22) + 12345
    g = torch.Generator(device=cuda_device).manual_seed(hash(kind) % 1000 + int(ratio * 1000))
    w = torch.randn(n, device=cuda_device, generator=g) * 0.02
    if kind == "outliers":
        idx = torch.randint(0, n, (n // 500,), device=cuda_device, generator=g)
        w[idx] *= 20
    elif kind == "ties":
        w = torch.round(w * 400) / 400                      # a few dozen distinct values
    elif kind == "two_values":
        w = torch.where(torch.rand(n, device=cuda_device, generator=g) < 0.03, torch.tensor(1.5, device=cuda_device), torch.tensor(-0.25, device=cuda_device))
    elif kind == "nan_inf":
        w[::1000] = float("nan")
        w[5::3000] = float("inf")
        w[7::3000] = float("-inf")
    elif kind == "sorted":
        w = torch.sort(w.abs()).values                      # the largest values all sit at the end of the buffer
    elif kind == "tiny_range":
        w = 1.0 + torch.rand(n, device=cuda_device, generator=g) * 1e-5   # every key shares its top 14 bits
    thr, k = cf.select_kth_abs(w, ratio, single_pass=True)
    thr3, k3 = cf.select_kth_abs(w, ratio, single_pass=False)
    keys = (w.view(torch.int32) & 0x7FFFFFFF)
    want = torch.sort(keys, descending=True).values[k - 1]
    assert k == k3
    assert int(thr.view(torch.int32).item()) == int(want.item()), (kind, ratio)
    assert int(thr3.view(torch.int32).item()) == int(want.item()), (kind, ratio)


@pytest.mark.parametrize("group", [2, 4, 32, 100, 128, 256])
@pytest.mark.parametrize("awq", [True, False])
def test_a2_groupwise(cuda_device, oracle, group, awq):
    from castforge_b200 import device as cf
    for n in (4, 1000, (1 << 18) + 77):
        w = weights(n, group + n, torch.float32).to(cuda_device)
        out, thr, k = cf.fakequant_group(w, 4, group, 0.01, awq)
        want, wthr, wk = oracle.fakequant_group(host_f32(w), 4, group, 0.01, awq, threads=0)
        if awq:
            assert k == wk and bits_equal(thr, np.array([wthr], np.float32))
        assert bits_equal(out, want), (group, awq, n)


def test_a2_golden(cuda_device, golden):
    from castforge_b200 import device as cf
    for case in ("a2_awq_2x2", "a2_ramp_awq1", "a2_ramp_awq0"):
        g = golden[case]
        w = torch.from_numpy(f32(g["w_bits"]).copy()).to(cuda_device)
        out, thr, k = cf.fakequant_group(w, g["bits"], g["group"], g["ratio"], bool(g["awq"]))
        assert out.cpu().numpy().view(np.uint32).tolist() == g["out_bits"], case
        if g["awq"]:
            assert k == g["k"]


# ------------------------------------------------------------------------------------------- A3
@pytest.mark.parametrize("block", [4, 32, 100, 128])
@pytest.mark.parametrize("fmt", [(False, True), (False, False), (True, True)])
def test_a3_fp8grid(cuda_device, oracle, block, fmt):
    from castforge_b200 import device as cf
    e5m2, mx = fmt
    n = (1 << 17) + 19
    w = weights(n, block, torch.float32)
    # block maxima straddling powers of two exercise ceil(log2f(.))
    fmax = 57344.0 if e5m2 else 448.0
    for i, e in enumerate(range(-20, 12)):
        base = np.float32(2.0 ** e) * np.float32(fmax)
        for j, v in enumerate((base, np.nextafter(base, np.float32(0)), np.nextafter(base, np.float32(1e30)),
                               np.float32(base * (1 + 3 * 2.0 ** -23)), np.float32(base * (1 + 100 * 2.0 ** -23)))):
            pos = (i * 5 + j) * max(block, 4) * 3
            if pos + max(block, 4) <= n:
                w[pos:pos + max(block, 4)] = 0
                w[pos] = float(v)
    wd = w.to(cuda_device)
    got = cf.fakequant_fp8grid(wd, block, e5m2, mx)
    want = oracle.fakequant_fp8grid(w.numpy(), block, e5m2, mx, threads=0)
    assert bits_equal(got, want)


def test_a3_a4_a5_golden(cuda_device, golden):
    from castforge_b200 import device as cf
    for case in ("a3_ramp_e5m20_mx1", "a3_ramp_e5m20_mx0", "a3_ramp_e5m21_mx1"):
        g = golden[case]
        w = torch.from_numpy(f32(g["w_bits"]).copy()).to(cuda_device)
        got = cf.fakequant_fp8grid(w, g["block"], bool(g["e5m2"]), bool(g["mxfp8"]))
        assert got.cpu().numpy().view(np.uint32).tolist() == g["out_bits"], case
    g = golden["a4_ramp_b16"]
    w = torch.from_numpy(f32(g["w_bits"]).copy()).to(cuda_device)
    assert cf.fakequant_e2m1(w, g["block"]).cpu().numpy().view(np.uint32).tolist() == g["out_bits"]
    for case in ("a5_8x6_b4", "a5_8x6_b5", "a5_6x4_b4"):
        g = golden[case]
        w = torch.from_numpy(f32(g["w_bits"]).copy()).reshape(g["K"], g["N"]).to(cuda_device)
        assert cf.fwht_cols_(w, g["block"]) == g["applied"]
        assert w.cpu().numpy().view(np.uint32).ravel().tolist() == g["out_bits"], case


# ------------------------------------------------------------------------------------------- A4
@pytest.mark.parametrize("block", [4, 16, 32, 24])
def test_a4_e2m1(cuda_device, oracle, block):
    from castforge_b200 import device as cf
    n = (1 << 17) + 3
    w = weights(n, 40 + block, torch.float32)
    w[5] = float("nan")
    w[100:100 + 8] = torch.tensor([6.0, 0.25, 0.75, 2.5, 5.0, -1.25, -0.0, 3.5])  # exact ties in one block
    got = cf.fakequant_e2m1(w.to(cuda_device), block)
    want = oracle.fakequant_e2m1(w.numpy(), block, threads=0)
    assert bits_equal(got, want)


# ------------------------------------------------------------------------------------------- A5
@pytest.mark.parametrize("shape_block", [((256, 96), 64), ((512, 33), 128), ((4096, 40), 4096), ((64, 64), 3), ((96, 8), 64),
                                         ((8, 100), 2), ((64, 70), 8), ((64, 31), 16), ((96, 65), 32), ((1024, 48), 256),
                                         ((1024, 33), 512), ((2048, 40), 1024), ((4096, 33), 2048)])
def test_a5_hadamard(cuda_device, oracle, shape_block):
    from castforge_b200 import device as cf
    (K, N), block = shape_block
    w = weights(K * N, K, torch.float32, scale=1.0).reshape(K, N)
    wd = w.clone().to(cuda_device)
    applied = cf.fwht_cols_(wd, block)
    want, b = oracle.fwht_cols(w.numpy(), K, N, block, threads=0)
    assert applied == b
    assert bits_equal(wd, want)


# ------------------------------------------------------------------------------------------- E2
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("n", [128, 300, 301, 1 << 18, (1 << 18) + 1, 4096 * 256])
def test_e2_int4_asym(cuda_device, oracle, dtype, group, n):
    from castforge_b200 import device as cf
    w = weights(n, n % 1000 + group, DT[dtype]).to(cuda_device)
    codes, scales, zps = cf.quant_int4_asym(w, group)
    c, s, z = oracle.quant_int4_asym(host_f32(w), group, threads=0)
    assert np.array_equal(scales.view(torch.int16).cpu().numpy().view(np.uint16), s)
    assert np.array_equal(zps.cpu().numpy(), z)
    assert np.array_equal(codes.cpu().numpy(), c)


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_e2_e3_source_aligned_to_16_bytes_only(cuda_device, oracle, dtype):
    """The entry points ask for a 16-byte aligned source; the kernels' 32-byte loads must not assume more."""
    from castforge_b200 import device as cf
    n = 1 << 18
    esz = 4 if dtype == "f32" else 2
    big = weights(n + 64, 7, DT[dtype]).to(cuda_device)
    w = big[16 // esz: 16 // esz + n]                       # starts 16 bytes into a 512-byte aligned allocation
    assert w.data_ptr() % 32 == 16 and w.is_contiguous()
    codes, scales, zps = cf.quant_int4_asym(w, 128)
    c, s, z = oracle.quant_int4_asym(host_f32(w), 128, threads=0)
    assert np.array_equal(scales.view(torch.int16).cpu().numpy().view(np.uint16), s)
    assert np.array_equal(zps.cpu().numpy(), z) and np.array_equal(codes.cpu().numpy(), c)
    codes, a8, a2 = cf.quant_nf4(w, 64, 256)
    c, b8, b2 = oracle.quant_nf4(host_f32(w), 64, 256, threads=0)
    assert bits_equal(a2, b2) and np.array_equal(a8.cpu().numpy(), b8) and np.array_equal(codes.cpu().numpy(), c)


def test_e2_special_values(cuda_device, oracle):
    from castforge_b200 import device as cf
    w = weights(4096, 3, torch.float32)
    w[0:128] = 0.0                    # all-zero group -> scale 1.0
    w[130] = float("nan")
    w[256:384] = 1e-9                 # (hi-lo)/15 flushes to f16 zero -> scale 1.0
    w[384:512] = torch.linspace(-1, 1, 128)
    w[512:640] = 5.0                  # all-positive group (range anchored at 0)
    w[640:768] = -3.0
    codes, scales, zps = cf.quant_int4_asym(w.to(cuda_device), 128)
    c, s, z = oracle.quant_int4_asym(w.numpy(), 128)
    assert np.array_equal(scales.view(torch.int16).cpu().numpy().view(np.uint16), s)
    assert np.array_equal(zps.cpu().numpy(), z) and np.array_equal(codes.cpu().numpy(), c)


# ------------------------------------------------------------------------------------------- E3
@pytest.mark.parametrize("dtype", ["bf16", "f32", "f16"])
@pytest.mark.parametrize("block", [32, 64, 128, 256])
@pytest.mark.parametrize("n", [64, 1000, 64 * 256 * 3 + 17, 4096 * 512])
def test_e3_nf4(cuda_device, oracle, dtype, block, n):
    from castforge_b200 import device as cf
    w = weights(n, n % 977 + block, DT[dtype]).to(cuda_device)
    codes, a8, a2 = cf.quant_nf4(w, block, 256)
    c, b8, b2 = oracle.quant_nf4(host_f32(w), block, 256, threads=0)
    assert bits_equal(a2, b2)
    assert np.array_equal(a8.cpu().numpy(), b8)
    assert np.array_equal(codes.cpu().numpy(), c)


def test_e3_nf4_dense_sweep_of_normalised_values(cuda_device, oracle):
    """Blocks whose absmax is exactly 1 make x == v: sweep x finely around every midpoint."""
    from castforge_b200 import device as cf
    mids = np.array([-0.8480964, -0.6106329, -0.45999518, -0.33967936, -0.23460737, -0.13791169, -0.04552499,
                     0.039790157, 0.12025523, 0.20352119, 0.2920137, 0.38931245, 0.5016633, 0.64278674, 0.8614783], np.float32)
    vals = []
    for m in mids:
        x = m
        lo = [x]
        for _ in range(20):
            lo.append(np.nextafter(lo[-1], np.float32(-2)))
        hi = [x]
        for _ in range(20):
            hi.append(np.nextafter(hi[-1], np.float32(2)))
        vals += lo + hi
    vals += list(np.linspace(-1, 1, 4001, dtype=np.float32))
    vals = np.array(vals, np.float32)
    blocks = []
    for i in range(0, len(vals), 63):
        blk = np.zeros(64, np.float32)
        chunk = vals[i:i + 63]
        blk[:len(chunk)] = chunk
        blk[63] = 1.0
        blocks.append(blk)
    w = torch.from_numpy(np.concatenate(blocks))
    codes, a8, a2 = cf.quant_nf4(w.to(cuda_device), 64, 256)
    c, b8, b2 = oracle.quant_nf4(w.numpy(), 64, 256)
    assert np.array_equal(codes.cpu().numpy(), c) and np.array_equal(a8.cpu().numpy(), b8)


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("block", [32, 64, 256])
def test_e3_nf4_list_equals_single_tensor_calls(cuda_device, dtype, block):
    """cfb200_quant_nf4_tensors (one launch pair for a whole list): every tensor's codes, 8-bit maxima and second-level
    scales EQUAL the single-tensor call's -- ragged sizes, a tensor shorter than one block, sizes that end inside a block."""
    from castforge_b200 import device as cf
    sizes = [64 * 256 * 3, 7, 64 * 1000 + 17, 1, 4096 * 130, 33, 64 * 256]
    ws = [weights(n, n % 31 + block, DT[dtype]).to(cuda_device) for n in sizes]
    got = cf.quant_nf4_tensors(ws, block, 256)
    for w, (c, a8, a2) in zip(ws, got):
        c1, b8, b2 = cf.quant_nf4(w, block, 256)
        assert torch.equal(c, c1) and torch.equal(a8, b8) and torch.equal(a2.view(torch.int32), b2.view(torch.int32))


def test_e3_workspace_too_small_is_rejected(cuda_device):
    from castforge_b200 import device as cf, CfbError
    w = weights(64 * 1000, 1, torch.bfloat16).to(cuda_device)
    with pytest.raises(CfbError) as ei:
        cf.quant_nf4(w, 64, 256, workspace=torch.empty(16, dtype=torch.uint8, device=cuda_device))
    assert ei.value.code == 5


# ------------------------------------------------------------------------------------------- E4
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_e4_tensor_list_equals_single_tensor_casts(cuda_device, dtype):
    """cfb200_cast_e4m3_tensors (the cooperative list launch): codes and {scale, absmax} EQUAL cfb200_cast_e4m3_tensor
    tensor by tensor -- ragged sizes, tails shorter than a vector, tensors larger than the on-chip ring, NaN / inf, zeros."""
    from castforge_b200 import device as cf
    sizes = [4096 * 1024 + 3, 7, 1, 33 * 1000, 12_000_017, 64, 2_000_000]
    ws = [weights(n, n % 13 + 5, DT[dtype]).to(cuda_device) for n in sizes]
    ws[3][17] = float("nan")
    ws[6][5] = float("inf")
    ws[5].zero_()
    codes, sa = cf.cast_e4m3_tensors(ws)
    import ctypes
    import castforge_b200
    for i, w in enumerate(ws):
        c1, s1 = cf.cast_e4m3_tensor(w)
        assert torch.equal(codes[i], c1), (dtype, i)
        assert torch.equal(sa[i].view(torch.int32), s1.view(torch.int32)), (dtype, i)
    flag = ctypes.c_int32(-1)
    assert castforge_b200.load().cfb200_quant_sym_status(ctypes.byref(flag)) == 0 and flag.value == 0


def test_e4_hardware_cast_matches_codec_on_covering_set(cuda_device, oracle):
    """Every code's exact value, each midpoint between adjacent codes, one ulp either side of it,
    values around the saturation point, zeros, NaN and infinities.  With the row absmax equal to
    448 the scale is exactly 1, so the hardware conversion sees these values unchanged."""
    from castforge_b200 import device as cf
    vals = [0.0, -0.0, float("nan"), float("inf"), float("-inf"), 448.0, 449.0, 463.9, 464.0, 465.0, 480.0, 1e9]
    dec = [oracle.e4m3_decode(c) for c in range(0x7F)]
    for i, x in enumerate(dec):
        nxt = dec[i + 1] if i + 1 < len(dec) else 480.0
        mid = np.float32((x + nxt) / 2)
        for v in (x, mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(1e9))):
            vals += [float(v), -float(v)]
    vals = np.array(vals, np.float32)
    cols = 1024
    row = np.zeros(cols, np.float32)
    finite = vals[np.isfinite(vals) & (np.abs(vals) <= 448)]
    row[:len(finite)] = finite
    row[-1] = 448.0
    x = torch.from_numpy(row).reshape(1, cols).to(cuda_device)
    codes, scales = cf.cast_e4m3_rows(x)
    assert float(scales[0]) == 1.0
    want = np.array([oracle.e4m3_encode_rne(float(v)) for v in row], np.uint8)
    assert np.array_equal(codes.cpu().numpy().ravel(), want)
    # NaN / inf / beyond-range inputs through the per-tensor path (absmax ignores NaN, inf saturates)
    w = torch.from_numpy(np.concatenate([vals, np.zeros(1000, np.float32)])).to(cuda_device)
    c2, sa = cf.cast_e4m3_tensor(w)
    wc, ws = oracle.cast_e4m3_rows(w.cpu().numpy(), 1, w.numel())
    assert bits_equal(sa[:1], ws) and np.array_equal(c2.cpu().numpy().ravel(), wc.ravel())


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("shape", [(7, 4096), (128, 14336), (33, 1000), (4, 40000)])
def test_e4_per_token_cast(cuda_device, oracle, dtype, shape):
    from castforge_b200 import device as cf
    rows, cols = shape
    x = weights(rows * cols, rows, DT[dtype], scale=1.0).reshape(rows, cols)
    x[:, ::97] *= 50
    xd = x.to(cuda_device)
    codes, scales = cf.cast_e4m3_rows(xd)
    wc, ws = oracle.cast_e4m3_rows(host_f32(xd), rows, cols, threads=0)
    assert bits_equal(scales, ws) and np.array_equal(codes.cpu().numpy(), wc)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_e4_per_tensor_cast(cuda_device, oracle, dtype):
    from castforge_b200 import device as cf
    w = weights((1 << 20) + 5, 9, DT[dtype]).to(cuda_device)
    codes, sa = cf.cast_e4m3_tensor(w)
    wc, ws = oracle.cast_e4m3_rows(host_f32(w), 1, w.numel(), threads=0)
    assert bits_equal(sa[:1], ws) and np.array_equal(codes.cpu().numpy().ravel(), wc.ravel())
