"""KV-cache page codecs: the K16/V8 codec (src/passes/serving/kv_attention.rs:52-222) and the float8_e4m3fn slice
codec (src/passes/serving/mutable_loads.rs:431-441).  CPU: the oracle against the reference's own test of the codec
(tests/commercial_readiness_tests.rs:565-623) and hand-derived codes.  GPU: the CUDA kernels against the oracle, bit
for bit."""
import numpy as np
import pytest

SCOPES = {"tensor": 0, "layer_head": 1, "page_head": 2}


def reference_fixture():
    """The caches of test_asym_k16_v8_kv_codec_and_scoped_scales: [2, 4, 2, 8], page 1 / head 1 of v zeroed."""
    P, T, H, D = 2, 4, 2, 8
    total = P * T * H * D
    i = np.arange(total, dtype=np.float32)
    k = ((i - np.float32(64.0)) * np.float32(0.05)).astype(np.float32).reshape(P, T, H, D)
    v = ((i - np.float32(32.0)) * np.float32(0.1)).astype(np.float32).reshape(P, T, H, D)
    v[1, :, 1, :] = 0.0
    return k, v


@pytest.mark.parametrize("scope", ["tensor", "layer_head", "page_head"])
def test_oracle_on_the_reference_test_case(oracle, scope):
    k, v = reference_fixture()
    kb, vc, vs = oracle.kv_encode_k16v8(k, v, SCOPES[scope])
    assert vs.size == {"tensor": 1, "layer_head": 2, "page_head": 4}[scope]
    if scope == "page_head":
        assert vs[3] == 1.0                                       # KV_ZERO_SCALE_SENTINEL for the zeroed (page, head)
    # byte footprint: 128 keys x 2 B + 128 codes + scales  (payload_bytes, kv_attention.rs:42-44)
    assert 2 * (kb.size + vc.size) == 512 and kb.size * 2 + vc.size + vs.size * 4 <= 400
    kd, vd = oracle.kv_decode_k16v8(kb, vc, vs, SCOPES[scope])
    assert np.abs(k - kd).max() < 5e-3
    assert not np.isnan(vd).any() and np.abs(v - vd).max() < 0.08


def test_oracle_hand_derived_codes(oracle):
    # one page, one token, two heads of four: head 0 absmax 2 -> scale 2/127; head 1 all zero -> scale 1
    v = np.array([[[[2.0, -1.1, 0.5, float("nan")], [0.0, -0.0, 0.0, 0.0]]]], np.float32)
    k = np.array([[[[1.0, -2.5, 65504.0, 1e-8], [70000.0, float("inf"), 0.333251953125, 0.3333]]]], np.float32)
    kb, vc, vs = oracle.kv_encode_k16v8(k, v, 2)
    s = np.float32(2.0) / np.float32(127.0)
    assert vs.tolist() == [float(s), 1.0]
    # 2/s = 127; -1.1/s = -69.85 -> -70; 0.5/s = 31.75 -> 32; NaN -> 0
    assert vc.reshape(-1).tolist() == [127, -70, 32, 0, 0, 0, 0, 0]
    # truncating f16: 1e-8 flushes to 0, 70000 overflows to inf, 0.3333 lies between 0x3555 and 0x3556 and stays 0x3555
    assert kb.reshape(-1).tolist() == [0x3C00, 0xC100, 0x7BFF, 0x0000, 0x7C00, 0x7C00, 0x3555, 0x3555]
    # per tensor: the symmetric clamp is +-127, never -128
    v2 = np.array([[[[-3.0, 3.0, 1.0, -1.0]]]], np.float32)
    _, vc2, vs2 = oracle.kv_encode_k16v8(v2, v2, 0)
    assert vc2.reshape(-1).tolist() == [-127, 127, 42, -42] and vs2[0] == np.float32(3.0) / np.float32(127.0)


def test_oracle_e4m3_slice_known_answers(oracle):
    # known answers of the reference codec (tests/serving_storage_routing_tests.rs:2228-2235 style): 1.0 -> 0x38,
    # 448 and beyond saturate to 0x7E, NaN -> 0x7F, the smallest subnormal 2^-9 -> 0x01
    x = np.array([0.0, -0.0, 1.0, -1.0, 448.0, 1e9, -1e9, float("nan"), 2.0 ** -9, 0.4375], np.float32)
    for which in (0, 1):
        assert oracle.e4m3_slice_encode(x, which).tolist() == [0x00, 0x80, 0x38, 0xB8, 0x7E, 0x7E, 0xFE, 0x7F, 0x01, 0x2E]
    back = oracle.e4m3_slice_decode(np.arange(256, dtype=np.uint8))
    assert np.isnan(back[0x7F]) and np.isnan(back[0xFF]) and back[0x7E] == 448.0 and back[0x01] == 2.0 ** -9
    finite = np.array([c for c in range(256) if c & 0x7F != 0x7F], np.uint8)
    assert np.array_equal(oracle.e4m3_slice_encode(oracle.e4m3_slice_decode(finite)), finite)   # every code round-trips


# ---------------------------------------------------------------------------------------------------------------------
def make_caches(shape, seed, dtype):
    import torch
    rng = np.random.default_rng(seed)
    k = rng.standard_normal(shape).astype(np.float32) * rng.choice([1e-6, 0.1, 1.0, 300.0, 1e5], size=shape).astype(np.float32)
    v = rng.standard_normal(shape).astype(np.float32) * (1.0 + 4.0 * rng.random((1, 1, shape[2], 1), dtype=np.float32))
    P, T, H, D = shape
    v[P // 2, :, H - 1, :] = 0.0                                    # an all-zero (page, head): sentinel scale
    flat = v.reshape(-1)
    flat[rng.integers(0, flat.size, 7)] = np.nan                    # NaN is ignored by the absmax and encodes as 0
    kf = k.reshape(-1)
    kf[rng.integers(0, kf.size, 5)] = [np.inf, -np.inf, np.nan, 65520.0, 6e-8]
    tk, tv = torch.from_numpy(k).to(dtype), torch.from_numpy(v).to(dtype)
    return tk, tv


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("scope", ["tensor", "layer_head", "page_head"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 8), (5, 16, 8, 128), (3, 7, 3, 24), (1, 1, 1, 8), (300, 16, 8, 64), (2, 33, 12, 40)])
def test_k16v8_cuda_matches_oracle(oracle, cuda_device, shape, scope, dtype_name):
    import torch
    from castforge_b200 import device as D
    dtype = getattr(torch, dtype_name)
    tk, tv = make_caches(shape, sum(shape) + SCOPES[scope], dtype)
    kb, vc, vs = D.kv_encode_k16v8(tk.to(cuda_device), tv.to(cuda_device), scope)
    wkb, wvc, wvs = oracle.kv_encode_k16v8(tk.float().numpy(), tv.float().numpy(), SCOPES[scope])
    assert np.array_equal(vs.cpu().numpy().view(np.uint32), wvs.view(np.uint32))
    assert np.array_equal(vc.cpu().numpy(), wvc)
    assert np.array_equal(kb.cpu().numpy().view(np.uint16), wkb)
    ko, vo = D.kv_decode_k16v8(kb, vc, vs, scope)
    wko, wvo = oracle.kv_decode_k16v8(wkb, wvc, wvs, SCOPES[scope])
    assert np.array_equal(vo.cpu().numpy().view(np.uint32), wvo.view(np.uint32))
    got_k, want_k = ko.cpu().numpy(), wko
    nan = np.isnan(want_k)
    assert np.array_equal(np.isnan(got_k), nan) and np.array_equal(got_k[~nan].view(np.uint32), want_k[~nan].view(np.uint32))


@pytest.mark.gpu
def test_k16v8_inf_values_and_infinite_scale(oracle, cuda_device):
    """An infinite value makes its scope's scale infinite: finite values encode as 0, the infinity itself as
    inf / inf = NaN -> 0."""
    import torch
    from castforge_b200 import device as D
    v = np.ones((2, 2, 2, 8), np.float32)
    v[0, 0, 0, 0] = np.inf
    v[1, 1, 1, 3] = -np.inf
    for scope in SCOPES:
        t = torch.from_numpy(v).to(cuda_device)
        kb, vc, vs = D.kv_encode_k16v8(t, t, scope)
        wkb, wvc, wvs = oracle.kv_encode_k16v8(v, v, SCOPES[scope])
        assert np.array_equal(vs.cpu().numpy().view(np.uint32), wvs.view(np.uint32))
        assert np.array_equal(vc.cpu().numpy(), wvc) and np.array_equal(kb.cpu().numpy().view(np.uint16), wkb)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16", "float16"])
def test_k16v8_tiny_absmax_scopes(oracle, cuda_device, dtype_name):
    """Heads whose absmax is subnormal, below 1e-12, or so small that absmax / 127 underflows to 0 (v / 0 = +-inf -> +-127,
    0 / 0 = NaN -> 0): these leave the branch-free path."""
    import torch
    from castforge_b200 import device as D
    dtype = getattr(torch, dtype_name)
    rng = np.random.default_rng(11)
    v = rng.standard_normal((3, 4, 6, 16)).astype(np.float32)
    for h, mag in enumerate([1.0, 1e-13, 1e-30, 3e-39, 1e-44, 6e-8]):
        v[:, :, h, :] *= np.float32(mag)
    v[0, 0, 4, :4] = [1.4e-45, -1.4e-45, 0.0, 2.8e-45]
    t = torch.from_numpy(v).to(dtype)
    for scope in ("layer_head", "page_head", "tensor"):
        kb, vc, vs = D.kv_encode_k16v8(t.to(cuda_device), t.to(cuda_device), scope)
        wkb, wvc, wvs = oracle.kv_encode_k16v8(t.float().numpy(), t.float().numpy(), SCOPES[scope])
        assert np.array_equal(vs.cpu().numpy().view(np.uint32), wvs.view(np.uint32))
        assert np.array_equal(vc.cpu().numpy(), wvc)
        assert np.array_equal(kb.cpu().numpy().view(np.uint16), wkb)


@pytest.mark.gpu
def test_k16v8_rejects_what_the_reference_rejects(cuda_device):
    import torch
    from castforge_b200 import device as D
    from castforge_b200._lib import CfbError
    with pytest.raises(CfbError):
        D.kv_encode_k16v8(torch.zeros((0, 4, 2, 8), device=cuda_device), torch.zeros((0, 4, 2, 8), device=cuda_device))
    with pytest.raises(CfbError):   # head_dim not a multiple of the 16-byte vector
        D.kv_encode_k16v8(torch.zeros((1, 4, 2, 6), device=cuda_device), torch.zeros((1, 4, 2, 6), device=cuda_device))


@pytest.mark.gpu
def test_e4m3_slice_cuda(oracle, cuda_device):
    """Every code's value, every midpoint between neighbours and one ulp either side, the saturation edge, NaN and the
    infinities, plus a ragged length; decoding of all 256 bytes."""
    import torch
    from castforge_b200 import device as D
    vals = oracle.e4m3_slice_decode(np.arange(0x7F, dtype=np.uint8)).astype(np.float64)     # 0 .. 448 ascending
    mids = ((vals[:-1] + vals[1:]) / 2).astype(np.float32)
    pts = np.concatenate([vals.astype(np.float32), mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(1e9)),
                          np.array([464.0, np.nextafter(np.float32(464.0), np.float32(0)), 480.0, 1e30, np.inf, np.nan, 1e-30],
                                   np.float32)]).astype(np.float32)
    x = np.concatenate([pts, -pts])
    rng = np.random.default_rng(3)
    x = np.concatenate([x, (rng.standard_normal(100_003) * rng.choice([1e-3, 1.0, 200.0], 100_003)).astype(np.float32)])
    got = D.e4m3_slice_encode(torch.from_numpy(x).to(cuda_device)).cpu().numpy()
    assert np.array_equal(got, oracle.e4m3_slice_encode(x, 1))
    # the reference-exact entry point: every power of two of the normal range with the 12 values below and above it
    # (where the reference's floor(log2f) lands one binade high), on top of the set above
    edge = []
    for k in range(-7, 10):
        b = np.float32(2.0 ** k).view(np.uint32)
        edge += [np.uint32(int(b) + d) for d in range(-12, 13)]
    xe = np.concatenate([x, np.array(edge, np.uint32).view(np.float32), -np.array(edge, np.uint32).view(np.float32)])
    want_ref = oracle.e4m3_slice_encode(xe, 0)
    got_ref = D.e4m3_slice_encode_ref(torch.from_numpy(xe).to(cuda_device)).cpu().numpy()
    assert np.array_equal(got_ref, want_ref)
    assert int((want_ref != oracle.e4m3_slice_encode(xe, 1)).sum()) > 0      # the set does contain slips
    codes = np.concatenate([np.arange(256, dtype=np.uint8), rng.integers(0, 256, 1001, dtype=np.uint8)])
    back = D.e4m3_slice_decode(torch.from_numpy(codes).to(cuda_device)).cpu().numpy()
    want = oracle.e4m3_slice_decode(codes)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(back), nan) and np.array_equal(back[~nan].view(np.uint32), want[~nan].view(np.uint32))
    assert D.e4m3_slice_encode(torch.zeros(0, device=cuda_device)).numel() == 0


@pytest.mark.gpu
def test_k16v8_round_trip_bound_on_a_serving_sized_cache(cuda_device):
    """4096 pages x 16 tokens x 8 heads x 128 (bf16, 134 MB per cache): |v - code * scale| <= scale / 2 per (page, head),
    keys within one f16 truncation step."""
    import torch
    from castforge_b200 import device as D
    g = torch.Generator(device=cuda_device).manual_seed(2)
    shape = (4096, 16, 8, 128)
    k = torch.randn(shape, device=cuda_device, generator=g).to(torch.bfloat16)
    v = (torch.randn(shape, device=cuda_device, generator=g) * 3).to(torch.bfloat16)
    kb, vc, vs = D.kv_encode_k16v8(k, v, "page_head")
    ko, vo = D.kv_decode_k16v8(kb, vc, vs, "page_head")
    amax = v.float().abs().amax(dim=(1, 3))
    assert torch.equal(vs.reshape(4096, 8), amax / torch.tensor(127.0, device=cuda_device))   # f32 / f32, IEEE
    # half a step, plus the f32 rounding of code * scale and of the quotient (both relative to the absmax, not the step)
    bound = (vs.reshape(4096, 1, 8, 1) * 0.5 + amax.reshape(4096, 1, 8, 1) * 2.0 ** -21).expand(shape)
    assert bool(((v.float() - vo).abs() <= bound).all())
    # a bf16 key is exact in f16 unless it is below the smallest normal f16 (2^-14), which the truncating cast flushes to 0
    kf = k.float()
    assert torch.equal(ko, torch.where(kf.abs() >= 2.0 ** -14, kf, torch.zeros_like(kf) * kf.sign()))
