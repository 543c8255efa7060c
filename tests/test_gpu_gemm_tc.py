"""GPU: tcgen05/TMEM GEMMs against the CPU oracle (small) and f64 products of the same operands (large).

Tolerance of this path: max-abs error <= 1e-2 * RMS of the reference output.  FP8 and bf16
products are exact in f32, so those are held to 1e-4; the W4A16 kernel rounds each dequantised
weight to bf16 once (relative 2^-9), which costs up to ~9e-3 of the RMS at K = 4096.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_err(got, ref):
    ref = ref.double()
    return float((got.double() - ref).abs().max() / ref.pow(2).mean().sqrt())


@pytest.mark.parametrize("shape", [(128, 128, 64), (128, 128, 512), (256, 384, 1024), (200, 130, 72), (1, 128, 256), (513, 1000, 4096)])
def test_bf16_nt(cuda_device, shape):
    from castforge_b200 import device as cf
    M, N, K = shape
    g = torch.Generator(device=cuda_device).manual_seed(M + N + K)
    a = torch.randn(M, K, device=cuda_device, generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, device=cuda_device, generator=g).to(torch.bfloat16)
    ref = a.double() @ b.double().T
    assert rel_err(cf.gemm_bf16_nt(a, b, 1.0, True), ref) < 1e-4
    assert rel_err(cf.gemm_bf16_nt(a, b, 0.5, False).float(), 0.5 * ref) < 3e-2   # rounding of the bf16 OUTPUT format (2^-9 of the largest value)


def test_bf16_symmetric_upper_only(cuda_device):
    """X^T X for the GPTQ Hessian: only tiles touching the upper triangle are computed."""
    from castforge_b200 import device as cf
    g = torch.Generator(device=cuda_device).manual_seed(5)
    xt = torch.randn(512, 2048, device=cuda_device, generator=g).to(torch.bfloat16)    # [features, tokens]
    h = cf.gemm_bf16_nt(xt, xt, 1.0, True, upper_only=True)
    ref = xt.double() @ xt.double().T
    iu = torch.triu_indices(512, 512, device=cuda_device)
    # diagonal entries are ~20x the RMS; f32 accumulation of 2048 positive terms is good to ~1e-5 of the VALUE
    assert float((h.double()[iu[0], iu[1]] - ref[iu[0], iu[1]]).abs().max() / ref.pow(2).mean().sqrt()) < 1e-3
    assert float(h[384:, :128].abs().max()) == 0.0      # strictly-lower tiles untouched (output was zero-filled)


@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 512, 1024), (300, 700, 4096), (7, 256, 512), (4096, 4096, 4096)])
def test_fp8_gemm(cuda_device, oracle, shape):
    """FP8 serving path: per-token activation scale x per-tensor weight scale, E4M3 x E4M3 -> f32 accumulate."""
    from castforge_b200 import device as cf
    M, N, K = shape
    g = torch.Generator(device=cuda_device).manual_seed(M * 3 + N)
    x = torch.randn(M, K, device=cuda_device, generator=g)
    x[:, :: 100] *= 50                                   # 1 % of channels x50
    w = (torch.randn(N, K, device=cuda_device, generator=g) * 0.02)
    ac, asc = cf.cast_e4m3_rows(x.to(torch.bfloat16))
    wc, wsa = cf.cast_e4m3_tensor(w.to(torch.bfloat16))
    c32 = cf.gemm_fp8(ac, asc, wc, float(wsa[0]), out_f32=True)
    ref = (ac.view(torch.float8_e4m3fn).double() @ wc.view(torch.float8_e4m3fn).double().T) * asc.double()[:, None] * float(wsa[0])
    assert rel_err(c32, ref) < 1e-4
    cbf = cf.gemm_fp8(ac, asc, wc, float(wsa[0]), out_f32=False)
    assert cbf.dtype == torch.bfloat16 and rel_err(cbf.float(), ref) < 3e-2          # bf16 output format rounding only
    if M * N * K <= 300 * 700 * 4096:                    # the CPU oracle on the same codes
        want = oracle.gemm_e4m3(ac.cpu().numpy(), asc.cpu().numpy(), wc.cpu().numpy(), float(wsa[0]), M, N, K)
        assert rel_err(c32.cpu(), torch.from_numpy(want)) < 1e-4


@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 384, 1024), (16, 256, 512), (2048, 4096, 4096),
                                   (128, 4096, 4096), (200, 4096, 4096), (63, 999, 1024), (96, 1024, 14336)])
def test_w4a16_prefill(cuda_device, oracle, shape):
    """W4A16 prefill path: INT4 asymmetric group-128 weights (0.1 % outliers x20), bf16 activations.  The shapes with
    M <= 256 and few column tiles run the split-K schedule (f32 partial sums + reduction launch)."""
    from castforge_b200 import device as cf
    M, N, K = shape
    g = torch.Generator(device=cuda_device).manual_seed(M + 7 * N)
    w = torch.randn(N, K, device=cuda_device, generator=g) * 0.02
    idx = torch.randint(0, N * K, (max(1, N * K // 1000),), device=cuda_device, generator=g)
    w.view(-1)[idx] *= 20
    a = torch.randn(M, K, device=cuda_device, generator=g).to(torch.bfloat16)
    codes, scales, zps = cf.quant_int4_asym(w.reshape(-1), 128)
    c = cf.gemm_w4a16(a, codes, scales, zps, N, 128, out_f32=True)
    if M * N * K <= 256 * 384 * 1024:
        want = oracle.gemm_w4a16(a.float().cpu().numpy(), codes.cpu().numpy(), scales.view(torch.int16).cpu().numpy().view(np.uint16),
                                 zps.cpu().numpy(), M, N, K, 128)
        ref = torch.from_numpy(want).to(cuda_device)
    else:
        ng = K // 128
        q = torch.stack([codes & 0xF, codes >> 4], 1).reshape(N, ng, 128).double()
        zz = torch.stack([zps & 0xF, zps >> 4], 1).reshape(-1)[: N * ng].reshape(N, ng, 1).double()
        wd = ((q - zz) * scales.double().reshape(N, ng, 1)).reshape(N, K)
        ref = a.double() @ wd.T
    assert rel_err(c, ref) < 1e-2
    cb = cf.gemm_w4a16(a, codes, scales, zps, N, 128, out_f32=False)
    assert cb.dtype == torch.bfloat16 and rel_err(cb.float(), ref) < 3e-2       # + bf16 output rounding


@pytest.mark.parametrize("adt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", [(128, 256, 512), (300, 1024, 4096)])
def test_w4a16_with_static_quantize_prologue(cuda_device, oracle, adt, shape):
    """The `w8a8` execute path: castforge.static_quantize on the activation operand (eval.rs:1369-1382) folded into the
    GEMM's staging pass.  Reference = f64 product of the interpreter's static_quantize output (bit-exact kernel of the same
    op) with the dequantised weights; the bar is the tensor-core GEMM tolerance, 1e-2 x RMS."""
    from castforge_b200 import device as cf
    M, N, K = shape
    g = torch.Generator(device=cuda_device).manual_seed(M + N)
    w = torch.randn(N, K, device=cuda_device, generator=g) * 0.02
    a32 = torch.randn(M, K, device=cuda_device, generator=g)
    a32[:, ::97] *= 6                                     # some values beyond the clamp at +-127 * scale
    a = a32 if adt == "f32" else a32.to(torch.bfloat16)
    sc = 0.03125 * 1.1
    codes, scales, zps = cf.quant_int4_asym(w.reshape(-1), 128)
    got = cf.gemm_w4a16_static_quantize(a, sc, 8, codes, scales, zps, N, 128, out_f32=True)
    asq = cf.static_quantize(a.float().reshape(-1), sc, 8).reshape(M, K)
    assert float(asq.abs().max()) <= 127 * sc * (1 + 1e-6) and int(torch.unique(asq).numel()) <= 255
    ng = K // 128
    q = torch.stack([codes & 0xF, codes >> 4], 1).reshape(N, ng, 128).double()
    zz = torch.stack([zps & 0xF, zps >> 4], 1).reshape(-1)[: N * ng].reshape(N, ng, 1).double()
    wd = ((q - zz) * scales.double().reshape(N, ng, 1)).reshape(N, K)
    assert rel_err(got, asq.double() @ wd.T) < 1e-2
    # and it is what the unfused sequence (static_quantize launch, bf16 copy, GEMM) computes, up to that copy's rounding
    unfused = cf.gemm_w4a16(asq.to(torch.bfloat16), codes, scales, zps, N, 128, out_f32=True)
    assert rel_err(got, unfused.double()) < 1e-2


@pytest.fixture
def pair_knob():
    """Sets the "gemm_pair" knob (0 = one CTA per tile, 2 = the two-CTA kernel wherever it can run) and restores the default."""
    from castforge_b200 import load
    def set_knob(v):
        assert load().cfb200_tune(b"gemm_pair", v) == 0
    yield set_knob
    set_knob(1)


@pytest.mark.parametrize("shape", [(129, 100, 64), (256, 256, 64), (300, 700, 4096), (1000, 520, 264), (513, 1000, 4096), (2048, 4096, 1024)])
def test_pair_kernel_bf16_and_fp8_match_the_one_cta_kernel(cuda_device, pair_knob, shape):
    """The two-CTA (cta_group::2, 256 x 256 tile) kernel against the one-CTA kernel on the same operands: both sum the same
    K slices in the same order, so the results are the same bits; and against the f64 product."""
    from castforge_b200 import device as cf
    M, N, K = shape
    g = torch.Generator(device=cuda_device).manual_seed(M * 5 + N + K)
    a = torch.randn(M, K, device=cuda_device, generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, device=cuda_device, generator=g).to(torch.bfloat16)
    pair_knob(0)
    one = cf.gemm_bf16_nt(a, b, 0.75, True)
    one_bf = cf.gemm_bf16_nt(a, b, 0.75, False)
    pair_knob(2)
    two = cf.gemm_bf16_nt(a, b, 0.75, True)
    two_bf = cf.gemm_bf16_nt(a, b, 0.75, False)
    assert rel_err(two, 0.75 * (a.double() @ b.double().T)) < 1e-4
    assert torch.equal(two, one) and torch.equal(two_bf, one_bf)      # same K slices in the same order: the same bits
    if K % 16 == 0:
        ac, asc = cf.cast_e4m3_rows(a)
        wc, wsa = cf.cast_e4m3_tensor((b.float() * 0.02).to(torch.bfloat16))
        pair_knob(0)
        f_one = cf.gemm_fp8(ac, asc, wc, float(wsa[0]), out_f32=True)
        pair_knob(2)
        f_two = cf.gemm_fp8(ac, asc, wc, float(wsa[0]), out_f32=True)
        ref = (ac.view(torch.float8_e4m3fn).double() @ wc.view(torch.float8_e4m3fn).double().T) * asc.double()[:, None] * float(wsa[0])
        assert rel_err(f_two, ref) < 1e-4 and torch.equal(f_two, f_one)


def test_pair_kernel_symmetric_upper_only(cuda_device, pair_knob):
    """Upper-triangle-only product through the two-CTA kernel: tiles strictly below the diagonal stay untouched."""
    from castforge_b200 import device as cf
    g = torch.Generator(device=cuda_device).manual_seed(6)
    xt = torch.randn(1280, 1024, device=cuda_device, generator=g).to(torch.bfloat16)
    pair_knob(2)
    h = cf.gemm_bf16_nt(xt, xt, 1.0, True, upper_only=True)
    ref = xt.double() @ xt.double().T
    iu = torch.triu_indices(1280, 1280, device=cuda_device)
    assert float((h.double()[iu[0], iu[1]] - ref[iu[0], iu[1]]).abs().max() / ref.pow(2).mean().sqrt()) < 1e-3
    assert float(h[768:, :256].abs().max()) == 0.0


@pytest.mark.parametrize("knob", [0, 2])
def test_bf16_product_into_a_block_with_triangle_and_accumulate(cuda_device, pair_knob, knob):
    """cfb200_gemm_bf16_nt_ex: operands and result are blocks of wider matrices (row pitches), C -= A B^T on the tiles that
    touch the lower triangle only, through both kernels."""
    from castforge_b200 import device as cf
    g = torch.Generator(device=cuda_device).manual_seed(9 + knob)
    big = torch.randn(1600, 2000, device=cuda_device, generator=g)
    wide = torch.randn(1300, 1024, device=cuda_device, generator=g).to(torch.bfloat16)
    a = wide[:, 256:256 + 512]                       # [1300, 512], row pitch 1024
    c = big[128:128 + 1300, 512:512 + 1300]          # [1300, 1300] block, row pitch 2000
    before = c.clone()
    pair_knob(knob)
    cf.gemm_bf16_nt_into(c, a, a, alpha=-1.0, triangle=2, accumulate=True)
    want = before.double() - a.double() @ a.double().T
    low = torch.tril(torch.ones(1300, 1300, device=cuda_device, dtype=torch.bool))
    assert float((c.double() - want)[low].abs().max()) < 1e-3          # f32 accumulation of 512 products of N(0,1) values
    tile = 256 if knob else 128
    far = torch.triu(torch.ones(1300, 1300, device=cuda_device, dtype=torch.bool), diagonal=2 * tile)   # surely in a skipped tile
    assert torch.equal(c[far], before[far])
    outside = big.clone()
    outside[128:128 + 1300, 512:512 + 1300] = 0
    ref = torch.randn(1600, 2000, device=cuda_device, generator=torch.Generator(device=cuda_device).manual_seed(9 + knob))
    ref[128:128 + 1300, 512:512 + 1300] = 0
    assert torch.equal(outside, ref)                                   # nothing outside the block was written


@pytest.mark.parametrize("shape", [(257, 256, 128), (300, 1000, 1024), (1024, 4096, 4096), (2048, 520, 14336)])
def test_pair_kernel_w4a16_matches_the_one_cta_kernel(cuda_device, pair_knob, shape):
    """W4A16 prefill through the two-CTA kernel (each CTA unpacks its 128 of the tile's 256 weight rows) against the one-CTA
    kernel: the unpacked f16 weights are the same bits and the K order is the same."""
    from castforge_b200 import device as cf
    M, N, K = shape
    g = torch.Generator(device=cuda_device).manual_seed(M + 11 * N)
    w = torch.randn(N, K, device=cuda_device, generator=g) * 0.02
    w.view(-1)[torch.randint(0, N * K, (max(1, N * K // 1000),), device=cuda_device, generator=g)] *= 20
    a = torch.randn(M, K, device=cuda_device, generator=g).to(torch.bfloat16)
    codes, scales, zps = cf.quant_int4_asym(w.reshape(-1), 128)
    pair_knob(0)
    one = cf.gemm_w4a16(a, codes, scales, zps, N, 128, out_f32=True)
    pair_knob(2)
    two = cf.gemm_w4a16(a, codes, scales, zps, N, 128, out_f32=True)
    two_bf = cf.gemm_w4a16(a, codes, scales, zps, N, 128, out_f32=False)
    ng = K // 128
    q = torch.stack([codes & 0xF, codes >> 4], 1).reshape(N, ng, 128).double()
    zz = torch.stack([zps & 0xF, zps >> 4], 1).reshape(-1)[: N * ng].reshape(N, ng, 1).double()
    wd = ((q - zz) * scales.double().reshape(N, ng, 1)).reshape(N, K)
    ref = a.double() @ wd.T
    assert rel_err(two, ref) < 1e-2 and rel_err(two_bf.float(), ref) < 4e-2     # + bf16 output rounding (2^-9 of the largest value)
    assert torch.equal(two, one)       # every unpacked weight and every hand-over arrived: any race would show as garbage


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("NK", [(4096, 4096), (264, 1024), (14336, 4096), (40, 128), (4096, 14336), (8200, 4096), (76040, 4096)])
def test_w4a16_decode(cuda_device, oracle, M, NK):
    """W4A16 decode (M <= 16): exact dequantisation in the register-ring kernel, offset-corrected in the ring kernel."""
    from castforge_b200 import device as cf
    N, K = NK
    g = torch.Generator(device=cuda_device).manual_seed(M + N)
    w = torch.randn(N, K, device=cuda_device, generator=g) * 0.02
    idx = torch.randint(0, N * K, (max(1, N * K // 1000),), device=cuda_device, generator=g)
    w.view(-1)[idx] *= 20
    a = torch.randn(M, K, device=cuda_device, generator=g).to(torch.bfloat16)
    codes, scales, zps = cf.quant_int4_asym(w.reshape(-1), 128)
    c = cf.gemv_w4a16(a, codes, scales, zps, N, 128, out_f32=True)
    ng = K // 128
    q = torch.stack([codes & 0xF, codes >> 4], 1).reshape(N, ng, 128).double()
    zz = torch.stack([zps & 0xF, zps >> 4], 1).reshape(-1)[: N * ng].reshape(N, ng, 1).double()
    wd = ((q - zz) * scales.double().reshape(N, ng, 1)).reshape(N, K)
    ref = a.double() @ wd.T
    # the register-ring kernel dequantises exactly (only the f32 summation order differs); the shared-memory ring
    # kernel of the large shapes feeds 1024 + q to the tensor cores and removes the offset afterwards, which costs
    # about 7 of the accumulator's 24 bits
    ring = N * K // 2 >= (16 << 20)  # weights of 16 MB and more take the shared-memory ring kernel
    assert rel_err(c, ref) < (1e-3 if ring else 1e-5)  # max error over all outputs / output RMS; the bar is 1e-2
    if N * K <= 264 * 1024:
        want = oracle.gemm_w4a16(a.float().cpu().numpy(), codes.cpu().numpy(), scales.view(torch.int16).cpu().numpy().view(np.uint16),
                                 zps.cpu().numpy(), M, N, K, 128)
        assert rel_err(c.cpu(), torch.from_numpy(want)) < 1e-5
    cb = cf.gemv_w4a16(a, codes, scales, zps, N, 128, out_f32=False)
    assert rel_err(cb.float(), ref) < 3e-2      # bf16 output format
    # both decode kernels (shared-memory ring for large shapes, register ring otherwise) and no wait ran out
    import ctypes
    import castforge_b200
    lib = castforge_b200.load()
    assert lib.cfb200_tune(b"gemv_ring", 0) == 0
    try:
        c2 = cf.gemv_w4a16(a, codes, scales, zps, N, 128, out_f32=True)
    finally:
        assert lib.cfb200_tune(b"gemv_ring", 1) == 0
    assert rel_err(c2, ref) < 1e-5
    flag = ctypes.c_int32(-1)
    assert lib.cfb200_gemv_w4a16_status(ctypes.byref(flag)) == 0 and flag.value == 0


def test_gemm_argument_errors(cuda_device):
    from castforge_b200 import device as cf, CfbError
    a = torch.zeros(128, 100, dtype=torch.uint8, device=cuda_device)     # K not a multiple of 16
    with pytest.raises(CfbError):
        cf.gemm_fp8(a, None, a, 1.0)
