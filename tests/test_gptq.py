"""E5 (GPTQ INT4, group 128): the f64 oracle against an independent numpy statement of the algorithm
(CPU), and the CUDA path against the oracle (GPU).

Two oracles.  `gptq` keeps its state in f64 (the algorithm as published); the CUDA path keeps f32 state, so against it
a code can differ where a value lands within rounding error of a quantisation boundary, and a differing code changes
the errors pushed to the right of it: those tests bound the fraction of differing codes and compare the quantity GPTQ
minimises, the layer output error ||X (W - W_hat)||.  `gptq_walk_f32` restates the column walk in the device's own f32
operation order, given the factor U the device computed: codes, scales and zero points must then be EQUAL, at the
small shapes and at BASELINE config 5's sizes (K = 4096 and K = 14336, T = 262144 calibration tokens) on sampled
rows.  The factor itself is checked against f64 (np.linalg at small K; at config size through U^T U (H + damp) v = v on
random vectors, which needs no second factorisation)."""
import numpy as np
import pytest


def make_case(seed, N, K, T):
    rng = np.random.default_rng(seed)
    mix = rng.standard_normal((K, K)).astype(np.float32) / np.sqrt(K)
    mix += np.eye(K, dtype=np.float32)
    X = rng.standard_normal((T, K)).astype(np.float32) @ mix
    X *= (1.0 + 3.0 * rng.random(K, dtype=np.float32))  # uneven channel magnitudes
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    return W, X


def bf16_round(a):
    import torch
    return torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()


def unpack(codes, n):
    c = np.asarray(codes, np.uint8)
    out = np.empty(c.size * 2, np.uint8)
    out[0::2] = c & 0xF
    out[1::2] = c >> 4
    return out[:n]


def numpy_gptq(W, X, group=128, damp=0.01):
    """Independent restatement: np.linalg for the factorisation, the E2 group formula in f32."""
    N, K = W.shape
    H = (X.astype(np.float64).T @ X.astype(np.float64)) / X.shape[0]
    H[np.diag_indices(K)] += damp * np.mean(np.diag(H))
    U = np.linalg.cholesky(np.linalg.inv(H)).T
    Wc = W.astype(np.float64).copy()
    Q = np.zeros((N, K), np.uint8)
    Wdq = np.zeros((N, K), np.float32)
    f32 = np.float32
    for j in range(K):
        if j % group == 0:
            blk = Wc[:, j:j + group].astype(np.float32)
            lo = np.minimum(blk.min(axis=1), f32(0))
            hi = np.maximum(blk.max(axis=1), f32(0))
            s32 = ((hi - lo) / f32(15)).astype(np.float32)
            bits = s32.view(np.uint32)
            exp = ((bits >> 23) & 0xFF).astype(np.int32) - 127 + 15
            h = np.where(exp <= 0, 0, (exp.astype(np.uint32) << 10) | ((bits & 0x7FFFFF) >> 13)).astype(np.uint16)
            h = np.where((h & 0x7FFF) == 0, np.uint16(0x3C00), h)
            s = h.view(np.float16).astype(np.float32)
            r = (-lo / s).astype(np.float32)
            zf = np.clip(np.sign(r) * np.floor(np.abs(r) + f32(0.5)), 0, 15).astype(np.float32)
        wj = Wc[:, j].astype(np.float32)
        r = (wj / s).astype(np.float32)
        qf = np.clip(np.sign(r) * np.floor(np.abs(r) + f32(0.5)) + zf, 0, 15).astype(np.float32)
        wq = ((qf - zf) * s).astype(np.float32)
        Q[:, j] = qf.astype(np.uint8)
        Wdq[:, j] = wq
        e = (Wc[:, j] - wq.astype(np.float64)) / U[j, j]
        Wc[:, j + 1:] -= np.outer(e, U[j, j + 1:])
    return Q, Wdq


def out_err(X, W, Wh):
    return float(np.linalg.norm(X.astype(np.float64) @ (W.astype(np.float64) - Wh.astype(np.float64)).T))


def test_oracle_matches_numpy_statement(oracle):
    W, X = make_case(11, 24, 256, 512)
    codes, scales, zps, wdq = oracle.gptq(W, X)
    Q, Wdq = numpy_gptq(W, X)
    q = unpack(codes, W.size).reshape(W.shape)
    assert (q != Q).mean() < 2e-3  # two f64 factorisations: only exact-boundary values may differ
    assert abs(out_err(X, W, wdq) - out_err(X, W, Wdq)) <= 1e-3 * out_err(X, W, Wdq)
    # the dequantised output is what the codes decode to
    np.testing.assert_array_equal(oracle.dequant_int4_asym(codes, scales, zps, W.size, 128).reshape(W.shape), wdq)


def test_oracle_beats_round_to_nearest(oracle):
    W, X = make_case(12, 32, 256, 1024)
    _, _, _, wdq = oracle.gptq(W, X)
    c, s, z = oracle.quant_int4_asym(W.reshape(-1), 128)
    rtn = oracle.dequant_int4_asym(c, s, z, W.size, 128).reshape(W.shape)
    assert out_err(X, W, wdq) < 0.9 * out_err(X, W, rtn)


def test_f32_order_walk_agrees_with_the_f64_oracle(oracle):
    """The f32-order walk is the same algorithm: given the f64 factor (rounded to f32) it lands within boundary effects
    of the f64 oracle, and what it returns decodes to its own dequantised rows."""
    W, X = make_case(21, 48, 256, 1024)
    T, K = X.shape
    H = (X.astype(np.float64).T @ X.astype(np.float64)) / T
    H[np.diag_indices(K)] += 0.01 * np.mean(np.diag(H))
    U = np.linalg.cholesky(np.linalg.inv(H)).T.astype(np.float32)
    codes, scales, zpb, wdq = oracle.gptq_walk_f32(W, U, want_dequant=True)
    oc, osc, oz, owdq = oracle.gptq(W, X)
    assert (unpack(codes, W.size) != unpack(oc, W.size)).mean() < 0.02
    assert abs(out_err(X, W, wdq) - out_err(X, W, owdq)) <= 0.02 * out_err(X, W, owdq)
    zp_packed = (zpb[0::2] | (zpb[1::2] << 4)).astype(np.uint8)
    np.testing.assert_array_equal(oracle.dequant_int4_asym(codes, scales, zp_packed, W.size, 128).reshape(W.shape), wdq)


def _unpack_zps(zps, ngroups):
    z = np.asarray(zps, np.uint8)
    out = np.empty(z.size * 2, np.uint8)
    out[0::2] = z & 0xF
    out[1::2] = z >> 4
    return out[:ngroups]


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,T", [(64, 256, 1024), (200, 512, 2048), (8, 128, 256), (96, 1024, 4096)])
def test_gptq_cuda_equals_f32_order_oracle(oracle, cuda_device, N, K, T):
    """Codes, scales, zero points and dequantised weights EQUAL the f32-order oracle's, given the device's factor."""
    import torch
    from castforge_b200 import device as D
    W, X = make_case(N + K + 1, N, K, T)
    W, X = bf16_round(W), bf16_round(X)
    xd = torch.from_numpy(X).to(cuda_device, torch.bfloat16)
    wd = torch.from_numpy(W).to(cuda_device, torch.bfloat16)
    U = D.gptq_prepare(D.gptq_hessian(xd), 0.01)
    codes, scales, zps, wdq = D.gptq_quantize(wd, U)
    torch.cuda.synchronize()
    oc, osc, ozb, owdq = oracle.gptq_walk_f32(W, U.cpu().numpy(), want_dequant=True)
    np.testing.assert_array_equal(codes.cpu().numpy(), oc)
    np.testing.assert_array_equal(scales.cpu().numpy().view(np.uint16), osc)
    np.testing.assert_array_equal(_unpack_zps(zps.cpu().numpy(), N * (K // 128)), ozb)
    np.testing.assert_array_equal(wdq.cpu().numpy(), owdq)


@pytest.mark.gpu
@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336)])
def test_gptq_config5_sizes(oracle, cuda_device, N, K):
    """BASELINE config 5 at its own sizes: gate / up (14336 x 4096) and down (4096 x 14336), 128 x 2048 = 262144
    calibration tokens, bf16 N(0, 1) activations with a per-channel scale drawn log-uniformly from [0.1, 10], 1 %
    damping, group 128.  Hessian entries against f64 sums, the factor through U^T U (H + damp) v = v, and the codes /
    scales / zero points of 64 sampled output rows EQUAL to the f32-order oracle's (rows are independent)."""
    import torch
    from castforge_b200 import device as D
    T = 128 * 2048
    g = torch.Generator(device=cuda_device).manual_seed(K)
    ch = torch.exp((torch.rand(K, device=cuda_device, generator=g) * 2 - 1) * float(np.log(10.0)))
    X = torch.empty(T, K, dtype=torch.bfloat16, device=cuda_device)
    for t0 in range(0, T, 16384):
        X[t0:t0 + 16384] = (torch.randn(16384, K, device=cuda_device, generator=g) * ch).to(torch.bfloat16)
    W = (torch.randn(N, K, device=cuda_device, generator=g) * 0.02).to(torch.bfloat16)
    H = D.gptq_hessian(X)
    # Hessian: 48 sampled entries (diagonal and off-diagonal) against f64 sums of the same bf16 values
    rng = np.random.default_rng(K)
    ii = rng.integers(0, K, 48)
    jj = np.where(np.arange(48) % 2 == 0, ii, rng.integers(0, K, 48))
    cols = torch.from_numpy(np.unique(np.concatenate([ii, jj]))).to(cuda_device)
    Xs = X[:, cols].double().cpu().numpy()
    pos = {int(c): k for k, c in enumerate(cols.cpu().numpy())}
    Hh = H.cpu().numpy()
    for i, j in zip(ii, jj):
        want = float(Xs[:, pos[int(i)]] @ Xs[:, pos[int(j)]]) / T
        # 32 chunk sums of 512 truncating tensor-core additions each, then round-to-nearest additions: measured 3e-5
        assert abs(float(Hh[i, j]) - want) <= 1e-4 * np.sqrt(Hh[i, i] * Hh[j, j]) + 1e-7, (i, j, Hh[i, j], want)
    del X, Xs
    torch.cuda.empty_cache()
    U = D.gptq_prepare(H, 0.01)
    Uh = U.cpu().numpy()
    assert np.all(np.diag(Uh) > 0) and float(np.abs(np.tril(Uh, -1)).max()) == 0.0
    # factor: (U^T U) (H + damp I) v = v in f64 for random v (U^T U = inverse of the damped Hessian)
    Hd = Hh.astype(np.float64)
    Hd[np.diag_indices(K)] += 0.01 * float(np.mean(np.diag(Hh).astype(np.float64)))
    V = rng.standard_normal((K, 4))
    Y = Uh.T.astype(np.float64) @ (Uh.astype(np.float64) @ (Hd @ V))
    resid = float(np.linalg.norm(Y - V) / np.linalg.norm(V))
    assert resid < 5e-3, resid   # f32 factorisation of a matrix with condition number ~1e3
    del Hd
    codes, scales, zps, wdq = D.gptq_quantize(W, U, want_dequant=True)
    torch.cuda.synchronize()
    rows = np.sort(rng.choice(N, 64, replace=False))
    Wr = W[torch.from_numpy(rows).to(cuda_device)].float().cpu().numpy()
    oc, osc, ozb, owdq = oracle.gptq_walk_f32(Wr, Uh, want_dequant=True)
    ng = K // 128
    ch_, sh_, zh_ = codes.cpu().numpy().reshape(N, K // 2), scales.cpu().numpy().view(np.uint16).reshape(N, ng), _unpack_zps(zps.cpu().numpy(), N * ng).reshape(N, ng)
    np.testing.assert_array_equal(ch_[rows], oc.reshape(64, K // 2))
    np.testing.assert_array_equal(sh_[rows], osc.reshape(64, ng))
    np.testing.assert_array_equal(zh_[rows], ozb.reshape(64, ng))
    np.testing.assert_array_equal(wdq[torch.from_numpy(rows).to(cuda_device)].cpu().numpy(), owdq)
    # the layer-output error (||X d||^2 = T d H d^T) against round-to-nearest in the same format, on those rows.
    # Config 5's activations are independent across channels, so with T >> K the Hessian is close to diagonal and
    # there is almost nothing for the error propagation to exploit (measured: 0.3 % better at K = 4096): the walk must
    # simply not be worse.  The correlated cases above (make_case) are where it has to win by a margin.
    c2, s2, z2 = oracle.quant_int4_asym(Wr.reshape(-1), 128)
    rtn = oracle.dequant_int4_asym(c2, s2, z2, Wr.size, 128).reshape(64, K)
    H64 = Hh.astype(np.float64)
    def err(d):
        d = d.astype(np.float64)
        return float(np.sqrt(np.einsum("rk,rk->", d @ H64, d)))
    assert err(Wr - owdq) <= 1.001 * err(Wr - rtn)


@pytest.mark.gpu
def test_gptq_factor_with_tensor_core_products_against_f64(cuda_device):
    """K = 2048 is the smallest size at which the factorisation's large products (trailing update of a 512-column panel,
    inverse level 1024) run on the bf16 tensor cores with three-way split operands: U against numpy's f64 factor."""
    import torch
    from castforge_b200 import device as D
    K, T = 2048, 8192
    W, X = make_case(77, 8, K, T)
    xd = torch.from_numpy(bf16_round(X)).to(cuda_device, torch.bfloat16)
    H = D.gptq_hessian(xd)
    U = D.gptq_prepare(H, 0.01).cpu().numpy()
    Hd = H.cpu().numpy().astype(np.float64)
    Hd[np.diag_indices(K)] += 0.01 * float(np.mean(np.diag(Hd)))
    Uref = np.linalg.cholesky(np.linalg.inv(Hd)).T
    assert np.all(np.diag(U) > 0) and float(np.abs(np.tril(U, -1)).max()) == 0.0
    assert np.abs(U - Uref).max() <= 1e-4 * np.abs(Uref).max()


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,T", [(64, 256, 1024), (200, 512, 2048), (8, 128, 256)])
def test_gptq_cuda_vs_oracle(oracle, cuda_device, N, K, T):
    import torch
    from castforge_b200 import device as D
    W, X = make_case(N + K, N, K, T)
    W, X = bf16_round(W), bf16_round(X)
    xd = torch.from_numpy(X).to(cuda_device, torch.bfloat16)
    wd = torch.from_numpy(W).to(cuda_device, torch.bfloat16)
    H = D.gptq_hessian(xd)
    Href = (X.astype(np.float64).T @ X.astype(np.float64)) / T
    assert np.abs(H.cpu().numpy() - Href).max() <= 1e-4 * np.abs(Href).max()
    U = D.gptq_prepare(H, 0.01)
    Hd = Href + 0.01 * np.mean(np.diag(Href)) * np.eye(K)
    Uref = np.linalg.cholesky(np.linalg.inv(Hd)).T
    assert np.abs(U.cpu().numpy() - Uref).max() <= 2e-3 * np.abs(Uref).max()
    codes, scales, zps, wdq = D.gptq_quantize(wd, U)
    torch.cuda.synchronize()
    oc, osc, oz, owdq = oracle.gptq(W, X)
    q = unpack(codes.cpu().numpy(), N * K)
    assert (q != unpack(oc, N * K)).mean() < 0.02
    assert (scales.cpu().numpy().view(np.uint16) != osc).mean() < 0.02
    wdq = wdq.cpu().numpy()
    # the codes, scales and zero points decode to the returned matrix, bit for bit
    np.testing.assert_array_equal(
        oracle.dequant_int4_asym(codes.cpu().numpy(), scales.cpu().numpy().view(np.uint16), zps.cpu().numpy(), N * K, 128).reshape(N, K), wdq)
    e_gpu, e_or = out_err(X, W, wdq), out_err(X, W, owdq)
    assert abs(e_gpu - e_or) <= 0.02 * e_or
    c, s, z = oracle.quant_int4_asym(W.reshape(-1), 128)
    rtn = oracle.dequant_int4_asym(c, s, z, W.size, 128).reshape(N, K)
    assert e_gpu < 0.9 * out_err(X, W, rtn)


@pytest.mark.gpu
def test_gptq_cuda_layer_shape_property(oracle, cuda_device):
    """A layer-sized case (K = 4096): too large for the f64 oracle, checked through the property
    GPTQ exists for -- a lower layer output error than round-to-nearest in the same format."""
    import torch
    from castforge_b200 import device as D
    N, K, T = 512, 4096, 8192
    g = torch.Generator(device="cpu").manual_seed(5)
    mix = torch.randn(K, 64, generator=g) @ torch.randn(64, K, generator=g) / 8 + torch.eye(K)
    X = (torch.randn(T, K, generator=g) @ mix).to(cuda_device, torch.bfloat16)
    W = (torch.randn(N, K, generator=g) * 0.02).to(cuda_device, torch.bfloat16)
    U = D.gptq_prepare(D.gptq_hessian(X), 0.01)
    codes, scales, zps, wdq = D.gptq_quantize(W, U)
    c2, s2, z2 = D.quant_int4_asym(W.reshape(-1), 128)
    rtn = torch.from_numpy(oracle.dequant_int4_asym(c2.cpu().numpy(), s2.cpu().numpy().view(np.uint16), z2.cpu().numpy(), N * K, 128)).reshape(N, K).to(cuda_device)
    Xf, Wf = X.float(), W.float()
    e_gptq = torch.linalg.norm(Xf @ (Wf - wdq).T).item()
    e_rtn = torch.linalg.norm(Xf @ (Wf - rtn).T).item()
    assert e_gptq < 0.8 * e_rtn
    assert int(unpack(codes.cpu().numpy(), N * K).max()) <= 15
