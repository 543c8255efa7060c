"""Torch-tensor front end of the cfb200_* device entry points.

torch is used for device memory and streams only; every computation goes through the C ABI of
libcastforge_b200.so.  All functions run on the tensor's device and torch's current stream.
"""
from __future__ import annotations

import ctypes

import torch

from ._lib import check, load

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise TypeError(f"unsupported weight dtype {t.dtype}")
    return _DT[t.dtype]


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _src(t: torch.Tensor) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError("device entry points need CUDA tensors")
    return t.contiguous()


def quant_sym_tensor(w: torch.Tensor, bits: int = 8, codes: torch.Tensor | None = None,
                     scale_absmax: torch.Tensor | None = None):
    """A1: per-tensor symmetric quantization.  Returns (codes int8, scale_absmax f32[2])."""
    w = _src(w)
    with torch.cuda.device(w.device):
        if codes is None:
            codes = torch.empty(w.numel(), dtype=torch.int8, device=w.device)
        if scale_absmax is None:
            scale_absmax = torch.empty(2, dtype=torch.float32, device=w.device)
        check(load().cfb200_quant_sym_tensor(_p(w), _dt(w), w.numel(), bits, _p(codes), _p(scale_absmax), _stream(w)))
    return codes, scale_absmax


def quant_sym_tensors(ws: list[torch.Tensor], bits: int = 8, l2_group_bytes: int = 0, time_stages: bool = False):
    """A1 over a list of same-dtype device tensors in one call.

    Returns (codes list, scale_absmax f32[len, 2]) and, with time_stages, the per-launch events.
    """
    if not ws:
        return [], None
    ws = [_src(w) for w in ws]
    dev, dt = ws[0].device, _dt(ws[0])
    if any(w.device != dev or _dt(w) != dt for w in ws):
        raise ValueError("quant_sym_tensors needs tensors of one dtype on one device")
    lib = load()
    cnt = len(ws)
    with torch.cuda.device(dev):
        codes = [torch.empty(w.numel(), dtype=torch.int8, device=dev) for w in ws]
        sa = torch.empty((cnt, 2), dtype=torch.float32, device=dev)
        srcs = (ctypes.c_void_p * cnt)(*[w.data_ptr() for w in ws])
        outs = (ctypes.c_void_p * cnt)(*[c.data_ptr() for c in codes])
        ns = (ctypes.c_size_t * cnt)(*[w.numel() for w in ws])
        events, evp = None, None
        if time_stages:
            nst = ctypes.c_int32(0)
            check(lib.cfb200_quant_sym_tensors_plan(cnt, ns, dt, l2_group_bytes, ctypes.byref(nst)))
            events = [torch.cuda.Event(enable_timing=True) for _ in range(nst.value + 1)]
            for e in events:
                e.record(torch.cuda.current_stream(dev))  # materialise the handles
            evp = (ctypes.c_void_p * len(events))(*[e.cuda_event for e in events])
        check(lib.cfb200_quant_sym_tensors(cnt, srcs, dt, ns, bits, outs, _p(sa), l2_group_bytes, evp, _stream(ws[0])))
    return (codes, sa, events) if time_stages else (codes, sa)


def fakequant_tensor(w: torch.Tensor, bits: int = 8):
    """A6 (QAT-STE): returns (out f32, scale_absmax f32[2])."""
    w = _src(w)
    assert w.dtype == torch.float32
    with torch.cuda.device(w.device):
        out = torch.empty_like(w)
        sa = torch.empty(2, dtype=torch.float32, device=w.device)
        check(load().cfb200_fakequant_tensor(_p(w), w.numel(), bits, _p(out), _p(sa), _stream(w)))
    return out, sa


def absmax(w: torch.Tensor) -> torch.Tensor:
    w = _src(w)
    with torch.cuda.device(w.device):
        out = torch.empty(1, dtype=torch.float32, device=w.device)
        check(load().cfb200_absmax(_p(w), _dt(w), w.numel(), _p(out), _stream(w)))
    return out


def quant_sym_apply(w: torch.Tensor, absmax_dev: torch.Tensor, bits: int = 8):
    """A1 apply step with a given absmax (one device f32): returns (codes int8, scale_absmax f32[2])."""
    w = _src(w)
    assert absmax_dev.is_cuda and absmax_dev.dtype == torch.float32 and absmax_dev.numel() >= 1
    with torch.cuda.device(w.device):
        codes = torch.empty(w.numel(), dtype=torch.int8, device=w.device)
        sa = torch.empty(2, dtype=torch.float32, device=w.device)
        check(load().cfb200_quant_sym_apply(_p(w), _dt(w), w.numel(), bits, _p(absmax_dev), _p(codes), _p(sa), _stream(w)))
    return codes, sa


def smoothquant_apply(w: torch.Tensor, bits: int, smooth_scale: float, eff_qscale: float) -> torch.Tensor:
    w = _src(w)
    assert w.dtype == torch.float32
    with torch.cuda.device(w.device):
        out = torch.empty_like(w)
        check(load().cfb200_smoothquant_apply(_p(w), w.numel(), bits, smooth_scale, eff_qscale, _p(out), _stream(w)))
    return out


def quant_per_channel(w: torch.Tensor, bits: int = 8):
    """E1: per-row symmetric quantization of a [rows, cols] matrix -> (codes int8, scales f32[rows])."""
    w = _src(w)
    rows, cols = w.shape
    with torch.cuda.device(w.device):
        codes = torch.empty((rows, cols), dtype=torch.int8, device=w.device)
        scales = torch.empty(rows, dtype=torch.float32, device=w.device)
        check(load().cfb200_quant_per_channel(_p(w), _dt(w), rows, cols, bits, _p(codes), _p(scales), _stream(w)))
    return codes, scales


def select_kth_abs(w: torch.Tensor, salient_ratio: float, single_pass: bool = True):
    """A2 threshold: (thr f32[1] on device, k).  single_pass: give the call the larger workspace that lets it read a
    large tensor once (sample, bracket, candidates) instead of three times; the result is the same exact value."""
    w = _src(w)
    assert w.dtype == torch.float32
    lib = load()
    with torch.cuda.device(w.device):
        nbytes = lib.cfb200_select_kth_workspace_bytes_for(w.numel()) if single_pass else lib.cfb200_select_kth_workspace_bytes()
        ws = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
        thr = torch.empty(1, dtype=torch.float32, device=w.device)
        k = ctypes.c_uint64(0)
        check(lib.cfb200_select_kth_abs(_p(w), w.numel(), salient_ratio, _p(thr), ctypes.byref(k), _p(ws), ws.numel(), _stream(w)))
    return thr, int(k.value)


def fakequant_group(w: torch.Tensor, bits: int = 4, group_size: int = 32, salient_ratio: float = 0.01,
                    awq_salient: bool = True):
    """A2: returns (out f32, thr tensor or None, k)."""
    w = _src(w)
    assert w.dtype == torch.float32
    thr, k = (select_kth_abs(w, salient_ratio) if awq_salient else (None, 0))
    with torch.cuda.device(w.device):
        out = torch.empty_like(w)
        check(load().cfb200_fakequant_group(_p(w), w.numel(), bits, group_size, int(awq_salient), _p(thr), _p(out), _stream(w)))
    return out, thr, k


def fakequant_fp8grid(w: torch.Tensor, block_size: int = 32, e5m2: bool = False, mxfp8: bool = True) -> torch.Tensor:
    w = _src(w)
    assert w.dtype == torch.float32
    with torch.cuda.device(w.device):
        out = torch.empty_like(w)
        check(load().cfb200_fakequant_fp8grid(_p(w), w.numel(), block_size, int(e5m2), int(mxfp8), _p(out), _stream(w)))
    return out


def fakequant_e2m1(w: torch.Tensor, block: int = 16) -> torch.Tensor:
    w = _src(w)
    assert w.dtype == torch.float32
    with torch.cuda.device(w.device):
        out = torch.empty_like(w)
        check(load().cfb200_fakequant_e2m1(_p(w), w.numel(), block, _p(out), _stream(w)))
    return out


def fwht_cols_(w: torch.Tensor, block_size: int) -> int:
    """A5, in place on a contiguous [K, N] f32 matrix.  Returns the block used (0 = untouched)."""
    assert w.is_cuda and w.is_contiguous() and w.dtype == torch.float32 and w.dim() == 2
    applied = ctypes.c_uint64(0)
    with torch.cuda.device(w.device):
        check(load().cfb200_fwht_cols(_p(w), w.shape[0], w.shape[1], block_size, ctypes.byref(applied), _stream(w)))
    return int(applied.value)


def quant_int4_asym(w: torch.Tensor, group: int = 128):
    """E2: returns (codes u8[ceil(n/2)], scales f16 bits as int16[ngroups], zero_points u8[ceil(ngroups/2)])."""
    w = _src(w)
    n = w.numel()
    ng = (n + group - 1) // group
    with torch.cuda.device(w.device):
        codes = torch.empty((n + 1) // 2, dtype=torch.uint8, device=w.device)
        scales = torch.empty(ng, dtype=torch.float16, device=w.device)
        zps = torch.empty((ng + 1) // 2, dtype=torch.uint8, device=w.device)
        check(load().cfb200_quant_int4_asym(_p(w), _dt(w), n, group, _p(codes), _p(scales), _p(zps), _stream(w)))
    return codes, scales, zps


def quant_nf4(w: torch.Tensor, block: int = 64, dq_block: int = 256, workspace: torch.Tensor | None = None):
    """E3: returns (codes u8, absmax8 u8[nblocks], absmax2 f32[nsuper])."""
    w = _src(w)
    n = w.numel()
    nb = (n + block - 1) // block
    nsb = (nb + dq_block - 1) // dq_block
    lib = load()
    with torch.cuda.device(w.device):
        codes = torch.empty((n + 1) // 2, dtype=torch.uint8, device=w.device)
        a8 = torch.empty(nb, dtype=torch.uint8, device=w.device)
        a2 = torch.empty(nsb, dtype=torch.float32, device=w.device)
        if workspace is None:
            workspace = torch.empty(max(1, lib.cfb200_quant_nf4_workspace_bytes(n, block)), dtype=torch.uint8, device=w.device)
        check(lib.cfb200_quant_nf4(_p(w), _dt(w), n, block, dq_block, _p(codes), _p(a8), _p(a2), _p(workspace), workspace.numel(), _stream(w)))
    return codes, a8, a2


def quant_nf4_tensors(ws: list[torch.Tensor], block: int = 64, dq_block: int = 256):
    """E3 over a list of same-dtype device tensors in two launches.  Returns a list of (codes, absmax8, absmax2)."""
    if not ws:
        return []
    ws = [_src(w) for w in ws]
    dev, dt = ws[0].device, _dt(ws[0])
    lib = load()
    cnt = len(ws)
    with torch.cuda.device(dev):
        outs = []
        for w in ws:
            n = w.numel()
            nb = (n + block - 1) // block
            outs.append((torch.empty((n + 1) // 2, dtype=torch.uint8, device=dev), torch.empty(nb, dtype=torch.uint8, device=dev),
                         torch.empty((nb + dq_block - 1) // dq_block, dtype=torch.float32, device=dev)))
        ns = (ctypes.c_size_t * cnt)(*[w.numel() for w in ws])
        arr = lambda xs: (ctypes.c_void_p * cnt)(*[x.data_ptr() for x in xs])
        need = lib.cfb200_quant_nf4_tensors_workspace_bytes(cnt, ns, block)
        wsb = torch.empty(need + 256, dtype=torch.uint8, device=dev)
        wp = ctypes.c_void_p(wsb.data_ptr() + (-wsb.data_ptr()) % 256)
        check(lib.cfb200_quant_nf4_tensors(cnt, arr(ws), dt, ns, block, dq_block, arr([o[0] for o in outs]), arr([o[1] for o in outs]),
                                           arr([o[2] for o in outs]), wp, need, _stream(ws[0])))
    return outs


def cast_e4m3_rows(x: torch.Tensor):
    """E4 per-row (per-token) cast of [rows, cols] -> (codes u8, scales f32[rows])."""
    x = _src(x)
    rows, cols = x.shape
    with torch.cuda.device(x.device):
        codes = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
        scales = torch.empty(rows, dtype=torch.float32, device=x.device)
        check(load().cfb200_cast_e4m3_rows(_p(x), _dt(x), rows, cols, _p(codes), _p(scales), _stream(x)))
    return codes, scales


def cast_e4m3_tensor(w: torch.Tensor):
    """E4 per-tensor cast -> (codes u8 like w, scale_absmax f32[2])."""
    w = _src(w)
    with torch.cuda.device(w.device):
        codes = torch.empty(w.shape, dtype=torch.uint8, device=w.device)
        sa = torch.empty(2, dtype=torch.float32, device=w.device)
        check(load().cfb200_cast_e4m3_tensor(_p(w), _dt(w), w.numel(), _p(codes), _p(sa), _stream(w)))
    return codes, sa


# ---- execute side (interpreter semantics, f32) -------------------------------------------------
EPILOGUES = {None: 0, "none": 0, "bias": 1, "bias_relu": 2, "relu": 2, "bias_tanh": 3, "tanh": 3, "bias_silu": 4,
             "silu": 4, "bias_gelu": 5, "gelu": 5, "bias_scale": 6}


def cast_e4m3_tensors(ws: list[torch.Tensor], l2_group_bytes: int = 0):
    """E4 per-tensor E4M3FN cast over a list of same-dtype device tensors in one cooperative launch.
    Returns (codes list, scale_absmax f32[len, 2])."""
    if not ws:
        return [], None
    ws = [_src(w) for w in ws]
    dev, dt = ws[0].device, _dt(ws[0])
    cnt = len(ws)
    with torch.cuda.device(dev):
        codes = [torch.empty(w.numel(), dtype=torch.uint8, device=dev) for w in ws]
        sa = torch.empty((cnt, 2), dtype=torch.float32, device=dev)
        srcs = (ctypes.c_void_p * cnt)(*[w.data_ptr() for w in ws])
        outs = (ctypes.c_void_p * cnt)(*[c.data_ptr() for c in codes])
        ns = (ctypes.c_size_t * cnt)(*[w.numel() for w in ws])
        check(load().cfb200_cast_e4m3_tensors(cnt, srcs, dt, ns, outs, _p(sa), l2_group_bytes, _stream(ws[0])))
    return codes, sa


def _f32dev(t):
    assert t.is_cuda and t.dtype == torch.float32
    return t.contiguous()


def matmul_f32(a: torch.Tensor, b: torch.Tensor, packed_rhs: bool = False, epilogue=None, bias=None, z=None) -> torch.Tensor:
    """A8: the interpreter's f32 GEMM, bit-exact (ascending k, unfused multiply/add)."""
    a, b = _f32dev(a), _f32dev(b)
    M, K = a.shape
    N = b.shape[0] if packed_rhs else b.shape[1]
    with torch.cuda.device(a.device):
        c = torch.empty((M, N), dtype=torch.float32, device=a.device)
        bias_c = _f32dev(bias) if bias is not None else None
        z_c = _f32dev(z) if z is not None else None
        check(load().cfb200_matmul_f32(_p(a), _p(b), M, N, K, int(packed_rhs), EPILOGUES[epilogue], _p(bias_c),
                                       bias_c.numel() if bias_c is not None else 0, _p(z_c), z_c.numel() if z_c is not None else 0,
                                       _p(c), _stream(a)))
    return c


def qmatmul_i8(a: torch.Tensor, wq: torch.Tensor, scale: float, zero_point: int = 0, packed_rhs: bool = False, epilogue=None,
               bias=None, z=None) -> torch.Tensor:
    """castforge.fused_qmatmul: int8 codes dequantized on the fly as (q - zp) * scale, then the same GEMM."""
    a = _f32dev(a)
    assert wq.is_cuda and wq.dtype == torch.int8
    wq = wq.contiguous()
    M, K = a.shape
    N = wq.shape[0] if packed_rhs else wq.shape[1]
    with torch.cuda.device(a.device):
        c = torch.empty((M, N), dtype=torch.float32, device=a.device)
        bias_c = _f32dev(bias) if bias is not None else None
        z_c = _f32dev(z) if z is not None else None
        check(load().cfb200_qmatmul_i8(_p(a), _p(wq), scale, zero_point, M, N, K, int(packed_rhs), EPILOGUES[epilogue], _p(bias_c),
                                       bias_c.numel() if bias_c is not None else 0, _p(z_c), z_c.numel() if z_c is not None else 0,
                                       _p(c), _stream(a)))
    return c


def dequant_i8(q: torch.Tensor, scale: float, zero_point: int = 0) -> torch.Tensor:
    q = q.contiguous()
    with torch.cuda.device(q.device):
        out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
        check(load().cfb200_dequant_i8(_p(q), q.numel(), scale, zero_point, _p(out), _stream(q)))
    return out


def static_quantize(x: torch.Tensor, scale_attr: float, bits: int = 8) -> torch.Tensor:
    x = _f32dev(x)
    with torch.cuda.device(x.device):
        out = torch.empty_like(x)
        check(load().cfb200_static_quantize(_p(x), x.numel(), scale_attr, bits, _p(out), _stream(x)))
    return out


def rmsnorm(x: torch.Tensor, weight=None, residual=None, eps: float = 1e-5) -> torch.Tensor:
    x = _f32dev(x)
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    with torch.cuda.device(x.device):
        out = torch.empty_like(x)
        w = _f32dev(weight) if weight is not None else None
        r = _f32dev(residual) if residual is not None else None
        check(load().cfb200_rmsnorm(_p(x), _p(r), _p(w), w.numel() if w is not None else 0, rows, cols, eps, _p(out), _stream(x)))
    return out


def rope(x: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor) -> torch.Tensor:
    x, cos_t, sin_t = _f32dev(x), _f32dev(cos_t), _f32dev(sin_t)
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    with torch.cuda.device(x.device):
        out = torch.empty_like(x)
        check(load().cfb200_rope(_p(x), _p(cos_t), _p(sin_t), rows, cols, _p(out), _stream(x)))
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    gate, up = _f32dev(gate), _f32dev(up)
    with torch.cuda.device(gate.device):
        out = torch.empty_like(gate)
        check(load().cfb200_swiglu(_p(gate), _p(up), gate.numel(), _p(out), _stream(gate)))
    return out


def attention_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, scale: float, mask=None) -> torch.Tensor:
    """Multi-head attention over [seq, heads*d] activations (heads are column slices)."""
    q, k, v = _f32dev(q), _f32dev(k), _f32dev(v)
    seq_q, hid = q.shape
    seq_kv = k.shape[0]
    d = hid // heads
    with torch.cuda.device(q.device):
        out = torch.empty_like(q)
        m = _f32dev(mask) if mask is not None else None
        check(load().cfb200_attention(_p(q), _p(k), _p(v), _p(m), heads, seq_q, seq_kv, d, d, hid, hid, hid, hid, d, d, d, d,
                                      scale, _p(out), _stream(q)))
    return out


# ---- tensor-core GEMMs ---------------------------------------------------------------------------
class DeviceKernelError(RuntimeError):
    """A kernel reported an error status (a bounded wait ran out)."""


def _check_flag(flag: torch.Tensor, what: str):
    code = int(flag.item())  # synchronises
    if code != 0:
        raise DeviceKernelError(f"{what}: kernel error status {code}")


def gemm_fp8(a_codes: torch.Tensor, a_scales, w_codes: torch.Tensor, w_scale: float, out_f32: bool = False, check: bool = True):
    """C[M,N] = (A_e4m3 @ W_e4m3^T) * a_scales[:,None] * w_scale; A [M,K], W [N,K] uint8 E4M3 codes."""
    assert a_codes.is_cuda and a_codes.dtype == torch.uint8 and w_codes.dtype == torch.uint8
    a_codes, w_codes = a_codes.contiguous(), w_codes.contiguous()
    M, K = a_codes.shape
    N = w_codes.shape[0]
    dev = a_codes.device
    with torch.cuda.device(dev):
        c = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        from ._lib import check as _chk
        _chk(load().cfb200_gemm_fp8(_p(a_codes), _p(a_scales), _p(w_codes), float(w_scale), M, N, K, _p(c), int(out_f32), _p(flag), _stream(a_codes)))
        if check:
            _check_flag(flag, "cfb200_gemm_fp8")
    return c


def gemm_bf16_nt(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, out_f32: bool = True, upper_only: bool = False, check: bool = True):
    """C = alpha * A @ B^T for bf16 A [M,K], B [N,K]."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    a, b = a.contiguous(), b.contiguous()
    M, K = a.shape
    N = b.shape[0]
    dev = a.device
    with torch.cuda.device(dev):
        c = torch.zeros((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        from ._lib import check as _chk
        _chk(load().cfb200_gemm_bf16_nt(_p(a), _p(b), M, N, K, float(alpha), _p(c), int(out_f32), int(upper_only), _p(flag), _stream(a)))
        if check:
            _check_flag(flag, "cfb200_gemm_bf16_nt")
    return c


def gemm_bf16_nt_into(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, triangle: int = 0, accumulate: bool = False):
    """c (f32, row-major, possibly a block of a wider matrix: any row stride) = or += alpha * a @ b^T for bf16 a [M,K], b [N,K]
    whose rows may be strided too (cfb200_gemm_bf16_nt_ex).  triangle: 0 all tiles, 1 / 2 only tiles touching the upper /
    lower triangle.  Returns c."""
    assert c.is_cuda and c.dtype == torch.float32 and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert c.stride(1) == 1 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = a.shape
    N = b.shape[0]
    assert c.shape == (M, N) and b.shape[1] == K
    with torch.cuda.device(c.device):
        flag = torch.zeros(1, dtype=torch.int32, device=c.device)
        from ._lib import check as _chk
        _chk(load().cfb200_gemm_bf16_nt_ex(_p(a), a.stride(0), _p(b), b.stride(0), M, N, K, float(alpha), _p(c), c.stride(0), 1, int(triangle),
                                           int(bool(accumulate)), _p(flag), _stream(c)))
        if int(flag.item()) != 0:
            raise RuntimeError("gemm_bf16_nt_into: a bounded wait ran out inside the kernel")
    return c


def gemm_w4a16(a: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, zps: torch.Tensor, N: int, group: int = 128,
               out_f32: bool = False, check: bool = True):
    """C[M,N] = A_bf16 @ dequant(W)^T with W [N,K] in the packed INT4 layout of quant_int4_asym."""
    assert a.is_cuda and a.dtype == torch.bfloat16
    a = a.contiguous()
    M, K = a.shape
    dev = a.device
    with torch.cuda.device(dev):
        c = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        from ._lib import check as _chk
        ws = torch.empty(load().cfb200_gemm_w4a16_workspace_bytes(M, N, K), dtype=torch.uint8, device=dev)
        _chk(load().cfb200_gemm_w4a16(_p(a), _p(codes), _p(scales), _p(zps), M, N, K, group, _p(c), int(out_f32), _p(ws), ws.numel(),
                                      _p(flag), _stream(a)))
        if check:
            _check_flag(flag, "cfb200_gemm_w4a16")
    return c


def gemm_w4a16_static_quantize(a: torch.Tensor, a_scale: float, a_bits: int, codes: torch.Tensor, scales: torch.Tensor, zps: torch.Tensor,
                               N: int, group: int = 128, out_f32: bool = False):
    """gemm_w4a16 with castforge.static_quantize{scale, bits} applied to the f32 / bf16 activations in the staging pass."""
    assert a.is_cuda and a.dtype in (torch.bfloat16, torch.float32)
    a = a.contiguous()
    M, K = a.shape
    dev = a.device
    with torch.cuda.device(dev):
        c = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        from ._lib import check as _chk
        ws = torch.empty(load().cfb200_gemm_w4a16_workspace_bytes(M, N, K), dtype=torch.uint8, device=dev)
        _chk(load().cfb200_gemm_w4a16_static_quantize(_p(a), _dt(a), float(a_scale), a_bits, _p(codes), _p(scales), _p(zps), M, N, K, group,
                                                      _p(c), int(out_f32), _p(ws), ws.numel(), _p(flag), _stream(a)))
        _check_flag(flag, "cfb200_gemm_w4a16_static_quantize")
    return c


def gemv_w4a16(a: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, zps: torch.Tensor, N: int, group: int = 128,
               out_f32: bool = False):
    """Decode-shape (M <= 16) W4A16 product; same operands as gemm_w4a16."""
    assert a.is_cuda and a.dtype == torch.bfloat16
    a = a.contiguous()
    M, K = a.shape
    with torch.cuda.device(a.device):
        c = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
        from ._lib import check as _chk
        _chk(load().cfb200_gemv_w4a16(_p(a), _p(codes), _p(scales), _p(zps), M, N, K, group, _p(c), int(out_f32), _stream(a)))
    return c


def gptq_hessian(x: torch.Tensor) -> torch.Tensor:
    """H [K,K] f32 = X^T X / T for bf16 calibration activations X [T,K]."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2
    x = x.contiguous()
    T, K = x.shape
    dev = x.device
    with torch.cuda.device(dev):
        h = torch.empty((K, K), dtype=torch.float32, device=dev)
        ws = torch.empty(load().cfb200_gptq_hessian_workspace_bytes(T, K), dtype=torch.uint8, device=dev)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        from ._lib import check as _chk
        _chk(load().cfb200_gptq_hessian(_p(x), T, K, _p(h), _p(ws), ws.numel(), _p(flag), _stream(x)))
        _check_flag(flag, "cfb200_gptq_hessian")
    return h


def gptq_prepare(h: torch.Tensor, damp_ratio: float = 0.01) -> torch.Tensor:
    """Upper Cholesky factor of the inverse of the damped Hessian."""
    assert h.is_cuda and h.dtype == torch.float32 and h.dim() == 2 and h.shape[0] == h.shape[1]
    h = h.contiguous()
    K = h.shape[0]
    with torch.cuda.device(h.device):
        u = torch.empty_like(h)
        ws = torch.empty(load().cfb200_gptq_prepare_workspace_bytes(K), dtype=torch.uint8, device=h.device)
        from ._lib import check as _chk
        _chk(load().cfb200_gptq_prepare(_p(h), K, float(damp_ratio), _p(u), _p(ws), ws.numel(), _stream(h)))
    return u


def gptq_quantize(w: torch.Tensor, u: torch.Tensor, want_dequant: bool = True):
    """GPTQ INT4 (group 128) of W [N,K] with the factor from gptq_prepare.  Returns codes, scales, zps, Wdq."""
    assert w.is_cuda and w.dim() == 2 and u.dtype == torch.float32
    w = w.contiguous()
    N, K = w.shape
    dev = w.device
    with torch.cuda.device(dev):
        codes = torch.empty(N * K // 2, dtype=torch.uint8, device=dev)
        ng = N * (K // 128)
        scales = torch.empty(ng, dtype=torch.uint16, device=dev)
        zps = torch.empty((ng + 1) // 2, dtype=torch.uint8, device=dev)
        wdq = torch.empty((N, K), dtype=torch.float32, device=dev) if want_dequant else None
        ws = torch.empty(load().cfb200_gptq_quantize_workspace_bytes(N, K), dtype=torch.uint8, device=dev)
        from ._lib import check as _chk
        _chk(load().cfb200_gptq_quantize(_p(w), _dt(w), N, K, _p(u), _p(codes), _p(scales), _p(zps), _p(wdq) if want_dequant else None,
                                         _p(ws), ws.numel(), _stream(w)))
    return codes, scales, zps, wdq


# ---- GGUF block formats -------------------------------------------------------------------------
def gguf_pack_q8_0(codes: torch.Tensor, scale: float) -> torch.Tensor:
    """Per-tensor INT8 codes + scale -> GGUF Q8_0 blocks (34 bytes per 32 codes)."""
    assert codes.is_cuda and codes.dtype == torch.int8
    codes = codes.contiguous().reshape(-1)
    n = codes.numel()
    with torch.cuda.device(codes.device):
        out = torch.empty(load().cfb200_gguf_q8_0_bytes(n), dtype=torch.uint8, device=codes.device)
        check(load().cfb200_gguf_pack_q8_0(_p(codes), n, float(scale), _p(out), _stream(codes)))
    return out


def gguf_unpack(blocks: torch.Tensor, n: int, kind: str = "q8_0") -> torch.Tensor:
    """GGUF Q8_0 / Q4_0 blocks -> n f32 values."""
    assert blocks.is_cuda and blocks.dtype == torch.uint8
    blocks = blocks.contiguous()
    with torch.cuda.device(blocks.device):
        out = torch.empty(n, dtype=torch.float32, device=blocks.device)
        fn = load().cfb200_gguf_unpack_q8_0 if kind == "q8_0" else load().cfb200_gguf_unpack_q4_0
        check(fn(_p(blocks), n, _p(out), _stream(blocks)))
    return out


# ---- KV-cache page codecs ------------------------------------------------------------------------
KV_SCOPES = {"tensor": 0, "layer_head": 1, "page_head": 2}


def kv_encode_k16v8(k: torch.Tensor, v: torch.Tensor, scope: str = "page_head"):
    """K16/V8 page codec over [num_pages, page_tokens, num_kv_heads, head_dim] caches.

    Returns (k_f16_bits int16, v_codes int8, v_scales f32)."""
    k, v = _src(k), _src(v)
    if k.shape != v.shape or k.dim() != 4 or k.dtype != v.dtype:
        raise ValueError("k and v must be 4-D caches of one shape and dtype")
    P, T, H, D = k.shape
    sc = KV_SCOPES[scope]
    with torch.cuda.device(k.device):
        kb = torch.empty(k.shape, dtype=torch.int16, device=k.device)
        vc = torch.empty(k.shape, dtype=torch.int8, device=k.device)
        vs = torch.empty(max(1, load().cfb200_kv_scale_count(sc, P, H)), dtype=torch.float32, device=k.device)
        check(load().cfb200_kv_encode_k16v8(_p(k), _p(v), _dt(k), P, T, H, D, sc, _p(kb), _p(vc), _p(vs), _stream(k)))
    return kb, vc, vs


def kv_decode_k16v8(kb: torch.Tensor, vc: torch.Tensor, vs: torch.Tensor, scope: str = "page_head"):
    """Inverse of kv_encode_k16v8: (k f32, v f32)."""
    assert kb.is_cuda and kb.dtype == torch.int16 and vc.dtype == torch.int8 and vs.dtype == torch.float32
    kb, vc, vs = kb.contiguous(), vc.contiguous(), vs.contiguous()
    P, T, H, D = kb.shape
    with torch.cuda.device(kb.device):
        ko = torch.empty(kb.shape, dtype=torch.float32, device=kb.device)
        vo = torch.empty(kb.shape, dtype=torch.float32, device=kb.device)
        check(load().cfb200_kv_decode_k16v8(_p(kb), _p(vc), _p(vs), P, T, H, D, KV_SCOPES[scope], _p(ko), _p(vo), _stream(kb)))
    return ko, vo


def e4m3_slice_encode(x: torch.Tensor) -> torch.Tensor:
    """f32 slice -> float8_e4m3fn bytes (no scale)."""
    assert x.is_cuda and x.dtype == torch.float32
    x = x.contiguous().reshape(-1)
    with torch.cuda.device(x.device):
        out = torch.empty(x.numel(), dtype=torch.uint8, device=x.device)
        check(load().cfb200_e4m3_slice_encode(_p(x), x.numel(), _p(out), _stream(x)))
    return out


def e4m3_slice_encode_ref(x: torch.Tensor) -> torch.Tensor:
    """The reference codec byte for byte (its log2f binade slips included)."""
    x = _src(x)
    assert x.dtype == torch.float32
    with torch.cuda.device(x.device):
        out = torch.empty(x.numel(), dtype=torch.uint8, device=x.device)
        check(load().cfb200_e4m3_slice_encode_ref(_p(x), x.numel(), _p(out), _stream(x)))
    return out


def e4m3_slice_decode(codes: torch.Tensor) -> torch.Tensor:
    """float8_e4m3fn bytes -> f32."""
    assert codes.is_cuda and codes.dtype == torch.uint8
    codes = codes.contiguous().reshape(-1)
    with torch.cuda.device(codes.device):
        out = torch.empty(codes.numel(), dtype=torch.float32, device=codes.device)
        check(load().cfb200_e4m3_slice_decode(_p(codes), codes.numel(), _p(out), _stream(codes)))
    return out


# ---- weight surgery upstream of quantize ----------------------------------------------------------
MERGE_METHODS = {"linear": 0, "slerp": 1, "ties": 2}


def merge_f32(a: torch.Tensor, b: torch.Tensor, method: str = "linear", t: float = 0.5, want_coef: bool = False):
    """merge_f32_tensors on two f32 device tensors of one shape.  Returns out (and the two coefficients used)."""
    a, b = _src(a), _src(b)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.shape != b.shape:
        raise ValueError("merge_f32 needs two f32 tensors of one shape")
    with torch.cuda.device(a.device):
        out = torch.empty_like(a)
        coef = torch.empty(2, dtype=torch.float32, device=a.device) if want_coef else None
        ws = torch.empty(load().cfb200_merge_workspace_bytes(), dtype=torch.uint8, device=a.device)
        check(load().cfb200_merge_f32(_p(a), _p(b), a.numel(), MERGE_METHODS[method], float(t), _p(out), _p(coef), _p(ws), ws.numel(),
                                      _stream(a)))
    return (out, coef) if want_coef else out


def task_vector_merge(base: torch.Tensor, finetuned: list[torch.Tensor], lam: float = 1.0, drop_rate: float = 0.0) -> torch.Tensor:
    """base + sum lam * DARE-pruned (finetuned[c] - base), all f32 device tensors of one shape."""
    base = _src(base)
    fts = [_src(f) for f in finetuned]
    if base.dtype != torch.float32 or any(f.dtype != torch.float32 or f.shape != base.shape for f in fts):
        raise ValueError("task_vector_merge needs f32 tensors of one shape")
    n = base.numel()
    with torch.cuda.device(base.device):
        out = torch.empty_like(base)
        ws = torch.empty(load().cfb200_task_vector_merge_workspace_bytes(n), dtype=torch.uint8, device=base.device)
        ptrs = (ctypes.c_void_p * max(1, len(fts)))(*[f.data_ptr() for f in fts])
        check(load().cfb200_task_vector_merge(_p(base), ptrs, len(fts), n, float(lam), float(drop_rate), _p(out), _p(ws), ws.numel(),
                                              _stream(base)))
    return out


def prune_2to4_(w: torch.Tensor) -> torch.Tensor:
    """2:4 magnitude mask, in place, over the flattened f32 tensor."""
    assert w.is_cuda and w.dtype == torch.float32 and w.is_contiguous()
    with torch.cuda.device(w.device):
        check(load().cfb200_prune_2to4(_p(w), w.numel(), _stream(w)))
    return w


def prune_columns_l1(w: torch.Tensor, sparsity: float | None = None, keep_cols: int | None = None):
    """Structured L1 column pruning of a 2-D f32 matrix.  Returns (pruned [rows, keep], kept column indices int32)."""
    w = _src(w)
    assert w.dtype == torch.float32 and w.dim() == 2
    rows, cols = w.shape
    if keep_cols is None:
        keep_cols = load().cfb200_prune_keep_cols(cols, float(0.5 if sparsity is None else sparsity))
    keep = min(max(int(keep_cols), 1), cols)
    with torch.cuda.device(w.device):
        out = torch.empty((rows, keep), dtype=torch.float32, device=w.device)
        kept = torch.empty(keep, dtype=torch.int32, device=w.device)
        ws = torch.empty(load().cfb200_prune_columns_workspace_bytes(cols), dtype=torch.uint8, device=w.device)
        check(load().cfb200_prune_columns_l1(_p(w), rows, cols, keep, _p(out), _p(kept), _p(ws), ws.numel(), _stream(w)))
    return out, kept


def transpose_f32(w: torch.Tensor) -> torch.Tensor:
    """[K, N] -> [N, K] (pack-weights)."""
    w = _src(w)
    assert w.dtype == torch.float32 and w.dim() == 2
    K, N = w.shape
    with torch.cuda.device(w.device):
        out = torch.empty((N, K), dtype=torch.float32, device=w.device)
        check(load().cfb200_transpose_f32(_p(w), K, N, _p(out), _stream(w)))
    return out


def lora_bake_(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    """W [k, n] += alpha * (A [k, r] @ B [r, n]) in place, with the reference's summation order."""
    assert w.is_cuda and w.dtype == torch.float32 and w.is_contiguous() and w.dim() == 2
    a, b = _src(a), _src(b)
    k, n = w.shape
    r = a.shape[1]
    assert a.shape == (k, r) and b.shape == (r, n) and a.dtype == b.dtype == torch.float32
    with torch.cuda.device(w.device):
        check(load().cfb200_lora_bake(_p(w), _p(a), _p(b), k, n, r, float(alpha), _stream(w)))
    return w


def column_norms(w: torch.Tensor) -> torch.Tensor:
    """max(||column||_2, 1e-8) of a 2-D f32 matrix, summed in row order."""
    w = _src(w)
    assert w.dtype == torch.float32 and w.dim() == 2
    with torch.cuda.device(w.device):
        out = torch.empty(w.shape[1], dtype=torch.float32, device=w.device)
        check(load().cfb200_column_norms(_p(w), w.shape[0], w.shape[1], _p(out), _stream(w)))
    return out


def dora_renorm_(w: torch.Tensor, orig_mags: torch.Tensor | None = None) -> torch.Tensor:
    """Every column becomes orig_mags[j] * (column / its norm), in place.  Returns the norms."""
    assert w.is_cuda and w.dtype == torch.float32 and w.is_contiguous() and w.dim() == 2
    with torch.cuda.device(w.device):
        norms = torch.empty(w.shape[1], dtype=torch.float32, device=w.device)
        check(load().cfb200_dora_renorm(_p(w), w.shape[0], w.shape[1], _p(orig_mags), _p(norms), _stream(w)))
    return norms


def fold_scale_(w: torch.Tensor, scale: torch.Tensor, axis: int) -> torch.Tensor:
    """W[r][c] *= scale[(r if axis == 0 else c) % len(scale)] in place (norm / batch-norm folding)."""
    assert w.is_cuda and w.dtype == torch.float32 and w.is_contiguous() and w.dim() == 2
    scale = _src(scale)
    assert scale.dtype == torch.float32
    with torch.cuda.device(w.device):
        check(load().cfb200_fold_scale(_p(w), w.shape[0], w.shape[1], _p(scale), scale.numel(), int(axis), _stream(w)))
    return w
