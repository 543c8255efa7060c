"""numpy front end of the CPU oracle (oracle/libcf_oracle.so).  Test infrastructure only."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
SO = ROOT / "oracle" / "libcf_oracle.so"

c_f = ctypes.c_float
c_sz = ctypes.c_size_t
c_i = ctypes.c_int
vp = ctypes.c_void_p


def _ptr(a):
    return a.ctypes.data_as(vp)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.cfo_f16_bits_to_f32.restype = c_f
        lib.cfo_f16_bits_to_f32.argtypes = [ctypes.c_uint16]
        lib.cfo_f32_to_f16_bits.restype = ctypes.c_uint16
        lib.cfo_f32_to_f16_bits.argtypes = [c_f]
        lib.cfo_bf16_bits_to_f32.restype = c_f
        lib.cfo_bf16_bits_to_f32.argtypes = [ctypes.c_uint16]
        lib.cfo_f32_to_bf16_bits.restype = ctypes.c_uint16
        lib.cfo_f32_to_bf16_bits.argtypes = [c_f]
        lib.cfo_parse_scale.restype = c_f
        lib.cfo_parse_scale.argtypes = [ctypes.c_char_p]
        lib.cfo_format_scale.argtypes = [c_f, ctypes.c_char_p]
        lib.cfo_e4m3_encode_ref.restype = ctypes.c_uint8
        lib.cfo_e4m3_encode_ref.argtypes = [c_f]
        lib.cfo_e4m3_encode_rne.restype = ctypes.c_uint8
        lib.cfo_e4m3_encode_rne.argtypes = [c_f]
        lib.cfo_e4m3_decode.restype = c_f
        lib.cfo_e4m3_decode.argtypes = [ctypes.c_uint8]
        lib.cfo_fwht_cols.restype = ctypes.c_uint64
        lib.cfo_max_threads.restype = c_i

    # ---- helpers -------------------------------------------------------------------------
    @staticmethod
    def _f32(a):
        return np.ascontiguousarray(a, dtype=np.float32).ravel()

    def max_threads(self):
        return int(self.lib.cfo_max_threads())

    def to_f32(self, raw: np.ndarray, dtype: int, threads=1):
        """raw: float32 array (dtype 0) or uint16 bit patterns (dtype 1 f16, 2 bf16)."""
        raw = np.ascontiguousarray(raw).ravel()
        out = np.empty(raw.size, np.float32)
        self.lib.cfo_to_f32(_ptr(raw), c_i(dtype), c_sz(raw.size), _ptr(out), c_i(threads))
        return out

    def format_scale(self, s: float) -> str:
        buf = ctypes.create_string_buffer(64)
        self.lib.cfo_format_scale(c_f(s), buf)
        return buf.value.decode()

    def parse_scale(self, s: str) -> float:
        return float(self.lib.cfo_parse_scale(s.encode()))

    # ---- A1 / A6 ---------------------------------------------------------------------------
    def quant_sym(self, v, bits, threads=1):
        v = self._f32(v)
        q = np.empty(v.size, np.int8)
        sc = c_f()
        buf = ctypes.create_string_buffer(64)
        self.lib.cfo_quant_sym(_ptr(v), c_sz(v.size), c_i(bits), _ptr(q), ctypes.byref(sc), buf, c_i(threads))
        return q, np.float32(sc.value), buf.value.decode()

    def fakequant_tensor(self, v, bits, threads=1):
        v = self._f32(v)
        out = np.empty_like(v)
        sc = c_f()
        self.lib.cfo_fakequant_tensor(_ptr(v), c_sz(v.size), c_i(bits), _ptr(out), ctypes.byref(sc), c_i(threads))
        return out, np.float32(sc.value)

    def smoothquant(self, v, bits, alpha, threads=1):
        v = self._f32(v)
        out = np.empty_like(v)
        params = np.empty(2, np.float32)
        self.lib.cfo_smoothquant(_ptr(v), c_sz(v.size), c_i(bits), c_f(alpha), _ptr(out), _ptr(params), c_i(threads))
        return out, params

    # ---- A2 ----------------------------------------------------------------------------------
    def salient_threshold(self, v, ratio, faithful=0):
        v = self._f32(v)
        thr = c_f()
        k = ctypes.c_uint64()
        self.lib.cfo_salient_threshold(_ptr(v), c_sz(v.size), c_f(ratio), c_i(faithful), ctypes.byref(thr), ctypes.byref(k))
        return np.float32(thr.value), int(k.value)

    def fakequant_group(self, v, bits, group, ratio, awq, faithful=0, threads=1):
        v = self._f32(v)
        out = np.empty_like(v)
        thr = c_f()
        k = ctypes.c_uint64()
        self.lib.cfo_fakequant_group(_ptr(v), c_sz(v.size), c_i(bits), c_sz(group), c_f(ratio), c_i(int(awq)),
                                     c_i(faithful), _ptr(out), ctypes.byref(thr), ctypes.byref(k), c_i(threads))
        return out, np.float32(thr.value), int(k.value)

    # ---- A3 / A4 / A5 ----------------------------------------------------------------------------
    def fakequant_fp8grid(self, v, block, e5m2, mxfp8, threads=1):
        v = self._f32(v)
        out = np.empty_like(v)
        self.lib.cfo_fakequant_fp8grid(_ptr(v), c_sz(v.size), c_sz(block), c_i(int(e5m2)), c_i(int(mxfp8)), _ptr(out), c_i(threads))
        return out

    def fakequant_e2m1(self, v, blk, threads=1):
        v = self._f32(v)
        out = np.empty_like(v)
        self.lib.cfo_fakequant_e2m1(_ptr(v), c_sz(v.size), c_sz(blk), _ptr(out), c_i(threads))
        return out

    def fwht_cols(self, w, K, N, block, threads=1):
        w = self._f32(w).copy()
        b = self.lib.cfo_fwht_cols(_ptr(w), c_sz(K), c_sz(N), c_sz(block), c_i(threads))
        return w.reshape(K, N), int(b)

    # ---- A8 ----------------------------------------------------------------------------------
    def dequant_i8(self, q, sc, zp=0):
        q = np.ascontiguousarray(q, np.int8).ravel()
        out = np.empty(q.size, np.float32)
        self.lib.cfo_dequant_i8(_ptr(q), c_sz(q.size), c_f(sc), ctypes.c_int64(zp), _ptr(out))
        return out

    def matmul_2d(self, A, B, M, N, K, packed_rhs=False, epilogue=0, bias=None, z=None, threads=1):
        A = self._f32(A)
        B = self._f32(B)
        C = np.empty(M * N, np.float32)
        bias_a = self._f32(bias) if bias is not None else np.zeros(1, np.float32)
        z_a = self._f32(z) if z is not None else None
        self.lib.cfo_matmul_2d(_ptr(A), _ptr(B), c_sz(M), c_sz(N), c_sz(K), c_i(int(packed_rhs)), c_i(epilogue),
                               _ptr(bias_a), c_sz(bias_a.size), _ptr(z_a) if z_a is not None else vp(0),
                               c_sz(z_a.size if z_a is not None else 0), _ptr(C), c_i(threads))
        return C.reshape(M, N)

    def static_quantize(self, x, scale, bits):
        x = self._f32(x)
        out = np.empty_like(x)
        self.lib.cfo_static_quantize(_ptr(x), c_sz(x.size), c_f(scale), c_i(bits), _ptr(out))
        return out

    # ---- A9 ----------------------------------------------------------------------------------
    def rmsnorm(self, x, rows, cols, eps, res=None, w=None):
        x = self._f32(x)
        out = np.empty_like(x)
        r = self._f32(res) if res is not None else None
        ww = self._f32(w) if w is not None else None
        self.lib.cfo_rmsnorm(_ptr(x), _ptr(r) if r is not None else vp(0), _ptr(ww) if ww is not None else vp(0),
                             c_sz(ww.size if ww is not None else 0), c_sz(rows), c_sz(cols), c_f(eps), _ptr(out))
        return out.reshape(rows, cols)

    def rope(self, x, cs, sn, rows, cols):
        x = self._f32(x)
        out = np.empty_like(x)
        self.lib.cfo_rope(_ptr(x), _ptr(self._f32(cs)), _ptr(self._f32(sn)), c_sz(rows), c_sz(cols), _ptr(out))
        return out.reshape(rows, cols)

    def swiglu(self, g, u):
        g = self._f32(g)
        out = np.empty_like(g)
        self.lib.cfo_swiglu(_ptr(g), _ptr(self._f32(u)), c_sz(g.size), _ptr(out))
        return out

    def attention(self, q, k, v, mask, batch, seq_q, seq_kv, d_k, d_v, ld, hs, scale, out_size):
        """q/k/v/out share row stride ld and head stride hs (column-sliced heads)."""
        q, k, v = self._f32(q), self._f32(k), self._f32(v)
        out = np.zeros(out_size, np.float32)
        m = self._f32(mask) if mask is not None else None
        self.lib.cfo_attention(_ptr(q), _ptr(k), _ptr(v), _ptr(m) if m is not None else vp(0), c_i(batch), c_i(seq_q),
                               c_i(seq_kv), c_i(d_k), c_i(d_v), c_sz(ld), c_sz(ld), c_sz(ld), c_sz(ld), c_sz(hs), c_sz(hs),
                               c_sz(hs), c_sz(hs), c_f(scale), _ptr(out))
        return out

    # ---- E-schemes -----------------------------------------------------------------------------
    def quant_per_channel(self, v, rows, cols, bits, threads=1):
        v = self._f32(v)
        q = np.empty(rows * cols, np.int8)
        s = np.empty(rows, np.float32)
        self.lib.cfo_quant_per_channel(_ptr(v), c_sz(rows), c_sz(cols), c_i(bits), _ptr(q), _ptr(s), c_i(threads))
        return q.reshape(rows, cols), s

    def quant_int4_asym(self, v, group, threads=1):
        v = self._f32(v)
        n = v.size
        ng = (n + group - 1) // group
        codes = np.zeros((n + 1) // 2, np.uint8)
        scales = np.empty(ng, np.uint16)
        zps = np.zeros((ng + 1) // 2, np.uint8)
        self.lib.cfo_quant_int4_asym(_ptr(v), c_sz(n), c_sz(group), _ptr(codes), _ptr(scales), _ptr(zps), c_i(threads))
        return codes, scales, zps

    def dequant_int4_asym(self, codes, scales, zps, n, group):
        out = np.empty(n, np.float32)
        self.lib.cfo_dequant_int4_asym(_ptr(np.ascontiguousarray(codes)), _ptr(np.ascontiguousarray(scales)),
                                       _ptr(np.ascontiguousarray(zps)), c_sz(n), c_sz(group), _ptr(out))
        return out

    def quant_nf4(self, v, block, dq_block, threads=1):
        v = self._f32(v)
        n = v.size
        nb = (n + block - 1) // block
        codes = np.zeros((n + 1) // 2, np.uint8)
        a8 = np.empty(nb, np.uint8)
        a2 = np.empty((nb + dq_block - 1) // dq_block, np.float32)
        self.lib.cfo_quant_nf4(_ptr(v), c_sz(n), c_sz(block), c_sz(dq_block), _ptr(codes), _ptr(a8), _ptr(a2), c_i(threads))
        return codes, a8, a2

    def dequant_nf4(self, codes, a8, a2, n, block, dq_block):
        out = np.empty(n, np.float32)
        self.lib.cfo_dequant_nf4(_ptr(np.ascontiguousarray(codes)), _ptr(np.ascontiguousarray(a8)),
                                 _ptr(np.ascontiguousarray(a2)), c_sz(n), c_sz(block), c_sz(dq_block), _ptr(out))
        return out

    def nf4_levels(self):
        out = np.empty(16, np.float32)
        self.lib.cfo_nf4_levels(_ptr(out))
        return out

    def e4m3_encode_ref(self, x):
        return int(self.lib.cfo_e4m3_encode_ref(c_f(x)))

    def e4m3_encode_rne(self, x):
        return int(self.lib.cfo_e4m3_encode_rne(c_f(x)))

    def e4m3_decode(self, b):
        return float(self.lib.cfo_e4m3_decode(ctypes.c_uint8(b)))

    def cast_e4m3_rows(self, v, rows, cols, threads=1):
        v = self._f32(v)
        codes = np.empty(rows * cols, np.uint8)
        s = np.empty(rows, np.float32)
        self.lib.cfo_cast_e4m3_rows(_ptr(v), c_sz(rows), c_sz(cols), _ptr(codes), _ptr(s), c_i(threads))
        return codes.reshape(rows, cols), s

    def gemm_e4m3(self, A, sa, W, sw, M, N, K, threads=0):
        C = np.empty(M * N, np.float32)
        self.lib.cfo_gemm_e4m3(_ptr(np.ascontiguousarray(A, np.uint8)), _ptr(np.ascontiguousarray(sa, np.float32)),
                               _ptr(np.ascontiguousarray(W, np.uint8)), c_f(sw), c_sz(M), c_sz(N), c_sz(K), _ptr(C), c_i(threads))
        return C.reshape(M, N)

    def gemm_w4a16(self, A, codes, scales, zps, M, N, K, group, threads=0):
        C = np.empty(M * N, np.float32)
        self.lib.cfo_gemm_w4a16(_ptr(self._f32(A)), _ptr(np.ascontiguousarray(codes)), _ptr(np.ascontiguousarray(scales)),
                                _ptr(np.ascontiguousarray(zps)), c_sz(M), c_sz(N), c_sz(K), c_sz(group), _ptr(C), c_i(threads))
        return C.reshape(M, N)

    def gptq(self, W, X, group=128, damp=0.01, threads=0):
        """E5 in f64.  W [N,K], X [T,K] (f32 values).  Returns codes, scales, zps, Wdq."""
        W = np.ascontiguousarray(W, np.float32)
        X = np.ascontiguousarray(X, np.float32)
        N, K = W.shape
        T = X.shape[0]
        codes = np.zeros(N * K // 2, np.uint8)
        ng = N * (K // group)
        scales = np.zeros(ng, np.uint16)
        zps = np.zeros((ng + 1) // 2, np.uint8)
        wdq = np.empty((N, K), np.float32)
        self.lib.cfo_gptq.restype = ctypes.c_int
        rc = self.lib.cfo_gptq(_ptr(W), _ptr(X), c_sz(N), c_sz(K), c_sz(T), c_sz(group), ctypes.c_double(damp), _ptr(codes), _ptr(scales),
                               _ptr(zps), _ptr(wdq), c_i(threads))
        if rc:
            raise ValueError("Hessian not positive definite")
        return codes, scales, zps, wdq

    def gptq_walk_f32(self, W, U, want_dequant=False, threads=0):
        """E5 column walk in the device kernels' f32 operation order.  W [rows, K] f32 values, U [K, K] f32 (the factor
        the device computed).  Returns codes [rows * K / 2], scales u16 [rows * K / 128], zero points (one byte per
        group) and, on request, the dequantised rows."""
        W = np.ascontiguousarray(W, np.float32)
        U = np.ascontiguousarray(U, np.float32)
        rows, K = W.shape
        assert U.shape == (K, K) and K % 128 == 0
        codes = np.zeros(rows * K // 2, np.uint8)
        scales = np.zeros(rows * (K // 128), np.uint16)
        zps = np.zeros(rows * (K // 128), np.uint8)
        wdq = np.empty((rows, K), np.float32) if want_dequant else None
        self.lib.cfo_gptq_walk_f32.restype = None
        self.lib.cfo_gptq_walk_f32(_ptr(W), c_sz(rows), c_sz(K), _ptr(U), _ptr(codes), _ptr(scales), _ptr(zps),
                                   _ptr(wdq) if want_dequant else None, c_i(threads))
        return codes, scales, zps, wdq

    def gguf_pack_q8_0(self, codes, scale):
        codes = np.ascontiguousarray(codes, np.int8).reshape(-1)
        out = np.zeros(((max(codes.size, 1) + 31) // 32) * 34, np.uint8)
        self.lib.cfo_gguf_pack_q8_0.restype = ctypes.c_size_t
        nb = self.lib.cfo_gguf_pack_q8_0(_ptr(codes), c_sz(codes.size), c_f(scale), _ptr(out))
        assert nb == out.size
        return out

    def gguf_unpack(self, blocks, n, kind="q8_0"):
        blocks = np.ascontiguousarray(blocks, np.uint8)
        out = np.empty(n, np.float32)
        fn = self.lib.cfo_gguf_unpack_q8_0 if kind == "q8_0" else self.lib.cfo_gguf_unpack_q4_0
        fn(_ptr(blocks), c_sz(n), _ptr(out))
        return out

    def kv_encode_k16v8(self, k, v, scope):
        """k, v: f32 arrays [P, T, H, D]; scope 0 / 1 / 2.  Returns (k_bits u16, v_codes i8, v_scales f32)."""
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        P, T, H, D = k.shape
        slots = 1 if scope == 0 else H if scope == 1 else P * H
        kb = np.empty(k.shape, np.uint16)
        vc = np.empty(k.shape, np.int8)
        vs = np.empty(slots, np.float32)
        rc = self.lib.cfo_kv_encode_k16v8(_ptr(k), _ptr(v), c_sz(P), c_sz(T), c_sz(H), c_sz(D), ctypes.c_int(scope),
                                          _ptr(kb), _ptr(vc), _ptr(vs))
        assert rc == 0
        return kb, vc, vs

    def kv_decode_k16v8(self, kb, vc, vs, scope):
        kb = np.ascontiguousarray(kb, np.uint16)
        vc = np.ascontiguousarray(vc, np.int8)
        vs = np.ascontiguousarray(vs, np.float32)
        P, T, H, D = kb.shape
        ko = np.empty(kb.shape, np.float32)
        vo = np.empty(kb.shape, np.float32)
        self.lib.cfo_kv_decode_k16v8(_ptr(kb), _ptr(vc), _ptr(vs), c_sz(P), c_sz(T), c_sz(H), c_sz(D), ctypes.c_int(scope),
                                     _ptr(ko), _ptr(vo))
        return ko, vo

    def e4m3_slice_encode(self, x, which=1):
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        out = np.empty(x.size, np.uint8)
        self.lib.cfo_e4m3_slice_encode(_ptr(x), c_sz(x.size), ctypes.c_int(which), _ptr(out))
        return out

    def e4m3_slice_decode(self, codes):
        codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
        out = np.empty(codes.size, np.float32)
        self.lib.cfo_e4m3_slice_decode(_ptr(codes), c_sz(codes.size), _ptr(out))
        return out

    def merge_f32(self, a, b, method, t):
        """method 0 linear / 1 slerp / 2 ties.  Returns (out, coefficients used)."""
        a = np.ascontiguousarray(a, np.float32).reshape(-1)
        b = np.ascontiguousarray(b, np.float32).reshape(-1)
        out = np.empty(a.size, np.float32)
        coef = np.empty(2, np.float32)
        self.lib.cfo_merge_f32(_ptr(a), _ptr(b), c_sz(a.size), ctypes.c_int(method), c_f(t), _ptr(out), _ptr(coef))
        return out, coef

    def dare_prune(self, delta, drop_rate):
        delta = np.ascontiguousarray(delta, np.float32).reshape(-1)
        out = np.empty(delta.size, np.float32)
        self.lib.cfo_dare_prune(_ptr(delta), c_sz(delta.size), c_f(drop_rate), _ptr(out))
        return out

    def task_vector_merge(self, base, fts, lam, drop_rate):
        base = np.ascontiguousarray(base, np.float32).reshape(-1)
        fts = [np.ascontiguousarray(f, np.float32).reshape(-1) for f in fts]
        ptrs = (ctypes.c_void_p * max(1, len(fts)))(*[f.ctypes.data for f in fts])
        out = np.empty(base.size, np.float32)
        self.lib.cfo_task_vector_merge(_ptr(base), ptrs, ctypes.c_int(len(fts)), c_sz(base.size), c_f(lam), c_f(drop_rate), _ptr(out))
        return out

    def apply_2to4_mask(self, vals):
        out = np.array(vals, np.float32).reshape(-1).copy()
        self.lib.cfo_apply_2to4_mask(_ptr(out), c_sz(out.size))
        return out

    def prune_keep_cols(self, cols, sparsity):
        self.lib.cfo_prune_keep_cols.restype = ctypes.c_size_t
        return int(self.lib.cfo_prune_keep_cols(c_sz(cols), c_f(sparsity)))

    def prune_columns_l1(self, w, keep_cols):
        w = np.ascontiguousarray(w, np.float32)
        rows, cols = w.shape
        out = np.empty(rows * cols, np.float32)
        kept = np.empty(max(cols, 1), np.int32)
        self.lib.cfo_prune_columns_l1.restype = ctypes.c_size_t
        keep = int(self.lib.cfo_prune_columns_l1(_ptr(w), c_sz(rows), c_sz(cols), c_sz(keep_cols), _ptr(out), _ptr(kept)))
        return out[: rows * keep].reshape(rows, keep).copy(), kept[:keep].copy()

    def transpose_f32(self, w):
        w = np.ascontiguousarray(w, np.float32)
        K, N = w.shape
        out = np.empty((N, K), np.float32)
        self.lib.cfo_transpose_f32(_ptr(w), c_sz(K), c_sz(N), _ptr(out))
        return out

    def lora_bake(self, w, a, b, alpha):
        w = np.array(w, np.float32).copy()
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        k, n = w.shape
        self.lib.cfo_lora_bake(_ptr(w), _ptr(a), _ptr(b), c_sz(k), c_sz(n), c_sz(a.shape[1]), c_f(alpha))
        return w

    def column_norms(self, w):
        w = np.ascontiguousarray(w, np.float32)
        out = np.empty(w.shape[1], np.float32)
        self.lib.cfo_column_norms(_ptr(w), c_sz(w.shape[0]), c_sz(w.shape[1]), _ptr(out))
        return out

    def dora_renorm(self, w, orig_mags=None):
        w = np.array(w, np.float32).copy()
        norms = np.empty(w.shape[1], np.float32)
        om = None if orig_mags is None else np.ascontiguousarray(orig_mags, np.float32)
        self.lib.cfo_dora_renorm(_ptr(w), c_sz(w.shape[0]), c_sz(w.shape[1]), _ptr(om) if om is not None else None, _ptr(norms))
        return w, norms


_inst = None


def build():
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "-s"], check=True)
    return SO


def load() -> Oracle:
    global _inst
    if _inst is None:
        src = ROOT / "oracle" / "cf_oracle.cpp"
        if not SO.exists() or SO.stat().st_mtime < src.stat().st_mtime:
            build()
        _inst = Oracle(ctypes.CDLL(str(SO)))
    return _inst
