// Dense contractions on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only.
//
//   C[M,N] = alpha * row_scale[m] * col_scale[n] * sum_k A[m,k] * B[n,k]      (A, B both K-major)
//
// used for  * FP8 E4M3 x E4M3 -> bf16 (kind::f8f6f4; per-token activation scale x weight scale)
//           * bf16 x bf16 -> f32/bf16 (kind::f16; the GPTQ Hessian X^T X on a transposed X)
//           * W4A16 prefill: B tiles are dequantised from packed INT4 into shared memory by four
//             producer warps instead of arriving by TMA (B_MODE == kBDequantW4).
//
// One CTA computes one 128 x BN tile.  Warp roles (192 threads):
//   warp 0   TMA producer: one elected lane issues cp.async.bulk.tensor loads of
//            the A tile (and the B tile) of each k-block into a kStages-deep shared-memory ring;
//   warp 1   allocates TMEM, then one elected lane issues tcgen05.mma (128 x BN x UMMA_K, operands
//            described by shared-memory matrix descriptors with the 128-byte swizzle TMA wrote),
//            tcgen05.commit releases each ring slot and finally signals the accumulator;
//   warps 2-5 epilogue: tcgen05.ld the f32 accumulator (one TMEM lane = one output row per
//            thread), apply the scales, convert and store.  In the W4 mode the same four warps
//            first serve as dequant producers for the B ring.
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records an error code
// in global memory and leaves its loop; TMEM is always freed before the CTA returns.
#include <mutex>

#include "tc_common.cuh"

namespace cfb {
namespace {
using namespace tc;

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------
// AM: 128-row A tiles per CTA (1 or 2).  With 2, a B tile -- in the W4 mode an unpacked one -- feeds two accumulators.
template <int BN, int KIND, int B_MODE, int STAGES, int AM = 1>
__global__ void __launch_bounds__(B_MODE == kBDequantW4 ? kThreadsTc + 32 * kW4ExtraWarps : kThreadsTc, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs args) {
  constexpr int ELEM = (KIND == kKindE4M3) ? 1 : 2;
  constexpr int BK = kBKBytes / ELEM;           // elements of K per k-block
  constexpr int UMMA_K = 32 / ELEM;             // 32 bytes of K per instruction
  constexpr uint32_t A_TILE = kBM * kBKBytes;   // 16 KB
  constexpr uint32_t A_BYTES = AM * A_TILE;
  constexpr uint32_t B_BYTES = BN * kBKBytes;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: [tiles (1024-aligned)] [full barriers] [empty barriers] [accum full x2] [accum empty x2] [tmem slot] [abort]
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* accum_full = bars + 2 * STAGES;       // [2]: accumulator buffer complete
  uint64_t* accum_empty = bars + 2 * STAGES + 2;  // [2]: accumulator buffer drained by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  GT_DECL();
  const int num_kb = (args.K + BK - 1) / BK;
  // The CTA is persistent: it walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (tile_n fastest) with two
  // accumulator buffers in TMEM, so the epilogue of one tile runs under the main loop of the next.
  const int tiles_n = (args.N + BN - 1) / BN, tiles_m = (args.M + AM * kBM - 1) / (AM * kBM);
  const int S = args.split_k > 1 ? args.split_k : 1;
  const int num_tiles = tiles_n * tiles_m * S;
  const int kb_per = (num_kb + S - 1) / S;
  // symmetric product: a tile entirely below the diagonal is skipped (the same test in every role)
  int kb_lo = 0, kb_hi = num_kb, slice = 0;  // the k-blocks of the current work item
  auto tile_origin = [&](int t, int& m0, int& n0) -> bool {
    slice = t % S;
    const int tt = t / S;
    kb_lo = slice * kb_per;
    kb_hi = min(num_kb, kb_lo + kb_per);
    m0 = (tt / tiles_n) * (AM * kBM);
    n0 = (tt % tiles_n) * BN;
    // triangle 1: a tile entirely below the diagonal is skipped; 2: a tile entirely above it (AM == 1 only)
    return !((args.upper_only == 1 && n0 + BN <= m0) || (args.upper_only == 2 && m0 + AM * kBM <= n0));
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), B_MODE == kBDequantW4 ? 1 + 4 : 1);  // TMA (+ the four warps of one unpacking team)
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&accum_full[i]), 1);
      mbar_init(smem_u32(&accum_empty[i]), 4);  // one arrival per epilogue warp
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tcgen05_alloc(smem_u32(tmem_slot), 2 * AM * BN);
    tcgen05_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;  // k-blocks issued so far, over all tiles
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0;
        if (!tile_origin(t, m0, n0)) continue;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, args.error_flag, 1, s_abort)) { ok = false; break; }
          const uint32_t a_dst = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          mbar_expect_tx(smem_u32(&full_bar[s]), B_MODE == kBTma ? STAGE_BYTES : A_BYTES);
#pragma unroll
          for (int am = 0; am < AM; ++am) tma_load_2d(a_dst + am * A_TILE, &tmA, kb * BK, m0 + am * kBM, smem_u32(&full_bar[s]));
          if (B_MODE == kBTma) tma_load_2d(a_dst + A_BYTES, &tmB, kb * BK, n0, smem_u32(&full_bar[s]));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // A and B always share one format (a kind::f16 descriptor with a_format = bf16 and
      // b_format = f16 faulted on B200): the W4 mode runs with BOTH operands in f16
      const uint32_t idesc = make_idesc<KIND>(kBM, BN);
      bool ok = true;
      uint32_t it = 0, done = 0;  // k-blocks consumed; tiles computed by this CTA
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0;
        if (!tile_origin(t, m0, n0)) continue;
        const uint32_t buf = done & 1u, aph = (done >> 1) & 1u;
        // the epilogue must have drained this accumulator buffer (two tiles ago)
        long long gt0 = GT_NOW();
        ok = mbar_wait(smem_u32(&accum_empty[buf]), aph ^ 1u, args.error_flag, 5, s_abort);
        GT_ADD(1, GT_NOW() - gt0);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * (AM * BN);
        for (int kb = kb_lo; kb < kb_hi && ok; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          gt0 = GT_NOW();
          ok = mbar_wait(smem_u32(&full_bar[s]), ph, args.error_flag, 2, s_abort);
          GT_ADD(0, GT_NOW() - gt0);
          GT_ADD(2, 1);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t db = make_kmajor_desc(a_addr + A_BYTES);
#pragma unroll
          for (int am = 0; am < AM; ++am) {
            const uint64_t da = make_kmajor_desc(a_addr + am * A_TILE);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // advancing K by 32 bytes inside the swizzle span = +2 in the (address >> 4) field
              tcgen05_mma<KIND>(tmem_d + am * BN, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb != kb_lo || k != 0) ? 1u : 0u);
            }
          }
          tcgen05_commit(smem_u32(&empty_bar[s]));  // slot reusable once these MMAs have read it
        }
        tcgen05_commit(smem_u32(&accum_full[buf]));  // accumulator complete (or whatever was issued)
        ++done;
      }
    }
  } else {
    // ---------------- warps 2..5 (and 6..9 in the W4 mode) ----------------
    const int ew = warp - 2;         // 0..3 (0..7)
    uint32_t it = 0, done = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m0, n0;
      if (!tile_origin(t, m0, n0)) continue;
      if (B_MODE == kBDequantW4) {
        // Unpacking warps: two teams of four (warps 2..5 and 6..9).  A team owns every other k-block, so two
        // k-blocks are being unpacked at any time; inside a team thread r owns row r of the B tile (64 codes of a
        // k-block).  The codes, scale and zero point of the team's NEXT k-block are fetched while the current one
        // is unpacked.
        const int groups_per_row = args.K / args.group;
        const int team = ew >> 2, prow = (ew & 3) * 32 + lane;
        struct Pre { uint4 p0, p1; uint32_t sc, zb, zsh; };
        Pre pre[BN / 128];
        auto prefetch = [&](int kb) {
          const int k0 = kb * BK;
          const int g = (args.group == 128) ? (k0 >> 7) : k0 / args.group;
#pragma unroll
          for (int rr = 0; rr < BN / 128; ++rr) {
            const int n = n0 + rr * 128 + prow;
            if (n < args.N && k0 < args.K) {
              const uint4* src = reinterpret_cast<const uint4*>(args.w_codes + (size_t)n * (args.K / 2) + k0 / 2);
              pre[rr].p0 = __ldg(src);
              pre[rr].p1 = __ldg(src + 1);  // 64 codes
              const size_t gi = (size_t)n * groups_per_row + g;
              pre[rr].sc = __ldg(args.w_scales + gi);
              pre[rr].zb = __ldg(args.w_zps + (gi >> 1));  // raw byte: taking the nibble here would wait for the load
              pre[rr].zsh = (uint32_t)(gi & 1) * 4u;
            }
          }
        };
        if (kb_lo + team < kb_hi) prefetch(kb_lo + team);
        for (int kb = kb_lo + team; kb < kb_hi; kb += kW4Teams) {
          const uint32_t itk = it + (uint32_t)(kb - kb_lo);
          const int s = (int)(itk % STAGES);
          const uint32_t ph = (itk / STAGES) & 1u;
          Pre cur[BN / 128];
#pragma unroll
          for (int rr = 0; rr < BN / 128; ++rr) cur[rr] = pre[rr];
          if (kb + kW4Teams < kb_hi) prefetch(kb + kW4Teams);
          const long long gu0 = GT_NOW();
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, args.error_flag, 3, s_abort)) { ok = false; break; }
          const long long gu1 = GT_NOW();
          const uint32_t b_tile = smem_u32(tiles + (size_t)s * STAGE_BYTES + A_BYTES);
          const int k0 = kb * BK;  // BK == 64 16-bit elements
#pragma unroll
          for (int rr = 0; rr < BN / 128; ++rr) {
            const int r = rr * 128 + prow;
            const int n = n0 + r;
            const uint32_t row = b_tile + (uint32_t)r * 128u;
            if (n < args.N && k0 < args.K) w4_unpack_row(cur[rr].p0, cur[rr].p1, cur[rr].sc, (int)((cur[rr].zb >> cur[rr].zsh) & 0xFu), row, r & 7);
            else w4_zero_row(row);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&full_bar[s]));
          if ((ew & 3) == 0 && lane == 0) {
            const long long gu3 = GT_NOW();
            GT_ADD(0, gu1 - gu0);
            GT_ADD(1, gu2 - gu1);
            GT_ADD(2, gu3 - gu2);
            GT_ADD(3, 1);
          }
        }
        it += (uint32_t)(kb_hi - kb_lo);
        if (!ok) break;
      }
      if (ew >= 4) continue;  // the extra unpacking warps of the W4 mode have no epilogue duty
      // ---------------- epilogue of this tile ----------------
      const uint32_t buf = done & 1u, aph = (done >> 1) & 1u;
      ++done;
      const long long ge0 = GT_NOW();
      if (!mbar_wait(smem_u32(&accum_full[buf]), aph, args.error_flag, 4, s_abort)) { ok = false; break; }
      const long long ge1 = GT_NOW();
      tcgen05_fence_after();
      const int quad = warp & 3;               // the TMEM lane quadrant this warp may read
#pragma unroll 1
      for (int am = 0; am < AM; ++am) {
      const int row = m0 + am * kBM + quad * 32 + lane;
      const float rs = (args.row_scale && row < args.M) ? args.row_scale[row] * args.alpha : args.alpha;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tcgen05_ld_32x32(tmem_base + buf * (AM * BN) + am * BN + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, r);
        tcgen05_wait_ld();
        if (row < args.M) {
          const int col0 = n0 + c0;
          if (S > 1) {  // raw partial sums of this k slice; scales and the output format are applied by the reduction
            float* dst = args.partial + ((size_t)slice * args.M + row) * args.N + col0;
            if (col0 + 32 <= args.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                                                  __uint_as_float(r[j + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < args.N) dst[j] = __uint_as_float(r[j]);
            }
          } else if (col0 < args.N) {
            store_row32(args, row, col0, r, rs);
          }
        }
      }
      }
      // this warp's quadrant of the buffer is in registers / memory: hand the buffer back to the MMA warp
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&accum_empty[buf]));
      if (ew == 0 && lane == 0) {
        GT_ADD(4, ge1 - ge0);
        GT_ADD(5, GT_NOW() - ge1);
        GT_ADD(6, 1);
      }
    }
  }
  // ---------------- teardown: free TMEM ----------------
  GT_FLUSH();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tcgen05_dealloc(tmem_base, 2 * AM * BN);
  }
}

// bf16 -> f16 (round to nearest, saturating at +-65504; NaN stays NaN) for the W4 mode's activations
__device__ __forceinline__ __half bf16_to_f16_sat(__nv_bfloat16 b) {
  const float v = __bfloat162float(b);
  return __float2half_rn((v != v) ? v : fminf(fmaxf(v, -65504.0f), 65504.0f));
}
__global__ void bf16_to_f16_kernel(const __nv_bfloat16* __restrict__ x, size_t n, __half* __restrict__ out) {
  // eight elements (16 bytes in, 16 bytes out) per thread and trip when the source is 16-byte aligned (the workspace is)
  const size_t n8 = (reinterpret_cast<uintptr_t>(x) & 15) == 0 ? n / 8 : 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(x) + i);
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&r);
    uint4 o;
    __half* h = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k) h[k] = bf16_to_f16_sat(b[k]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
  for (size_t i = n8 * 8 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = bf16_to_f16_sat(x[i]);
}

// The same staging pass with castforge.static_quantize (src/codegen/eval.rs:1369-1382) applied on the way: the f32 value
// clamp(round(x / sc), +-qmax) * sc -- IEEE division, half-away rounding, separately rounded product, exactly as the
// interpreter evaluates the op -- is what gets rounded to f16, so the activation matrix makes no extra trip through memory.
template <bool F32IN>
__global__ void static_quantize_to_f16_kernel(const void* __restrict__ x, size_t n, float sc, float qmax, __half* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = F32IN ? reinterpret_cast<const float*>(x)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    float q = roundf(__fdiv_rn(v, sc));
    q = (q != q) ? q : fminf(fmaxf(q, -qmax), qmax);
    const float r = __fmul_rn(q, sc);
    out[i] = __float2half_rn((r != r) ? r : fminf(fmaxf(r, -65504.0f), 65504.0f));
  }
}

#ifdef CFB_GEMM_TRACE
}  // namespace
extern "C" int32_t cfb200_debug_gemm_trace(unsigned long long* out64, int reset) {
  if (out64 && cudaMemcpyFromSymbol(out64, g_gtrace, sizeof(g_gtrace)) != cudaSuccess) return 1;
  if (out64 && cudaMemcpyFromSymbol(out64 + 2 * 18 * 8, g_gstamp, sizeof(g_gstamp)) != cudaSuccess) return 1;
  if (reset) {
    unsigned long long z[2 * 18 * 8] = {};
    if (cudaMemcpyToSymbol(g_gtrace, z, sizeof(z)) != cudaSuccess) return 1;
  }
  return 0;
}
namespace {
#endif

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D K-major operand [rows, K] with row pitch `ld` elements: box = 128 bytes of K x box_rows rows
int32_t make_tmap(CUtensorMap* tm, const void* base, int elem_bytes, size_t rows, size_t K, size_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(CFB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * elem_bytes) % 16 != 0)
    return set_error(CFB200_ERR_MISALIGNED, "TMA operand needs a 16-byte aligned base and row pitch");
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(kBKBytes / elem_bytes), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(tm, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(CFB200_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
  return CFB200_OK;
}

template <int BN, int KIND, int B_MODE, int STAGES, int AM = 1>
int32_t launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, cudaStream_t st) {
  constexpr int ELEM = (KIND == kKindE4M3) ? 1 : 2;
  (void)ELEM;
  const size_t smem = (size_t)STAGES * (AM * kBM + BN) * kBKBytes + 1024 /*alignment slack*/ + (2 * STAGES + 4) * 8 + 16;
  static thread_local int attr_dev = -1;
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    CFB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, KIND, B_MODE, STAGES, AM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_dev = dev;
  }
  const size_t num_tiles = ((a.N + BN - 1) / BN) * ((a.M + AM * kBM - 1) / (AM * kBM)) * (a.split_k > 1 ? a.split_k : 1);
  const unsigned grid = (unsigned)std::min<size_t>(num_tiles, (size_t)sm_count());  // persistent: one CTA per SM
  gemm_tc_kernel<BN, KIND, B_MODE, STAGES, AM><<<grid, B_MODE == kBDequantW4 ? kThreadsTc + 32 * kW4ExtraWarps : kThreadsTc, smem, st>>>(tmA, tmB, a);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}


// Which kernel a product of this shape takes ("gemm_pair" knob: 0 = never the pair kernel, 1 = where it pays, 2 = wherever
// it can run).  The pair kernel needs more than one 128-row tile of A, and enough 256 x 256 tiles to occupy most of the
// device's 74 pairs; below that the one-CTA kernel's 128 x 128 tiles spread the work over more SMs.
bool use_pair_kernel(size_t M, size_t N, size_t min_tiles) {
  const long long knob = tunable(kTuneGemmPair);
  if (knob == 0 || M <= (size_t)kBM) return false;
  if (knob >= 2) return true;
  return ((M + 2 * kBM - 1) / (2 * kBM)) * ((N + kPairBN - 1) / kPairBN) >= min_tiles;
}

}  // namespace
}  // namespace cfb

using namespace cfb;

namespace cfb {
namespace {
using namespace tc;
// Self-test of the give-up path of the tensor-core kernels: the same bounded wait on a barrier that nothing completes,
// with a short limit; the caller's error word receives the code, as it does from a kernel.
// which: 0 = the plain wait, 1 = the sleeping wait of the epilogue warps, 2 = the wait that sees the other CTA's arrivals
__global__ void tc_wait_probe_kernel(int* error_flag, unsigned limit, int which) {
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&s_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (which == 0) mbar_wait(smem_u32(&s_bar), 0u, error_flag, 7, &s_abort, limit);
    else if (which == 1) mbar_wait_idle(smem_u32(&s_bar), 0u, error_flag, 8, &s_abort, limit);
    else mbar_wait_cluster(smem_u32(&s_bar), 0u, error_flag, 9, &s_abort, limit);
  }
}
}  // namespace
int32_t tc_expired_wait_selftest(int32_t* observed, int which) {
  int* flag = nullptr;
  CFB_CUDA(cudaMalloc(&flag, sizeof(int)));
  cudaMemset(flag, 0, sizeof(int));
  tc_wait_probe_kernel<<<1, 32>>>(flag, 1u << 12, which);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpy(observed, flag, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(flag);
  if (e != cudaSuccess) return set_error(CFB200_ERR_CUDA, "wait probe failed: %s", cudaGetErrorString(e));
  return CFB200_OK;
}
}  // namespace cfb

extern "C" int32_t cfb200_gemm_fp8(const uint8_t* A, const float* a_scales, const uint8_t* W, float w_scale, size_t M, size_t N,
                                   size_t K, void* C, int32_t out_f32, int32_t* error_flag, void* stream) {
  CFB_CHECK_ARG(A && W && C, "NULL buffer");
  CFB_CHECK_ARG(M > 0 && N > 0 && K > 0 && K % 16 == 0, "fp8 GEMM needs K a positive multiple of 16 (got %zu)", K);
  CFB_CHECK_ARG(M < (1u << 31) && N < (1u << 31) && K < (1u << 31), "dimension too large");
  CUtensorMap tmA, tmB;
  int32_t rc = make_tmap(&tmA, A, 1, M, K, K, kBM);
  if (rc) return rc;
  rc = make_tmap(&tmB, W, 1, N, K, K, 256);
  if (rc) return rc;
  GemmArgs g = {};
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.row_scale = a_scales; g.alpha = w_scale; g.C = C; g.ldc = (int)N; g.out_f32 = out_f32; g.error_flag = error_flag;
  if (use_pair_kernel(M, N, 56)) {
    rc = make_tmap(&tmB, W, 1, N, K, K, 128);
    if (rc) return rc;
    return tc::launch_pair_fp8(tmA, tmB, g, (cudaStream_t)stream);
  }
  return launch_gemm<256, kKindE4M3, kBTma, 4>(tmA, tmB, g, (cudaStream_t)stream);
}

// The bf16 product with explicit row pitches (lda, ldb in elements: the operands may be column ranges of wider
// matrices) and an optional C += (f32 output only).
// The bf16 product with explicit row pitches (lda, ldb, ldc in elements: the operands and the result may be blocks of
// wider matrices), a triangle selector (0 = all tiles, 1 = only tiles that touch the upper triangle, 2 = the lower) and an
// optional C += (f32 output only).
extern "C" int32_t cfb200_gemm_bf16_nt_ex(const void* A, size_t lda, const void* B, size_t ldb, size_t M, size_t N, size_t K,
                                          float alpha, void* C, size_t ldc, int32_t out_f32, int32_t triangle, int32_t accumulate,
                                          int32_t* error_flag, void* stream) {
  CFB_CHECK_ARG(A && B && C, "NULL buffer");
  CFB_CHECK_ARG(M > 0 && N > 0 && K > 0 && K % 8 == 0, "bf16 GEMM needs K a positive multiple of 8 (got %zu)", K);
  CFB_CHECK_ARG(M < (1u << 31) && N < (1u << 31) && K < (1u << 31) && ldc < (1u << 31), "dimension too large");
  CFB_CHECK_ARG(lda >= K && ldb >= K && ldc >= N, "row pitch shorter than the row");
  CFB_CHECK_ARG(!accumulate || out_f32, "accumulation needs an f32 output");
  CFB_CHECK_ARG(triangle >= 0 && triangle <= 2, "triangle is 0, 1 or 2");
  CUtensorMap tmA, tmB;
  int32_t rc = make_tmap(&tmA, A, 2, M, K, lda, kBM);
  if (rc) return rc;
  rc = make_tmap(&tmB, B, 2, N, K, ldb, 128);
  if (rc) return rc;
  GemmArgs g = {};
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.alpha = alpha; g.C = C; g.ldc = (int)ldc; g.out_f32 = out_f32; g.upper_only = triangle; g.accumulate = accumulate;
  g.error_flag = error_flag;
  if (use_pair_kernel(M, N, 56)) return tc::launch_pair_bf16(tmA, tmB, g, (cudaStream_t)stream);
  return launch_gemm<128, kKindBF16, kBTma, 6>(tmA, tmB, g, (cudaStream_t)stream);
}

extern "C" int32_t cfb200_gemm_bf16_nt_ld(const void* A, size_t lda, const void* B, size_t ldb, size_t M, size_t N, size_t K,
                                          float alpha, void* C, int32_t out_f32, int32_t upper_only, int32_t accumulate,
                                          int32_t* error_flag, void* stream) {
  return cfb200_gemm_bf16_nt_ex(A, lda, B, ldb, M, N, K, alpha, C, N, out_f32, upper_only ? 1 : 0, accumulate, error_flag, stream);
}

extern "C" int32_t cfb200_gemm_bf16_nt(const void* A, const void* B, size_t M, size_t N, size_t K, float alpha, void* C,
                                       int32_t out_f32, int32_t upper_only, int32_t* error_flag, void* stream) {
  return cfb200_gemm_bf16_nt_ld(A, K, B, K, M, N, K, alpha, C, out_f32, upper_only, 0, error_flag, stream);
}

namespace cfb {
namespace {
// Few output tiles (M <= 256 and a narrow N): the k-blocks of each tile are dealt to `S` CTAs, which leave f32 partial
// sums for a reduction launch.  Returns S (1 = no split); every slice gets at least 8 k-blocks.
int w4_split_k(size_t M, size_t N, size_t K) {
  if (M > 256) return 1;
  const int tiles = (int)((N + 127) / 128), num_kb = (int)(K / 64), sms = sm_count();
  const int cap = (int)tunable(kTuneW4SplitK);
  int S = sms / tiles;
  if (S > num_kb / 8) S = num_kb / 8;
  if (cap > 0 && S > cap) S = cap;
  if (S < 2) return 1;
  const int kb_per = (num_kb + S - 1) / S;
  return (num_kb + kb_per - 1) / kb_per;  // no empty slice
}
size_t w4_f16_bytes(size_t M, size_t K) { return (M * K * 2 + 255) & ~(size_t)255; }

// C[m][n] = sum over slices of partial[s][m][n], written as f32 or bf16 (four columns per thread)
__global__ void __launch_bounds__(256) split_k_reduce_kernel(const float* __restrict__ partial, int S, size_t mn, void* C, int out_f32) {
  const size_t i = ((size_t)blockIdx.x * 256 + threadIdx.x) * 4;
  if (i >= mn) return;
  if ((mn & 3) == 0) {  // every slice then starts on a 16-byte boundary
    float4 acc = *reinterpret_cast<const float4*>(partial + i);
    for (int s = 1; s < S; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)s * mn + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (out_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(C) + i) = acc;
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(C) + i) =
          make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
  } else {
    for (size_t j = i; j < mn && j < i + 4; ++j) {
      float acc = partial[j];
      for (int s = 1; s < S; ++s) acc += partial[(size_t)s * mn + j];
      if (out_f32) reinterpret_cast<float*>(C)[j] = acc;
      else reinterpret_cast<__nv_bfloat16*>(C)[j] = __float2bfloat16_rn(acc);
    }
  }
}
}  // namespace
}  // namespace cfb

extern "C" size_t cfb200_gemm_w4a16_workspace_bytes(size_t M, size_t N, size_t K) {
  const int S = w4_split_k(M, N, K);
  return w4_f16_bytes(M, K) + (S > 1 ? (size_t)S * M * N * 4 : 0);
}

namespace cfb {
namespace {
// a_mode: 0 = bf16 activations as they are; 1 / 2 = static_quantize(scale, bits) of bf16 / f32 activations in the staging pass
int32_t gemm_w4a16_impl(const void* A, int a_mode, float a_scale, int a_bits, const uint8_t* w_codes, const uint16_t* w_scales,
                        const uint8_t* w_zps, size_t M, size_t N, size_t K, size_t group, void* C, int32_t out_f32, void* workspace,
                        size_t workspace_bytes, int32_t* error_flag, void* stream) {
  CFB_CHECK_ARG(A && w_codes && w_scales && w_zps && C, "NULL buffer");
  CFB_CHECK_ARG(M > 0 && N > 0 && K > 0 && K % 64 == 0, "W4A16 GEMM needs K a positive multiple of 64 (got %zu)", K);
  CFB_CHECK_ARG(group >= 64 && group % 64 == 0 && K % group == 0, "group must be a multiple of 64 dividing K (got %zu)", group);
  CFB_CHECK_ALIGNED(w_codes, 16);
  CFB_CHECK_ALIGNED(workspace, 16);
  const size_t need = cfb200_gemm_w4a16_workspace_bytes(M, N, K);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(CFB200_ERR_WORKSPACE, "gemm_w4a16 needs %zu bytes of workspace (f16 copy of the activations, split-K partial sums)", need);
  cudaStream_t st = (cudaStream_t)stream;
  // Both operands of one tensor-core instruction are f16 here: the bf16 activations are first copied to f16 (saturating
  // at +-65504).  DO NOT give A as bf16 beside an f16 B in one kind::f16 instruction descriptor: that launch ended in
  // a device error (lost context) both times it ran.  kind::f16 takes ONE 16-bit format for both operands.
  const size_t n = M * K;
  size_t blocks = (n + 255) / 256, cap = (size_t)sm_count() * 16;
  const unsigned cgrid = (unsigned)(blocks < cap ? blocks : cap);
  if (a_mode == 0) {
    const size_t vblocks = (n / 8 + 255) / 256 + 1;
    bf16_to_f16_kernel<<<(unsigned)(vblocks < cap ? vblocks : cap), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(A), n, reinterpret_cast<__half*>(workspace));
  } else {
    const float sc = a_scale > 0.0f ? a_scale : 1.0f / 127.0f;  // the interpreter's default for a missing scale attribute
    const float qmax = a_bits == 4 ? 7.0f : 127.0f;
    if (a_mode == 2) static_quantize_to_f16_kernel<true><<<cgrid, 256, 0, st>>>(A, n, sc, qmax, reinterpret_cast<__half*>(workspace));
    else static_quantize_to_f16_kernel<false><<<cgrid, 256, 0, st>>>(A, n, sc, qmax, reinterpret_cast<__half*>(workspace));
  }
  CFB_LAUNCH_CHECK();
  CUtensorMap tmA;
  int32_t rc = make_tmap(&tmA, workspace, 2, M, K, K, kBM);
  if (rc) return rc;
  GemmArgs g = {};
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.alpha = 1.0f; g.C = C; g.ldc = (int)N; g.out_f32 = out_f32; g.error_flag = error_flag;
  g.w_codes = w_codes; g.w_scales = w_scales; g.w_zps = w_zps; g.group = (int)group;
  g.split_k = w4_split_k(M, N, K);
  if (g.split_k > 1) g.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + w4_f16_bytes(M, K));
  // more than one 128-row tile of activations: a CTA takes two of them, so that every unpacked weight tile is used twice
  rc = (M > 256 && use_pair_kernel(M, N, 32)) ? tc::launch_pair_w4(tmA, g, st)
       : M > 128 ? launch_gemm<128, kKindF16, kBDequantW4, 4, 2>(tmA, tmA, g, st)
                 : launch_gemm<128, kKindF16, kBDequantW4, 6>(tmA, tmA, g, st);
  if (rc || g.split_k <= 1) return rc;
  const size_t mn = M * N;
  split_k_reduce_kernel<<<(unsigned)((mn / 4 + 256) / 256), 256, 0, st>>>(g.partial, g.split_k, mn, C, out_f32);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}
}  // namespace
}  // namespace cfb

extern "C" int32_t cfb200_gemm_w4a16(const void* A, const uint8_t* w_codes, const uint16_t* w_scales, const uint8_t* w_zps,
                                     size_t M, size_t N, size_t K, size_t group, void* C, int32_t out_f32, void* workspace,
                                     size_t workspace_bytes, int32_t* error_flag, void* stream) {
  return gemm_w4a16_impl(A, 0, 0.0f, 8, w_codes, w_scales, w_zps, M, N, K, group, C, out_f32, workspace, workspace_bytes, error_flag, stream);
}

extern "C" int32_t cfb200_gemm_w4a16_static_quantize(const void* A, int32_t a_dtype, float a_scale, int32_t a_bits,
                                                     const uint8_t* w_codes, const uint16_t* w_scales, const uint8_t* w_zps, size_t M,
                                                     size_t N, size_t K, size_t group, void* C, int32_t out_f32, void* workspace,
                                                     size_t workspace_bytes, int32_t* error_flag, void* stream) {
  CFB_CHECK_ARG(a_dtype == CFB200_F32 || a_dtype == CFB200_BF16, "activations must be f32 or bf16 (got dtype %d)", a_dtype);
  return gemm_w4a16_impl(A, a_dtype == CFB200_F32 ? 2 : 1, a_scale, a_bits, w_codes, w_scales, w_zps, M, N, K, group, C, out_f32, workspace,
                         workspace_bytes, error_flag, stream);
}
