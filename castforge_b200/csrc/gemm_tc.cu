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
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace cfb {
namespace {

constexpr int kBM = 128;
constexpr int kBKBytes = 128;  // one 128-byte swizzle span of K per k-block
constexpr int kThreadsTc = 192;        // TMA warp, MMA warp, 4 epilogue warps
#ifndef CFB_W4_TEAMS
#define CFB_W4_TEAMS 3
#endif
constexpr int kW4Teams = CFB_W4_TEAMS;  // W4 mode: teams of four unpacking warps, each on its own k-block
constexpr int kW4ExtraWarps = 4 * (kW4Teams - 1);
constexpr unsigned kSpinLimit = 1u << 22;

enum { kKindE4M3 = 0, kKindBF16 = 1, kKindF16 = 2 };
enum { kBTma = 0, kBDequantW4 = 1 };

struct GemmArgs {
  int M, N, K;              // K in elements
  const float* row_scale;   // [M] or NULL
  const float* col_scale;   // [N] or NULL
  float alpha;
  void* C;                  // [M, ldc] bf16 or f32
  int ldc;
  int out_f32;
  int upper_only;           // 1: skip tiles strictly below the diagonal (symmetric products); 2: strictly above it
  int accumulate;           // f32 output only: C += result instead of C = result
  int* error_flag;          // device int, set non-zero when a bounded wait ran out
  int split_k;              // > 1: a tile's k-blocks are dealt to split_k CTAs, raw f32 partial sums go to `partial`
  float* partial;           // [split_k][M][N] f32 (split_k > 1 only)
  // W4 mode
  const uint8_t* w_codes;   // [N, K/2]
  const uint16_t* w_scales; // [N, K/group] f16 bits
  const uint8_t* w_zps;     // flat nibbles, group index = n * (K/group) + g
  int group;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait; false = gave up (error recorded)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code, volatile int* s_abort,
                                          unsigned limit = kSpinLimit) {
  for (unsigned i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *s_abort) return false;
  }
  *s_abort = 1;
  if (error_flag) atomicCAS(error_flag, 0, code);
  return false;
}

// the same bounded wait for a warp that expects to wait long (an epilogue warp during a tile's main loop): it sleeps
// between polls and leaves the issue slots of its scheduler to the warps that feed the tensor core
__device__ __forceinline__ bool mbar_wait_idle(uint32_t bar, uint32_t parity, int* error_flag, int code, volatile int* s_abort,
                                               unsigned limit = kSpinLimit) {
  for (unsigned i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(64);
    if ((i & 1023u) == 1023u && *s_abort) return false;
  }
  *s_abort = 1;
  if (error_flag) atomicCAS(error_flag, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tcgen05_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int KIND>
__device__ __forceinline__ void tcgen05_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  if (KIND == kKindE4M3) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 32 TMEM lanes (one per thread of the warp) x 32 consecutive 32-bit columns
__device__ __forceinline__ void tcgen05_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled,
// 8-row groups 1024 bytes apart (exactly what TMA SWIZZLE_128B writes).
//   bits [0,14)  start address >> 4        bits [32,46) stride byte offset >> 4 (1024 -> 64)
//   bits [16,30) leading byte offset >> 4 (unused for swizzled K-major; 1)
//   bits [46,48) descriptor version = 1    bits [61,64) swizzle mode: 2 = 128 bytes
__device__ __forceinline__ uint64_t make_kmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor: f32 accumulate, A and B K-major.
//   [4,6) c_format 1 = f32   [7,10) a_format   [10,13) b_format   (f16 kind: 0 f16, 1 bf16;
//   f8f6f4 kind: 0 e4m3, 1 e5m2)   15/16 a/b major (0 = K)   [17,23) N >> 3   [24,29) M >> 4
template <int KIND>
__device__ __forceinline__ uint32_t make_idesc(int mma_m, int mma_n) {
  // one format for BOTH operands (a descriptor with different A and B formats faulted on the device: never build one)
  const uint32_t fmt = (KIND == kKindBF16) ? 1u : 0u;  // e4m3 and f16 are both format 0 of their kind
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------
// AM: 128-row A tiles per CTA (1 or 2).  With 2, a B tile -- in the W4 mode an unpacked one -- feeds two accumulators.
// 32 accumulator columns of one output row -> C (scales, output format, optional C +=)
__device__ __forceinline__ void store_row32(const GemmArgs& args, int row, int col0, const uint32_t (&r)[32], float rs) {
  if (args.out_f32) {
    float* dst = reinterpret_cast<float*>(args.C) + (size_t)row * args.ldc + col0;
    if (col0 + 32 <= args.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
      float4* d4 = reinterpret_cast<float4*>(dst);
      float4 o[8];
      if (args.accumulate) {  // all eight loads of the old values first: behind each other's stores they would run one memory latency at a time
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __ldcg(d4 + j);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v;
        v.x = __uint_as_float(r[4 * j]) * rs * (args.col_scale ? args.col_scale[col0 + 4 * j] : 1.0f);
        v.y = __uint_as_float(r[4 * j + 1]) * rs * (args.col_scale ? args.col_scale[col0 + 4 * j + 1] : 1.0f);
        v.z = __uint_as_float(r[4 * j + 2]) * rs * (args.col_scale ? args.col_scale[col0 + 4 * j + 2] : 1.0f);
        v.w = __uint_as_float(r[4 * j + 3]) * rs * (args.col_scale ? args.col_scale[col0 + 4 * j + 3] : 1.0f);
        if (args.accumulate) {
          v.x = __fadd_rn(o[j].x, v.x); v.y = __fadd_rn(o[j].y, v.y); v.z = __fadd_rn(o[j].z, v.z); v.w = __fadd_rn(o[j].w, v.w);
        }
        d4[j] = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < args.N) {
          const float v = __uint_as_float(r[j]) * rs * (args.col_scale ? args.col_scale[col0 + j] : 1.0f);
          dst[j] = args.accumulate ? __fadd_rn(dst[j], v) : v;
        }
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(args.C) + (size_t)row * args.ldc + col0;
    if (col0 + 32 <= args.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
          const float v0 = __uint_as_float(r[j + 2 * tt]) * rs * (args.col_scale ? args.col_scale[col0 + j + 2 * tt] : 1.0f);
          const float v1 = __uint_as_float(r[j + 2 * tt + 1]) * rs * (args.col_scale ? args.col_scale[col0 + j + 2 * tt + 1] : 1.0f);
          const __nv_bfloat162 b2 = __floats2bfloat162_rn(v0, v1);
          pk[tt] = *reinterpret_cast<const uint32_t*>(&b2);
        }
        *reinterpret_cast<uint4*>(dst + j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < args.N)
          dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]) * rs * (args.col_scale ? args.col_scale[col0 + j] : 1.0f));
    }
  }
}

#ifdef CFB_GEMM_TRACE
// Cycle accounting of CTA 0's warps, for builds made with -DCFB_GEMM_TRACE only.
// Every thread sums into registers; lane 0 of each warp of CTAs 0 and 1 writes its eight sums when the kernel ends.
__device__ unsigned long long g_gtrace[2 * 18 * 8];
#define GT_DECL() long long gt_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; const long long gt_start = clock64()
#define GT_NOW() clock64()
#define GT_ADD(i, v) do { gt_acc[i] += (long long)(v); } while (0)
#define GT_FLUSH()                                                                                                          \
  do {                                                                                                                      \
    if (blockIdx.x < 2 && (threadIdx.x & 31) == 0) {                                                                        \
      gt_acc[7] = clock64() - gt_start;                                                                                     \
      for (int i_ = 0; i_ < 8; ++i_) g_gtrace[(blockIdx.x * 18 + (threadIdx.x >> 5)) * 8 + i_] = (unsigned long long)gt_acc[i_]; \
    }                                                                                                                       \
  } while (0)
// wall-clock stamps (globaltimer, ns) of the hand-overs of ONE k-block of CTAs 0 and 1
__device__ unsigned long long g_gstamp[2 * 16];
constexpr uint32_t kStampIt = 670;
__device__ __forceinline__ unsigned long long gt_wall() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define GT_STAMP(itv, slot) do { if ((itv) == kStampIt && blockIdx.x < 2) g_gstamp[blockIdx.x * 16 + (slot)] = gt_wall(); } while (0)
#else
#define GT_STAMP(itv, slot) do { } while (0)
#define GT_DECL() do { } while (0)
#define GT_NOW() 0ll
#define GT_ADD(i, v) do { } while (0)
#define GT_FLUSH() do { } while (0)
#endif

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
            uint4 out[8];
            if (n < args.N && k0 < args.K) {
              const uint4 p0 = cur[rr].p0, p1 = cur[rr].p1;
              const float sc = __half2float(__ushort_as_half((unsigned short)cur[rr].sc));
              const int zp = (int)((cur[rr].zb >> cur[rr].zsh) & 0xFu);
              const uint32_t words[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
              // Fast form (f16 operands, scale >= 2^-10 so that scale / 16 is a normal f16): byte j of a word holds
              // codes 2j (low nibble) and 2j+1 (high nibble).  One PRMT copies the byte into both halves, one LOP3
              // keeps the low nibble in the low half and the high nibble in the high half on top of the f16
              // pattern of 1024: the halves read 1024 + q and 1024 + 16 q.  Subtracting (1024 + zp, 1024 + 16 zp) is
              // exact, and one packed multiply by (scale, scale / 16) rounds (q - zp) * scale once, to the same f16
              // the slow form produces.
              const bool fast = (KIND == kKindF16) && sc >= 0.0009765625f && sc < 65504.0f;
              if (fast) {
                const __half2 zpair = __halves2half2(__ushort_as_half((unsigned short)(0x6400 + zp)), __float2half_rn(1024.0f + 16.0f * (float)zp));
                const __half2 spair = __floats2half2_rn(sc, sc * 0.0625f);
#pragma unroll
                for (int w8 = 0; w8 < 8; ++w8) {
                  uint32_t o[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    uint32_t x;
                    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(x) : "r"(words[w8]), "r"(0u), "r"((uint32_t)(j | 0x40 | (j << 8) | 0x4000)));
                    x = (x & 0x00F0000Fu) | 0x64006400u;
                    const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&x), zpair), spair);
                    o[j] = *reinterpret_cast<const uint32_t*>(&v);
                  }
                  out[w8] = make_uint4(o[0], o[1], o[2], o[3]);
                }
              } else {
#pragma unroll
                for (int w8 = 0; w8 < 8; ++w8) {  // 8 codes per word -> one 16-byte chunk of 16-bit floats
                  uint32_t o[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const int q0 = (int)((words[w8] >> (8 * j)) & 0xF), q1 = (int)((words[w8] >> (8 * j + 4)) & 0xF);
                    // f16 keeps 11 significant bits of (q - zp) * scale (the product has at most 15);
                    // in bf16 the 8-bit rounding alone used most of the 1e-2 error budget
                    if (KIND == kKindF16) {
                      const __half2 v = __floats2half2_rn((float)(q0 - zp) * sc, (float)(q1 - zp) * sc);
                      o[j] = *reinterpret_cast<const uint32_t*>(&v);
                    } else {
                      const __nv_bfloat162 v = __floats2bfloat162_rn((float)(q0 - zp) * sc, (float)(q1 - zp) * sc);
                      o[j] = *reinterpret_cast<const uint32_t*>(&v);
                    }
                  }
                  out[w8] = make_uint4(o[0], o[1], o[2], o[3]);
                }
              }
            } else {
#pragma unroll
              for (int c = 0; c < 8; ++c) out[c] = make_uint4(0, 0, 0, 0);
            }
            // 128-byte swizzle: 16-byte chunk c of row r lives at chunk (c ^ (r & 7))
            const uint32_t row = b_tile + (uint32_t)r * 128u;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row + (uint32_t)((c ^ (r & 7)) << 4)), "r"(out[c].x), "r"(out[c].y),
                           "r"(out[c].z), "r"(out[c].w) : "memory");
          }
          const long long gu2 = GT_NOW();
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

// ---------------------------------------------------------------------------------------------
// the pair kernel: the two CTAs of a cluster (two SMs) work on ONE 256 x 256 tile
// ---------------------------------------------------------------------------------------------
// With one CTA per tile the tensor pipe waits on shared memory: a 128 x 128 x 16 instruction reads 8 KB of operands
// for 65 cycles of arithmetic, which is all a shared memory of 128 bytes per cycle can deliver, and the TMA (and, in
// the W4 mode, the unpacking warps) write into the same memory.  `cta_group::2` halves the operand reads per flop: each
// CTA of the pair holds 128 rows of A and 128 of the tile's 256 rows of B, one instruction issued by the leader CTA
// multiplies 256 x 256 x 16 on both SMs, and every SM's accumulator (its 128 rows x 256 columns) sits in its own TMEM.
//   leader (cluster rank 0): its full barriers collect BOTH CTAs' TMA bytes (and unpack arrivals); its MMA thread issues
//   for the pair and commits to the empty / accumulator-full barriers of both CTAs; its accumulator-empty barriers take
//   the arrivals of both CTAs' epilogue warps.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {  // the same offset in CTA `rank` of the cluster
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_peer(uint32_t cluster_addr) {  // default semantics: release at CTA scope
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {  // sees arrivals from the peer CTA
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int* error_flag, int code, volatile int* s_abort,
                                                  unsigned limit = kSpinLimit) {
  for (unsigned i = 0; i < limit; ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *s_abort) return false;
  }
  *s_abort = 1;
  if (error_flag) atomicCAS(error_flag, 0, code);
  return false;
}
// TMA load into this CTA's shared memory whose completion is counted on a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tmap, int x, int y, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ void tcgen05_alloc_pair(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrives on the barrier at this offset in BOTH CTAs once the pair's earlier MMAs have completed
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"((uint16_t)3)
               : "memory");
}
template <int KIND>
__device__ __forceinline__ void tcgen05_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  if (KIND == kKindE4M3) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

constexpr int kPairBN = 256;  // columns of the pair's tile = accumulator columns per CTA
constexpr int kPairW4Threads = kThreadsTc + 32 * 4 * kW4Teams;  // TMA, MMA, 4 epilogue warps, kW4Teams teams of 4 unpacking warps

template <int KIND, int B_MODE, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(B_MODE == kBDequantW4 ? kPairW4Threads : kThreadsTc, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs args) {
  constexpr int ELEM = (KIND == kKindE4M3) ? 1 : 2;
  constexpr int BK = kBKBytes / ELEM;
  constexpr int UMMA_K = 32 / ELEM;
  constexpr uint32_t A_TILE = kBM * kBKBytes;  // this CTA's 128 rows of A: 16 KB
  constexpr uint32_t B_TILE = 128 * kBKBytes;  // this CTA's 128 of the tile's 256 rows of B: 16 KB
  constexpr uint32_t STAGE_BYTES = A_TILE + B_TILE;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the carve is the same in both CTAs (the dynamic shared memory starts at the same offset), which the pair instructions rely on
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                      // used in the leader only
  uint64_t* empty_bar = bars + STAGES;            // one per CTA: its TMA (and unpacking) warps wait here
  uint64_t* accum_full = bars + 2 * STAGES;       // [2] per CTA: its epilogue waits here
  uint64_t* accum_empty = bars + 2 * STAGES + 2;  // [2] used in the leader only: 4 + 4 epilogue warps arrive
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  GT_DECL();
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_kb = (args.K + BK - 1) / BK;
  const int tiles_n = (args.N + kPairBN - 1) / kPairBN, tiles_m = (args.M + 2 * kBM - 1) / (2 * kBM);
  const int num_tiles = tiles_n * tiles_m;
  // Tiles are walked in bands of kBand tile rows, down the band first: the pairs at work at one time then cover a
  // squarish patch of C (8 x 9 tiles with 74 pairs) and share their A and B slabs in L2, instead of two full tile rows.
  constexpr int kBand = 8;
  auto tile_origin = [&](int t, int& m0, int& n0) -> bool {
    const int band = t / (kBand * tiles_n), r = t - band * (kBand * tiles_n);
    const int rows = min(kBand, tiles_m - band * kBand);  // the last band may be shorter
    m0 = (band * kBand + r % rows) * (2 * kBM);
    n0 = (r / rows) * kPairBN;
    return !((args.upper_only == 1 && n0 + kPairBN <= m0) || (args.upper_only == 2 && m0 + 2 * kBM <= n0));
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // the leader's TMA thread (+ in the W4 mode the four unpacking warps of a team in each CTA)
      mbar_init(smem_u32(&full_bar[s]), B_MODE == kBDequantW4 ? 1 + 8 : 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&accum_full[i]), 1);
      mbar_init(smem_u32(&accum_empty[i]), 8);
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the MMA warp of EACH CTA takes part in the pair's allocation
    tcgen05_alloc_pair(smem_u32(tmem_slot), 2 * kPairBN);
    tcgen05_relinquish_pair();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them from the other side
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (each CTA loads its own halves; completion is counted in the leader) ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int m0, n0;
        if (!tile_origin(t, m0, n0)) continue;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, args.error_flag, 11, s_abort)) { ok = false; break; }
          GT_STAMP(it, 0);
          GT_STAMP(it - STAGES, 10);
          const uint32_t a_dst = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t lead_full = mapa_u32(smem_u32(&full_bar[s]), 0);
          if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * (B_MODE == kBTma ? STAGE_BYTES : A_TILE));
          tma_load_2d_pair(a_dst, &tmA, kb * BK, m0 + (int)rank * kBM, lead_full);
          if (B_MODE == kBTma) tma_load_2d_pair(a_dst + A_TILE, &tmB, kb * BK, n0 + (int)rank * 128, lead_full);
          GT_STAMP(it, 1);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one thread of the leader CTA issues for the pair ----------------
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = make_idesc<KIND>(2 * kBM, kPairBN);
      bool ok = true;
      uint32_t it = 0, done = 0;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int m0, n0;
        if (!tile_origin(t, m0, n0)) continue;
        const uint32_t buf = done & 1u, aph = (done >> 1) & 1u;
        long long gt0 = GT_NOW();
        ok = mbar_wait_cluster(smem_u32(&accum_empty[buf]), aph ^ 1u, args.error_flag, 15, s_abort);
        GT_ADD(1, GT_NOW() - gt0);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kPairBN;
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          gt0 = GT_NOW();
          ok = mbar_wait_cluster(smem_u32(&full_bar[s]), ph, args.error_flag, 12, s_abort);
          GT_ADD(0, GT_NOW() - gt0);
          GT_ADD(2, 1);
          if (!ok) break;
          GT_STAMP(it, 7);
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t da = make_kmajor_desc(a_addr), db = make_kmajor_desc(a_addr + A_TILE);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tcgen05_mma_pair<KIND>(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb != 0 || k != 0) ? 1u : 0u);
          tcgen05_commit_pair(smem_u32(&empty_bar[s]));
          GT_STAMP(it, 8);
        }
        tcgen05_commit_pair(smem_u32(&accum_full[buf]));
        ++done;
      }
    }
  } else if (B_MODE == kBDequantW4 && warp >= 6) {
    // ---------------- W4 mode, warps 6..: teams of four unpacking warps, each team on every kW4Teams-th k-block ----------------
    // Thread r of a team owns row r of this CTA's 128 rows of the B tile.  A thread keeps the codes, scale and zero point of
    // its next TWO k-blocks in registers; the loads that refill a set are issued right after the set's k-block has been
    // handed over, so that no load is in flight when the next hand-over's fence runs (a fence waits for them).
    const int team = (warp - 6) >> 2, prow = ((warp - 6) & 3) * 32 + lane;
    const int groups_per_row = args.K / args.group;
    struct Pre { uint4 p0, p1; uint32_t sc, zb, zsh; };
    uint32_t it = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs) {
      int m0, n0;
      if (!tile_origin(t, m0, n0)) continue;
      const int n = n0 + (int)rank * 128 + prow;
      const bool live = n < args.N;
      auto fetch = [&](int kb, Pre& d) {
        const int k0 = kb * BK;
        const int g = (args.group == 128) ? (k0 >> 7) : k0 / args.group;
        if (live) {
          const uint4* src = reinterpret_cast<const uint4*>(args.w_codes + (size_t)n * (args.K / 2) + k0 / 2);
          d.p0 = __ldg(src);
          d.p1 = __ldg(src + 1);
          const size_t gi = (size_t)n * groups_per_row + g;
          d.sc = __ldg(args.w_scales + gi);
          d.zb = __ldg(args.w_zps + (gi >> 1));  // the raw byte: taking the nibble here would make the warp wait for the load
          d.zsh = (uint32_t)(gi & 1) * 4u;
        }
      };
      auto step = [&](int kb, Pre& cur) -> bool {
        const uint32_t itk = it + (uint32_t)kb;
        const int s = (int)(itk % STAGES);
        const uint32_t ph = (itk / STAGES) & 1u;
        const long long gu0 = GT_NOW();
        if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, args.error_flag, 13, s_abort)) return false;
        const long long gu1 = GT_NOW();
        if (prow == 0) GT_STAMP(itk, 2);
        const uint32_t row = smem_u32(tiles + (size_t)s * STAGE_BYTES + A_TILE) + (uint32_t)prow * 128u;
        // 128-byte swizzle: 16-byte chunk c of row r lives at chunk (c ^ (r & 7))
        auto put = [&](int c, uint32_t o0, uint32_t o1, uint32_t o2, uint32_t o3) {
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row + (uint32_t)((c ^ (prow & 7)) << 4)), "r"(o0), "r"(o1), "r"(o2), "r"(o3)
                       : "memory");
        };
        if (live) {
          const float sc = __half2float(__ushort_as_half((unsigned short)cur.sc));
          const int zp = (int)((cur.zb >> cur.zsh) & 0xFu);
          const uint32_t words[8] = {cur.p0.x, cur.p0.y, cur.p0.z, cur.p0.w, cur.p1.x, cur.p1.y, cur.p1.z, cur.p1.w};
          // the packed form of the one-CTA kernel: PRMT + LOP3 put (1024 + q, 1024 + 16 q) into an f16 pair, an exact
          // subtraction and ONE rounding multiply by (scale, scale / 16) give (q - zp) * scale
          if (sc >= 0.0009765625f && sc < 65504.0f) {
            const __half2 zpair = __halves2half2(__ushort_as_half((unsigned short)(0x6400 + zp)), __float2half_rn(1024.0f + 16.0f * (float)zp));
            const __half2 spair = __floats2half2_rn(sc, sc * 0.0625f);
#pragma unroll
            for (int w8 = 0; w8 < 8; ++w8) {
              uint32_t o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t x;
                asm("prmt.b32 %0, %1, %2, %3;" : "=r"(x) : "r"(words[w8]), "r"(0u), "r"((uint32_t)(j | 0x40 | (j << 8) | 0x4000)));
                x = (x & 0x00F0000Fu) | 0x64006400u;
                const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&x), zpair), spair);
                o[j] = *reinterpret_cast<const uint32_t*>(&v);
              }
              put(w8, o[0], o[1], o[2], o[3]);
            }
          } else {
#pragma unroll
            for (int w8 = 0; w8 < 8; ++w8) {
              uint32_t o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int q0 = (int)((words[w8] >> (8 * j)) & 0xF), q1 = (int)((words[w8] >> (8 * j + 4)) & 0xF);
                const __half2 v = __floats2half2_rn((float)(q0 - zp) * sc, (float)(q1 - zp) * sc);
                o[j] = *reinterpret_cast<const uint32_t*>(&v);
              }
              put(w8, o[0], o[1], o[2], o[3]);
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) put(c, 0u, 0u, 0u, 0u);
        }
        const long long gu2 = GT_NOW();
        if (prow == 0) GT_STAMP(itk, 3);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        // Both CTAs' teams arrive on the LEADER's full barrier.  The arrival carries the default (CTA-scope) release: the
        // fence above has already put this warp's rows where the tensor core reads them, in this SM's own shared memory,
        // and a cluster-scope release here cost every unpacking warp over 1000 cycles per k-block.
        if (lane == 0) mbar_arrive_peer(mapa_u32(smem_u32(&full_bar[s]), 0));
        if (prow == 0) GT_STAMP(itk, 4);
        if (kb + 2 * kW4Teams < num_kb) fetch(kb + 2 * kW4Teams, cur);
        if (((warp - 6) & 3) == 0 && lane == 0) {
          const long long gu3 = GT_NOW();
          GT_ADD(0, gu1 - gu0);
          GT_ADD(1, gu2 - gu1);
          GT_ADD(2, gu3 - gu2);
          GT_ADD(3, 1);
        }
        return true;
      };
      Pre ra, rb;
      if (team < num_kb) fetch(team, ra);
      if (team + kW4Teams < num_kb) fetch(team + kW4Teams, rb);
      for (int kb = team; kb < num_kb; kb += 2 * kW4Teams) {
        if (!step(kb, ra)) { ok = false; break; }
        if (kb + kW4Teams < num_kb && !step(kb + kW4Teams, rb)) { ok = false; break; }
      }
      it += (uint32_t)num_kb;
    }
  } else {
    // ---------------- warps 2..5: epilogue of this CTA's 128 rows x 256 columns ----------------
    uint32_t done = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs) {
      int m0, n0;
      if (!tile_origin(t, m0, n0)) continue;
      const uint32_t buf = done & 1u, aph = (done >> 1) & 1u;
      ++done;
      const long long ge0 = GT_NOW();
      if (!mbar_wait_idle(smem_u32(&accum_full[buf]), aph, args.error_flag, 14, s_abort)) { ok = false; break; }
      const long long ge1 = GT_NOW();
      tcgen05_fence_after();
      const int quad = warp & 3;
      const int row = m0 + (int)rank * kBM + quad * 32 + lane;
      const float rs = (args.row_scale && row < args.M) ? args.row_scale[row] * args.alpha : args.alpha;
#pragma unroll 1
      for (int c0 = 0; c0 < kPairBN; c0 += 32) {
        uint32_t r[32];
        tcgen05_ld_32x32(tmem_base + buf * kPairBN + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, r);
        tcgen05_wait_ld();
        if (row < args.M && n0 + c0 < args.N) store_row32(args, row, n0 + c0, r, rs);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&accum_empty[buf]), 0));
      if (warp == 2 && lane == 0) {
        GT_ADD(4, ge1 - ge0);
        GT_ADD(5, GT_NOW() - ge1);
        GT_ADD(6, 1);
      }
    }
  }
  // ---------------- teardown: neither CTA leaves (or frees TMEM) while the other may still use its memory ----------------
  GT_FLUSH();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    tcgen05_dealloc_pair(tmem_base, 2 * kPairBN);
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

template <int KIND, int B_MODE, int STAGES>
int32_t launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, cudaStream_t st) {
  constexpr int kThreads = B_MODE == kBDequantW4 ? kPairW4Threads : kThreadsTc;
  const size_t smem = (size_t)STAGES * (kBM + 128) * kBKBytes + 1024 /*alignment slack*/ + (2 * STAGES + 4) * 8 + 16;
  static thread_local int attr_dev = -1;
  static thread_local int max_pairs = 0;
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    CFB_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<KIND, B_MODE, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sm_count() & ~1u);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    CFB_CUDA(cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<KIND, B_MODE, STAGES>, &cfg));
    max_pairs = n;
    attr_dev = dev;
  }
  if (max_pairs <= 0) return set_error(CFB200_ERR_CUDA, "no cluster of two CTAs of the pair kernel fits on this device");
  const size_t num_tiles = ((a.N + kPairBN - 1) / kPairBN) * ((a.M + 2 * kBM - 1) / (2 * kBM));
  const unsigned pairs = (unsigned)std::min<size_t>(num_tiles, (size_t)max_pairs);
  gemm_pair_kernel<KIND, B_MODE, STAGES><<<2 * pairs, kThreads, smem, st>>>(tmA, tmB, a);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

}  // namespace
}  // namespace cfb

using namespace cfb;

namespace cfb {
namespace {
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
    return launch_gemm_pair<kKindE4M3, kBTma, 7>(tmA, tmB, g, (cudaStream_t)stream);
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
  if (use_pair_kernel(M, N, 56)) return launch_gemm_pair<kKindBF16, kBTma, 7>(tmA, tmB, g, (cudaStream_t)stream);
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
  rc = (M > 256 && use_pair_kernel(M, N, 32)) ? launch_gemm_pair<kKindF16, kBDequantW4, 7>(tmA, tmA, g, st)
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
