// Shared pieces of the tensor-core GEMM kernels (gemm_tc.cu: one CTA per tile; gemm_pair.cu: two CTAs of a cluster per
// tile): tile constants, the argument block, PTX wrappers for mbarriers, TMA and tcgen05, the shared-memory and
// instruction descriptors, the epilogue's row store and the cycle-trace macros of -DCFB_GEMM_TRACE builds.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace cfb {
namespace tc {

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
static __device__ unsigned long long g_gtrace[2 * 18 * 8];
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
static __device__ unsigned long long g_gstamp[2 * 16];
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

// ---------------------------------------------------------------------------------------------
// W4 mode: one weight row of a k-block
// ---------------------------------------------------------------------------------------------
// 64 INT4 codes (32 bytes: p0, p1; byte j of a word holds codes 2j in its low and 2j + 1 in its high nibble) -> 64 f16
// values (q - zp) * scale, written as the row's eight 16-byte chunks of a 128-byte-swizzled K-major tile (chunk c of row r
// lives at chunk c ^ (r & 7)).  Fast form (scale >= 2^-10, so that scale / 16 is a normal f16): one PRMT copies a byte into
// both halves of a word, one LOP3 keeps the low nibble in the low half and the high nibble in the high half on top of the
// f16 pattern of 1024: the halves read 1024 + q and 1024 + 16 q.  Subtracting (1024 + zp, 1024 + 16 zp) is exact, and one
// packed multiply by (scale, scale / 16) rounds (q - zp) * scale once -- to the same f16 the slow form produces.
__device__ __forceinline__ void w4_unpack_row(const uint4& p0, const uint4& p1, uint32_t scale_f16_bits, int zp, uint32_t row_addr, int r7) {
  const float sc = __half2float(__ushort_as_half((unsigned short)scale_f16_bits));
  const uint32_t words[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
  auto put = [&](int c, uint32_t o0, uint32_t o1, uint32_t o2, uint32_t o3) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row_addr + (uint32_t)((c ^ r7) << 4)), "r"(o0), "r"(o1), "r"(o2), "r"(o3) : "memory");
  };
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
  } else {  // f16 keeps 11 significant bits of (q - zp) * scale (the product has at most 15)
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
}
// a row past the end of the weight: zeros
__device__ __forceinline__ void w4_zero_row(uint32_t row_addr) {
#pragma unroll
  for (int c = 0; c < 8; ++c) asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(row_addr + (uint32_t)(c << 4)), "r"(0u) : "memory");
}

// waits that observe arrivals from the other CTA of a pair (acquire at cluster scope)
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

constexpr int kPairBN = 256;  // columns of the pair kernel's tile = accumulator columns per CTA

// the pair kernel's launchers (gemm_pair.cu); tmB is not used by the W4 one
int32_t launch_pair_fp8(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, cudaStream_t st);
int32_t launch_pair_bf16(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, cudaStream_t st);
int32_t launch_pair_w4(const CUtensorMap& tmA, const GemmArgs& a, cudaStream_t st);

}  // namespace tc
}  // namespace cfb
