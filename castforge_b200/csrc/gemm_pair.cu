// The pair kernel of the tensor-core GEMMs: the two CTAs of a cluster (two SMs) work on ONE 256 x 256 tile through
// tcgen05 cta_group::2 (bf16 / f16 / E4M3 operands by TMA; in the W4 mode the weight tile is unpacked from INT4 by
// warps of both CTAs).  Entry points and the one-CTA kernel are in gemm_tc.cu.
#include "tc_common.cuh"

namespace cfb {
namespace {
using namespace tc;

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
        if (live) w4_unpack_row(cur.p0, cur.p1, cur.sc, (int)((cur.zb >> cur.zsh) & 0xFu), row, prow & 7);
        else w4_zero_row(row);
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

namespace tc {
int32_t launch_pair_fp8(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, cudaStream_t st) {
  return launch_gemm_pair<kKindE4M3, kBTma, 7>(tmA, tmB, a, st);
}
int32_t launch_pair_bf16(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, cudaStream_t st) {
  return launch_gemm_pair<kKindBF16, kBTma, 7>(tmA, tmB, a, st);
}
int32_t launch_pair_w4(const CUtensorMap& tmA, const GemmArgs& a, cudaStream_t st) {
  return launch_gemm_pair<kKindF16, kBDequantW4, 7>(tmA, tmA, a, st);
}
}  // namespace tc
}  // namespace cfb

#ifdef CFB_GEMM_TRACE
extern "C" int32_t cfb200_debug_pair_trace(unsigned long long* out64, int reset) {
  using namespace cfb::tc;
  if (out64 && cudaMemcpyFromSymbol(out64, g_gtrace, sizeof(g_gtrace)) != cudaSuccess) return 1;
  if (out64 && cudaMemcpyFromSymbol(out64 + 2 * 18 * 8, g_gstamp, sizeof(g_gstamp)) != cudaSuccess) return 1;
  if (reset) {
    unsigned long long z[2 * 18 * 8] = {};
    if (cudaMemcpyToSymbol(g_gtrace, z, sizeof(z)) != cudaSuccess) return 1;
  }
  return 0;
}
#endif
