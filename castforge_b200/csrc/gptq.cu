// E5: GPTQ 4-bit, group 128, act-order off (no reference counterpart; written from the published
// description of the algorithm).
//   1. Hessian   H = X^T X / T over T calibration tokens      -> tcgen05 bf16 GEMM on a transposed X
//   2. damping   H += 0.01 * mean(diag H) * I
//   3. U = upper Cholesky factor of H^-1 (H^-1 = U^T U), obtained without forming H^-1:
//      with P the index reversal, P H P = L L^T (lower Cholesky) and U = P L^-1 P.
//   4. for each block of 128 columns (= one quantisation group): every output row is independent;
//      a warp walks its row's 128 columns in order, quantises column j with the group's
//      scale / zero point (the asymmetric INT4 formula of cfb200_quant_int4_asym, computed from the
//      row's CURRENT values at the block start), and pushes the error e = (w - q) / U[j,j] into the
//      columns to its right: w[l] -= e * U[j,l].  The block's errors are then applied to all
//      later columns with one GEMM (W[:, end:] -= E * U[block, end:]).
// The factorisation needs f32 precision (~K^3 flops against the Hessian's 2*T*K^2).  Its 64-column steps and small
// products run as f32 on the CUDA cores; the large products (the trailing update of a 512-column panel, the upper levels
// of the triangular inverse) run on the bf16 tensor cores with every f32 operand split into three bf16 numbers (see
// split3).  The column walk and its error propagation are f32 on the CUDA cores in a fixed operation order, which the
// CPU oracle repeats bit for bit.
#include <math.h>

#include "common.cuh"

namespace cfb {
namespace {

#ifndef CFB_GPTQ_SPLITK
#define CFB_GPTQ_SPLITK 1024
#endif
constexpr int kNB = 64;  // factorisation block

// ---- bf16 transpose [R, C] -> [C, R] ------------------------------------------------------------
__global__ void transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, size_t R, size_t C, __nv_bfloat16* __restrict__ out) {
  __shared__ __nv_bfloat16 tile[64][66];
  const size_t r0 = (size_t)blockIdx.y * 64, c0 = (size_t)blockIdx.x * 64;
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const size_t r = r0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (r < R && c < C) ? in[r * C + c] : __float2bfloat16(0.0f);
    const size_t c2 = c + 32;
    tile[i][threadIdx.x + 32] = (r < R && c2 < C) ? in[r * C + c2] : __float2bfloat16(0.0f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const size_t c = c0 + i;
    for (int h = 0; h < 2; ++h) {
      const size_t r = r0 + threadIdx.x + 32 * h;
      if (c < C && r < R) out[c * R + r] = tile[threadIdx.x + 32 * h][i];
    }
  }
}

// ---- generic f32 GEMM: C[m,n] = beta*C[m,n] + alpha * sum_k A(m,k) * B(k,n), element strides ------
// 128 x 128 tile per CTA, 8 x 8 outputs per thread (two 4-wide halves 64 apart, so that the shared-memory reads are
// conflict-free 16-byte loads), k-tile 16 in two shared-memory buffers (one barrier per k-tile), the next k-tile's global
// loads in flight while the current one is multiplied.  Operands are addressed through (row stride, column stride) so that
// transposes cost nothing; a thread fetches four consecutive elements along whichever dimension is contiguous in memory
// with one 16-byte load where the tile lies inside the operand and the addresses allow it.  Every output element is one
// chain of fused multiply-adds in ascending k, whatever path its operands took.
constexpr int kSgBM = 128, kSgBN = 128, kSgBK = 16;

// FLUSH > 0 (a multiple of the k-tile; beta = 1): the sum restarts every FLUSH values of k and each partial sum goes into C
// with its own rounded addition, C = C + alpha * partial, exactly as K / FLUSH separate calls with K = FLUSH would leave
// it -- but C is read and written once.  The running C values live in registers meanwhile.
template <int FLUSH>
__global__ void __launch_bounds__(256)
sgemm_kernel(int M, int N, int K, float alpha, const float* __restrict__ A, long rsA, long csA, const float* __restrict__ B,
             long rsB, long csB, float beta, float* __restrict__ C, long ldc, int mode, long batchA, long batchB, long batchC) {
  A += (long)blockIdx.z * batchA;  // batched: the operands of problem z lie batch* elements further on
  B += (long)blockIdx.z * batchB;
  C += (long)blockIdx.z * batchC;
  // rows padded by 4 floats: a k-fast operand is stored 16 k apart per thread, which would hit one bank without it
  __shared__ __align__(16) float sA[2][kSgBK][kSgBM + 4], sB[2][kSgBK][kSgBN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * kSgBM, n0 = blockIdx.x * kSgBN;
  // mode bit 0: only tiles that touch the lower triangle of C are wanted (symmetric update);
  // mode bit 1: B is lower triangular (B(k, n) = 0 for k < n), so the k loop of a tile starts at its first column;
  // mode bit 2: A is lower triangular (A(m, k) = 0 for k > m), so the k loop of a tile ends with its last row
  if ((mode & 1) && n0 > m0 + kSgBM - 1) return;
  const int k_begin = (mode & 2) ? (n0 / kSgBK) * kSgBK : 0;
  if (mode & 4) K = min(K, m0 + kSgBM);
  const bool a_m_fast = (rsA == 1), b_n_fast = (csB == 1);
  // 16-byte loads: the operand's contiguous dimension has stride 1, the other stride and the base keep 16-byte alignment,
  // and the tile's rows / columns all exist (k is checked per k-tile)
  const bool a_vec = (a_m_fast ? (csA % 4 == 0) : (csA == 1 && rsA % 4 == 0)) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && m0 + kSgBM <= M;
  const bool b_vec = (b_n_fast ? (rsB % 4 == 0) : (rsB == 1 && csB % 4 == 0)) && ((reinterpret_cast<uintptr_t>(B) & 15) == 0) && n0 + kSgBN <= N;
  // a tile of an operand is 128 (m or n) x 16 (k) = 2048 elements = 512 groups of four along the contiguous dimension:
  // two groups per thread.  Group q: along-m/n-fast: (kk = q / 32, mm = 4 * (q % 32)); k-fast: (mm = q / 4, kk = 4 * (q % 4)).
  float4 va[2], vb[2];
  float ra[8], rb[8];
  bool a_v = false, b_v = false;  // how the tile in flight was fetched
  auto gload = [&](int k0) {
    a_v = a_vec && k0 + kSgBK <= K;
    b_v = b_vec && k0 + kSgBK <= K;
    if (a_v) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int q = tid + u * 256;
        const int mm = a_m_fast ? 4 * (q & 31) : (q >> 2), kk = a_m_fast ? (q >> 5) : 4 * (q & 3);
        va[u] = *reinterpret_cast<const float4*>(A + (long)(m0 + mm) * rsA + (long)(k0 + kk) * csA);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = tid + i * 256;
        const int amm = a_m_fast ? (e & 127) : (e >> 4), akk = a_m_fast ? (e >> 7) : (e & 15);
        ra[i] = (m0 + amm < M && k0 + akk < K) ? A[(long)(m0 + amm) * rsA + (long)(k0 + akk) * csA] : 0.0f;
      }
    }
    if (b_v) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int q = tid + u * 256;
        const int nn = b_n_fast ? 4 * (q & 31) : (q >> 2), kk = b_n_fast ? (q >> 5) : 4 * (q & 3);
        vb[u] = *reinterpret_cast<const float4*>(B + (long)(k0 + kk) * rsB + (long)(n0 + nn) * csB);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = tid + i * 256;
        const int bnn = b_n_fast ? (e & 127) : (e >> 4), bkk = b_n_fast ? (e >> 7) : (e & 15);
        rb[i] = (n0 + bnn < N && k0 + bkk < K) ? B[(long)(k0 + bkk) * rsB + (long)(n0 + bnn) * csB] : 0.0f;
      }
    }
  };
  auto sstore = [&](int buf) {
    if (a_v) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int q = tid + u * 256;
        if (a_m_fast) {
          *reinterpret_cast<float4*>(&sA[buf][q >> 5][4 * (q & 31)]) = va[u];
        } else {
          const int mm = q >> 2, kk = 4 * (q & 3);
          sA[buf][kk][mm] = va[u].x; sA[buf][kk + 1][mm] = va[u].y; sA[buf][kk + 2][mm] = va[u].z; sA[buf][kk + 3][mm] = va[u].w;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = tid + i * 256;
        const int amm = a_m_fast ? (e & 127) : (e >> 4), akk = a_m_fast ? (e >> 7) : (e & 15);
        sA[buf][akk][amm] = ra[i];
      }
    }
    if (b_v) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int q = tid + u * 256;
        if (b_n_fast) {
          *reinterpret_cast<float4*>(&sB[buf][q >> 5][4 * (q & 31)]) = vb[u];
        } else {
          const int nn = q >> 2, kk = 4 * (q & 3);
          sB[buf][kk][nn] = vb[u].x; sB[buf][kk + 1][nn] = vb[u].y; sB[buf][kk + 2][nn] = vb[u].z; sB[buf][kk + 3][nn] = vb[u].w;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = tid + i * 256;
        const int bnn = b_n_fast ? (e & 127) : (e >> 4), bkk = b_n_fast ? (e >> 7) : (e & 15);
        sB[buf][bkk][bnn] = rb[i];
      }
    }
  };
  float acc[8][8] = {};
  float crun[FLUSH > 0 ? 8 : 1][FLUSH > 0 ? 8 : 1];
  if (FLUSH > 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
        crun[FLUSH > 0 ? i : 0][FLUSH > 0 ? j : 0] = (m < M && n < N) ? C[(long)m * ldc + n] : 0.0f;
      }
    }
  }
  int buf = 0;
  if (k_begin < K) {
    gload(k_begin);
    sstore(0);
  }
  __syncthreads();
  for (int k0 = k_begin; k0 < K; k0 += kSgBK) {
    const bool more = k0 + kSgBK < K;
    if (more) gload(k0 + kSgBK);
#pragma unroll
    for (int kk = 0; kk < kSgBK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&sA[buf][kk][ty * 4]), a1 = *reinterpret_cast<const float4*>(&sA[buf][kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&sB[buf][kk][tx * 4]), b1 = *reinterpret_cast<const float4*>(&sB[buf][kk][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (FLUSH > 0 && (k0 + kSgBK) % (FLUSH > 0 ? FLUSH : 1) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float& cr = crun[FLUSH > 0 ? i : 0][FLUSH > 0 ? j : 0];
          cr = beta * cr + alpha * acc[i][j];
          acc[i][j] = 0.0f;
        }
    }
    if (more) sstore(buf ^ 1);  // the other buffer: everyone left it at the previous barrier
    __syncthreads();
    buf ^= 1;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (n < N) {
        float* c = C + (long)m * ldc + n;
        if (FLUSH > 0) *c = crun[FLUSH > 0 ? i : 0][FLUSH > 0 ? j : 0];
        else *c = (beta == 0.0f ? 0.0f : beta * *c) + alpha * acc[i][j];
      }
    }
  }
}

void sgemm(cudaStream_t st, int M, int N, int K, float alpha, const float* A, long rsA, long csA, const float* B, long rsB, long csB,
           float beta, float* C, long ldc, int mode = 0, int batch = 1, long batchA = 0, long batchB = 0, long batchC = 0,
           int flush = 0) {
  if (M <= 0 || N <= 0 || batch <= 0) return;
  dim3 grid((N + kSgBN - 1) / kSgBN, (M + kSgBM - 1) / kSgBM, batch);
  if (flush == 128) sgemm_kernel<128><<<grid, 256, 0, st>>>(M, N, K, alpha, A, rsA, csA, B, rsB, csB, beta, C, ldc, mode, batchA, batchB, batchC);
  else sgemm_kernel<0><<<grid, 256, 0, st>>>(M, N, K, alpha, A, rsA, csA, B, rsB, csB, beta, C, ldc, mode, batchA, batchB, batchC);
}

// ---- small helpers on K x K matrices ---------------------------------------------------------------
__global__ void mirror_upper_kernel(float* __restrict__ H, int n) {  // H[j][i] = H[i][j] for i < j
  const int i = blockIdx.y * 16 + threadIdx.y, j = blockIdx.x * 16 + threadIdx.x;
  if (i < n && j < n && i < j) H[(size_t)j * n + i] = H[(size_t)i * n + j];
}
__global__ void diag_mean_kernel(const float* __restrict__ H, int n, float* __restrict__ out) {
  __shared__ double part[256];
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += 256) s += (double)H[(size_t)i * n + i];
  part[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = (float)(part[0] / n);
}
// out = reversed(in) with optional damping of the diagonal: out[i][j] = in[n-1-i][n-1-j] (+ damp on i == j)
__global__ void reverse_kernel(const float* __restrict__ in, int n, const float* __restrict__ mean_diag, float damp_ratio,
                               float* __restrict__ out, int keep_upper_only) {
  const int i = blockIdx.y * 16 + threadIdx.y, j = blockIdx.x * 16 + threadIdx.x;
  if (i >= n || j >= n) return;
  float v = in[(size_t)(n - 1 - i) * n + (n - 1 - j)];
  if (i == j && mean_diag) {
    v += damp_ratio * mean_diag[0];
    if (!(v > 0.0f)) v = 1.0f;  // dead input channel: keep the factorisation defined
  }
  if (keep_upper_only && j < i) v = 0.0f;
  out[(size_t)i * n + j] = v;
}

// Cholesky of one kNB x kNB diagonal block in shared memory + the inverse of its factor.
// 256 threads = 64 rows x 4 column quarters.  Factor (right-looking): in step j every thread scales its own row's
// entry of column j (read from the still unscaled block, so one barrier per step is enough: the scaled column goes to a
// second array) and updates its 16 columns of that row.  Inverse: forward substitution, one column per group of four
// lanes (each takes a quarter of the dot product, two shuffles add them up), rows in order -- only the four lanes of
// a column depend on one another, so a warp-level barrier per row is all it needs.
__global__ void __launch_bounds__(256) chol_diag_kernel(float* __restrict__ A, int n, int k0, float* __restrict__ dinv) {
  static_assert(kNB == 64, "thread layout assumes 64 x 64 blocks");
  __shared__ float a[kNB][kNB + 1], l[kNB][kNB + 1];
  float (*x)[kNB + 1] = a;  // the inverse is written over the block once the factor is complete (a is dead then)
  const int nb = min(kNB, n - k0);
  for (int i = threadIdx.x; i < kNB * kNB; i += 256) {
    const int r = i >> 6, c = i & 63;
    a[r][c] = (r < nb && c < nb) ? A[(size_t)(k0 + r) * n + k0 + c] : (r == c ? 1.0f : 0.0f);
    l[r][c] = 0.0f;
  }
  __syncthreads();
  {
    const int row = threadIdx.x >> 2, c0 = (threadIdx.x & 3) * 16;
    for (int j = 0; j < kNB; ++j) {
      const float d = sqrtf(fmaxf(a[j][j], 1e-30f));
      const float inv = 1.0f / d;
      if (row >= j) {
        const float lij = row == j ? d : a[row][j] * inv;
        if (j >= c0 && j < c0 + 16) l[row][j] = lij;  // the owner of (row, j) keeps the finished entry
        // all 16 columns unrolled and predicated: the loads go out together instead of one dependent trip per column
        float cj[16], cur[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          cj[u] = a[c0 + u][j];
          cur[u] = a[row][c0 + u];
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int c = c0 + u;
          if (c > j && c <= row) a[row][c] = fmaf(-lij, cj[u] * inv, cur[u]);
        }
      }
      __syncthreads();
    }
  }
  {  // (the loop above ends on a barrier: every read of `a` is done before x overwrites it)
    // column c of X = L^-1: x[i][c] = (delta_ic - sum_{j=c}^{i-1} l[i][j] x[j][c]) / l[i][i]
    const int c = threadIdx.x >> 2, q = threadIdx.x & 3;
    for (int i = 0; i < kNB; ++i) {
      float lv[16], xv[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {  // j = c + q + 4u < i; out-of-range slots read row / column 63 and are not used
        const int j = min(c + q + 4 * u, kNB - 1);
        lv[u] = l[i][j];
        xv[u] = x[j][c];
      }
      float s = 0.0f;
#pragma unroll
      for (int u = 0; u < 16; ++u)
        if (c + q + 4 * u < i) s = fmaf(lv[u], xv[u], s);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (q == 0) x[i][c] = (i < c) ? 0.0f : ((i == c ? 1.0f : 0.0f) - s) / l[i][i];
      __syncwarp();
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kNB * kNB; i += 256) {
    const int r = i >> 6, c = i & 63;
    if (r < nb && c < nb) A[(size_t)(k0 + r) * n + k0 + c] = (c <= r) ? l[r][c] : 0.0f;
    dinv[i] = (r < nb && c < nb) ? x[r][c] : 0.0f;
  }
}

// panel below a factored diagonal block: P <- P * Linv_kk^T, one CTA per 64 rows (in place)
__global__ void __launch_bounds__(256) panel_trsm_kernel(float* __restrict__ A, int n, int k0, const float* __restrict__ dinv) {
  __shared__ float p[kNB][kNB + 1], li[kNB][kNB + 1];
  const int r0 = k0 + kNB + blockIdx.x * kNB;
  for (int i = threadIdx.x; i < kNB * kNB; i += 256) {
    const int r = i / kNB, c = i % kNB;
    p[r][c] = (r0 + r < n) ? A[(size_t)(r0 + r) * n + k0 + c] : 0.0f;
    li[r][c] = dinv[i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kNB * kNB; i += 256) {
    const int r = i / kNB, c = i % kNB;
    float s = 0.0f;
    for (int j = 0; j <= c; ++j) s = fmaf(p[r][j], li[c][j], s);  // (P * Linv^T)[r][c] = sum_j P[r][j] * Linv[c][j]
    if (r0 + r < n) A[(size_t)(r0 + r) * n + k0 + c] = s;
  }
}

__global__ void fill_kernel(float* p, size_t n, float v) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}
__global__ void copy_block_kernel(const float* __restrict__ dinv, float* __restrict__ X, int n, int k0) {
  for (int i = threadIdx.x; i < kNB * kNB; i += blockDim.x) {
    const int r = i / kNB, c = i % kNB;
    if (k0 + r < n && k0 + c < n) X[(size_t)(k0 + r) * n + k0 + c] = dinv[i];
  }
}

// ---- f32 products on the bf16 tensor cores ---------------------------------------------------------
// x = h + m + l with h = bf16(x), m = bf16(x - h), l = bf16(x - h - m): 24 significant bits in three bf16 numbers.  A
// product a * b is summed as  (h l + l h + m m) + (h m + m h) + h h,  six bf16 x bf16 products that are exact in the
// tensor core's f32 accumulator; what is left out (m l, l m, l l) is below 2^-24 of a * b.  The six terms of a K-slice
// become six K-blocks of ONE bf16 GEMM, smallest terms first, so that the accumulator's truncating additions act on the
// small partial sums while they are alone and on h h only for the slice's own length (kSplitK / 16 additions); slices are
// summed by the GEMM epilogue's rounded C +=.  Measured on damped Hessians of condition number ~850 (K = 4096) and at
// K = 14336: || U^T U (H + damp) v - v || / || v || = 5e-7 and 2e-6 in f64 (3e-7 and 1e-6 with 512-column slices).
constexpr int kSplitK = CFB_GPTQ_SPLITK;  // f32 columns per slice
constexpr int kSplitW = 6 * kSplitK;      // bf16 columns of a slice's operand
constexpr int kTcMin = 1024;              // products with fewer rows and columns than this stay on the CUDA cores

__device__ __forceinline__ void split3(float x, __nv_bfloat16& h, __nv_bfloat16& m, __nv_bfloat16& l) {
  h = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(h);  // exact
  m = __float2bfloat16_rn(r1);
  l = __float2bfloat16_rn(r1 - __bfloat162float(m));
}
// block order along the bf16 K axis: left operand  h l m | h m | h,  right operand  l h m | m h | h
__device__ __forceinline__ void put_left(__nv_bfloat16* row, int k, int kc, __nv_bfloat16 h, __nv_bfloat16 m, __nv_bfloat16 l) {
  row[k] = h; row[kc + k] = l; row[2 * kc + k] = m; row[3 * kc + k] = h; row[4 * kc + k] = m; row[5 * kc + k] = h;
}
__device__ __forceinline__ void put_right(__nv_bfloat16* row, int k, int kc, __nv_bfloat16 h, __nv_bfloat16 m, __nv_bfloat16 l) {
  row[k] = l; row[kc + k] = h; row[2 * kc + k] = m; row[3 * kc + k] = m; row[4 * kc + k] = h; row[5 * kc + k] = h;
}
// src [R, kc] f32 (row pitch ld) -> left and / or right operand [R, 6 * kc] bf16 (row pitch 6 * kSplitK; kc <= kSplitK,
// the columns kc .. of a block that a short last slice leaves are never read: the GEMM's K is 6 * kc with blocks kc apart)
__global__ void split_rows_kernel(const float* __restrict__ src, long ld, int R, int kc, __nv_bfloat16* __restrict__ left,
                                  __nv_bfloat16* __restrict__ right) {
  const long total = (long)R * kc;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / kc), k = (int)(i - (long)r * kc);
    __nv_bfloat16 h, m, l;
    split3(src[(long)r * ld + k], h, m, l);
    if (left) put_left(left + (long)r * (6 * kc), k, kc, h, m, l);
    if (right) put_right(right + (long)r * (6 * kc), k, kc, h, m, l);
  }
}
// src [kc, R] f32 (row pitch ld: the operand's K runs down the rows) -> right operand [R, 6 * kc] bf16, through a
// 32 x 32 shared-memory tile so that both sides are accessed along their rows
__global__ void split_cols_kernel(const float* __restrict__ src, long ld, int R, int kc, __nv_bfloat16* __restrict__ right) {
  __shared__ float tile[32][33];
  const int r0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int k = k0 + j, r = r0 + threadIdx.x;
    tile[j][threadIdx.x] = (k < kc && r < R) ? src[(long)k * ld + r] : 0.0f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int r = r0 + j, k = k0 + threadIdx.x;
    if (r < R && k < kc) {
      __nv_bfloat16 h, m, l;
      split3(tile[threadIdx.x][j], h, m, l);
      put_right(right + (long)r * (6 * kc), k, kc, h, m, l);
    }
  }
}

// ---- the column walk ---------------------------------------------------------------------------------
// truncating f32 -> f16 of the reference (tensor_store.rs:85-101), 0/inf/NaN -> 1.0 (as in the INT4 kernel)
__device__ __forceinline__ unsigned f16_trunc_scale_bits(float v) {
  const unsigned bits = __float_as_uint(v);
  const unsigned sign = (bits >> 16) & 0x8000u;
  const int exp = (int)((bits >> 23) & 0xffu);
  const unsigned mant = bits & 0x7fffffu;
  unsigned h;
  if (exp == 255) h = sign | 0x7c00u | (mant ? 0x0200u : 0u);
  else {
    const int ne = exp - 127 + 15;
    if (ne >= 31) h = sign | 0x7c00u;
    else if (ne <= 0) h = sign;
    else h = sign | ((unsigned)ne << 10) | (mant >> 13);
  }
  if ((h & 0x7fffu) == 0 || (h & 0x7c00u) == 0x7c00u) h = 0x3c00u;
  return h;
}

// One block of 128 columns starting at column b.  Warp per row; lane l holds columns l, l+32, l+64, l+96.
__global__ void __launch_bounds__(256)
gptq_block_kernel(float* __restrict__ W, int N, int K, int b, const float* __restrict__ U, uint8_t* __restrict__ codes,
                  uint16_t* __restrict__ scales, uint8_t* __restrict__ zp_bytes, float* __restrict__ Err, int err_pitch) {
  extern __shared__ float su[];  // U[b..b+128)[b..b+128), row-major, pitch 129
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = i >> 7, c = i & 127;
    su[r * 129 + c] = (c >= r) ? U[(size_t)(b + r) * K + b + c] : 0.0f;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = K / 128, g = b / 128;
  for (int row = blockIdx.x * 8 + warp; row < N; row += gridDim.x * 8) {
    float w[4], e[4];
    int q[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) w[s] = W[(size_t)row * K + b + s * 32 + lane];
    float lo = fminf(fminf(fminf(w[0], w[1]), fminf(w[2], w[3])), 0.0f), hi = fmaxf(fmaxf(fmaxf(w[0], w[1]), fmaxf(w[2], w[3])), 0.0f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(kFullMask, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(kFullMask, hi, o));
    }
    const unsigned sh = f16_trunc_scale_bits(__fdiv_rn(__fsub_rn(hi, lo), 15.0f));
    const float sc = __half2float(__ushort_as_half((unsigned short)sh));
    float zf = roundf(__fdiv_rn(-lo, sc));
    zf = (zf != zf) ? 0.0f : fminf(fmaxf(zf, 0.0f), 15.0f);
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll 4
      for (int jj = 0; jj < 32; ++jj) {
        const int j = s * 32 + jj;
        const float wj = __shfl_sync(kFullMask, w[s], jj);
        float qf = roundf(__fdiv_rn(wj, sc)) + zf;
        qf = (qf != qf) ? 0.0f : fminf(fmaxf(qf, 0.0f), 15.0f);
        const float wq = __fmul_rn(qf - zf, sc);
        const float ej = __fdiv_rn(wj - wq, su[j * 129 + j]);
        if (lane == jj) { q[s] = (int)qf; e[s] = ej; w[s] = wq; }
        // push the error into the columns to the right of j (upper triangle of U: others are zero)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int col = t * 32 + lane;
          if (t >= s && col > j) w[t] = fmaf(-ej, su[j * 129 + col], w[t]);
        }
      }
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int col = b + s * 32 + lane;
      W[(size_t)row * K + col] = w[s];  // the dequantised weight
      Err[(size_t)row * err_pitch + s * 32 + lane] = e[s];
      const int hi_n = __shfl_down_sync(kFullMask, q[s], 1);
      if ((lane & 1) == 0) codes[((size_t)row * K + col) >> 1] = (uint8_t)(q[s] | (hi_n << 4));
    }
    if (lane == 0) {
      scales[(size_t)row * groups + g] = (uint16_t)sh;
      zp_bytes[(size_t)row * groups + g] = (uint8_t)zf;
    }
  }
}

__global__ void pack_zp_kernel(const uint8_t* __restrict__ zp_bytes, size_t ngroups, uint8_t* __restrict__ zps) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (ngroups + 1) / 2; i += (size_t)gridDim.x * blockDim.x) {
    const uint8_t lo = zp_bytes[2 * i], hi = (2 * i + 1 < ngroups) ? zp_bytes[2 * i + 1] : 0;
    zps[i] = (uint8_t)(lo | (hi << 4));
  }
}

__global__ void widen_kernel(const void* __restrict__ src, int dt, size_t n, float* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = dt == CFB200_F32 ? load_elem<CFB200_F32>(src, i) : dt == CFB200_F16 ? load_elem<CFB200_F16>(src, i) : load_elem<CFB200_BF16>(src, i);
}

}  // namespace
}  // namespace cfb

using namespace cfb;

extern "C" int32_t cfb200_gemm_bf16_nt_ld(const void* A, size_t lda, const void* B, size_t ldb, size_t M, size_t N, size_t K,
                                          float alpha, void* C, int32_t out_f32, int32_t upper_only, int32_t accumulate,
                                          int32_t* error_flag, void* stream);

extern "C" int32_t cfb200_gemm_bf16_nt_ex(const void* A, size_t lda, const void* B, size_t ldb, size_t M, size_t N, size_t K,
                                          float alpha, void* C, size_t ldc, int32_t out_f32, int32_t triangle, int32_t accumulate,
                                          int32_t* error_flag, void* stream);

namespace cfb {
namespace {
// C[M, N] (pitch ldc) += alpha * A[M, K] * B on the tensor cores, f32 operands split three ways (see split3).  B is given
// by rows ([N, K], pitch ldb: b_rows) or by columns ([K, N], pitch ldb: b_cols); b_rows == A means a symmetric update
// (both operands from one split pass).  a_lower: A is lower triangular, so slice k0 only has rows >= k0; b_lower: B (by
// columns) is lower triangular, so slice k0 only reaches columns < k0 + slice.  wl / wr: [max(M, N), kSplitW] bf16 each.
int32_t tc_product(cudaStream_t st, int M, int N, int K, float alpha, const float* A, long lda, const float* b_rows,
                   const float* b_cols, long ldb, float* C, long ldc, int triangle, bool a_lower, bool b_lower,
                   __nv_bfloat16* wl, __nv_bfloat16* wr, int32_t* flag) {
  for (int k0 = 0; k0 < K; k0 += kSplitK) {
    const int kc = std::min(kSplitK, K - k0);
    const int m_lo = a_lower ? k0 : 0, m_eff = M - m_lo;
    const int n_eff = b_lower ? std::min(N, k0 + kc) : N;
    if (m_eff <= 0 || n_eff <= 0) continue;
    const bool same = (b_rows == A) && !b_cols;
    auto blocks = [](long total) { return (unsigned)std::min<long>((total + 255) / 256, (long)sm_count() * 16); };
    split_rows_kernel<<<blocks((long)m_eff * kc), 256, 0, st>>>(A + (long)m_lo * lda + k0, lda, m_eff, kc, wl, same ? wr : nullptr);
    if (b_cols) {
      split_cols_kernel<<<dim3((unsigned)((n_eff + 31) / 32), (unsigned)((kc + 31) / 32)), dim3(32, 8), 0, st>>>(b_cols + (long)k0 * ldb, ldb, n_eff, kc, wr);
    } else if (!same) {
      split_rows_kernel<<<blocks((long)n_eff * kc), 256, 0, st>>>(b_rows + k0, ldb, n_eff, kc, nullptr, wr);
    }
    CFB_LAUNCH_CHECK();
    const int32_t rc = cfb200_gemm_bf16_nt_ex(wl, (size_t)6 * kc, wr, (size_t)6 * kc, (size_t)m_eff, (size_t)n_eff, (size_t)6 * kc, alpha,
                                              C + (long)m_lo * ldc, (size_t)ldc, 1, triangle, 1, flag, st);
    if (rc) return rc;
  }
  return CFB200_OK;
}
// a bounded wait of a tensor-core launch that ran out makes the factor unusable: say so in the result itself
__global__ void poison_if_flag_kernel(const int32_t* flag, float* U) {
  if (*flag != 0) U[0] = __int_as_float(0x7fc00000);
}
}  // namespace
}  // namespace cfb

// H (K x K f32) = X^T X / T for X [T, K] bf16.  xt_workspace: T*K bf16 (the transposed copy).
extern "C" size_t cfb200_gptq_hessian_workspace_bytes(size_t T, size_t K) { return T * K * 2; }

extern "C" int32_t cfb200_gptq_hessian_scaled(const void* X, size_t T, size_t K, float alpha, float* H, void* xt_workspace,
                                              size_t workspace_bytes, int32_t* error_flag, void* stream);

extern "C" int32_t cfb200_gptq_hessian(const void* X, size_t T, size_t K, float* H, void* xt_workspace, size_t workspace_bytes,
                                       int32_t* error_flag, void* stream) {
  CFB_CHECK_ARG(T > 0, "bad argument");
  return cfb200_gptq_hessian_scaled(X, T, K, 1.0f / (float)T, H, xt_workspace, workspace_bytes, error_flag, stream);
}

// H = alpha * X^T X: the building block of a Hessian accumulated over several token shards (alpha = 1 / total tokens).
extern "C" int32_t cfb200_gptq_hessian_scaled(const void* X, size_t T, size_t K, float alpha, float* H, void* xt_workspace,
                                              size_t workspace_bytes, int32_t* error_flag, void* stream) {
  CFB_CHECK_ARG(X && H && T > 0 && K > 0, "bad argument");
  CFB_CHECK_ARG(T % 8 == 0, "the token count must be a multiple of 8 (got %zu)", T);
  if (!xt_workspace || workspace_bytes < T * K * 2) return set_error(CFB200_ERR_WORKSPACE, "gptq_hessian needs %zu bytes of workspace", T * K * 2);
  cudaStream_t st = (cudaStream_t)stream;
  dim3 tg((unsigned)((K + 63) / 64), (unsigned)((T + 63) / 64)), tb(32, 8);
  transpose_bf16_kernel<<<tg, tb, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(X), T, K, reinterpret_cast<__nv_bfloat16*>(xt_workspace));
  CFB_LAUNCH_CHECK();
  CFB_CUDA(cudaMemsetAsync(H, 0, K * K * sizeof(float), st));
  // The tensor cores add every 16-token product block into the f32 accumulator with truncation, which biases a sum of
  // T / 16 same-sign terms downwards (measured -1.4e-3 relative on the diagonal at T = 262144).  Tokens therefore go
  // through in chunks of 8192: each chunk's sum is short (512 blocks), and the chunks are added to H with
  // round-to-nearest f32 additions in the epilogue.
  constexpr size_t kChunk = 8192;
  int32_t rc = CFB200_OK;
  const char* xt = reinterpret_cast<const char*>(xt_workspace);
  for (size_t t0 = 0; t0 < T && rc == CFB200_OK; t0 += kChunk) {
    const size_t tc = T - t0 < kChunk ? T - t0 : kChunk;
    rc = cfb200_gemm_bf16_nt_ld(xt + t0 * 2, T, xt + t0 * 2, T, K, K, tc, alpha, H, 1, 1, t0 > 0, error_flag, stream);
  }
  if (rc) return rc;
  dim3 mg((unsigned)((K + 15) / 16), (unsigned)((K + 15) / 16)), mb(16, 16);
  mirror_upper_kernel<<<mg, mb, 0, st>>>(H, (int)K);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

// U = upper Cholesky factor of (H + damp * mean(diag H) * I)^-1.  workspace: 2*K*K + 64*64 + 4 floats.
extern "C" size_t cfb200_gptq_prepare_workspace_bytes(size_t K) {
  // reversed matrix / factor, its inverse, a diagonal block, four words (mean, give-up flag), two split operands
  return (2 * K * K + kNB * kNB + 4) * sizeof(float) + 2 * K * (size_t)kSplitW * sizeof(__nv_bfloat16);
}

extern "C" int32_t cfb200_gptq_prepare(const float* H, size_t K, float damp_ratio, float* U, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  CFB_CHECK_ARG(H && U && K > 0 && K < (1u << 20), "bad argument");
  if (!workspace || workspace_bytes < cfb200_gptq_prepare_workspace_bytes(K))
    return set_error(CFB200_ERR_WORKSPACE, "gptq_prepare needs %zu bytes of workspace", cfb200_gptq_prepare_workspace_bytes(K));
  cudaStream_t st = (cudaStream_t)stream;
  const int n = (int)K;
  float* A = reinterpret_cast<float*>(workspace);  // reversed, damped H -> its lower Cholesky factor
  float* Xi = A + K * K;                           // inverse of that factor
  float* dinv = Xi + K * K;
  float* mean = dinv + kNB * kNB;
  int32_t* flag = reinterpret_cast<int32_t*>(mean + 2);
  __nv_bfloat16* wl = reinterpret_cast<__nv_bfloat16*>(mean + 4);  // 16-byte aligned: every part before it is a multiple of 16 bytes
  __nv_bfloat16* wr = wl + K * (size_t)kSplitW;
  CFB_CUDA(cudaMemsetAsync(flag, 0, sizeof(int32_t), st));
  dim3 g16((unsigned)((K + 15) / 16), (unsigned)((K + 15) / 16)), b16(16, 16);
  diag_mean_kernel<<<1, 256, 0, st>>>(H, n, mean);
  reverse_kernel<<<g16, b16, 0, st>>>(H, n, mean, damp_ratio, A, 0);
  fill_kernel<<<1024, 256, 0, st>>>(Xi, K * K, 0.0f);
  // Blocked Cholesky on two levels.  Inside an outer panel of kOuter columns the 64-column steps update only the rest of
  // the panel; what lies right of the panel gets ONE update per panel with all kOuter columns (a K = 512 product instead
  // of eight K = 64 products: an eighth of the passes over the trailing matrix, and a multiply loop long enough to pay
  // for a tile's loads and stores).
  constexpr int kOuter = 8 * kNB;
  for (int p0 = 0; p0 < n; p0 += kOuter) {
    const int p1 = std::min(n, p0 + kOuter);
    for (int k0 = p0; k0 < p1; k0 += kNB) {
      chol_diag_kernel<<<1, 256, 0, st>>>(A, n, k0, dinv);
      copy_block_kernel<<<1, 256, 0, st>>>(dinv, Xi, n, k0);
      const int r = n - k0 - kNB;
      if (r <= 0) continue;
      panel_trsm_kernel<<<(r + kNB - 1) / kNB, 256, 0, st>>>(A, n, k0, dinv);
      const int c = p1 - k0 - kNB;  // columns of the panel right of this step
      if (c > 0) {
        const float* P = A + (size_t)(k0 + kNB) * n + k0;  // r x kNB
        float* T = A + (size_t)(k0 + kNB) * n + k0 + kNB;   // r x c, lower-triangle tiles only
        sgemm(st, r, c, kNB, -1.0f, P, n, 1, P, 1, n, 1.0f, T, n, 1);
      }
    }
    const int r2 = n - p1;
    if (r2 > 0) {
      const float* P = A + (size_t)p1 * n + p0;  // r2 x (p1 - p0)
      float* T = A + (size_t)p1 * n + p1;        // trailing r2 x r2
      if (r2 >= kTcMin) {
        const int32_t rc = tc_product(st, r2, r2, p1 - p0, -1.0f, P, n, P, nullptr, n, T, n, 2, false, false, wl, wr, flag);
        if (rc) return rc;
      } else {
        sgemm(st, r2, r2, p1 - p0, -1.0f, P, n, 1, P, 1, n, 1.0f, T, n, 1);
      }
    }
  }
  // L^-1 by doubling: the diagonal 64-blocks are inverted already; at block size s every pair of neighbouring
  // diagonal blocks [[X11, 0], [X21, X22]] gets X21 = -X22 * (L21 * X11), all pairs of a level in one batched launch.
  for (int sz = kNB; sz < n; sz *= 2) {
    const int pairs = n / (2 * sz), rem = n - pairs * 2 * sz;
    const long step = (long)2 * sz * n + 2 * sz;  // from one pair's blocks to the next pair's
    float* tmp = U;                               // U is free until the end; T of a pair sits where its X21 goes
    const long o21 = (long)sz * n;                // offset of block (2,1) from a pair's origin; (2,2) is at o21 + sz
    if (sz >= kTcMin) {  // large blocks: both products on the tensor cores, pair by pair
      for (int pi = 0; pi <= pairs; ++pi) {
        const int sb = pi < pairs ? sz : rem - sz;  // rows of the pair's second block (the last pair may be short)
        if (sb <= 0) break;
        const long o = (long)pi * step;
        CFB_CUDA(cudaMemset2DAsync(tmp + o + o21, (size_t)n * sizeof(float), 0, (size_t)sz * sizeof(float), (size_t)sb, st));
        int32_t rc = tc_product(st, sb, sz, sz, 1.0f, A + o + o21, n, nullptr, Xi + o, n, tmp + o + o21, n, 0, false, true, wl, wr, flag);  // T = L21 * X11
        if (rc) return rc;
        rc = tc_product(st, sb, sz, sb, -1.0f, Xi + o + o21 + sz, n, nullptr, tmp + o + o21, n, Xi + o + o21, n, 0, true, false, wl, wr, flag);  // X21 = -X22 * T
        if (rc) return rc;
      }
      continue;
    }
    sgemm(st, sz, sz, sz, 1.0f, A + o21, n, 1, Xi, n, 1, 0.0f, tmp + o21, n, 2, pairs, step, step, step);          // T = L21 * X11
    sgemm(st, sz, sz, sz, -1.0f, Xi + o21 + sz, n, 1, tmp + o21, n, 1, 0.0f, Xi + o21, n, 4, pairs, step, step, step);  // X21 = -X22 * T
    if (rem > sz) {  // a last pair whose second block is short
      const int sb = rem - sz;
      const long o = (long)pairs * step;
      sgemm(st, sb, sz, sz, 1.0f, A + o + o21, n, 1, Xi + o, n, 1, 0.0f, tmp + o + o21, n, 2);
      sgemm(st, sb, sz, sb, -1.0f, Xi + o + o21 + sz, n, 1, tmp + o + o21, n, 1, 0.0f, Xi + o + o21, n, 4);
    }
  }
  reverse_kernel<<<g16, b16, 0, st>>>(Xi, n, nullptr, 0.0f, U, 1);  // U = P L^-1 P (upper)
  poison_if_flag_kernel<<<1, 1, 0, st>>>(flag, U);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

// Quantize W [N, K] (rows independent: a rank may own any row range).  workspace: N*K + N*128 floats + N*K/128 bytes.
constexpr size_t kWalkPanel = 1024;  // columns whose errors are kept before the columns right of them are updated
extern "C" size_t cfb200_gptq_quantize_workspace_bytes(size_t N, size_t K) {
  return (N * K + N * kWalkPanel) * sizeof(float) + N * (K / 128) + 256;
}

extern "C" int32_t cfb200_gptq_quantize(const void* W, int32_t w_dtype, size_t N, size_t K, const float* U, uint8_t* codes,
                                        uint16_t* scales, uint8_t* zero_points, float* w_dequant /* nullable, [N,K] f32 */,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  CFB_CHECK_ARG(W && U && codes && scales && zero_points && N > 0 && K > 0, "bad argument");
  CFB_CHECK_ARG(dtype_ok(w_dtype), "unknown dtype %d", w_dtype);
  CFB_CHECK_ARG(K % 128 == 0, "K must be a multiple of the group size 128 (got %zu)", K);
  if (!workspace || workspace_bytes < cfb200_gptq_quantize_workspace_bytes(N, K))
    return set_error(CFB200_ERR_WORKSPACE, "gptq_quantize needs %zu bytes of workspace", cfb200_gptq_quantize_workspace_bytes(N, K));
  cudaStream_t st = (cudaStream_t)stream;
  float* Wf = reinterpret_cast<float*>(workspace);
  float* Err = Wf + N * K;
  uint8_t* zpb = reinterpret_cast<uint8_t*>(Err + N * kWalkPanel);
  widen_kernel<<<2048, 256, 0, st>>>(W, w_dtype, N * K, Wf);
  static thread_local int attr_dev = -1;
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  const size_t smem = 128 * 129 * sizeof(float);
  if (attr_dev != dev) {
    CFB_CUDA(cudaFuncSetAttribute(gptq_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_dev = dev;
  }
  const int grid = (int)std::min<size_t>((N + 7) / 8, (size_t)sm_count() * 3);
  // Every column block's errors reach every later column as ONE rounded subtraction of that block's 128-term sum, block
  // after block (the order the CPU oracle repeats).  Inside a panel of kWalkPanel columns the columns still to be walked
  // are updated after each block; the columns right of the panel get the panel's blocks in one launch that restarts its
  // sum every 128 terms and subtracts each partial sum in turn -- the same operations in the same order, with one pass
  // over those columns per panel instead of one per block.
  for (size_t p0 = 0; p0 < K; p0 += kWalkPanel) {
    const size_t p1 = std::min(K, p0 + kWalkPanel);
    for (size_t b = p0; b < p1; b += 128) {
      float* eb = Err + (b - p0);
      gptq_block_kernel<<<grid, 256, smem, st>>>(Wf, (int)N, (int)K, (int)b, U, codes, scales, zpb, eb, (int)kWalkPanel);
      const size_t c = p1 - b - 128;
      if (c > 0)  // W[:, b+128 : p1] -= Err_b * U[b:b+128, b+128 : p1]
        sgemm(st, (int)N, (int)c, 128, -1.0f, eb, (long)kWalkPanel, 1, U + b * K + b + 128, (long)K, 1, 1.0f, Wf + b + 128, (long)K);
    }
    const size_t rest = K - p1;
    if (rest > 0)  // W[:, p1:] -= Err_b * U[b:b+128, p1:] for every block b of the panel, in order
      sgemm(st, (int)N, (int)rest, (int)(p1 - p0), -1.0f, Err, (long)kWalkPanel, 1, U + p0 * K + p1, (long)K, 1, 1.0f, Wf + p1, (long)K, 0, 1, 0, 0,
            0, 128);
  }
  pack_zp_kernel<<<256, 256, 0, st>>>(zpb, N * (K / 128), zero_points);
  if (w_dequant) CFB_CUDA(cudaMemcpyAsync(w_dequant, Wf, N * K * sizeof(float), cudaMemcpyDeviceToDevice, st));
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}
