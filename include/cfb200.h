/*
 * cfb200.h -- device entry points of the B200 (sm_100a) quantize-and-execute path.
 *
 * This is the C ABI a host `Pass` binds to run CastForge's weight-quantization arithmetic and
 * its dequantize-fused GEMM on the GPU.  CastForge itself has no such interface (its passes
 * loop over host vectors in-process), so every declaration cites the reference routine whose
 * arithmetic it replaces (paths relative to the CastForge source tree).
 *
 * Conventions
 *  - every function returns 0 on success or a CFB200_ERR_* code; cfb200_last_error() gives the
 *    message for the calling thread;
 *  - all pointers are DEVICE pointers unless the name says `host`; buffers are caller-owned;
 *    nothing is allocated unless a function says so;
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream); work is enqueued, not
 *    synchronised;
 *  - input/output base pointers must be 16-byte aligned;
 *  - dtype codes: CFB200_F32 / CFB200_F16 / CFB200_BF16 (storage of the source weights;
 *    widening to f32 follows src/ir/tensor_store.rs:58-111);
 *  - "flat" groups/blocks chunk the row-major buffer, so they run along the last dimension and
 *    the final one may be short (src/passes/quantize/schemes.rs:532, formats.rs:466).
 */
#ifndef CFB200_H
#define CFB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { CFB200_F32 = 0, CFB200_F16 = 1, CFB200_BF16 = 2 };

enum {
  CFB200_OK = 0,
  CFB200_ERR_INVALID = 1,     /* bad argument (shape, option, NULL pointer) */
  CFB200_ERR_MISALIGNED = 2,  /* a pointer is not 16-byte aligned */
  CFB200_ERR_CUDA = 3,        /* a CUDA runtime call or launch failed */
  CFB200_ERR_UNSUPPORTED = 4, /* valid request this build does not implement */
  CFB200_ERR_WORKSPACE = 5,   /* caller-provided workspace too small */
  CFB200_ERR_DEVICE = 6       /* a kernel reported an error status (e.g. a bounded wait ran out) */
};

/* Message of the last failing call on this thread ("" if none).  Never freed by the caller. */
const char* cfb200_last_error(void);
/* Library version string (static). */
const char* cfb200_version(void);

/* Performance knob (process-wide, never changes results).  Keys: "a1_persist" (1, default: f16 / bf16
 * lists and large tensors run as one cooperative launch; 2: f32 too; 0: one launch per tensor group), "a1_group_mb"
 * (L2 budget of a tensor group, default 64), "a1_retain_mb" (MB of a group's tail that the first
 * pass leaves in L2 at normal priority, default 60; negative = everything), "a1_tail_first" (1, default: the quantize
 * pass re-reads that tail before the lines that were let go; 0: oldest lines first), "a1_keep_mb",
 * "a1_demote", "a1_merge" (variants of the launch-per-group path), "a1_bar_sleep" (ns between polls of the cooperative
 * launch's grid barrier, default 0), "gemv_ring" (1, default: decode
 * shapes with 16 MB of packed weights or more use the shared-memory ring kernel; 0: never; n > 1: from n MB), "gemv_ring_rounds", "w4_split_k" (W4A16 prefill
 * with M <= 256: 0 = automatic split-K, 1 = never, n = at most n slices; changes the summation
 * order of the f32 accumulation and nothing else), "gemm_pair" (the bf16 / FP8 / W4A16-prefill products: 1, default =
 * two CTAs of a cluster (two SMs, tcgen05 cta_group::2) per 256 x 256 tile where the product has at least 56 such tiles
 * (W4A16: M > 256 and 32 tiles); 0 = always one CTA per tile; 2 = pairs wherever M > 128 (W4A16: M > 256)), "colpar_p2p"
 * (column-parallel products: 1, default = products of 8 MB and more are rejoined by a peer-load kernel over CUDA-IPC
 * mappings where the ranks are separate processes on one node; 0 = always ncclAllGather; n > 1 = from n MB; negative =
 * peer loads for every size). */
int32_t cfb200_tune(const char* key, int64_t value);

/* ---- A1: per-tensor symmetric INT8 / INT4 ------------------------------------------------
 * Replaces quantize_symmetric_f32 (src/passes/quantize/formats.rs:664-698) as driven by
 * QuantizeWeightsPass::run (src/passes/quantize/schemes.rs:324-452).
 * codes: n int8 (one code per byte for bits == 4 too).  scale_absmax: 2 floats,
 * [0] = scale (absmax < 1e-12 ? 1 : absmax / qmax), [1] = absmax.  Zero point is always 0.
 * bits: 4 -> range [-8,7]; anything else means 8 -> [-128,127] (formats.rs:654-660). */
int32_t cfb200_quant_sym_tensor(const void* src, int32_t src_dtype, size_t n, int32_t bits,
                                int8_t* codes, float* scale_absmax, void* stream);

/* The same in two steps, for callers that shard one tensor across devices by row blocks:
 * cfb200_absmax on each shard, a max across shards (host or NCCL), then this call with the
 * global absmax (one device float; it may alias scale_absmax + 1). */
int32_t cfb200_quant_sym_apply(const void* src, int32_t src_dtype, size_t n, int32_t bits,
                               const float* absmax, int8_t* codes, float* scale_absmax,
                               void* stream);

/* A whole list of device-resident tensors (what QuantizeWeightsPass::run loops over,
 * src/passes/quantize/schemes.rs:324-452) in one call.  srcs/ns/codes are HOST arrays of `count`
 * device pointers / element counts; scale_absmax is a DEVICE array of 2*count floats
 * ({scale, absmax} per tensor).  Consecutive tensors are grouped while their bytes fit
 * l2_group_bytes (0 = default).  By default a list of f16 / bf16 tensors runs as ONE cooperative launch per
 * 1024 tensors (absmax pass, grid barrier, quantize pass per group, the quantize pass of a group
 * overlapped with the absmax pass of the next); for f32 sources, or with cfb200_tune("a1_persist", 0),
 * the two passes of successive groups share launches, groups + 1 in total.  The _plan call returns the number of
 * launches as n_stages.  The default mode copies a descriptor table from host memory, so it must
 * not be called while `stream` is being captured into a CUDA graph.  Calls may come from several host threads and
 * streams: the eight descriptor slots of a device are recycled as their launches finish (the call blocks until one is free).
 * stage_events: NULL, or n_stages + 1 cudaEvent_t handles; handle k is recorded before launch k
 * and the last one after the final launch (for per-launch timing on `stream`). */
int32_t cfb200_quant_sym_tensors_plan(int32_t count, const size_t* ns, int32_t src_dtype,
                                      size_t l2_group_bytes, int32_t* n_stages);
int32_t cfb200_quant_sym_tensors(int32_t count, const void* const* srcs, int32_t src_dtype,
                                 const size_t* ns, int32_t bits, int8_t* const* codes,
                                 float* scale_absmax, size_t l2_group_bytes,
                                 void* const* stage_events, void* stream);

/* The cooperative launch above bounds every wait it makes (its bulk copies, its grid barrier).  If one runs out, the
 * CTAs stop, wait for the copies they still have in flight and return, and the codes and scales of that call are
 * incomplete although the call itself returned 0.  This call synchronises the current device and reports whether
 * that has ever happened on it (0 = never; sticky until the process ends).  cfb200_store_run_pipeline checks it
 * before it reports success.  (No counterpart in the reference: its pass cannot fail half-way.) */
int32_t cfb200_quant_sym_status(int32_t* flag_host);

/* Self-test of the give-up path that every spin-wait in the kernels has.  A one-warp kernel waits, with a limit of a
 * few thousand polls, on a barrier that nothing completes, gives up and reports exactly as the real kernels do:
 * which == 0: through the sticky flag of the cooperative A1 launch -- *observed_host receives what
 * cfb200_quant_sym_status then reads (1), and the flag is cleared again; which == 1: through a caller error word as
 * the tensor-core GEMMs use it -- *observed_host receives the code written there (7); which == 2 and 3: the same for
 * the two other waits of the pair kernel (the sleeping wait of its epilogue warps, code 8; the wait that observes the
 * other CTA's arrivals, code 9).  Touches no caller memory, leaves nothing in flight, runs in microseconds.
 * (which >= 1 allocates and frees four bytes of device memory.) */
int32_t cfb200_selftest_expired_wait(int32_t which, int32_t* observed_host);

/* ---- A6: per-tensor fake quantization (QAT-STE) --------------------------------------------
 * Replaces run_qat_ste's arithmetic (src/passes/quantize/formats.rs:764-769): f32 in, f32 out,
 * out = clamp(round(v/scale)) * scale.  scale_absmax as above. */
int32_t cfb200_fakequant_tensor(const float* src, size_t n, int32_t bits, float* out,
                                float* scale_absmax, void* stream);

/* SmoothQuant migration (src/passes/quantize/schemes.rs:229-243).  The two per-tensor scalars
 * depend on powf and are computed by the host from the absmax this call leaves in
 * absmax_out[0]; pass 1 = cfb200_absmax, pass 2 = this function with the scalars.
 * out = clamp(round(v*smooth / effq)) * effq / smooth. */
int32_t cfb200_absmax(const void* src, int32_t src_dtype, size_t n, float* absmax_out,
                      void* stream);
int32_t cfb200_smoothquant_apply(const float* src, size_t n, int32_t bits, float smooth_scale,
                                 float eff_qscale, float* out, void* stream);

/* ---- E1: per-output-channel symmetric INT8 / INT4 (extension; no reference counterpart) ----
 * A1's formula applied independently to each row of a [rows, cols] row-major matrix.
 * scales: rows floats. */
int32_t cfb200_quant_per_channel(const void* src, int32_t src_dtype, size_t rows, size_t cols,
                                 int32_t bits, int8_t* codes, float* scales, void* stream);

/* ---- A2: group-wise fake quantization with the AWQ salient threshold ----------------------
 * Replaces QuantizeGroupwisePass::run (src/passes/quantize/schemes.rs:483-570).
 * cfb200_select_kth_abs finds the k-th largest |v| under IEEE total order (NaN largest),
 * k = clamp(ceil((float)n * clamp(ratio, .001, .5)), 1, n) -- schemes.rs:522-530 -- and writes
 * it to thr_out[0] (device); k is returned through k_host.  workspace: device scratch of at
 * least cfb200_select_kth_workspace_bytes() bytes (three histogram passes over the tensor).  With a 256-byte aligned
 * workspace of cfb200_select_kth_workspace_bytes_for(n) bytes, a tensor of a million elements or more and a rank in the top
 * 5 %, the tensor is read once instead: a sample brackets the threshold, one pass counts the keys above the bracket
 * and collects those inside it, the exact rank is found among them; the bracket is verified on the device and the
 * three passes run if it does not hold, so the answer is the exact k-th value either way.
 * cfb200_fakequant_group then applies, per flat group, scale = gmax<1e-12 ? 1 : gmax/qmax,
 * eff = (awq_salient && |v| >= thr) ? scale*0.5 : scale, out = clamp(round(v/eff))*eff. */
size_t cfb200_select_kth_workspace_bytes(void);
size_t cfb200_select_kth_workspace_bytes_for(size_t n);
int32_t cfb200_select_kth_abs(const float* src, size_t n, float salient_ratio, float* thr_out,
                              uint64_t* k_host, void* workspace, size_t workspace_bytes,
                              void* stream);
int32_t cfb200_fakequant_group(const float* src, size_t n, int32_t bits, size_t group_size,
                               int32_t awq_salient, const float* thr, float* out, void* stream);

/* ---- A3: FP8 "grid" fake quantization ---------------------------------------------------------
 * Replaces QuantizeFp8Pass::run (src/passes/quantize/schemes.rs:658-716): per flat block,
 * raw = amax<1e-12 ? 1 : amax/fp8_max; scale = mxfp8 ? 2^ceil(log2(raw)) : raw;
 * out = round(clamp(v/scale, +-fp8_max) / step) * step * scale, step = fp8_max/grid. */
int32_t cfb200_fakequant_fp8grid(const float* src, size_t n, size_t block_size, int32_t e5m2,
                                 int32_t mxfp8, float* out, void* stream);

/* ---- A4: E2M1 (FP4) fake quantization ---------------------------------------------------------
 * Replaces run_fp4_quantize / snap_e2m1 (src/passes/quantize/formats.rs:369-383, :414-479).
 * `block` is the resolved block length (nvfp4 with 32 requested -> 16, else max(block,4)). */
int32_t cfb200_fakequant_e2m1(const float* src, size_t n, size_t block, float* out, void* stream);

/* ---- A5: blocked Hadamard rotation down the columns of a [K, N] f32 matrix, in place --------
 * Replaces RotateHadamardPass::run's butterflies (src/passes/quantize/formats.rs:303-327).
 * b = clamp(next_pow2(block_size), 2, K); if K % b != 0 nothing is done and *applied_host = 0,
 * else *applied_host = b. */
int32_t cfb200_fwht_cols(float* w, size_t K, size_t N, size_t block_size, uint64_t* applied_host,
                         void* stream);

/* ---- E2: asymmetric INT4, flat groups, packed (extension; no reference counterpart) ---------
 * Per group: lo = min(0,min v), hi = max(0,max v); scale = truncating f16 of (hi-lo)/15
 * (src/ir/tensor_store.rs:85-101; 0/inf/NaN -> 1.0); zp = clamp(round(-lo/s),0,15);
 * q = clamp(round(v/s)+zp, 0, 15).  codes: ceil(n/2) bytes, element 2j in the low nibble
 * (src/ir/formats/gguf.rs:520-531); scales: one f16 bit pattern per group; zero_points: two
 * groups per byte, even group in the low nibble.  group in {32, 64, 128, 256}. */
int32_t cfb200_quant_int4_asym(const void* src, int32_t src_dtype, size_t n, size_t group,
                               uint8_t* codes, uint16_t* scales, uint8_t* zero_points,
                               void* stream);

/* ---- E3: NF4 with double-quantised absmax (extension; no reference counterpart) -------------
 * Per flat block: a = amax; x = v * (1/a) (a == 0 -> 0); code = #{midpoints m_j : x > m_j}
 * over the 15 midpoints of the NF4 levels; two codes per byte, low nibble first.
 * absmax8[b] = clamp(round(a / s2), 0, 255), s2 = max(a over dq_block blocks)/255 (0 -> 1),
 * absmax2[super-block] = s2.  block in {32, 64, 128, 256}; dq_block <= 1024.
 * workspace: device scratch of cfb200_quant_nf4_workspace_bytes(n, block) bytes (holds the
 * f32 block absmax values between the two kernels). */
size_t cfb200_quant_nf4_workspace_bytes(size_t n, size_t block);
int32_t cfb200_quant_nf4(const void* src, int32_t src_dtype, size_t n, size_t block,
                         size_t dq_block, uint8_t* codes, uint8_t* absmax8, float* absmax2,
                         void* workspace, size_t workspace_bytes, void* stream);

/* The same over a list of tensors (a whole store) in two launches instead of two per tensor.  srcs / ns / codes /
 * absmax8 / absmax2 are HOST arrays of `count` device pointers / element counts; results per tensor are identical to
 * cfb200_quant_nf4.  workspace: 256-byte aligned, cfb200_quant_nf4_tensors_workspace_bytes(count, ns, block) bytes
 * (a descriptor table, copied from host memory -- not callable under stream capture -- and the block maxima). */
size_t cfb200_quant_nf4_tensors_workspace_bytes(int32_t count, const size_t* ns, size_t block);
int32_t cfb200_quant_nf4_tensors(int32_t count, const void* const* srcs, int32_t src_dtype, const size_t* ns,
                                 size_t block, size_t dq_block, uint8_t* const* codes, uint8_t* const* absmax8,
                                 float* const* absmax2, void* workspace, size_t workspace_bytes, void* stream);

/* NF4 for callers that must not allocate.  (No counterpart in the reference: CastForge's passes
 * allocate host vectors freely.)  Some hosts cannot give this library a workspace: an engine whose
 * memory manager has already claimed the whole device, so a cudaMalloc would fail; a serving loop
 * in which any allocation would stall the device between requests; a plug-in interface that only
 * passes the tensors themselves.  For them the per-block maxima that cfb200_quant_nf4 keeps in a
 * caller workspace live in a 4 MiB array built into the library instead (present on every device
 * that loads the library, until the process ends).  Results are identical to cfb200_quant_nf4.
 *  - limit: ceil(n / block) <= 1 048 576 blocks (cfb200_quant_nf4_static_max_elements(block)
 *    elements, 67 108 864 at block 64); larger tensors are rejected with CFB200_ERR_INVALID;
 *  - neither this call nor anything it runs allocates or frees device or pinned memory;
 *  - the first call on each device looks up the array's device address (and uploads the 256-byte
 *    code table) with that device current; make that first call before starting a stream capture;
 *  - all calls on a device share the one array, which still holds the previous call's maxima.
 *    Each call rewrites every slot it later reads, so no clearing is needed, but two calls that
 *    overlap on the GPU (different streams, or different host threads) race: serialise them. */
size_t cfb200_quant_nf4_static_max_elements(size_t block);
int32_t cfb200_quant_nf4_static(const void* src, int32_t src_dtype, size_t n, size_t block,
                                size_t dq_block, uint8_t* codes, uint8_t* absmax8, float* absmax2,
                                void* stream);

/* ---- E4: true FP8 E4M3FN casts (extension) ---------------------------------------------------
 * Encoding = round-to-nearest-even, saturating to +-448, NaN -> 0x7F, i.e. the codec of
 * src/passes/serving/mutable_loads.rs:367-410.  Each row of [rows, cols] gets
 * scale = amax<1e-12 ? 1 : amax/448 and codes = e4m3(v * (1/scale)); rows == tokens gives the
 * dynamic per-token activation scale. */
int32_t cfb200_cast_e4m3_rows(const void* src, int32_t src_dtype, size_t rows, size_t cols,
                              uint8_t* codes, float* scales, void* stream);
/* Per-tensor variant for large weights (two streaming passes instead of one CTA per row).
 * scale_absmax: [0] = scale, [1] = absmax. */
int32_t cfb200_cast_e4m3_tensor(const void* src, int32_t src_dtype, size_t n, uint8_t* codes,
                                float* scale_absmax, void* stream);

/* The per-tensor cast over a whole list of device-resident tensors (the weights of a store on their way to the FP8
 * GEMM) in one cooperative launch per 1024 tensors, with the schedule of cfb200_quant_sym_tensors: arguments as there,
 * scale_absmax = {scale, absmax} per tensor; results identical to cfb200_cast_e4m3_tensor tensor by tensor.  Copies a
 * descriptor table from host memory: not under stream capture.  cfb200_quant_sym_status reports its waits too. */
int32_t cfb200_cast_e4m3_tensors(int32_t count, const void* const* srcs, int32_t src_dtype, const size_t* ns,
                                 uint8_t* const* codes, float* scale_absmax, size_t l2_group_bytes, void* stream);

/* ---- A8: interpreter dequantize + GEMM, bit-exact ----------------------------------------------
 * Replaces eval_matmul_2d (src/codegen/eval.rs:1465-1507) and the fused_qmatmul epilogues
 * (:1145-1179): C[m,n] = sum_k A[m,k]*B, products added in ascending k with separately rounded
 * multiply and add.  B is [K,N] row-major, or [N,K] when packed_rhs.  epilogue: 0 none, 1 bias,
 * 2 bias_relu (max with z), 3 bias_tanh, 4 bias_silu, 5 bias_gelu (tanh form), 6 bias_scale (* z);
 * bias and z are indexed modulo their lengths.  cfb200_qmatmul_i8 reads int8 codes and
 * dequantizes on the fly as (q - zp) * scale (eval.rs:314-317; `scale` is the PARSED 6-decimal
 * string of the quantized type, not the stored f32).  All buffers f32 on the device. */
int32_t cfb200_matmul_f32(const float* A, const float* B, size_t M, size_t N, size_t K,
                          int32_t packed_rhs, int32_t epilogue, const float* bias, size_t bias_len,
                          const float* z, size_t z_len, float* C, void* stream);
int32_t cfb200_qmatmul_i8(const float* A, const int8_t* Wq, float scale, int32_t zero_point,
                          size_t M, size_t N, size_t K, int32_t packed_rhs, int32_t epilogue,
                          const float* bias, size_t bias_len, const float* z, size_t z_len,
                          float* C, void* stream);
int32_t cfb200_dequant_i8(const int8_t* q, size_t n, float scale, int32_t zero_point, float* out,
                          void* stream);
/* castforge.static_quantize prologue (eval.rs:1369-1382): clamp(round(x/sc), +-qmax) * sc. */
int32_t cfb200_static_quantize(const float* x, size_t n, float scale_attr, int32_t bits,
                               float* out, void* stream);

/* ---- Tensor-core GEMMs (tcgen05 / TMEM) ---------------------------------------------------------
 * The reference evaluates every GEMM with the scalar loop above; these are the fast versions of
 * the same contractions for operands that are already narrow.  All compute
 * C[M,N] = sum_k A[m,k] * B[n,k] with both operands K-major (the `packed_rhs` orientation of
 * eval_matmul_2d, src/codegen/eval.rs:1496-1500) and f32 accumulation.  error_flag: NULL or a
 * device int the kernel sets non-zero if one of its bounded waits ran out (the call itself still
 * returns 0: check the flag after synchronising).
 *  cfb200_gemm_fp8:   A, W are E4M3FN codes (cfb200_cast_e4m3_rows / _tensor); C = acc *
 *                     a_scales[m] * w_scale; a_scales may be NULL.  K % 16 == 0.
 *  cfb200_gemm_bf16_nt: bf16 operands; C = alpha * acc; upper_only skips tiles strictly below
 *                     the diagonal (symmetric products such as the GPTQ Hessian).  K % 8 == 0.
 *  cfb200_gemm_w4a16: A bf16 [M,K]; W in the layout cfb200_quant_int4_asym produces for a [N,K]
 *                     matrix with groups along K, dequantised as (q - zp) * scale inside the
 *                     kernel.  Both operands run as f16 (11 significant bits), so the
 *                     activations are first copied to f16 (saturating at +-65504) into
 *                     `workspace` (cfb200_gemm_w4a16_workspace_bytes, which also covers the
 *                     f32 partial sums of the split-K schedule used when M <= 256 leaves too
 *                     few output tiles for the device; a reduction launch follows).
 *                     K % 64 == 0, group % 64 == 0.
 * C is bf16 (out_f32 == 0) or f32, row-major [M,N]. */
int32_t cfb200_gemm_fp8(const uint8_t* A, const float* a_scales, const uint8_t* W, float w_scale,
                        size_t M, size_t N, size_t K, void* C, int32_t out_f32,
                        int32_t* error_flag, void* stream);
int32_t cfb200_gemm_bf16_nt(const void* A, const void* B, size_t M, size_t N, size_t K, float alpha,
                            void* C, int32_t out_f32, int32_t upper_only, int32_t* error_flag,
                            void* stream);
/* cfb200_gemm_bf16_nt with explicit row pitches (lda, ldb in elements, multiples of 8: the operands may be column
 * ranges of wider matrices) and `accumulate` (f32 output only): C += alpha * acc, one rounded f32 addition per element. */
int32_t cfb200_gemm_bf16_nt_ld(const void* A, size_t lda, const void* B, size_t ldb, size_t M, size_t N, size_t K,
                               float alpha, void* C, int32_t out_f32, int32_t upper_only, int32_t accumulate,
                               int32_t* error_flag, void* stream);
/* The same product with a row pitch for C as well (ldc elements: C may be a block of a wider matrix) and a triangle
 * selector: 0 = every tile, 1 = only the tiles that touch the upper triangle, 2 = only those that touch the lower. */
int32_t cfb200_gemm_bf16_nt_ex(const void* A, size_t lda, const void* B, size_t ldb, size_t M, size_t N, size_t K,
                               float alpha, void* C, size_t ldc, int32_t out_f32, int32_t triangle, int32_t accumulate,
                               int32_t* error_flag, void* stream);
size_t cfb200_gemm_w4a16_workspace_bytes(size_t M, size_t N, size_t K);
int32_t cfb200_gemm_w4a16(const void* A, const uint8_t* w_codes, const uint16_t* w_scales,
                          const uint8_t* w_zps, size_t M, size_t N, size_t K, size_t group, void* C,
                          int32_t out_f32, void* workspace, size_t workspace_bytes,
                          int32_t* error_flag, void* stream);

/* cfb200_gemm_w4a16 with castforge.static_quantize{scale, bits} on the activation operand (the `w8a8` rewrite of
 * lower-mixed-precision, src/passes/quantize/formats.rs:541-611, evaluated by src/codegen/eval.rs:1369-1382) folded
 * into the pass that stages the activations as f16: each value becomes clamp(round(x / scale), +-qmax) * scale in f32,
 * with the interpreter's arithmetic, before it is rounded to f16 -- no separate launch, no extra copy of A.
 * a_dtype: CFB200_F32 or CFB200_BF16; a_scale <= 0 means the interpreter's default 1/127; a_bits 4 -> qmax 7, else 127. */
int32_t cfb200_gemm_w4a16_static_quantize(const void* A, int32_t a_dtype, float a_scale, int32_t a_bits,
                                          const uint8_t* w_codes, const uint16_t* w_scales, const uint8_t* w_zps,
                                          size_t M, size_t N, size_t K, size_t group, void* C, int32_t out_f32,
                                          void* workspace, size_t workspace_bytes, int32_t* error_flag, void* stream);

/* Decode shapes (1 <= M <= 16): the same W4A16 product, HBM-bound on the packed weights, which are
 * streamed once; dequantisation is exact (integer (q - zp) on the tensor cores, group scale
 * applied to the f32 group sum).  group must be 128, K % 128 == 0.  No workspace, one launch. */
int32_t cfb200_gemv_w4a16(const void* A, const uint8_t* w_codes, const uint16_t* w_scales,
                          const uint8_t* w_zps, size_t M, size_t N, size_t K, size_t group, void* C,
                          int32_t out_f32, void* stream);
/* Synchronises the device and reports whether a bounded wait inside a decode kernel has ever run
 * out on it (0 = never; sticky).  The waits are on the kernel's own bulk copies and cannot run out
 * on a healthy device; a non-zero flag means the outputs since then are not to be trusted. */
int32_t cfb200_gemv_w4a16_status(int32_t* flag_host);

/* ---- E5: GPTQ, 4 bits, group 128, columns in natural order (no reference counterpart) -----------
 * Three steps, each with a caller-provided workspace (the *_workspace_bytes queries):
 *  cfb200_gptq_hessian:  H[K,K] f32 = X^T X / T for calibration activations X [T,K] bf16
 *                        (T % 8 == 0), on the tensor cores through cfb200_gemm_bf16_nt.
 *  cfb200_gptq_prepare:  U[K,K] f32 = the upper Cholesky factor of
 *                        (H + damp_ratio * mean(diag H) * I)^-1; a zero diagonal entry (dead input
 *                        channel) is replaced by 1.  Products of 1024 rows and more inside the
 *                        factorisation run on the bf16 tensor cores with f32 operands split three
 *                        ways (f32-level accuracy); if a bounded wait of such a launch runs out,
 *                        U[0] is set to NaN, so a factor with a positive diagonal is a good one.
 *  cfb200_gptq_quantize: W [N,K] (dtype code) -> codes / scales / zero_points in the layout of
 *                        cfb200_quant_int4_asym with group 128 along K, each column's rounding
 *                        error pushed into the columns right of it through U.  Rows are
 *                        independent, so ranks may each take a row range with the same U.
 *                        w_dequant: NULL or [N,K] f32 receiving (q - zp) * scale. */
size_t cfb200_gptq_hessian_workspace_bytes(size_t T, size_t K);
int32_t cfb200_gptq_hessian(const void* X, size_t T, size_t K, float* H, void* xt_workspace,
                            size_t workspace_bytes, int32_t* error_flag, void* stream);
size_t cfb200_gptq_prepare_workspace_bytes(size_t K);
int32_t cfb200_gptq_prepare(const float* H, size_t K, float damp_ratio, float* U, void* workspace,
                            size_t workspace_bytes, void* stream);
size_t cfb200_gptq_quantize_workspace_bytes(size_t N, size_t K);
int32_t cfb200_gptq_quantize(const void* W, int32_t w_dtype, size_t N, size_t K, const float* U,
                             uint8_t* codes, uint16_t* scales, uint8_t* zero_points,
                             float* w_dequant, void* workspace, size_t workspace_bytes,
                             void* stream);

/* H = alpha * X^T X (cfb200_gptq_hessian is this with alpha = 1 / T): one token shard's share of a Hessian that
 * several ranks accumulate, alpha = 1 / total tokens. */
int32_t cfb200_gptq_hessian_scaled(const void* X, size_t T, size_t K, float alpha, float* H, void* xt_workspace,
                                   size_t workspace_bytes, int32_t* error_flag, void* stream);

/* ---- Several GPUs of one machine ------------------------------------------------------------------
 * One communicator per GPU: one process per GPU (cfb200_comm_unique_id on one rank, the 128 bytes handed to the others
 * by whatever the host has -- MPI, a file, torch.distributed --, cfb200_comm_init on every rank with its device
 * current), or one process that drives `ndev` devices from one host thread per device (cfb200_comm_init_local).
 * Communication is plain NCCL (opened with dlopen when the first of these calls is made; the rest of the library works
 * without it), collectives are enqueued on the caller's stream, no kernel reads another GPU's memory.
 * The reference has no counterpart: it stamps all_gather / all_reduce attributes on its graph
 * (src/passes/distributed/spmd.rs:416-478) and evaluates them as the identity (src/codegen/eval.rs:1449-1455).
 *
 * Placement (host arithmetic, the same answer on every rank, nothing exchanged):
 *  cfb200_shard_assign: owner[i] = rank that quantizes tensor i whole -- largest first onto the least-loaded rank, equal
 *    sizes in store order, ties to the lowest rank -- or -1 for a tensor of split_min_bytes or more (0 = never), which
 *    every rank takes a row block of.
 *  cfb200_shard_row_range: rows [begin, end) of `rank` when `rows` rows are dealt out in units of `align` rows; blocks
 *    differ by at most one unit, trailing ranks may be empty.
 *
 * cfb200_quant_sym_tensors_sharded: A1 over this rank's part of a store (QuantizeWeightsPass::run's loop,
 *  src/passes/quantize/schemes.rs:324-452, dealt over ranks).  Arguments as cfb200_quant_sym_tensors; is_row_block[i] != 0
 *  marks a buffer that holds this rank's rows of a tensor split over ALL ranks (every rank passes the split tensors in
 *  the same order; an empty block has ns[i] == 0).  Whole tensors need nothing from other ranks; for a row block the
 *  ranks take the maximum of their partial absmax (one float per split tensor, one grouped ncclAllReduce), so scale and
 *  codes are bit-identical to the one-GPU result.  scale_absmax[2 i] holds the tensor's scale on every rank.
 *
 * Column-parallel GEMMs: every rank holds N_local = N / world rows of the [N, K] weight (rank r: rows
 *  [r N_local, (r + 1) N_local), with their scales and zero points) and the whole activation matrix.  The rank's block of
 *  the product comes from cfb200_gemm_w4a16 (cfb200_gemv_w4a16 when M <= 16 and group == 128) or cfb200_gemm_fp8; the
 *  blocks are then rejoined so that every rank holds the whole bf16 product in C: layout 0 = row-major [M, N], layout 1 =
 *  [world][M][N_local].  Products of 8 MB and more between ranks that are separate processes on one node: the blocks are
 *  written to exchange buffers that the library allocates and the ranks map from one another (CUDA IPC; set up by the
 *  first call of a shape class, which synchronises the stream and must not run under stream capture), one small
 *  all-reduce says that every block is complete, and a copy kernel reads the peers' blocks over NVLink straight into C.
 *  Otherwise: one ncclAllGather (plus one interleaving launch for layout 0 with M > 1).  Either way the bits in C are
 *  the local kernels' bits.  N_local % 8 == 0; workspace (256-byte aligned) of
 *  cfb200_gemm_colpar_workspace_bytes(..., w4 = 1 or 0).  Calls on one communicator are issued in the same order on
 *  every rank (as for any collective).
 *
 * cfb200_gptq_hessian_sharded: every rank passes its T_local calibration tokens (T_local % 8 == 0, may be 0); H receives
 *  X^T X / T_total summed over ranks (one ncclAllReduce of K x K floats).  The factor U is then computed on every rank
 *  (cfb200_gptq_prepare) and each rank walks its own output rows with cfb200_gptq_quantize: no communication in the
 *  walk.  The sum over ranks adds in another order than one GPU does, so H agrees to rounding, not bit for bit; pass
 *  every token to every rank (T_local = T_total, world-size-1 behaviour) when bit-identical codes are wanted. */
typedef struct cfb200_comm cfb200_comm_t;
int32_t cfb200_comm_unique_id(void* id_out_128_host);
int32_t cfb200_comm_init(const void* id_128_host, int32_t world, int32_t rank, cfb200_comm_t** comm_out);
int32_t cfb200_comm_init_local(int32_t ndev, const int32_t* devices, cfb200_comm_t** comms_out);
int32_t cfb200_comm_world(const cfb200_comm_t* comm);
int32_t cfb200_comm_rank(const cfb200_comm_t* comm);
void cfb200_comm_free(cfb200_comm_t* comm);
int32_t cfb200_nccl_version(int32_t* version_out);
int32_t cfb200_shard_assign(int32_t count, const size_t* nbytes, int32_t world, size_t split_min_bytes, int32_t* owner);
int32_t cfb200_shard_row_range(size_t rows, int32_t world, int32_t rank, size_t align, size_t* row_begin, size_t* row_end);
int32_t cfb200_quant_sym_tensors_sharded(cfb200_comm_t* comm, int32_t count, const void* const* srcs, int32_t src_dtype,
                                         const size_t* ns, const int32_t* is_row_block, int32_t bits,
                                         int8_t* const* codes, float* scale_absmax, void* stream);
size_t cfb200_gemm_colpar_workspace_bytes(size_t M, size_t N_local, size_t K, int32_t world, int32_t w4);
int32_t cfb200_gemm_w4a16_colpar(cfb200_comm_t* comm, const void* A, const uint8_t* w_codes, const uint16_t* w_scales,
                                 const uint8_t* w_zps, size_t M, size_t N_local, size_t K, size_t group, void* C,
                                 int32_t layout, void* workspace, size_t workspace_bytes, int32_t* error_flag,
                                 void* stream);
int32_t cfb200_gemm_fp8_colpar(cfb200_comm_t* comm, const uint8_t* A, const float* a_scales, const uint8_t* W_local,
                               float w_scale, size_t M, size_t N_local, size_t K, void* C, int32_t layout,
                               void* workspace, size_t workspace_bytes, int32_t* error_flag, void* stream);
int32_t cfb200_gptq_hessian_sharded(cfb200_comm_t* comm, const void* X_local, size_t T_local, size_t T_total, size_t K,
                                    float* H, void* xt_workspace, size_t workspace_bytes, int32_t* error_flag,
                                    void* stream);

/* ---- GGUF block formats (the on-disk step after quantize) ----------------------------------------
 * cfb200_gguf_pack_q8_0: what export_gguf_bytes does with a per-tensor INT8 tensor
 * (src/ir/formats/gguf.rs:283-296): blocks of 34 bytes = the tensor's scale as f16 bits (truncating
 * f32_to_f16_bits, src/ir/tensor_store.rs:85-101, the same in every block) + 32 codes; the last
 * block is zero-padded and an empty tensor still yields one block.  out: cfb200_gguf_q8_0_bytes(n).
 * cfb200_gguf_unpack_q8_0 / _q4_0: decode_ggml_tensor (gguf.rs:536-552, :513-534): f32 = q * d
 * with d = f16_bits_to_f32(block scale); Q4_0 = 18-byte blocks, (nibble - 8) * d, low nibble first. */
size_t cfb200_gguf_q8_0_bytes(size_t n);
size_t cfb200_gguf_q4_0_bytes(size_t n);
int32_t cfb200_gguf_pack_q8_0(const int8_t* codes, size_t n, float scale, uint8_t* out, void* stream);
int32_t cfb200_gguf_unpack_q8_0(const uint8_t* blocks, size_t n, float* out, void* stream);
int32_t cfb200_gguf_unpack_q4_0(const uint8_t* blocks, size_t n, float* out, void* stream);

/* ---- KV-cache page codecs --------------------------------------------------------------------------
 * K16/V8 (AsymK16V8Codec, src/passes/serving/kv_attention.rs:52-222) over k, v of shape
 * [num_pages, page_tokens, num_kv_heads, head_dim] (contiguous, f32 as in the reference, or f16 /
 * bf16 widened first): k_f16_bits = truncating f32_to_f16_bits of every key
 * (src/ir/tensor_store.rs:85-101); v_codes = clamp(round(v / scale), -127, 127), NaN -> 0;
 * scale = absmax / 127, or 1.0 when the absmax of its scope is 0.  scope: 0 = one scale,
 * 1 = one per kv head, 2 = one per (page, kv head), laid out [page][head]; v_scales holds
 * cfb200_kv_scale_count(scope, ...) floats.  head_dim must be a multiple of 4 (f32) or 8 (16-bit
 * sources), num_kv_heads <= 1024; an empty shape is an error, as in the reference.  Scope 2 is one
 * launch that reads the cache once; the wider scopes take three.
 * cfb200_kv_decode_k16v8: k_out = f16_bits_to_f32, v_out = code * scale (f32, head_dim % 4 == 0).
 * cfb200_e4m3_slice_encode / _decode: the float8_e4m3fn slice codec
 * (src/passes/serving/mutable_loads.rs:431-441): one byte per f32 element, no scale, RNE onto the
 * E4M3FN grid, saturating at +-448, NaN -> 0x7F; decoding 0x7F / 0xFF gives NaN. */
size_t cfb200_kv_scale_count(int32_t scope, size_t num_pages, size_t num_kv_heads);
int32_t cfb200_kv_encode_k16v8(const void* k, const void* v, int32_t src_dtype, size_t num_pages,
                               size_t page_tokens, size_t num_kv_heads, size_t head_dim, int32_t scope,
                               uint16_t* k_f16_bits, int8_t* v_codes, float* v_scales, void* stream);
int32_t cfb200_kv_decode_k16v8(const uint16_t* k_f16_bits, const int8_t* v_codes, const float* v_scales,
                               size_t num_pages, size_t page_tokens, size_t num_kv_heads,
                               size_t head_dim, int32_t scope, float* k_out, float* v_out, void* stream);
int32_t cfb200_e4m3_slice_encode(const float* src, size_t n, uint8_t* codes, void* stream);
int32_t cfb200_e4m3_slice_decode(const uint8_t* codes, size_t n, float* out, void* stream);
/* The reference codec byte for byte.  f32_to_fp8_e4m3fn (mutable_loads.rs:391-393) takes its exponent from
 * floor(log2f(|v|)); for the few f32 values within 8 ulp below a power of two 2^k whose logarithm rounds up to k it
 * returns the byte of 1.125 * 2^k where round-to-nearest-even (cfb200_e4m3_slice_encode) gives 2^k.  This entry point
 * reproduces those bytes too: which inputs slip is taken from the host's own log2f on the first call on each device
 * (make that call outside stream capture).  Everything else is identical to cfb200_e4m3_slice_encode. */
int32_t cfb200_e4m3_slice_encode_ref(const float* src, size_t n, uint8_t* codes, void* stream);

/* ---- weight surgery upstream of quantize ----------------------------------------------------------
 * cfb200_merge_f32: merge_f32_tensors (src/passes/weights/merge.rs:396-440) over two f32 tensors of n
 * elements.  method 0 = linear `(1 - t) a + t b`, 1 = SLERP, 2 = TIES.  Linear and TIES are
 * bit-exact (every product and sum rounded on its own).  SLERP's two coefficients come from f64
 * sums of a.a, b.b, a.b and double-precision acos / sin rounded to f32 -- the reference adds in f32
 * in index order, so the coefficients agree to its own summation error (which grows like
 * sqrt(n) * 6e-8 relative); with near-zero norms it falls back to linear like the reference.  coef_out: NULL
 * or two device floats that receive the coefficients used.  workspace (SLERP only):
 * cfb200_merge_workspace_bytes().  out must not alias a or b.
 * cfb200_task_vector_merge: MergeTaskVectorsPass (merge.rs:271-290) with apply_dare_pruning
 * (:357-384): out = base + sum_c lambda * prune(finetuned[c] - base); prune zeroes the
 * floor(n * p) entries of smallest magnitude (p = clamp(drop_rate, 0, 0.99); ties: lowest index
 * first) and multiplies the rest by 1 / (1 - p); p <= 1e-6 prunes nothing.  Bit-exact.
 * `finetuned` is a host array of `count` device pointers.  NaN deltas are kept (the reference's
 * ordering is undefined for them).  out must not alias base or a finetuned tensor. */
size_t cfb200_merge_workspace_bytes(void);
int32_t cfb200_merge_f32(const float* a, const float* b, size_t n, int32_t method, float t, float* out,
                         float* coef_out, void* workspace, size_t workspace_bytes, void* stream);
size_t cfb200_task_vector_merge_workspace_bytes(size_t n);
int32_t cfb200_task_vector_merge(const float* base, const float* const* finetuned, int32_t count,
                                 size_t n, float lambda, float drop_rate, float* out, void* workspace,
                                 size_t workspace_bytes, void* stream);

/* cfb200_prune_2to4: apply_2to4_mask (src/passes/weights/prune.rs:548-565), in place: in every aligned
 * group of four the two entries of smallest magnitude become 0.0 (ties: lower index first); a
 * trailing group of fewer than four is untouched.
 * cfb200_prune_columns_l1: prune_2d_columns_by_l1 (prune.rs:568-603) on a row-major [rows, cols]
 * matrix: column scores = f32 sums of |w| down the rows in row order, the keep_cols best columns
 * (ties: lower index first; keep_cols is clamped to [1, cols]) are kept in ascending index order;
 * out = [rows, keep_cols], kept_idx = keep_cols column indices.  cfb200_prune_keep_cols gives the
 * count PruneStructuredPass::run derives from `sparsity` (prune.rs:339-341).  An empty matrix is an
 * error here (the reference returns its input).
 * cfb200_transpose_f32: pack-weights (src/passes/weights/fold.rs:549-554), [K, N] -> [N, K].
 * All three are bit-exact. */
int32_t cfb200_prune_2to4(float* w, size_t n, void* stream);
size_t cfb200_prune_keep_cols(size_t cols, float sparsity);
size_t cfb200_prune_columns_workspace_bytes(size_t cols);
int32_t cfb200_prune_columns_l1(const float* w, size_t rows, size_t cols, size_t keep_cols, float* out,
                                int32_t* kept_idx, void* workspace, size_t workspace_bytes,
                                void* stream);
int32_t cfb200_transpose_f32(const float* w, size_t K, size_t N, float* out, void* stream);

/* LoRA / DoRA baking (`merge-weights(method=lora | dora)`), bit-exact, in place on a row-major [k, n] f32 weight.
 * cfb200_lora_bake: BakeLoraPass::run (src/passes/weights/lora.rs:79-88): W += alpha * (A [k, r] @ B [r, n]), the
 * inner sum in f32 with p ascending and no fused multiply-add.
 * cfb200_column_norms: mags[j] = max(sqrt(sum over rows of v^2), 1e-8), the sum in f32 in row order (lora.rs:305-313)
 * -- call it on the base weight before the bake.
 * cfb200_dora_renorm: lora.rs:353-369: every column becomes orig_mags[j] * (v / norm_j), norm_j as above on the
 * current weight; orig_mags NULL keeps each column's own norm; `norms` (n floats) receives the norm_j. */
int32_t cfb200_lora_bake(float* W, const float* A, const float* B, size_t k, size_t n, size_t r, float alpha,
                         void* stream);
int32_t cfb200_column_norms(const float* W, size_t k, size_t n, float* mags, void* stream);
int32_t cfb200_dora_renorm(float* W, size_t k, size_t n, const float* orig_mags, float* norms, void* stream);
/* fold-weights(mode=norm | batchnorm), the weight side (src/passes/weights/fold.rs:235-240, :416-437): a [rows, cols]
 * f32 weight is multiplied in place by scale[i % scale_len], i the row (axis 0: a pre-GEMM norm gamma over K, or the
 * output channel of a packed [N, K] weight) or the column (axis 1: the output channel of a [K, N] weight). */
int32_t cfb200_fold_scale(float* W, size_t rows, size_t cols, const float* scale, size_t scale_len, int32_t axis,
                          void* stream);

/* ---- A9: block ops around the GEMMs (f32) ------------------------------------------------------
 * fused_rmsnorm / fused_residual_rmsnorm (eval.rs:1058-1089, :1180-1213; residual may be NULL,
 * weight may be NULL or of length cols or rows*cols), fused_rope half-split (:1096-1118),
 * fused_swiglu (:1090-1095), fused_attention (:1607-1668) over `batch` heads addressed by row
 * (ld_*) and head (hs_*) strides in floats; mask is NULL or [seq_q, seq_kv] added to the scores. */
int32_t cfb200_rmsnorm(const float* x, const float* residual, const float* weight, size_t weight_len,
                       size_t rows, size_t cols, float eps, float* out, void* stream);
int32_t cfb200_rope(const float* x, const float* cos_t, const float* sin_t, size_t rows, size_t cols,
                    float* out, void* stream);
int32_t cfb200_swiglu(const float* gate, const float* up, size_t n, float* out, void* stream);
int32_t cfb200_attention(const float* q, const float* k, const float* v, const float* mask,
                         int32_t batch, int32_t seq_q, int32_t seq_kv, int32_t d_k, int32_t d_v,
                         size_t ld_q, size_t ld_k, size_t ld_v, size_t ld_o, size_t hs_q, size_t hs_k,
                         size_t hs_v, size_t hs_o, float scale, float* out, void* stream);

/* ---- TensorStore handles (host memory) ---------------------------------------------------------------
 * The weight plane of the reference (src/ir/tensor_store.rs:13-39) as an opaque handle, with its
 * SafeTensors layout (scale / zero_point in the header, I8 payload: :300-309, :427-757), and the
 * pass manager entry that the reference only has in-process (src/passes/registry/manager.rs:281-331):
 * cfb200_store_run_pipeline parses a pipeline string with the reference's grammar and option rules
 * and runs each quantize-family pass over every eligible tensor, streaming host -> device -> host.
 * dtype codes: 0 F32, 1 F16, 2 BF16, 3 I8, 4 U8.  `borrow` != 0 keeps the caller's buffer (which
 * must outlive the store entry; pinned memory copies fastest) instead of copying it.
 * Extension schemes are selected by exact name: scheme=per_channel | int4_asym | nf4 | fp8_e4m3;
 * they add companion entries "<name>.scales", "<name>.zeros", "<name>.absmax8", "<name>.absmax2".
 * Strings returned through out-pointers are released with castforge_free_string. */
typedef struct cfb200_store cfb200_store_t;
cfb200_store_t* cfb200_store_new(void);
void cfb200_store_free(cfb200_store_t* store);
const char* cfb200_store_last_error(void);
int32_t cfb200_store_insert(cfb200_store_t* store, const char* name, int32_t dtype, const int64_t* shape,
                            int32_t rank, const void* host_data, int32_t borrow);
int32_t cfb200_store_len(cfb200_store_t* store);
int32_t cfb200_store_entry(cfb200_store_t* store, int32_t index, const char** name, int32_t* dtype,
                           int32_t* rank, const int64_t** shape, const void** data, size_t* nbytes,
                           int32_t* quantized, float* scale, int64_t* zero_point);
const char* cfb200_store_entry_attrs(cfb200_store_t* store, int32_t index);
int32_t cfb200_store_run_pipeline(cfb200_store_t* store, const char* pipeline_spec,
                                  char** out_telemetry_json, char** out_error);
int32_t cfb200_store_save_safetensors(cfb200_store_t* store, const char* path);
int32_t cfb200_store_load_safetensors(cfb200_store_t* store, const char* path);
int32_t cfb200_store_load_safetensors_bytes(cfb200_store_t* store, const void* bytes, size_t n);
/* load_safetensors_lazy_file (src/ir/tensor_store.rs:779-890): reads only the JSON header and registers
 * every tensor as a slice of the file (TensorBacking::ExternalFile); count_out (nullable) = tensors
 * registered.  A slice is read when cfb200_store_entry asks for its bytes, when the store is saved,
 * or -- the case this exists for -- by cfb200_store_run_pipeline, which reads each slice with several
 * threads straight into pinned staging memory one tensor ahead of the host -> device copies, so the
 * float weights never sit in host memory as a whole.  The file must stay in place meanwhile. */
int32_t cfb200_store_load_safetensors_lazy(cfb200_store_t* store, const char* path, int32_t* count_out);
/* The `{:.6}`-and-trim scale string of a quantized type (src/passes/quantize/formats.rs:680-688). */
int32_t cfb200_format_scale(float scale, char* out, size_t out_len);

#ifdef __cplusplus
}
#endif

#endif /* CFB200_H */
