/*
 * C ABI of libint64gemm.so — the B200 (sm_100a) implementation of the int64
 * fixed-point hot path of ZK-DeepSeek's integer DeepSeek-V3 forward pass.
 *
 * Two groups of entry points:
 *
 *  1. The 21 symbols the reference library exports (inference/int64_gemm.cu),
 *     with identical names and argument lists, so that the reference's
 *     inference/kernel.py can load this library unchanged.  They return void,
 *     launch on the legacy default stream and take C `int` extents like the
 *     originals.  Element indices are 64-bit inside, so tensors of 2^31 elements
 *     and more (where the reference's `int` indices overflow) are handled.  A
 *     rejected call writes nothing, keeps its status for zkds_last_status() and
 *     prints one line to stderr.
 *
 *  2. zkds_* entry points: same arithmetic, 64-bit extents, an explicit stream,
 *     an int status return, and the parameters the reference hard-codes.
 *
 * All pointers are device pointers unless a comment says HOST.  Tensors are
 * dense and row-major in the shapes given.  No entry point synchronises the
 * device except where a comment says so.
 *
 * Concurrency.  The contraction entry points keep their scratch (limb planes of the
 * operands they split, range words, split-K partial sums) in ONE arena per device,
 * owned by the library and reused by the next call.  Calls on one device must
 * therefore be issued from one host thread at a time and on one stream (or on
 * streams the caller orders with events so that two calls never overlap on the
 * GPU): two calls in flight at once would overwrite each other's planes.  Calls on
 * different devices are independent.  Prepared weight planes (zkds_planes_create)
 * are read-only afterwards and may be shared freely.
 */
#ifndef ZKDS_INT64_H
#define ZKDS_INT64_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status ------------------------------------------------------------------ */
#define ZKDS_OK 0
#define ZKDS_ERR_ARG 1
#define ZKDS_ERR_RANGE 2
#define ZKDS_ERR_CUDA 3
#define ZKDS_ERR_WORKSPACE 4
#define ZKDS_ERR_DEVICE 5
#define ZKDS_ERR_UNSUPPORTED 6

int zkds_last_status(void);         /* status of the most recent call on this thread */
int zkds_last_cuda_error(void);     /* cudaError_t behind the last ZKDS_ERR_CUDA */
const char* zkds_status_string(int status);
const char* zkds_version(void);
void zkds_shutdown(void);           /* frees the library's scratch arenas (synchronises) */
/* Health of the tensor-core kernels that have FINISHED on the current device (no sync):
 * ZKDS_ERR_DEVICE if one of them gave up a bounded wait, ZKDS_ERR_RANGE if an operand did
 * not fit the a_limbs/b_limbs the caller promised (the result of that call is wrong), else
 * ZKDS_OK.  clear != 0 resets the flags. */
int zkds_device_status(int clear);

/* ---- flags of the contraction entry points ----------------------------------- */
#define ZKDS_ALGO_AUTO 0        /* limb tensor-core kernel when it applies, else exact */
#define ZKDS_ALGO_EXACT 1       /* CUDA-core kernel with 128-bit accumulators */
#define ZKDS_ALGO_LIMB 2        /* tensor-core kernel or ZKDS_ERR_UNSUPPORTED */
#define ZKDS_ALGO_MASK 3
#define ZKDS_REMAINDER_LEGACY 4 /* R as the reference binary returns it: its mask
                                   "(1 << s) - 1" uses a 32-bit 1 (int64_gemm.cu:22), which is
                                   exact for s <= 31 and yields the low 32 bits of the sum for
                                   every s >= 32 (observed with its nvcc 12.9 build on a B200).
                                   Default: R = sum mod 2^s. */

#define ZKDS_LIMBS_DYNAMIC 8    /* a_limbs > 0 is an upper bound on the limbs of A: the count
                                   actually needed is derived on the device from the range seen
                                   while A is split (no host synchronisation).  Data beyond the
                                   bound raises the flag zkds_device_status reports. */

#define ZKDS_CAUSAL_SKIP 16      /* score entry points with causal != 0: output tiles that lie entirely
                                   in the masked region are neither computed nor written (their
                                   contents are undefined).  Only for callers that never read masked
                                   scores: zkds_softmax_causal / zkds_einsum_bsht_btc_bshc_causal. */

#define ZKDS_GROUP_ROWS_32 32    /* grouped entry points (tile_group != null): the caller promises that no group */
#define ZKDS_GROUP_ROWS_64 64    /* holds more than 32 (64) rows, i.e. only the first 32 (64) rows of every
                                   128-row tile are tokens and the rest is padding.  The kernel then fetches
                                   only those rows of A (decode: a few rows per expert, the weights stream
                                   from HBM and the A tiles from L2, so a smaller A box is less L2 traffic and
                                   a deeper pipeline); padding rows come out as zero rows do.  A token names
                                   an expert at most once, so a group never has more rows than there are tokens:
                                   up to that many tokens the bound is certain.  With the fused gather
                                   (row_index given) a row beyond the bound raises the flag zkds_device_status
                                   reports, like a limb bound that did not hold, so a caller may also promise
                                   optimistically and repeat the call without the flag when it is told so;
                                   without row_index such a row is lost silently. */

/* =============================================================================
 * Group 1 — the reference's symbols (same names, same argument lists)
 * ========================================================================== */

/* inference/int64_gemm.cu:36-47.  C = (sum_k (A/a_rescale)*(B/b_rescale)) >> c_rescale with
 * a 128-bit sum, R = remainder (legacy flavour).  A (B,M,K) int64, B (N,K) int32. */
void int64_32_bmm_broadcast_launcher(const int64_t* A, const int32_t* B, int64_t* C, int64_t* R,
                                     const int64_t a_rescale, const int64_t b_rescale,
                                     const int64_t c_rescale, int Bdim, int M, int K, int N);
/* inference/int64_gemm.cu:79-90.  Same with B (N,K) int64. */
void int64_64_bmm_broadcast_launcher(const int64_t* A, const int64_t* B, int64_t* C, int64_t* R,
                                     const int64_t a_rescale, const int64_t b_rescale,
                                     const int64_t c_rescale, int Bdim, int M, int K, int N);
/* inference/int64_gemm.cu:126-132, 173-179, 215-221: float bit pattern -> fixed point
 * (exported by the reference, called by nothing). */
void bf16_to_int32_2d(const uint16_t* input, int32_t* output, int rows, int cols, int rescale);
void wkv_b_bf16_to_int32(const uint16_t* input, int32_t* output, int rows, int cols);
void float32_to_int64_2d(const uint32_t* input, int64_t* output, int rows, int cols, int rescale);
/* inference/int64_gemm.cu:274-286.  RoPE complex multiply, products >> 42; headDim is the
 * number of PAIRS.  A, C (batch,seq,head,pairs,2); B (seq,pairs,2) broadcast. */
void complex_int64_mul(const int64_t* A, const int64_t* B, int64_t* C, int batchSize, int seqLen,
                       int headCount, int headDim);
/* inference/int64_gemm.cu:365-385.  C = floor(A*W / rms[row]); rms is a device array. */
void rms_norm_32(const int64_t* A, const int32_t* W, const int64_t* rms, int64_t* C, int seqLen,
                 int Dim);
void rms_norm_64(const int64_t* A, const int64_t* W, const int64_t* rms, int64_t* C, int seqLen,
                 int Dim);
/* inference/int64_gemm.cu:416-425, 458-467, 499-509, 539-549: the absorbed-MLA einsums.
 * The first three add rescale/2 before the shift, the fourth does not. */
void einsum_bshd_hdc_bshc(const int64_t* q_nope, const int32_t* wkv_b_1, int64_t* out,
                          int64_t rescale, int B, int S, int H, int D, int C);
void einsum_bshc_btc_bsht(const int64_t* A, const int64_t* B, int64_t* C, int64_t rescale, int Bsz,
                          int S, int H, int T, int Cdim);
void einsum_bsht_btc_bshc(const int64_t* A, const int64_t* B, int64_t* C, int64_t rescale, int Bsz,
                          int S, int H, int T, int Cdim);
void einsum_bshc_hdc_bshd(const int64_t* A, const int32_t* B, int64_t* C, int64_t rescale, int Bsz,
                          int S, int H, int D, int Cdim);
/* inference/int64_gemm.cu:661-670, 748-757.  Rows are the last dimension T.  R is
 * overwritten with the unnormalised weights, as in the reference. */
void softmax_q21(int64_t* R, int64_t* C, int64_t* EXP2_FRAC_LUT, int Bsz, int S, int H, int T);
void softmax_q19(int64_t* R, int64_t* C, int64_t* EXP2_FRAC_LUT, int Bsz, int S, int H, int T);
/* inference/int64_gemm.cu:672-680, 759-767.  Fill a HOST table of 256 entries. */
void softmax_init_q21(int64_t* EXP2_FRAC_LUT);
void softmax_init_q19(int64_t* EXP2_FRAC_LUT);
/* inference/int64_gemm.cu:821-830, 884-893, 949-958, 1019-1028 (no device printf). */
void silu_q25(int64_t* R, int64_t* C, int64_t* EXP2_FRAC_LUT_25, int Bsz, int S, int Dim);
void sigmoid_q25(int64_t* R, int64_t* C, int64_t* EXP2_FRAC_LUT_25, int Bsz, int S, int Dim);
void silu_q23(int64_t* R, int64_t* C, int64_t* EXP2_FRAC_LUT_23, int Bsz, int S, int Dim);
void sigmoid_q23(int64_t* R, int64_t* C, int64_t* EXP2_FRAC_LUT_23, int Bsz, int S, int Dim);
/* inference/int64_gemm.cu:832-839, 960-967.  Fill a HOST table of 256 entries. */
void silu_init_q25(int64_t* EXP2_FRAC_LUT);
void silu_init_q23(int64_t* EXP2_FRAC_LUT);

/* =============================================================================
 * Group 2 — status-returning entry points
 * ========================================================================== */

/* Replaces int64_{32,64}_bmm_broadcast_launcher (int64_gemm.cu:36-47, 79-90).
 * b_bits: 32 or 64.  R may be null.  a_limbs/b_limbs: number of signed 8-bit limbs that
 * cover |A/a_rescale| and |B/b_rescale| (0 = measure on the device, which costs one
 * reduction pass and a host synchronisation). */
int zkds_gemm(const int64_t* A, const void* B, int b_bits, int64_t* C, int64_t* R,
              int64_t a_rescale, int64_t b_rescale, int64_t c_rescale, int64_t Bdim, int64_t M,
              int64_t K, int64_t N, int a_limbs, int b_limbs, int flags, void* stream);

/* zkds_gemm for callers that must not allocate (this entry point has no counterpart in the
 * reference).  Same arithmetic and arguments as zkds_gemm, always on the tensor-core limb
 * kernel, but it calls no cudaMalloc, cudaFree, cudaHostAlloc or any other allocating
 * routine: the limb planes and status words it needs live in a fixed 64 MiB device array that
 * is part of the library image, so every GPU that loads the library holds those 64 MiB until
 * the process exits.  Meant for hosts whose own pool already owns the whole GPU (an
 * allocation here would fail or fragment it) or that cannot afford the device-wide
 * synchronisation an allocation implies.
 *   - Capacity: a_limbs*Bdim*M*K16 + b_limbs*N*K16 bytes (K16 = K rounded up to 16, each term
 *     rounded up to 1 KiB) must not exceed zkds_gemm_noalloc_capacity(); larger shapes are
 *     rejected with ZKDS_ERR_RANGE and a message on stderr.  zkds_gemm_noalloc_bytes computes
 *     the need of a shape.  Shapes the limb kernel cannot take give ZKDS_ERR_UNSUPPORTED
 *     (there is no fallback).
 *   - The first call on a device looks up the device address of that array
 *     (cudaGetSymbolAddress with the device current); that first call should come before
 *     any stream capture.  Note that EVERY call, not only the first, ends by waiting for its
 *     stream (last point below).
 *   - Every call uses the same array, which keeps the previous call's bytes; the status words
 *     are cleared at the start of each call.  Two calls whose GPU work overlaps (different
 *     streams or threads) race on it: serialise them.
 *   - The call waits for its own kernels before returning (it reads the status words back),
 *     so the returned status already covers operand-range overflow and device-side waits. */
int zkds_gemm_noalloc(const int64_t* A, const void* B, int b_bits, int64_t* C, int64_t* R,
                      int64_t a_rescale, int64_t b_rescale, int64_t c_rescale, int64_t Bdim, int64_t M,
                      int64_t K, int64_t N, int a_limbs, int b_limbs, int flags, void* stream);
unsigned long long zkds_gemm_noalloc_capacity(void);
unsigned long long zkds_gemm_noalloc_bytes(int64_t Bdim, int64_t M, int64_t K, int64_t N, int a_limbs,
                                           int b_limbs);

/* Replace the four einsum entry points (int64_gemm.cu:416-549). */
int zkds_einsum_bshd_hdc_bshc(const int64_t* q, const int32_t* W, int64_t* out, int64_t rescale,
                              int64_t B, int64_t S, int64_t H, int64_t D, int64_t C, int a_limbs,
                              int b_limbs, int flags, void* stream);
int zkds_einsum_bshc_btc_bsht(const int64_t* A, const int64_t* KV, int64_t* out, int64_t rescale,
                              int64_t B, int64_t S, int64_t H, int64_t T, int64_t C, int a_limbs,
                              int b_limbs, int flags, void* stream);
int zkds_einsum_bsht_btc_bshc(const int64_t* P, const int64_t* KV, int64_t* out, int64_t rescale,
                              int64_t B, int64_t S, int64_t H, int64_t T, int64_t C, int a_limbs,
                              int b_limbs, int flags, void* stream);
int zkds_einsum_bshc_hdc_bshd(const int64_t* A, const int32_t* W, int64_t* out, int64_t rescale,
                              int64_t B, int64_t S, int64_t H, int64_t D, int64_t C, int a_limbs,
                              int b_limbs, int flags, void* stream);

/* einsum_bshc_btc_bsht (int64_gemm.cu:458-467) with the element-wise tail of the attention
 * scores fused into its epilogue (model.py:897-905): v = quotient; v += addin[b,s,h,t] if addin;
 * v = floor(v * ep_mul / ep_div) if ep_div (wrapping int64 multiply, floor division as torch's //);
 * v += mask_value where causal and t > start_pos + s.  MLA uses it as
 * scores = (score1 + score2) * 94 // 695 + mask with score1 passed as addin. */
int zkds_einsum_bshc_btc_bsht_ex(const int64_t* A, const int64_t* KV, int64_t* out, int64_t rescale,
                                 int64_t B, int64_t S, int64_t H, int64_t T, int64_t C,
                                 const int64_t* addin, int64_t ep_mul, int64_t ep_div, int causal,
                                 int64_t start_pos, int64_t mask_value, int a_limbs, int b_limbs,
                                 int flags, void* stream);

/* Both score contractions of the absorbed MLA path and their element-wise tail in ONE tensor-core
 * pass (replaces two einsum_bshc_btc_bsht calls plus the torch ops of model.py:884-905):
 *   out[b,s,h,t] = floor((((r1/2 + q_abs[b,s,h,:].kv[b,t,:]) >> r1) +
 *                          ((r2/2 + q_pe[b,s,h,:].pe[b,t,:]) >> r2)) * ep_mul / ep_div)  (+ mask_value
 *                  where causal and t > start_pos + s).
 * q_abs [B,S,H,C1], kv [B,T,C1], q_pe [B,S,H,C2], pe [B,T,C2], out [B,S,H,T].  Neither partial score
 * tensor is materialised.  Returns ZKDS_ERR_UNSUPPORTED (silently) when C1 is not a multiple of 128
 * or the limb counts do not fit the kernel; callers then fall back to the separate entry points. */
int zkds_mla_scores(const int64_t* q_abs, const int64_t* kv, const int64_t* q_pe, const int64_t* pe,
                    int64_t* out, int64_t B, int64_t S, int64_t H, int64_t T, int64_t C1, int64_t C2,
                    int64_t rescale1, int64_t rescale2, int64_t ep_mul, int64_t ep_div, int causal,
                    int64_t start_pos, int64_t mask_value, int a_limbs, int b_limbs, int flags, void* stream);

/* Causal counterparts for prefill attention whose masked scores were skipped (ZKDS_CAUSAL_SKIP).
 * Row (b, s, h) owns columns t <= start_pos + s only.  The results equal what softmax_q19 and
 * einsum_bsht_btc_bshc give on fully written masked scores, because a masked score (-(64<<36) added)
 * always gets weight 0 (int64_gemm.cu:706-710).
 *  zkds_softmax_causal: Q19 softmax that reads and writes only the owned columns (T even, <= 8192;
 *    ZKDS_ERR_UNSUPPORTED otherwise, silently).
 *  zkds_einsum_bsht_btc_bshc_causal: P . KV that reads only the owned columns of P and skips the K
 *    blocks beyond them; a_limbs must be given (probabilities fit 3 limbs). */
int zkds_softmax_causal(const int64_t* X, int64_t* C, const int64_t* lut, int64_t B, int64_t S, int64_t H,
                        int64_t T, int64_t start_pos, void* stream);
int zkds_einsum_bsht_btc_bshc_causal(const int64_t* P, const int64_t* KV, int64_t* out, int64_t rescale,
                                     int64_t B, int64_t S, int64_t H, int64_t T, int64_t C, int64_t start_pos,
                                     int a_limbs, int b_limbs, int flags, void* stream);

/* softmax_q19 over the rows of `scores` [B,S,H,T] followed by einsum_bsht_btc_bshc with KV [B,T,C]
 * (model.py:911-926 with kernel.py:424-448 and :274-305; no single reference entry point): out
 * [B,S,H,C] = (rescale/2 + sum_t softmax(scores)[b,s,h,t] * KV[b,t,c]) >> rescale.  The softmax kernel
 * writes the probabilities straight into the int8 limb planes the tensor-core contraction reads, so they
 * never reach memory as int64 words; `scores` is left untouched.  causal_skip != 0: row (b, s, h) owns
 * columns t <= start_pos + s only (the rest is not read), as in the two entry points above.
 * a_limbs <= 0 means 3 (a Q19 probability is at most 2^19).  Returns ZKDS_ERR_UNSUPPORTED (silently)
 * when T is not a multiple of 4, T > 8176, `scores` is not 16-byte aligned or the limb kernel declines
 * the shape; callers then use softmax_q19 and the einsum separately. */
int zkds_softmax_pv(const int64_t* scores, const int64_t* KV, int64_t* out, const int64_t* lut,
                    int64_t rescale, int64_t B, int64_t S, int64_t H, int64_t T, int64_t C, int causal_skip,
                    int64_t start_pos, int a_limbs, int b_limbs, int flags, void* stream);

/* ---- the latent cache kept as limb planes (decode) ---------------------------------------------------------
 * The reference's attention reads the whole int64 latent cache every step (model.py:884-926); split into limb
 * planes per call, that is the whole cache re-read and re-written twice per layer and step.  These entry
 * points keep the planes resident instead: each step splits only its new positions, and the score and P . KV
 * contractions read the planes in place.  No reference counterpart.
 *   score planes [limbs][B][capacity][C1 + round16(C2)] int8   (a position is a row: latent | rope part)
 *   value planes [limbs][B][C1][capacity] int8                 (a position is a column)
 * capacity: positions the buffers hold, a multiple of 16; both buffers 16-byte aligned, allocated by the caller
 * (zero-initialised: the padding columns of the score planes are never written).  `limbs` is a promise like
 * a_limbs / b_limbs elsewhere: a value that does not fit raises the flag zkds_device_status reports. */
int zkds_cache_planes_append(const int64_t* kv_new, const int64_t* pe_new, int8_t* score_planes,
                             int8_t* value_planes, int64_t B, int64_t S, int64_t C1, int64_t C2,
                             int64_t start_pos, int64_t capacity, int limbs, void* stream);

/* zkds_mla_scores with the cache side (kv, pe) given as resident score planes holding positions [0, T);
 * b_limbs = the planes' limb count, a_limbs > 0. */
int zkds_mla_scores_cached(const int64_t* q_abs, const int64_t* q_pe, const int8_t* score_planes,
                           int64_t capacity, int64_t* out, int64_t B, int64_t S, int64_t H, int64_t T,
                           int64_t C1, int64_t C2, int64_t rescale1, int64_t rescale2, int64_t ep_mul,
                           int64_t ep_div, int causal, int64_t start_pos, int64_t mask_value, int a_limbs,
                           int b_limbs, int flags, void* stream);

/* zkds_softmax_pv with KV given as resident value planes holding positions [0, T). */
int zkds_softmax_pv_cached(const int64_t* scores, const int8_t* value_planes, int64_t capacity, int64_t* out,
                           const int64_t* lut, int64_t rescale, int64_t B, int64_t S, int64_t H, int64_t T,
                           int64_t C, int causal_skip, int64_t start_pos, int a_limbs, int b_limbs, int flags,
                           void* stream);

/* Grouped linear layer for the routed experts (replaces the per-expert Python loop of
 * MoE.forward, model.py:1355-1379): A is a flat [n_tiles*128, K] int64 matrix whose i-th
 * 128-row tile holds tokens of expert tile_group[i] (device array; negative = unused tile),
 * planes hold every expert's weight (nb = experts).  C [n_tiles*128, N] = (addend + A W_g^T) >> shift.
 * group_shift (device, may be null): per-expert shifts, [2g] for output columns < n_split and
 * [2g+1] from n_split on (n_split a multiple of 8) — each expert's w1, w3, w2 carry their own
 * shift (model.py:231-232) and w1|w3 may be stacked into one weight. */
int zkds_grouped_prepared(const int64_t* A, const void* planes, const int* tile_group, int64_t n_tiles,
                          int64_t* C, int64_t a_rescale, int64_t addend, int64_t shift,
                          const int* group_shift, int64_t n_split, int a_limbs, int flags, void* stream);

/* zkds_grouped_prepared with the row gather of the expert dispatch folded into the limb split: row m of
 * the grouped A matrix is row row_index[m] of A (int32, on the device; a negative entry is a padding row of
 * zeros), so the gathered [n_tiles*128, K] matrix is never written (model.py:1372-1378 builds it with
 * index_select).  a_limbs must be given (> 0).  No reference counterpart as a single entry point. */
int zkds_grouped_gather_prepared(const int64_t* A, const int* row_index, const void* planes, const int* tile_group,
                                 int64_t n_tiles, int64_t* C, int64_t a_rescale, int64_t addend, int64_t shift,
                                 const int* group_shift, int64_t n_split, int a_limbs, int flags, void* stream);

/* The down projection of a gated MLP with the gate folded into its limb split (model.py:1034-1049 and
 * 1271-1281: `(silu_q23(r1) * r2) >> 23` followed by w2): C[rows, N] = (sum_k h[m,k] * W2[n,k]) >> shift with
 * h = (silu_q23(r1) * r2) >> 23 (wrapping product, arithmetic shift) produced directly as int8 limb planes,
 * never stored as int64.  r1, r2: rows of K words with row stride ld (both halves of a stacked w1|w3 output);
 * lut: the Q23 table of silu_init_q23; planes: W2 (zkds_planes_create); tile_group / group_shift / n_split as
 * in zkds_grouped_prepared (rows a multiple of 128 then) or null for a plain linear layer; a_limbs > 0.
 * Returns ZKDS_ERR_UNSUPPORTED (silently) for odd K or ld, unaligned pointers or shapes the limb kernel
 * declines; callers then use zkds_glu_q23 and the linear entry point. */
int zkds_glu_prepared(const int64_t* r1, const int64_t* r2, int64_t ld, const int64_t* lut, int64_t rows,
                      const void* planes, const int* tile_group, int64_t* C, int64_t shift,
                      const int* group_shift, int64_t n_split, int a_limbs, int flags, void* stream);

/* ---- expert parallelism over peer memory (no reference counterpart: the reference sums every rank's expert
 * outputs with a full-tensor all_reduce, model.py:1381-1382).  One process per GPU; the buffers named "of
 * every GPU" are symmetric allocations that each process has mapped (peer pointers, plain loads and stores
 * over NVLink and nothing else).  A layer then runs: publish the local token rows -> zkds_peer_barrier -> the
 * owner's grouped GEMMs, whose limb split reads the rows of every GPU in place
 * (zkds_grouped_gather_parts_prepared) -> zkds_moe_combine_peer writes each token's weighted sum into its home
 * GPU -> zkds_peer_barrier -> zkds_moe_sum_slots on the home GPU.  No row is packed, sent or unpacked by a
 * separate collective. */

/* zkds_grouped_gather_prepared with the source rows spread over n_parts (<= 16) buffers of rows_per_part rows
 * each (parts: host array of device pointers, e.g. the token rows of every GPU): row_index[m] = g names row
 * g % rows_per_part of parts[g / rows_per_part]; negative or beyond the parts = a row of zeros. */
int zkds_grouped_gather_parts_prepared(const int64_t* const* parts, int n_parts, int64_t rows_per_part,
                                       const int* row_index, const void* planes, const int* tile_group,
                                       int64_t n_tiles, int64_t* C, int64_t shift, const int* group_shift,
                                       int64_t n_split, int a_limbs, int flags, void* stream);

/* zkds_moe_combine for the owner of some experts: tokens = n_parts * tokens_per_part gathered tokens, pos
 * [tokens, slots] (row of `out` for each (token, slot), -1 = expert of another GPU), w [tokens, slots].  For
 * every token g with at least one local expert, sum_slot floor(out[pos] * w / 2^23) is stored at
 * slot_bases[g / tokens_per_part] + ((g % tokens_per_part) * n_parts + my_part) * cols: the slot of this owner
 * in the token's home GPU (slot_bases: host array of the n_parts GPUs' slot buffers,
 * [tokens_per_part, n_parts, cols] int64 each, 16-byte aligned).  Other tokens' slots are not written. */
int zkds_moe_combine_peer(const int64_t* out, const int* pos, const int64_t* w, int64_t tokens, int slots,
                          int64_t cols, int64_t tokens_per_part, int64_t* const* slot_bases, int n_parts,
                          int my_part, void* stream);

/* The home GPU's side: y[t] = base[t] (or 0) + sum over the owners q of token t's experts, each once, of
 * slot_rows[t][q]; q = indices[t][slot] / experts_per_part (indices [tokens, slots] int64 global expert ids).
 * Only slots that an owner wrote during this exchange are read. */
int zkds_moe_sum_slots(const int64_t* base, const int64_t* slot_rows, const int64_t* indices, int64_t tokens,
                       int slots, int64_t cols, int n_parts, int experts_per_part, int64_t* y, void* stream);

/* Barrier between the n_parts GPUs on `stream`: flag_bases[i] = GPU i's array of n_parts 64-bit flags
 * (zero-initialised once, peer-mapped); epoch must grow by one with every call, the same on all GPUs.  Work
 * queued before the call on any GPU is complete and visible to work queued after it on every GPU.  The wait
 * is bounded (4 s): on expiry *status (device or mapped host word) becomes 1, the kernel returns and
 * the caller reports the error; nothing spins for ever.  Every GPU must run its kernel concurrently, so the
 * participants are different GPUs, never several processes on one. */
int zkds_peer_barrier(uint64_t* const* flag_bases, int n_parts, int my_part, uint64_t epoch, uint32_t* status,
                      void* stream);

/* Replaces complex_int64_mul (int64_gemm.cu:274-286) with the product shift as a
 * parameter (the reference hard-codes 42). */
int zkds_rope(const int64_t* A, const int64_t* table, int64_t* C, int64_t batch, int64_t seq,
              int64_t heads, int64_t pairs, int shift, void* stream);

/* Replaces RMS_Norm_int64's host loop plus rms_norm_32/64 (kernel.py:477-550,
 * int64_gemm.cu:365-385) with one fused pass: rms[m] = isqrt((eps + sum a^2) / dim),
 * C = floor(A*W / rms).  w_bits: 32 or 64.  rms_out (device, M entries) may be null.
 * A row whose rms is 0 (undefined in the reference) yields zeros. */
int zkds_rms_norm(const int64_t* A, const void* W, int w_bits, int64_t* C, int64_t* rms_out,
                  int64_t M, int64_t N, int64_t eps, int64_t dim, void* stream);
/* rms_norm_32/64 with 64-bit extents: normalise with the caller's per-row rms. */
int zkds_rms_norm_apply(const int64_t* A, const void* W, int w_bits, const int64_t* rms,
                        int64_t* C, int64_t M, int64_t N, void* stream);

/* Replaces softmax_q19 / softmax_q21 (int64_gemm.cu:661-670, 748-757).  frac: 19 or 21.
 * weights_out (may be null, may equal X) receives the unnormalised weights. */
int zkds_softmax(const int64_t* X, int64_t* weights_out, int64_t* C, const int64_t* lut,
                 int64_t rows, int64_t T, int frac, void* stream);

/* Replaces silu_q23/q25 and sigmoid_q23/q25 (int64_gemm.cu:821-1028).  frac: 23 or 25. */
int zkds_act(const int64_t* X, int64_t* C, const int64_t* lut, int64_t n, int frac, int silu,
             void* stream);

/* ---- static operands prepared once (no counterpart in the reference, which re-reads its
 * int32/int64 weights in every call, int64_gemm.cu:25,68) ------------------------------------
 * zkds_planes_create splits W[z*s_batch + n*s_row + k*s_k] / div (z < nb, n < rows, k < K;
 * bits 32 or 64) into signed 8-bit limb planes kept on the device until zkds_planes_destroy.
 * limbs = 0 measures the range (one reduction and a host synchronisation).  Allocates with
 * cudaMalloc. */
int zkds_planes_create(const void* W, int bits, int64_t nb, int64_t rows, int64_t K, int64_t s_batch,
                       int64_t s_row, int64_t s_k, int64_t div, int limbs, void** out, void* stream);
int zkds_planes_limbs(const void* planes);
int zkds_planes_destroy(void* planes);
/* C[z][m][n] = (addend + sum_k (A[z*a_s_batch + m*a_s_row + k] / a_rescale) * W(z or 0, n, k)) >> shift
 * on the tensor-core kernel, W given as prepared planes (N and K come from them; b_batched:
 * W differs per batch z).  R may be null. */
int zkds_contraction_prepared(const int64_t* A, int64_t a_s_batch, int64_t a_s_row, const void* planes,
                              int b_batched, int64_t* C, int64_t* R, int64_t c_s_batch, int64_t c_s_row,
                              int64_t batches, int64_t M, int64_t a_rescale, int64_t addend, int64_t shift,
                              int a_limbs, int flags, void* stream);

/* CUDA-event timing of the tensor-core kernel alone: zkds_timing(1) makes every later
 * contraction record an event pair around that kernel on its stream; zkds_last_kernel_ms
 * waits for the most recent pair and returns its duration (< 0 if there is none). */
void zkds_timing(int enable);
float zkds_last_kernel_ms(void);
/* zkds_timing(2) resets and starts accumulating, over every tensor-core launch, the kernel's
 * duration and the int8 work it issued (limb pairs x 2MNK); each launch is then waited for, so
 * this is a profiling pass.  zkds_timing_totals reads the sums. */
void zkds_timing_totals(double* ms, double* int8_ops, long long* launches);
/* i-th tensor-core launch since zkds_timing(2) (first 256 kept): out8 = {batches, M, N, K, limbs of
 * A used, limbs of B, milliseconds, flags: 1 grouped + 2 B differs per batch}; returns 0 when there
 * is no such record. */
int zkds_timing_record(long long i, double* out8);

/* Tail of the gated MLP (model.py:1034-1048, 1266-1280): h = (silu_q23(r1) * r2) >> 23 with a
 * wrapping int64 product.  r1, r2: rows x n with row stride ld (both halves of a fused w1|w3
 * GEMM output can be passed in place); h dense rows x n; s1_out (may be null) receives
 * silu_q23(r1) for the zk dump.  n and ld even, pointers 16-byte aligned. */
int zkds_glu_q23(const int64_t* r1, const int64_t* r2, int64_t ld, int64_t* h, int64_t* s1_out,
                 const int64_t* lut, int64_t rows, int64_t n, void* stream);
/* Expert dispatch (replaces x[idx] per expert, model.py:1372-1374): dst[r] = src[index[r]], zeros
 * where index[r] < 0.  cols even. */
int zkds_gather_rows(const int64_t* src, const int* index, int64_t* dst, int64_t rows, int64_t cols,
                     void* stream);
/* Expert combine (replaces y[idx] += y2 * w // 2^23 and the final y + z, model.py:1379-1383):
 * y[t] = base[t] + sum_slot floor(out[pos[t][slot]] * w[t][slot] / 2^23); pos < 0 skips the slot;
 * base may be null. */
int zkds_moe_combine(const int64_t* out, const int* pos, const int64_t* w, const int64_t* base,
                     int64_t* y, int64_t tokens, int slots, int64_t cols, void* stream);

/* Gate.forward after the sigmoid (replaces the torch ops of model.py:1140-1211): scores = sigma + bias
 * (bias int32, may be null); with n_groups > 1 the score of a group is the sum of its two largest scores
 * (its largest when bias is null), the topk_groups best groups stay and the others are masked with -(2^42);
 * indices [tokens][topk] = the topk best experts in descending order of score, lower index on ties;
 * raw_weights = sigma[indices]; weights = ((raw * 2^23) // sum raw) * 5 // 2 (floor divisions).
 * sigma [tokens][experts] int64.  Returns ZKDS_ERR_UNSUPPORTED (silently) for experts > 1024 or not a
 * multiple of n_groups, n_groups > 32, topk > 32. */
int zkds_gate_select(const int64_t* sigma, const int32_t* bias, int64_t tokens, int experts, int n_groups,
                     int topk_groups, int topk, int64_t* indices, int64_t* raw_weights, int64_t* weights,
                     void* stream);

/* Replaces the four *_init_* functions.  HOST table of 256 entries.
 * kind: 0 softmax Q19, 1 softmax Q21, 2 silu Q23, 3 silu Q25. */
int zkds_lut(int64_t* host_lut, int kind);

#ifdef __cplusplus
}
#endif
#endif /* ZKDS_INT64_H */
