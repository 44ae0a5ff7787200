// Internal launch interface between the C-ABI layer (capi.cu) and the kernel
// translation units.  Every launcher validates nothing: the C-ABI layer owns the
// argument checks.  All return a ZKDS_* status.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace zkds {

int sm_count();  // SM count of the current device (cached per device)

// Diagnostic switches, read from the environment ONCE (first use) and constant for the life of the
// process; all off by default.  They exist so that one run on one GPU can compare two variants.
struct Switches {
    bool wait_profile;            // ZKDS_WAIT_PROFILE: the persistent kernel reports where its warps waited
    bool trace;                   // ZKDS_TRACE: one line per timed launch
    bool no_persistent;           // ZKDS_NO_PERSISTENT
    bool no_persistent_grouped;   // ZKDS_NO_PERSISTENT_GROUPED
    bool no_merged;               // ZKDS_NO_MERGED
    bool no_split_release;        // ZKDS_NO_SPLIT_RELEASE
    bool no_backoff;              // ZKDS_NO_BACKOFF
    bool no_split_k;              // ZKDS_NO_SPLIT_K: few-tile GEMMs keep one CTA per output tile
    bool split_generic;           // ZKDS_SPLIT_GENERIC
    bool softmax_generic;         // ZKDS_SOFTMAX_GENERIC
    bool rms_staged, rms_nostage; // ZKDS_RMS_STAGED, ZKDS_RMS_NOSTAGE
    int epi_warps;                // ZKDS_EPI_WARPS = 8 | 16 (0: default)
    int tile_nt;                  // ZKDS_TILE_NT = forced tile width (0: default)
    int persistent_max_kb;        // ZKDS_PERSISTENT_MAX_KB (negative: default)
};
const Switches& switches();

// ---- streaming fixed-point kernels (fixedpoint.cu) ---------------------------
int launch_act(const int64_t* X, int64_t* C, const int64_t* lut, int64_t n, int frac, int silu,
               cudaStream_t st);
int launch_softmax(const int64_t* X, int64_t* Wout, int64_t* C, const int64_t* lut, int64_t rows,
                   int64_t T, int frac, cudaStream_t st);
// Q19 softmax over rows (b, s, h) that only looks at columns <= start + s of each row and writes
// only those (causal attention with the masked scores left unwritten)
int launch_softmax_causal(const int64_t* X, int64_t* C, const int64_t* lut, int64_t B, int64_t S, int64_t H,
                          int64_t T, int64_t start, cudaStream_t st);
// Q19 softmax whose probabilities are written as signed 8-bit limb planes (row pitch Kp, limb l at
// planes + l * plane_stride); valid_H > 0 restricts row (b, s, h) to columns <= valid_start + s
bool softmax_planes_supported(const int64_t* X, int64_t rows, int64_t T, int64_t Kp);
int launch_softmax_planes(const int64_t* X, const int64_t* lut, int8_t* planes, int L, int64_t rows, int64_t T,
                          int64_t Kp, int64_t plane_stride, unsigned* overflow, unsigned long long* absmax_out,
                          int64_t valid_H, int64_t valid_S, int64_t valid_start, cudaStream_t st);
int launch_rope(const int64_t* A, const int64_t* Tb, int64_t* C, int64_t batch, int64_t S,
                int64_t H, int64_t pairs, int shift, cudaStream_t st);
int launch_rmsnorm(const int64_t* A, const void* W, int w_bits, const int64_t* rms_in,
                   int64_t* rms_out, int64_t* C, int64_t M, int64_t N, int64_t eps, int64_t dim,
                   int fused, cudaStream_t st);

int launch_glu(const int64_t* r1, const int64_t* r2, int64_t ld, int64_t* h, int64_t* s1_out,
               const int64_t* lut, int64_t rows, int64_t n, cudaStream_t st);
// (silu_q23(r1) * r2) >> 23 written as limb planes (see launch_softmax_planes for the layout)
bool glu_planes_supported(const int64_t* r1, const int64_t* r2, int64_t ld, int64_t n);
int launch_glu_planes(const int64_t* r1, const int64_t* r2, int64_t ld, const int64_t* lut, int8_t* planes, int L,
                      int64_t rows, int64_t n, int64_t Kp, int64_t plane_stride, unsigned* overflow,
                      unsigned long long* absmax_out, cudaStream_t st);
int launch_gather_rows(const int64_t* src, const int* index, int64_t* dst, int64_t rows, int64_t cols,
                       cudaStream_t st);
// Gate.forward after the sigmoid (model.py:1140-1211): bias, grouped top-k selection, gathered and
// normalised weights; one warp per token.  ZKDS_ERR_UNSUPPORTED for shapes it does not take.
int launch_gate_select(const int64_t* sig, const int32_t* bias, int64_t T, int E, int n_groups, int topk_groups,
                       int topk, int64_t* indices, int64_t* raw, int64_t* w, cudaStream_t st);
int launch_moe_combine(const int64_t* out, const int* pos, const int64_t* w, const int64_t* base,
                       int64_t* y, int64_t tokens, int slots, int64_t cols, cudaStream_t st);
// expert parallelism over peer memory (see include/zkds_int64.h)
constexpr int kMaxRowParts = 16;
int launch_moe_combine_peer(const int64_t* out, const int* pos, const int64_t* w, int64_t tokens, int slots,
                            int64_t cols, int64_t tokens_per_part, int64_t* const* slot_bases, int n_parts,
                            int my_part, cudaStream_t st);
int launch_moe_sum_slots(const int64_t* base, const int64_t* slot_rows, const int64_t* indices, int64_t tokens,
                         int slots, int64_t cols, int n_parts, int experts_per_part, int64_t* y, cudaStream_t st);
int launch_peer_barrier(unsigned long long* const* flag_bases, int n_parts, int my_part, unsigned long long epoch,
                        unsigned* status, cudaStream_t st);

// ---- contractions ---------------------------------------------------------------
// One batched contraction  C[z][m][n] = (addend + sum_k A(z,m,k) * B(z,n,k)) >> shift
// with the sum held in 128 bits.  A is int64 with unit k-stride; B is int32 or int64
// with arbitrary n- and k-strides (so the MLA einsums map onto it without copies).
// a_div / b_div are C truncating divisors applied to each element before the product.
struct Contraction {
    const int64_t* A;
    const void* B;
    int b_bits;  // 32 or 64
    int64_t* C;
    int64_t* R;  // remainder output, may be null
    int64_t batches, M, N, K;
    int64_t a_sz, a_sm;
    int64_t b_sz, b_sn, b_sk;
    int64_t c_sz, c_sm;
    int64_t a_div, b_div;
    int64_t addend;
    int shift;     // 0..127
    int r_legacy;  // remainder flavour, see gemm_remainder()
    // ---- optional extensions (all zero = plain contraction) ----
    // epilogue: v = quotient; v += addin[z][m][n] (same layout as C); v = floor(v * ep_mul / ep_div)
    // when ep_div != 0 (wrapping multiply); rows are (s, h) pairs with causal_H heads per s:
    // v += mask_value where n > causal_start + m / causal_H
    const int64_t* addin;
    int64_t ep_mul, ep_div;
    int64_t causal_H, causal_start, mask_value;
    // a_limbs passed to the limb kernel is an upper bound; the count needed is derived on the
    // device from the range measured while splitting A (no host synchronisation)
    int dynamic_a;
    // grouped mode (limb kernel only): batches == 1, A is a flat [M, K] matrix, tile_group[i]
    // gives the B batch of the i-th 128-row tile (negative: tile skipped)
    const int* tile_group;
    // grouped mode, 0 / 32 / 64: the caller promises that only the first 32 (64) rows of every 128-row tile
    // hold data (no group has more rows than that); the kernel then loads only those rows of A and the other
    // rows of a tile come out as zero rows would
    int group_rows;
    // limb kernel only: row m of A is source row a_row_index[m] (negative: a row of zeros), so a row
    // gather needs no pass of its own
    const int* a_row_index;
    // with a_row_index: the source rows lie in a_n_parts (<= kMaxRowParts) pieces of a_rows_per_part rows each
    // (piece i at a_parts[i], which may be another GPU's memory mapped into this process): row g is row
    // g % a_rows_per_part of piece g / a_rows_per_part; an index beyond the pieces reads as a row of zeros.
    // 0 pieces: all rows at A.
    const void* a_parts[16];
    int a_n_parts;
    int64_t a_rows_per_part;
    // grouped mode: shift per group, [2g] for columns < n_split, [2g+1] from n_split on (values in
    // 0..127, n_split a multiple of 8); null = the uniform shift
    const int* group_shift;
    int64_t n_split;
    // causal skipping, rows = (s, h) pairs with skip_H heads per sequence position:
    //  skip_tiles: output tiles entirely beyond column skip_start + s are neither computed nor written;
    //  skip_k: A holds data only in columns <= skip_start + s (zero beyond, not read), and K blocks
    //          past that are not accumulated
    int skip_tiles, skip_k;
    int64_t skip_H, skip_start;
    // A holds Q19 softmax inputs (rows of K scores, contiguous): the limb planes are produced from
    // softmax(A) by the softmax kernel itself and the probabilities never reach memory as int64
    // (limb kernel only; softmax_S = sequence positions per batch when skip_k is set)
    const int64_t* softmax_lut;
    int64_t softmax_S;
    // A is r1 of a gated MLP (rows of K words, row stride a_sm): the limb planes are produced from
    // (silu_q23(A) * glu_r2) >> 23, glu_r2 with the same row stride, and the gated product never reaches
    // memory as int64 (limb kernel only, batches == 1)
    const int64_t* glu_r2;
    const int64_t* glu_lut;
};

// CUDA-core path: exact for every input, any shape (gemm_exact.cu)
int launch_contraction_exact(const Contraction& p, cudaStream_t st);

// Tensor-core path (limb_gemm.cu).  La/Lb: signed 8-bit limb counts that cover the
// operands after division; returns ZKDS_ERR_UNSUPPORTED when the shape or the limb
// counts fall outside what the kernel handles (caller then uses the exact path).
// pre_b: limb planes of B prepared ahead of time (static weights), or null to split B now.
struct Planes {
    int8_t* data;     // [L][nb][rows][pitch] int8
    int L;
    int64_t nb, rows, K;
    int64_t pitch;    // bytes between rows; 0 = K rounded up to 16 (resident cache planes are wider: their
                      // capacity, of which the first K columns are in use)
};
int launch_contraction_limb(const Contraction& p, int La, int Lb, const Planes* pre_b, cudaStream_t st);

// MLA attention scores in one tensor-core pass (limb_gemm.cu): A1/B1 contract over K1 with
// (addend1, shift1), A2/B2 over K2 with (addend2, shift2); the two quotients are added and the
// element-wise tail (ep_mul / ep_div, causal mask) applied.  All operands dense int64:
// A1 [b][M][K1], A2 [b][M][K2], B1 [b][N][K1], B2 [b][N][K2], out [b][M][N].
struct FusedScores {
    const int64_t *A1, *A2, *B1, *B2;
    int64_t* out;
    int64_t batches, M, N, K1, K2;
    int64_t addend1, addend2;
    int shift1, shift2;
    int64_t ep_mul, ep_div, causal_H, causal_start, mask_value;
    int dynamic_a;
    int skip_tiles;   // with causal_H: tiles whose every column is masked are neither computed nor written
    // B1 | B2 already split (resident cache planes): [Lb][batches][b_batch_rows][K1 + round16(K2)] int8, of
    // which rows [0, N) of every batch are in use; B1 and B2 are then ignored
    const int8_t* b_planes;
    int64_t b_batch_rows;
};
// new cache rows as limb planes in both layouts the attention contractions read (see zkds_cache_planes_append)
int launch_cache_planes_append(const int64_t* kv_new, const int64_t* pe_new, int8_t* score_planes,
                               int8_t* value_planes, int64_t B, int64_t S, int64_t C1, int64_t C2,
                               int64_t start_pos, int64_t cap, int L, cudaStream_t st);
int launch_scores_fused(const FusedScores& f, int La, int Lb, cudaStream_t st);

// planes[l][z][r][Kp] <- limb l of X[z*sz + r*sr + k*sk] / div
int planes_split(const void* X, int bits, int64_t nb, int64_t rows, int64_t K, int64_t sz, int64_t sr,
                 int64_t sk, int64_t div, int L, int8_t* dst, cudaStream_t st);
// smallest count of balanced signed 8-bit limbs (digits in [-128,127]) covering |v| <= maxabs
int limbs_needed(uint64_t maxabs);

// GEMM on the tensor-core kernel with every byte of scratch in a fixed device array of the
// module (no allocation of any kind); p.b_sz must be 0 (B shared by the batches)
int launch_gemm_noalloc(const Contraction& p, int La, int Lb, cudaStream_t st);
size_t gemm_noalloc_capacity();
size_t gemm_noalloc_bytes(int64_t Bdim, int64_t M, int64_t K, int64_t N, int a_limbs, int b_limbs);

// CUDA-event timing of the tensor-core kernel alone (events recorded on the launching stream)
void limb_timing_enable(int on);
float limb_last_kernel_ms();
// on == 2 also accumulates, per launch, the kernel's duration and limb-pairs x 2MNK (waits for
// every launch: a profiling pass, not a timed one)
void limb_timing_totals(double* ms, double* int8_ops, long long* launches);
// i-th launch since accumulation started: {batches, M, N, K, a limbs used, b limbs, ms, grouped}
int limb_timing_record(long long i, double* out8);

// ZKDS_ERR_DEVICE when a tensor-core kernel reported a wait that ran out, ZKDS_ERR_RANGE
// when an operand did not fit the limb count it was split into, else ZKDS_OK.  The flags
// live in host-mapped memory: reading them needs no synchronisation, but they describe only
// kernels that have finished.  clear != 0 resets them.
int limb_device_status(int clear);

// max |x / div| over a strided int64 / int32 operand, written to *out_dev (uint64)
int launch_absmax(const void* X, int bits, int64_t batches, int64_t rows, int64_t cols,
                  int64_t sz, int64_t sr, int64_t sc, int64_t div, uint64_t* out_dev,
                  cudaStream_t st);

// dead-code converters kept for ABI completeness (converters.cu)
int launch_bf16_to_int32(const uint16_t* in, int32_t* out, int rows, int cols, int rescale,
                         int wkv_b_variant, cudaStream_t st);
int launch_f32_to_int64(const uint32_t* in, int64_t* out, int rows, int cols, int rescale,
                        cudaStream_t st);

// scratch memory owned by the library, one arena per device, grown on demand and
// reused by the next call (capi.cu).  Returns null when the allocation fails.
void* workspace(size_t bytes, int slot);
// same; *fresh_bytes is the size of the block when this call had to allocate it (its contents are then
// undefined), 0 when the block of an earlier call is returned with whatever that call left in it
void* workspace_fresh(size_t bytes, int slot, size_t* fresh_bytes);

}  // namespace zkds
