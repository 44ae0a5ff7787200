// Fixed-point streaming kernels: SiLU / sigmoid (Q23, Q25), softmax (Q19, Q21),
// RoPE complex multiply and RMSNorm.  All are HBM-bound integer work: 128-bit
// vector loads/stores, warp-shuffle reductions, the row staged in shared memory
// where a row is read more than once.  Arithmetic follows the reference kernels
// bit for bit (inference/int64_gemm.cu:223-385, 605-768, 775-1017) with the slow
// integer divisions replaced by a double-precision estimate plus an exact
// integer correction.
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace zkds {

static constexpr int kThreads = 256;

// ------------------------------------------------------------------------------
// SiLU / sigmoid
// ------------------------------------------------------------------------------

// floor-toward-zero NUM / den for NUM = 2^(2*FRAC); den is any int64.
template <int FRAC>
__device__ __forceinline__ int64_t div_from_pow2(int64_t den)
{
    constexpr int64_t NUM = (int64_t)1 << (2 * FRAC);
    if (den > 0 && den < ((int64_t)1 << 52)) {
        int64_t q = (int64_t)((double)NUM / (double)den);
        int64_t rem = NUM - q * den;
        if (rem < 0) --q;
        else if (rem >= den) ++q;
        return q;
    }
    if (den == 0) return 0;  // unreachable for LUT-generated den; keeps the division defined
    return NUM / den;
}

template <int FRAC, bool SILU>
__device__ __forceinline__ int64_t act_one(int64_t r, const int64_t* lut)
{
    constexpr int64_t LIM = (int64_t)64 << FRAC;
    constexpr int64_t LOG2E = (FRAC == 23) ? 12102203ll : 48408813ll;
    if (r >= LIM) return r;  // the reference returns r here for sigmoid as well
    if (r <= -LIM) return 0;
    if (FRAC == 23) {
        // |r| < 2^29: everything up to the division runs in 32-bit registers
        const int32_t r32 = (int32_t)r;
        const int32_t y = (int32_t)(((int64_t)(-r32) * (int64_t)(int32_t)LOG2E) >> 23);   // |y| < 2^30
        const int32_t k = y >> 23;
        const uint32_t t = (uint32_t)lut[(y & 0x7FFFFF) >> 15];                       // < 2^24
        if (k < 8) {
            // denominator 2^23 + 2^y fits 32 bits: one double-precision estimate, exact correction
            const uint32_t u = k < 0 ? (k > -32 ? (t >> (-k)) : 0u) : (t << k);
            const uint32_t den = 8388608u + u;
            uint32_t q = (uint32_t)__double2uint_rz(70368744177664.0 / (double)den);
            const int64_t rem = (int64_t)70368744177664ll - (int64_t)((uint64_t)q * den);
            if (rem < 0) --q;
            else if (rem >= (int64_t)den) ++q;
            if (!SILU) return (int64_t)q;
            return ((int64_t)r32 * (int64_t)q) >> 23;
        }
    }
    // |r| < 2^(FRAC+6) and LOG2E < 2^(FRAC+1): the product fits in 64 bits
    int64_t y = (FRAC == 23) ? ((-r) * LOG2E) >> FRAC : -((r * LOG2E) >> FRAC);
    int64_t k = y >> FRAC;
    int64_t f = y & (((int64_t)1 << FRAC) - 1);
    int64_t t = lut[f >> (FRAC - 8)];
    int64_t u = 0;
    if (k > -63) {
        if (k < 0) u = t >> (int)(-k);
        else u = (k >= 64) ? 0 : (int64_t)((uint64_t)t << (int)k);
    }
    int64_t q = div_from_pow2<FRAC>((int64_t)(((uint64_t)1 << FRAC) + (uint64_t)u));
    if (!SILU) return q;
    return (int64_t)((uint64_t)r * (uint64_t)q) >> FRAC;
}

template <int FRAC, bool SILU, bool VEC>
__global__ void __launch_bounds__(kThreads)
act_kernel(const int64_t* X, int64_t* C, const int64_t* __restrict__ lut_g, int64_t n)
{
    __shared__ int64_t lut[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = lut_g[i];
    __syncthreads();
    constexpr int UNROLL = 4;
    if (VEC) {
        const int64_t nv = n >> 1;
        const longlong2* Xv = reinterpret_cast<const longlong2*>(X);
        longlong2* Cv = reinterpret_cast<longlong2*>(C);
        int64_t stride = (int64_t)gridDim.x * kThreads * UNROLL;
        for (int64_t base = (int64_t)blockIdx.x * kThreads * UNROLL; base < nv; base += stride) {
            longlong2 v[UNROLL];
#pragma unroll
            for (int j = 0; j < UNROLL; ++j) {
                int64_t i = base + j * kThreads + threadIdx.x;
                if (i < nv) v[j] = Xv[i];
            }
#pragma unroll
            for (int j = 0; j < UNROLL; ++j) {
                int64_t i = base + j * kThreads + threadIdx.x;
                if (i < nv) {
                    longlong2 o;
                    o.x = act_one<FRAC, SILU>(v[j].x, lut);
                    o.y = act_one<FRAC, SILU>(v[j].y, lut);
                    Cv[i] = o;
                }
            }
        }
        if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0)
            C[n - 1] = act_one<FRAC, SILU>(X[n - 1], lut);
    } else {
        int64_t stride = (int64_t)gridDim.x * kThreads;
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
            C[i] = act_one<FRAC, SILU>(X[i], lut);
    }
}

static int grid_for(int64_t work_items, int per_block, int sm_count, int waves)
{
    int64_t blocks = (work_items + per_block - 1) / per_block;
    int64_t cap = (int64_t)sm_count * waves;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

int launch_act(const int64_t* X, int64_t* C, const int64_t* lut, int64_t n, int frac, int silu,
               cudaStream_t st)
{
    if (n == 0) return ZKDS_OK;
    bool vec = (((uintptr_t)X | (uintptr_t)C) & 15) == 0;
    int sms = sm_count();
    int grid = grid_for(vec ? n / 2 : n, kThreads * (vec ? 4 : 1), sms, 8);
#define ZKDS_ACT(F, S)                                                           \
    do {                                                                         \
        if (vec) act_kernel<F, S, true><<<grid, kThreads, 0, st>>>(X, C, lut, n); \
        else act_kernel<F, S, false><<<grid, kThreads, 0, st>>>(X, C, lut, n);    \
    } while (0)
    if (frac == 23 && silu) ZKDS_ACT(23, true);
    else if (frac == 23) ZKDS_ACT(23, false);
    else if (frac == 25 && silu) ZKDS_ACT(25, true);
    else if (frac == 25) ZKDS_ACT(25, false);
    else return ZKDS_ERR_ARG;
#undef ZKDS_ACT
    return check_launch();
}

// ------------------------------------------------------------------------------
// softmax: one CTA per row, the row staged in shared memory
// ------------------------------------------------------------------------------

__device__ __forceinline__ int64_t block_max_i64(int64_t v, int64_t* red)
{
    v = warp_max_i64(v);
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) red[w] = v;
    __syncthreads();
    int nw = blockDim.x >> 5;
    int64_t r = (lane < nw) ? red[lane] : INT64_MIN;
    r = warp_max_i64(r);
    __syncthreads();
    return r;
}

__device__ __forceinline__ int64_t block_sum_i64(int64_t v, int64_t* red)
{
    v = warp_sum_i64(v);
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) red[w] = v;
    __syncthreads();
    int nw = blockDim.x >> 5;
    int64_t r = (lane < nw) ? red[lane] : 0;
    r = warp_sum_i64(r);
    __syncthreads();
    return r;
}

// unnormalised weight of one score, given the row maximum
template <int FRAC>
__device__ __forceinline__ int64_t softmax_weight(int64_t x, int64_t mx, const int64_t* lut)
{
    if (FRAC == 19) {
        uint64_t d = (uint64_t)mx - (uint64_t)x;
        if (d > (uint64_t)(64 << 19)) return 0;
        int64_t y = (int64_t)((d * 756388ull) >> 19);  // d <= 2^25: no overflow
        int64_t k = y >> 19, f = y & 0x7FFFF;
        int64_t t = lut[f >> 11];
        return (k >= 64) ? 0 : (t >> (int)k);
    } else {
        int64_t d = (int64_t)((uint64_t)x - (uint64_t)mx);
        if (d < -(int64_t)(64 << 21)) return 0;
        int64_t y = (int64_t)((uint64_t)d * 3025551ull + (uint64_t)(1 << 20)) >> 21;
        int64_t ny = (int64_t)(0 - (uint64_t)y);
        int64_t k = ny >> 21, f = ny & 0x1FFFFF;
        int64_t t = lut[f >> 13];
        return (k >= 64) ? 0 : (t >> (int)k);
    }
}

// exact num / den for 0 <= num < 2^52, 0 < den < 2^52 with a per-row reciprocal
__device__ __forceinline__ int64_t div_by_row(int64_t num, int64_t den, double inv)
{
    // the estimate is within one of the quotient: one exact correction either way
    int64_t q = (int64_t)((double)num * inv);
    int64_t rem = num - q * den;
    if (rem < 0) --q;
    else if (rem >= den) ++q;
    return q;
}

template <int FRAC>
__device__ __forceinline__ int64_t softmax_norm(int64_t w, int64_t sumW, double inv, bool fast)
{
    if (sumW == 0) return 0;
    int64_t num = (int64_t)((uint64_t)w << FRAC);
    if (FRAC == 21) num += sumW / 2;
    if (fast) return div_by_row(num, sumW, inv);
    return num / sumW;
}

// STAGE: row held in dynamic shared memory; otherwise C is used as scratch for the
// weights exactly as the reference uses its input buffer.
template <int FRAC, bool STAGE, bool VEC>
__global__ void __launch_bounds__(kThreads)
softmax_kernel(const int64_t* X, int64_t* Wout, int64_t* C, const int64_t* __restrict__ lut_g,
               int64_t T)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int64_t lut[256];
    __shared__ int64_t red[32];
    int64_t* row = reinterpret_cast<int64_t*>(smem_raw);
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = lut_g[i];
    const int64_t off = (int64_t)blockIdx.x * T;
    const int64_t* x = X + off;
    int64_t* c = C + off;
    int64_t* wo = Wout ? Wout + off : nullptr;

    int64_t mx = INT64_MIN;
    if (VEC) {
        const longlong2* xv = reinterpret_cast<const longlong2*>(x);
        longlong2* rv = reinterpret_cast<longlong2*>(row);
        for (int64_t i = threadIdx.x; i < (T >> 1); i += kThreads) {
            longlong2 v = xv[i];
            if (STAGE) rv[i] = v;
            mx = v.x > mx ? v.x : mx;
            mx = v.y > mx ? v.y : mx;
        }
    } else {
        for (int64_t i = threadIdx.x; i < T; i += kThreads) {
            int64_t v = x[i];
            if (STAGE) row[i] = v;
            mx = v > mx ? v : mx;
        }
    }
    mx = block_max_i64(mx, red);  // also orders the LUT and row stores

    int64_t sum = 0;
    if (VEC) {
        const longlong2* src = STAGE ? reinterpret_cast<const longlong2*>(row)
                                     : reinterpret_cast<const longlong2*>(x);
        longlong2* dst = STAGE ? reinterpret_cast<longlong2*>(row) : reinterpret_cast<longlong2*>(c);
        for (int64_t i = threadIdx.x; i < (T >> 1); i += kThreads) {
            longlong2 v = src[i];
            v.x = softmax_weight<FRAC>(v.x, mx, lut);
            v.y = softmax_weight<FRAC>(v.y, mx, lut);
            dst[i] = v;
            sum += v.x + v.y;
        }
    } else {
        const int64_t* src = STAGE ? row : x;
        int64_t* dst = STAGE ? row : c;
        for (int64_t i = threadIdx.x; i < T; i += kThreads) {
            int64_t w = softmax_weight<FRAC>(src[i], mx, lut);
            dst[i] = w;
            sum += w;
        }
    }
    const int64_t sumW = block_sum_i64(sum, red);
    // every weight is < 2^(FRAC+1) so num < 2^(2*FRAC+2); the double path needs sumW < 2^52
    const bool fast = sumW > 0 && sumW < ((int64_t)1 << 51);
    const double inv = fast ? 1.0 / (double)sumW : 0.0;

    if (VEC) {
        const longlong2* src = STAGE ? reinterpret_cast<const longlong2*>(row)
                                     : reinterpret_cast<const longlong2*>(c);
        longlong2* cv = reinterpret_cast<longlong2*>(c);
        longlong2* wv = reinterpret_cast<longlong2*>(wo);
        for (int64_t i = threadIdx.x; i < (T >> 1); i += kThreads) {
            longlong2 w = src[i];
            if (wo) wv[i] = w;
            longlong2 o;
            o.x = softmax_norm<FRAC>(w.x, sumW, inv, fast);
            o.y = softmax_norm<FRAC>(w.y, sumW, inv, fast);
            cv[i] = o;
        }
    } else {
        const int64_t* src = STAGE ? row : c;
        for (int64_t i = threadIdx.x; i < T; i += kThreads) {
            int64_t w = src[i];
            if (wo) wo[i] = w;
            c[i] = softmax_norm<FRAC>(w, sumW, inv, fast);
        }
    }
}

// Q19 softmax with the row in registers and 32-bit arithmetic wherever the values allow it:
// after the clip the difference d fits 26 bits, weights fit 20 bits, and the final division
// (w << 19) / sumW uses one 64-bit reciprocal per row (floor((2^64 - 1) / sumW), an estimate that
// is at most one below the quotient) plus an exact correction.  E = 16-byte pairs per thread.
// FULL: every row owns all T columns (no causal bound), so no element needs a validity test.
template <int E, bool FULL>
__global__ void __launch_bounds__(kThreads, (E <= 4 ? 6 : 1))
softmax_q19_reg_kernel(const int64_t* X, int64_t* Wout, int64_t* C, const int64_t* __restrict__ lut_g,
                       int T, int valid_H, int valid_S, int valid_start)
{
    __shared__ uint32_t lut[256];
    __shared__ int64_t red[32];
    __shared__ uint64_t s_magic;
    for (int i = threadIdx.x; i < 256; i += kThreads) lut[i] = (uint32_t)lut_g[i];
    const int64_t off = (int64_t)blockIdx.x * T;
    const longlong2* xv = reinterpret_cast<const longlong2*>(X + off);
    longlong2* cv = reinterpret_cast<longlong2*>(C + off);
    longlong2* wv = Wout ? reinterpret_cast<longlong2*>(Wout + off) : nullptr;
    // valid_H > 0: row (b, s, h) only counts columns <= valid_start + s; the rest is neither read
    // nor written
    int valid = T;
    if (!FULL && valid_H) {
        const int sidx = (int)((blockIdx.x / (unsigned)valid_H) % (unsigned)valid_S);
        valid = valid_start + sidx + 1 < T ? valid_start + sidx + 1 : T;
    }
    const int half = (valid + 1) >> 1;

    longlong2 v[E];
    int64_t mx = INT64_MIN;
#pragma unroll
    for (int j = 0; j < E; ++j) {
        const int i = threadIdx.x + j * kThreads;
        if (i < half) {
            v[j] = xv[i];
            if (!FULL && 2 * i + 1 >= valid) v[j].y = INT64_MIN;   // odd boundary: the second element is masked
            mx = v[j].x > mx ? v[j].x : mx;
            mx = v[j].y > mx ? v[j].y : mx;
        }
    }
    mx = block_max_i64(mx, red);

    uint32_t w[2 * E];
    uint64_t sum = 0;
#pragma unroll
    for (int j = 0; j < E; ++j) {
        const int i = threadIdx.x + j * kThreads;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t wi = 0;
            if (i < half && (FULL || 2 * i + h < valid)) {
                const uint64_t d = (uint64_t)mx - (uint64_t)(h ? v[j].y : v[j].x);
                if (d <= (uint64_t)(64 << 19)) {
                    const uint32_t y = (uint32_t)(((uint64_t)(uint32_t)d * 756388u) >> 19);
                    const uint32_t k = y >> 19;
                    const uint32_t t = lut[(y & 0x7FFFFu) >> 11];
                    wi = k >= 32u ? 0u : (t >> k);
                }
            }
            w[2 * j + h] = wi;
            sum += wi;
        }
    }
    const uint64_t sumW = (uint64_t)block_sum_i64((int64_t)sum, red);
    if (threadIdx.x == 0) s_magic = sumW ? 0xFFFFFFFFFFFFFFFFull / sumW : 0;
    __syncthreads();
    const uint64_t magic = s_magic;
    const uint32_t m_lo = (uint32_t)magic, m_hi = (uint32_t)(magic >> 32);
    const bool small = sumW < (1ull << 32);
    const uint32_t s32 = (uint32_t)sumW;

#pragma unroll
    for (int j = 0; j < E; ++j) {
        const int i = threadIdx.x + j * kThreads;
        if (i >= half) continue;
        longlong2 o;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t wi = w[2 * j + h];
            const uint64_t num = (uint64_t)wi << 19;
            // floor(num * magic / 2^64) = (wi * m_hi + ((wi * m_lo) >> 32)) >> 13
            uint64_t q = ((uint64_t)wi * m_hi + (((uint64_t)wi * m_lo) >> 32)) >> 13;
            if (small) {
                // magic = floor((2^64 - 1) / sumW) makes q the quotient or one below it (num < 2^40, so the
                // estimate's error num * (1 + (2^64 - 1) mod sumW) / (sumW * 2^64) stays below 1): one correction
                const uint64_t rem = num - q * s32;    // q < 2^20, s32 < 2^32
                q += rem >= sumW ? 1 : 0;
            } else if (sumW) {
                q = num / sumW;
            }
            if (h) o.y = (int64_t)q; else o.x = (int64_t)q;
        }
        cv[i] = o;
        if (wv) wv[i] = make_longlong2((int64_t)w[2 * j], (int64_t)w[2 * j + 1]);
    }
}

static int launch_softmax_q19_reg(const int64_t* X, int64_t* Wout, int64_t* C, const int64_t* lut,
                                  int64_t rows, int64_t T, cudaStream_t st, int vH = 0, int vS = 1,
                                  int vstart = 0)
{
    const int pairs = (int)((T / 2 + kThreads - 1) / kThreads);
    const unsigned g = (unsigned)rows;
    const bool full = vH == 0 && (T & 1) == 0;
#define ZKDS_SR(E)                                                                                          \
    do {                                                                                                    \
        if (full) softmax_q19_reg_kernel<E, true><<<g, kThreads, 0, st>>>(X, Wout, C, lut, (int)T, vH, vS, vstart);  \
        else softmax_q19_reg_kernel<E, false><<<g, kThreads, 0, st>>>(X, Wout, C, lut, (int)T, vH, vS, vstart);     \
    } while (0)
    if (pairs <= 1) ZKDS_SR(1);
    else if (pairs <= 2) ZKDS_SR(2);
    else if (pairs <= 4) ZKDS_SR(4);
    else if (pairs <= 8) ZKDS_SR(8);
    else ZKDS_SR(16);
#undef ZKDS_SR
    return check_launch();
}

// The same Q19 softmax, but the probabilities leave the kernel as signed 8-bit limb planes (the A
// operand of the tensor-core contraction that consumes them) instead of int64 words: plane l of row
// r lives at planes + l * plane_stride + r * Kp.  Balanced radix-256 digits as in the limb split;
// columns from `valid` (or T) up to Kp are written as zero.  E = groups of four columns per thread.
// MINB: CTAs per SM the kernel is compiled for.  The 4096-column case (E = 4, three limbs) asks for eight: 32
// registers and 68 bytes of spills instead of 48 registers and five CTAs, 6.95 against 7.48 ms on the 17 GB
// score tensor of the 4096-token prefill (six CTAs: 7.13 ms).
template <int E, int LL, int MINB, bool FULL>      // LL: limb count known at compile time, 0 = use L; FULL as above
__global__ void __launch_bounds__(kThreads, MINB)
softmax_q19_planes_kernel(const int64_t* X, const int64_t* __restrict__ lut_g, int8_t* __restrict__ planes,
                          int L, int T, int64_t Kp, int64_t plane_stride, unsigned* overflow,
                          unsigned long long* absmax_out, int valid_H, int valid_S, int valid_start)
{
    __shared__ uint32_t lut[256];
    __shared__ int64_t red[32];
    __shared__ uint64_t s_magic;
    for (int i = threadIdx.x; i < 256; i += kThreads) lut[i] = (uint32_t)lut_g[i];
    const longlong2* xv = reinterpret_cast<const longlong2*>(X + (int64_t)blockIdx.x * T);
    int8_t* drow = planes + (int64_t)blockIdx.x * Kp;
    int valid = T;
    if (!FULL && valid_H) {
        const int sidx = (int)((blockIdx.x / (unsigned)valid_H) % (unsigned)valid_S);
        valid = valid_start + sidx + 1 < T ? valid_start + sidx + 1 : T;
    }
    const int quads_valid = (valid + 3) >> 2;
    const int quads_all = (int)(Kp >> 2);

    int64_t v[4 * E];
    int64_t mx = INT64_MIN;
#pragma unroll
    for (int j = 0; j < E; ++j) {
        const int q = threadIdx.x + j * kThreads;
        if (q < quads_valid) {
            const longlong2 a = xv[2 * q], b = xv[2 * q + 1];
            v[4 * j] = a.x; v[4 * j + 1] = a.y; v[4 * j + 2] = b.x; v[4 * j + 3] = b.y;
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                if (!FULL && 4 * q + h >= valid) v[4 * j + h] = INT64_MIN;
                mx = v[4 * j + h] > mx ? v[4 * j + h] : mx;
            }
        }
    }
    mx = block_max_i64(mx, red);

    uint32_t w[4 * E];
    uint32_t sum32 = 0;              // at most 32 weights of at most 2^19 + 1 each
#pragma unroll
    for (int j = 0; j < E; ++j) {
        const int q = threadIdx.x + j * kThreads;
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            uint32_t wi = 0;
            if (q < quads_valid && (FULL || 4 * q + h < valid)) {
                const uint64_t d = (uint64_t)mx - (uint64_t)v[4 * j + h];
                if (d <= (uint64_t)(64 << 19)) {
                    const uint32_t y = (uint32_t)(((uint64_t)(uint32_t)d * 756388u) >> 19);
                    const uint32_t k = y >> 19;
                    const uint32_t t = lut[(y & 0x7FFFFu) >> 11];
                    wi = k >= 32u ? 0u : (t >> k);
                }
            }
            w[4 * j + h] = wi;
            sum32 += wi;
        }
    }
    const uint64_t sumW = (uint64_t)block_sum_i64((int64_t)sum32, red);
    if (threadIdx.x == 0) s_magic = sumW ? 0xFFFFFFFFFFFFFFFFull / sumW : 0;
    __syncthreads();
    const uint64_t magic = s_magic;
    const uint32_t m_lo = (uint32_t)magic, m_hi = (uint32_t)(magic >> 32);
    const bool small = sumW < (1ull << 32);
    const uint32_t s32 = (uint32_t)sumW;

    uint32_t seen = 0;
    bool ovf = false;
#pragma unroll
    for (int j = 0; j < E; ++j) {
        const int q = threadIdx.x + j * kThreads;
        if (q >= quads_all) continue;
        uint32_t u[4] = {0, 0, 0, 0};
        if (q < quads_valid) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const uint32_t wi = w[4 * j + h];
                const uint64_t num = (uint64_t)wi << 19;
                uint64_t qt = ((uint64_t)wi * m_hi + (((uint64_t)wi * m_lo) >> 32)) >> 13;
                if (small) {
                    const uint64_t rem = num - qt * s32;      // qt is the quotient or one below it (see above)
                    qt += rem >= sumW ? 1 : 0;
                } else if (sumW) {
                    qt = num / sumW;
                }
                u[h] = (uint32_t)qt;                 // 0 .. 2^19
                seen = u[h] > seen ? u[h] : seen;
            }
        }
        if (LL == 3) {
            // balanced digits of a value below 2^23 - 2^15: the bytes of u + 0x808080, each with its
            // top bit flipped (digit + 128 is what the biased sum holds at every position)
            uint32_t t[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                t[h] = u[h] + 0x00808080u;
                ovf |= (t[h] >> 24) != 0;
            }
#pragma unroll
            for (int l = 0; l < 3; ++l) {
                const uint32_t sel = 0x0040u + 0x0011u * (uint32_t)l;     // byte l of both operands
                const uint32_t lo = __byte_perm(t[0], t[1], sel), hi = __byte_perm(t[2], t[3], sel);
                *reinterpret_cast<uint32_t*>(drow + 4 * q + l * plane_stride) =
                    __byte_perm(lo, hi, 0x5410u) ^ 0x80808080u;
            }
        } else {
            constexpr int LMAX = LL ? LL : 9;
            uint32_t pl[LMAX];
#pragma unroll
            for (int l = 0; l < LMAX; ++l) pl[l] = 0;
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                int32_t x = (int32_t)u[h];
#pragma unroll
                for (int l = 0; l < LMAX; ++l) {
                    if (LL || l < L) {
                        pl[l] |= (uint32_t)(x & 0xFF) << (h * 8);
                        x = (x >> 8) + ((x >> 7) & 1);
                    }
                }
                ovf |= (x != 0);
            }
#pragma unroll
            for (int l = 0; l < LMAX; ++l)
                if (LL || l < L) *reinterpret_cast<uint32_t*>(drow + 4 * q + l * plane_stride) = pl[l];
        }
    }
    if (ovf) *overflow = 1u;
    if (absmax_out) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const uint32_t other = __shfl_xor_sync(0xffffffffu, seen, o);
            seen = other > seen ? other : seen;
        }
        if ((threadIdx.x & 31) == 0 && seen) atomicMax(absmax_out, (unsigned long long)seen);
    }
}

bool softmax_planes_supported(const int64_t* X, int64_t rows, int64_t T, int64_t Kp)
{
    return rows > 0 && rows <= 0x7fffffffll && T >= 4 && (T & 3) == 0 && Kp >= T && (Kp & 3) == 0 &&
           Kp <= 8 * 4 * kThreads && ((uintptr_t)X & 15) == 0;
}

int launch_softmax_planes(const int64_t* X, const int64_t* lut, int8_t* planes, int L, int64_t rows, int64_t T,
                          int64_t Kp, int64_t plane_stride, unsigned* overflow, unsigned long long* absmax_out,
                          int64_t valid_H, int64_t valid_S, int64_t valid_start, cudaStream_t st)
{
    if (!softmax_planes_supported(X, rows, T, Kp) || L < 1 || L > 9 || valid_H > 0x7fffffff ||
        valid_S > 0x7fffffff || valid_start > 0x7fffffff)
        return ZKDS_ERR_UNSUPPORTED;
    const int per = (int)(((Kp >> 2) + kThreads - 1) / kThreads);
    const unsigned g = (unsigned)rows;
    const int vS = valid_S > 0 ? (int)valid_S : 1;
#define ZKDS_SP(E)                                                                                        \
    do {                                                                                                  \
        if (L == 3 && valid_H == 0)                                                                       \
            softmax_q19_planes_kernel<E, 3, (E == 4 ? 6 : 1), true><<<g, kThreads, 0, st>>>(              \
                X, lut, planes, L, (int)T, Kp, plane_stride, overflow, absmax_out, (int)valid_H, vS,      \
                (int)valid_start);                                                                        \
        else if (L == 3)                                                                                  \
            softmax_q19_planes_kernel<E, 3, (E == 4 ? 8 : 1), false><<<g, kThreads, 0, st>>>(             \
                X, lut, planes, L, (int)T, Kp, plane_stride, overflow, absmax_out, (int)valid_H, vS,      \
                (int)valid_start);                                                                        \
        else                                                                                              \
            softmax_q19_planes_kernel<E, 0, 1, false><<<g, kThreads, 0, st>>>(X, lut, planes, L, (int)T, Kp, \
                                                                    plane_stride, overflow, absmax_out,   \
                                                                    (int)valid_H, vS, (int)valid_start);  \
    } while (0)
    if (per <= 1) ZKDS_SP(1);
    else if (per <= 2) ZKDS_SP(2);
    else if (per <= 4) ZKDS_SP(4);
    else ZKDS_SP(8);
#undef ZKDS_SP
    return check_launch();
}

int launch_softmax_causal(const int64_t* X, int64_t* C, const int64_t* lut, int64_t B, int64_t S, int64_t H,
                          int64_t T, int64_t start, cudaStream_t st)
{
    const int64_t rows = B * S * H;
    if (rows == 0 || T == 0) return ZKDS_OK;
    if (rows > 0x7fffffffll || T > 2 * 16 * kThreads || (T & 1) || H <= 0 || H > 0x7fffffff || S > 0x7fffffff ||
        start < 0 || start > 0x7fffffff || ((((uintptr_t)X | (uintptr_t)C) & 15) != 0))
        return ZKDS_ERR_UNSUPPORTED;
    return launch_softmax_q19_reg(X, nullptr, C, lut, rows, T, st, (int)H, (int)S, (int)start);
}

template <int FRAC>
static int launch_softmax_t(const int64_t* X, int64_t* Wout, int64_t* C, const int64_t* lut,
                            int64_t rows, int64_t T, cudaStream_t st)
{
    const size_t row_bytes = (size_t)T * 8;
    const bool stage = row_bytes <= 200 * 1024;
    const bool vec = (T % 2 == 0) && ((((uintptr_t)X | (uintptr_t)C | (uintptr_t)Wout) & 15) == 0);
    size_t smem = stage ? row_bytes : 0;
#define ZKDS_SM(S, V)                                                                        \
    do {                                                                                     \
        auto k = softmax_kernel<FRAC, S, V>;                                                 \
        if (smem > 48 * 1024)                                                                \
            ZKDS_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                           (int)smem));                                      \
        k<<<(unsigned)rows, kThreads, smem, st>>>(X, Wout, C, lut, T);                       \
    } while (0)
    if (stage && vec) ZKDS_SM(true, true);
    else if (stage) ZKDS_SM(true, false);
    else if (vec) ZKDS_SM(false, true);
    else ZKDS_SM(false, false);
#undef ZKDS_SM
    return check_launch();
}

int launch_softmax(const int64_t* X, int64_t* Wout, int64_t* C, const int64_t* lut, int64_t rows,
                   int64_t T, int frac, cudaStream_t st)
{
    if (rows == 0 || T == 0) return ZKDS_OK;
    if (rows > 0x7fffffffll) return ZKDS_ERR_RANGE;
    if (frac == 19) {
        const bool vec = (T % 2 == 0) && ((((uintptr_t)X | (uintptr_t)C | (uintptr_t)Wout) & 15) == 0);
        if (vec && T >= 64 && T <= 2 * 16 * kThreads && !switches().softmax_generic)
            return launch_softmax_q19_reg(X, Wout, C, lut, rows, T, st);
        return launch_softmax_t<19>(X, Wout, C, lut, rows, T, st);
    }
    if (frac == 21) return launch_softmax_t<21>(X, Wout, C, lut, rows, T, st);
    return ZKDS_ERR_ARG;
}

// ------------------------------------------------------------------------------
// RoPE: (a0 + i a1) * (b0 + i b1), every product reduced to bits [shift, shift+64)
// ------------------------------------------------------------------------------

__device__ __forceinline__ int64_t mul_shift(int64_t x, int64_t y, int shift)
{
    return sar128_lo(mul64x64(x, y), shift);
}

// grid.x enumerates (position, chunk); a position is one (batch, seq) row of H*pairs pairs
__global__ void __launch_bounds__(kThreads)
rope_kernel(const longlong2* __restrict__ A, const longlong2* __restrict__ Tb,
            longlong2* __restrict__ C, unsigned chunks, unsigned rowlen, unsigned S,
            unsigned pairs, int shift)
{
    const unsigned pos = blockIdx.x / chunks;
    const unsigned chunk = blockIdx.x - pos * chunks;
    const unsigned s = pos % S;
    const longlong2* a = A + (int64_t)pos * rowlen;
    longlong2* c = C + (int64_t)pos * rowlen;
    const longlong2* t = Tb + (int64_t)s * pairs;
    constexpr int UNROLL = 4;
    const unsigned base = chunk * (kThreads * UNROLL);
    longlong2 av[UNROLL], bv[UNROLL];
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
        unsigned i = base + j * kThreads + threadIdx.x;
        if (i < rowlen) {
            av[j] = a[i];
            bv[j] = t[i % pairs];
        }
    }
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
        unsigned i = base + j * kThreads + threadIdx.x;
        if (i < rowlen) {
            longlong2 o;
            // magnitudes (|v|, or |v| - 1 for v < 0) of the larger factor on each side
            const uint64_t ma = (uint64_t)(av[j].x ^ (av[j].x >> 63)) | (uint64_t)(av[j].y ^ (av[j].y >> 63));
            const uint64_t mb = (uint64_t)(bv[j].x ^ (bv[j].x >> 63)) | (uint64_t)(bv[j].y ^ (bv[j].y >> 63));
            if (shift < 64 && __clzll((long long)ma) + __clzll((long long)mb) >= 68) {
                // every product stays below 2^62: one-word multiplies, the arithmetic shift floors
                o.x = ((av[j].x * bv[j].x) >> shift) - ((av[j].y * bv[j].y) >> shift);
                o.y = ((av[j].x * bv[j].y) >> shift) + ((av[j].y * bv[j].x) >> shift);
            } else {
                o.x = (int64_t)((uint64_t)mul_shift(av[j].x, bv[j].x, shift) -
                                (uint64_t)mul_shift(av[j].y, bv[j].y, shift));
                o.y = (int64_t)((uint64_t)mul_shift(av[j].x, bv[j].y, shift) +
                                (uint64_t)mul_shift(av[j].y, bv[j].x, shift));
            }
            c[i] = o;
        }
    }
}

int launch_rope(const int64_t* A, const int64_t* Tb, int64_t* C, int64_t batch, int64_t S,
                int64_t H, int64_t pairs, int shift, cudaStream_t st)
{
    if (batch == 0 || S == 0 || H == 0 || pairs == 0) return ZKDS_OK;
    if (shift < 0 || shift > 127) return ZKDS_ERR_ARG;
    if ((((uintptr_t)A | (uintptr_t)Tb | (uintptr_t)C) & 15) != 0) return ZKDS_ERR_ARG;
    int64_t rowlen = H * pairs;
    int64_t chunks = (rowlen + kThreads * 4 - 1) / (kThreads * 4);
    int64_t blocks = batch * S * chunks;
    if (rowlen > 0x7fffffffll || blocks > 0x7fffffffll || S > 0x7fffffffll) return ZKDS_ERR_RANGE;
    rope_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(
        reinterpret_cast<const longlong2*>(A), reinterpret_cast<const longlong2*>(Tb),
        reinterpret_cast<longlong2*>(C), (unsigned)chunks, (unsigned)rowlen, (unsigned)S,
        (unsigned)pairs, shift);
    return check_launch();
}

// ------------------------------------------------------------------------------
// RMSNorm
// ------------------------------------------------------------------------------

struct u128w {
    uint64_t lo, hi;
};

__device__ __forceinline__ u128w warp_sum_u128(u128w v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        uint64_t lo = __shfl_xor_sync(0xffffffffu, v.lo, o);
        uint64_t hi = __shfl_xor_sync(0xffffffffu, v.hi, o);
        uint64_t nlo = v.lo + lo;
        v.hi = v.hi + hi + (nlo < lo ? 1ull : 0ull);
        v.lo = nlo;
    }
    return v;
}

// floor(sqrt(v)), v unsigned 128-bit
__device__ uint64_t isqrt_u128(unsigned __int128 v)
{
    if (v == 0) return 0;
    if ((v >> 62) == 0) {
        // fits 62 bits: double-precision estimate (within 2 of the root), exact correction
        const uint64_t x = (uint64_t)v;
        uint64_t r = (uint64_t)__double2ull_rz(sqrt((double)x));
        while (r * r > x) --r;
        while ((r + 1) * (r + 1) <= x) ++r;
        return r;
    }
    unsigned __int128 r = 0, bit;
    uint64_t hi = (uint64_t)(v >> 64);
    int top = hi ? 127 - __clzll((long long)hi) : 63 - __clzll((long long)(uint64_t)v);
    bit = (unsigned __int128)1 << (top & ~1);
    while (bit != 0) {
        if (v >= r + bit) { v -= r + bit; r = (r >> 1) + bit; }
        else r >>= 1;
        bit >>= 2;
    }
    return (uint64_t)r;
}

// the reference's quotient: trunc(P / r), minus one when the remainder is negative
__device__ __noinline__ int64_t div_slow(i128w P, int64_t r)
{
    if (r == 0) return 0;
    __int128 p = ((__int128)P.hi << 64) | (__int128)(unsigned __int128)P.lo;
    __int128 qq = p / (__int128)r, rr = p % (__int128)r;
    if (rr < 0) qq -= 1;
    return (int64_t)qq;
}

__device__ __noinline__ int64_t norm_one_wide(int64_t a, int64_t w, int64_t r, double inv);

// floor(a*w / r): the case of two 32-bit factors inline, everything else out of line
__device__ __forceinline__ int64_t norm_one_fast(int64_t a, int64_t w, int64_t r, double inv)
{
    if (r > 0 && a == (int64_t)(int32_t)a && w == (int64_t)(int32_t)w) {
        const int64_t p = (int64_t)(int32_t)a * (int64_t)(int32_t)w;
        const double qe = (double)p * inv;
        if (fabs(qe) < 562949953421312.0) {
            int64_t q = __double2ll_rd(qe);
            int64_t rem = p - q * r;
            if (rem < 0) { --q; rem += r; }
            else if (rem >= r) { ++q; rem -= r; }
            if (rem >= 0 && rem < r) return q;
        }
    }
    return norm_one_wide(a, w, r, inv);
}

// floor(a*w / r) for r > 0 through a double estimate corrected with the exact remainder
__device__ __forceinline__ int64_t norm_one(int64_t a, int64_t w, int64_t r, double inv)
{
    if (r > 0 && a == (int64_t)(int32_t)a && w == (int64_t)(int32_t)w) {
        // both factors fit 32 bits: the product fits 64 bits and everything stays in one word
        const int64_t p = (int64_t)(int32_t)a * (int64_t)(int32_t)w;
        const double qe = (double)p * inv;          // |p| < 2^62, |q| < 2^62 / r
        if (fabs(qe) < 562949953421312.0) {
            int64_t q = __double2ll_rd(qe);
            int64_t rem = p - q * r;
            if (rem < 0) { --q; rem += r; }
            else if (rem >= r) { ++q; rem -= r; }
            if (rem >= 0 && rem < r) return q;
        }
    }
    i128w P = mul64x64(a, w);
    if (r > 0) {
        // convert the magnitude so that the estimate keeps a 2^-52 relative error
        const bool neg = P.hi < 0;
        i128w U = neg ? sub128(i128w{0, 0}, P) : P;
        double pd = (double)(uint64_t)U.hi * 18446744073709551616.0 + (double)U.lo;
        double qe = neg ? -(pd * inv) : pd * inv;
        if (fabs(qe) < 562949953421312.0) {  // 2^49: estimate is within 1 of the quotient
            int64_t q = __double2ll_rd(qe);
            i128w rem = sub128(P, mul64x64(q, r));
            if (rem.hi < 0) { --q; rem = add128(rem, make_i128(r)); }
            else if (rem.hi > 0 || rem.lo >= (uint64_t)r) { ++q; rem = sub128(rem, make_i128(r)); }
            if (rem.hi == 0 && rem.lo < (uint64_t)r) return q;
        }
    }
    return div_slow(P, r);
}

__device__ __noinline__ int64_t norm_one_wide(int64_t a, int64_t w, int64_t r, double inv)
{
    return norm_one(a, w, r, inv);
}

// a^2 added to a two-word accumulator
__device__ __forceinline__ void add_square(uint64_t& lo, uint64_t& hi, int64_t v)
{
    if (v == (int64_t)(int32_t)v) {
        const uint64_t sq = (uint64_t)((int64_t)(int32_t)v * (int64_t)(int32_t)v);
        const uint64_t nlo = lo + sq;
        hi += (nlo < sq ? 1ull : 0ull);
        lo = nlo;
    } else {
        const i128w p = mul64x64(v, v);
        const uint64_t nlo = lo + p.lo;
        hi += (uint64_t)p.hi + (nlo < p.lo ? 1ull : 0ull);
        lo = nlo;
    }
}

// One CTA per row.  FUSED: compute rms = isqrt((eps + sum a^2) / dim) here and write
// it to rms_out; otherwise read the caller's rms[row].
template <typename WT, bool FUSED, bool STAGE>
__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(const int64_t* __restrict__ A, const WT* __restrict__ W, const int64_t* rms_in,
               int64_t* rms_out, int64_t* __restrict__ C, int64_t N, int64_t eps, int64_t dim)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ u128w red[32];
    __shared__ int64_t s_rms;
    int64_t* row = reinterpret_cast<int64_t*>(smem_raw);
    const int64_t off = (int64_t)blockIdx.x * N;
    const int64_t* a = A + off;
    int64_t* c = C + off;
    const bool vec = ((N & 1) == 0) && ((((uintptr_t)A | (uintptr_t)C) & 15) == 0);

    if (FUSED) {
        u128w acc = {0, 0};
        if (vec) {
            const longlong2* av = reinterpret_cast<const longlong2*>(a);
            longlong2* rv = reinterpret_cast<longlong2*>(row);
            for (int64_t i = threadIdx.x; i < (N >> 1); i += kThreads) {
                longlong2 v = av[i];
                if (STAGE) rv[i] = v;
                add_square(acc.lo, acc.hi, v.x);
                add_square(acc.lo, acc.hi, v.y);
            }
        } else {
            for (int64_t i = threadIdx.x; i < N; i += kThreads) {
                int64_t v = a[i];
                if (STAGE) row[i] = v;
                add_square(acc.lo, acc.hi, v);
            }
        }
        acc = warp_sum_u128(acc);
        int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
        if (lane == 0) red[wid] = acc;
        __syncthreads();
        if (wid == 0) {
            u128w t = (lane < (kThreads >> 5)) ? red[lane] : u128w{0, 0};
            t = warp_sum_u128(t);
            if (lane == 0) {
                unsigned __int128 tot = ((unsigned __int128)t.hi << 64) | t.lo;
                tot += (unsigned __int128)(__int128)eps;
                uint64_t r = 0;
                if (dim) {
                    if ((tot >> 64) == 0) r = isqrt_u128((unsigned __int128)((uint64_t)tot / (uint64_t)dim));
                    else r = isqrt_u128(tot / (unsigned __int128)(uint64_t)dim);
                }
                s_rms = (int64_t)r;
                if (rms_out) rms_out[blockIdx.x] = (int64_t)r;
            }
        }
        __syncthreads();
    } else {
        if (threadIdx.x == 0) s_rms = rms_in[blockIdx.x];
        __syncthreads();
    }
    const int64_t r = s_rms;
    const double inv = r > 0 ? 1.0 / (double)r : 0.0;
    const int64_t* src = (FUSED && STAGE) ? row : a;
    if (vec) {
        const longlong2* sv = reinterpret_cast<const longlong2*>(src);
        longlong2* cv = reinterpret_cast<longlong2*>(c);
        for (int64_t i = threadIdx.x; i < (N >> 1); i += kThreads) {
            longlong2 v = sv[i];
            longlong2 o;
            o.x = norm_one(v.x, (int64_t)W[2 * i], r, inv);
            o.y = norm_one(v.y, (int64_t)W[2 * i + 1], r, inv);
            cv[i] = o;
        }
    } else {
        for (int64_t i = threadIdx.x; i < N; i += kThreads)
            c[i] = norm_one(src[i], (int64_t)W[i], r, inv);
    }
}

// Rows of at most 16 * kRegThreads elements: the row lives in registers (E 16-byte pairs per
// thread, every load in flight at once), no shared-memory staging, two 512-thread CTAs per SM so one
// row streams while the other reduces.
constexpr int kRegThreads = 512;

template <typename WT, int E>
__global__ void __launch_bounds__(kRegThreads, 2)
rmsnorm_reg_kernel(const int64_t* __restrict__ A, const WT* __restrict__ W, int64_t* rms_out,
                   int64_t* __restrict__ C, int half, int64_t eps, int64_t dim)
{
    __shared__ u128w red[kRegThreads / 32];
    __shared__ int64_t s_rms;
    const int64_t off = (int64_t)blockIdx.x * half;
    const longlong2* av = reinterpret_cast<const longlong2*>(A) + off;
    longlong2* cv = reinterpret_cast<longlong2*>(C) + off;
    longlong2 v[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
        const int i = threadIdx.x + j * kRegThreads;
        v[j] = i < half ? av[i] : make_longlong2(0, 0);
    }
    u128w acc = {0, 0};
#pragma unroll
    for (int j = 0; j < E; ++j) {
        add_square(acc.lo, acc.hi, v[j].x);
        add_square(acc.lo, acc.hi, v[j].y);
    }
    acc = warp_sum_u128(acc);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = acc;
    __syncthreads();
    if (wid == 0) {
        u128w t = (lane < kRegThreads / 32) ? red[lane] : u128w{0, 0};
        t = warp_sum_u128(t);
        if (lane == 0) {
            unsigned __int128 tot = ((unsigned __int128)t.hi << 64) | t.lo;
            tot += (unsigned __int128)(__int128)eps;
            uint64_t r = 0;
            if (dim) {
                if ((tot >> 64) == 0) r = isqrt_u128((unsigned __int128)((uint64_t)tot / (uint64_t)dim));
                else r = isqrt_u128(tot / (unsigned __int128)(uint64_t)dim);
            }
            s_rms = (int64_t)r;
            if (rms_out) rms_out[blockIdx.x] = (int64_t)r;
        }
    }
    __syncthreads();
    const int64_t r = s_rms;
    const double inv = r > 0 ? 1.0 / (double)r : 0.0;
#pragma unroll
    for (int j = 0; j < E; ++j) {
        const int i = threadIdx.x + j * kRegThreads;
        if (i < half) {
            longlong2 o;
            o.x = norm_one_fast(v[j].x, (int64_t)W[2 * i], r, inv);
            o.y = norm_one_fast(v[j].y, (int64_t)W[2 * i + 1], r, inv);
            cv[i] = o;
        }
    }
}

template <typename WT>
static int launch_rmsnorm_reg(const int64_t* A, const WT* W, int64_t* rms_out, int64_t* C, int64_t M,
                              int64_t N, int64_t eps, int64_t dim, cudaStream_t st)
{
    const int half = (int)(N >> 1);
    const int per = (half + kRegThreads - 1) / kRegThreads;
    const unsigned g = (unsigned)M;
    if (per <= 1) rmsnorm_reg_kernel<WT, 1><<<g, kRegThreads, 0, st>>>(A, W, rms_out, C, half, eps, dim);
    else if (per <= 2) rmsnorm_reg_kernel<WT, 2><<<g, kRegThreads, 0, st>>>(A, W, rms_out, C, half, eps, dim);
    else if (per <= 4) rmsnorm_reg_kernel<WT, 4><<<g, kRegThreads, 0, st>>>(A, W, rms_out, C, half, eps, dim);
    else rmsnorm_reg_kernel<WT, 8><<<g, kRegThreads, 0, st>>>(A, W, rms_out, C, half, eps, dim);
    return check_launch();
}

template <typename WT>
static int launch_rmsnorm_t(const int64_t* A, const WT* W, const int64_t* rms_in, int64_t* rms_out,
                            int64_t* C, int64_t M, int64_t N, int64_t eps, int64_t dim, bool fused,
                            cudaStream_t st)
{
    if (fused && (N & 1) == 0 && N <= 16 * kRegThreads && ((((uintptr_t)A | (uintptr_t)C) & 15) == 0) &&
        !switches().rms_staged)
        return launch_rmsnorm_reg<WT>(A, W, rms_out, C, M, N, eps, dim, st);
    size_t row_bytes = (size_t)N * 8;
    bool stage = fused && row_bytes <= 200 * 1024 && !switches().rms_nostage;
    size_t smem = stage ? row_bytes : 0;
#define ZKDS_RMS(F, S)                                                                       \
    do {                                                                                     \
        auto k = rmsnorm_kernel<WT, F, S>;                                                   \
        if (smem > 48 * 1024)                                                                \
            ZKDS_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                           (int)smem));                                      \
        k<<<(unsigned)M, kThreads, smem, st>>>(A, W, rms_in, rms_out, C, N, eps, dim);       \
    } while (0)
    if (fused && stage) ZKDS_RMS(true, true);
    else if (fused) ZKDS_RMS(true, false);
    else ZKDS_RMS(false, false);
#undef ZKDS_RMS
    return check_launch();
}

int launch_rmsnorm(const int64_t* A, const void* W, int w_bits, const int64_t* rms_in,
                   int64_t* rms_out, int64_t* C, int64_t M, int64_t N, int64_t eps, int64_t dim,
                   int fused, cudaStream_t st)
{
    if (M == 0 || N == 0) return ZKDS_OK;
    if (M > 0x7fffffffll) return ZKDS_ERR_RANGE;
    if (w_bits == 32)
        return launch_rmsnorm_t<int32_t>(A, (const int32_t*)W, rms_in, rms_out, C, M, N, eps, dim,
                                         fused != 0, st);
    if (w_bits == 64)
        return launch_rmsnorm_t<int64_t>(A, (const int64_t*)W, rms_in, rms_out, C, M, N, eps, dim,
                                         fused != 0, st);
    return ZKDS_ERR_ARG;
}

// ------------------------------------------------------------------------------
// gated MLP tail, expert dispatch and combine
// ------------------------------------------------------------------------------

// h = (silu_q23(r1) * r2) >> 23 (wrapping product, arithmetic shift: model.py:1048, 1280);
// r1/r2 are rows of length n with row stride ld (so both halves of one fused w1|w3 GEMM output
// can be read in place); s1_out (optional, dense) receives silu(r1) for the zk dump.
__global__ void __launch_bounds__(kThreads)
glu_kernel(const int64_t* __restrict__ r1, const int64_t* __restrict__ r2, int64_t ld,
           int64_t* __restrict__ h, int64_t* __restrict__ s1_out, const int64_t* __restrict__ lut_g,
           int64_t rows, int64_t n)
{
    __shared__ int64_t lut[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = lut_g[i];
    __syncthreads();
    const int64_t nv = n >> 1;  // n is even (checked by the launcher)
    const int64_t total = rows * nv;
    for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * kThreads) {
        const int64_t row = t / nv, c = (t - row * nv) << 1;
        const longlong2 a = *reinterpret_cast<const longlong2*>(r1 + row * ld + c);
        const longlong2 b = *reinterpret_cast<const longlong2*>(r2 + row * ld + c);
        longlong2 sv, o;
        sv.x = act_one<23, true>(a.x, lut);
        sv.y = act_one<23, true>(a.y, lut);
        o.x = (int64_t)((uint64_t)sv.x * (uint64_t)b.x) >> 23;
        o.y = (int64_t)((uint64_t)sv.y * (uint64_t)b.y) >> 23;
        *reinterpret_cast<longlong2*>(h + row * n + c) = o;
        if (s1_out) *reinterpret_cast<longlong2*>(s1_out + row * n + c) = sv;
    }
}

int launch_glu(const int64_t* r1, const int64_t* r2, int64_t ld, int64_t* h, int64_t* s1_out,
               const int64_t* lut, int64_t rows, int64_t n, cudaStream_t st)
{
    if (rows == 0 || n == 0) return ZKDS_OK;
    if ((n & 1) || (ld & 1) ||
        ((((uintptr_t)r1 | (uintptr_t)r2 | (uintptr_t)h | (uintptr_t)s1_out) & 15) != 0))
        return ZKDS_ERR_ARG;
    int grid = grid_for(rows * (n / 2), kThreads, sm_count(), 16);
    glu_kernel<<<grid, kThreads, 0, st>>>(r1, r2, ld, h, s1_out, lut, rows, n);
    return check_launch();
}

// The gated product written as signed 8-bit limb planes (the A operand of the w2 contraction) instead
// of int64 words: plane l of row r at planes + l * plane_stride + r * Kp, balanced radix-256 digits as
// in the limb split, columns from n to Kp zero.  A CTA is a (rows x threads-per-row) grid, four
// consecutive columns per thread; the largest magnitude seen goes to absmax_out, a value the L limbs
// cannot hold raises *overflow.
template <int LL>      // limb count known at compile time, 0 = use L
__global__ void __launch_bounds__(kThreads)
glu_planes_kernel(const int64_t* __restrict__ r1, const int64_t* __restrict__ r2, int64_t ld,
                  const int64_t* __restrict__ lut_g, int8_t* __restrict__ planes, int L, int64_t rows, int64_t n,
                  int64_t Kp, int64_t plane_stride, unsigned* overflow, unsigned long long* absmax_out,
                  int tpr_log2)
{
    __shared__ int64_t lut[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = lut_g[i];
    __syncthreads();
    uint64_t seen = 0;
    uint32_t seen32 = 0;          // largest magnitude met on the 32-bit path
    bool ovf = false;
    const int64_t quads = Kp >> 2;
    const int tpr = 1 << tpr_log2;
    const int lane_q = threadIdx.x & (tpr - 1);
    const int64_t rpb = kThreads >> tpr_log2;
    for (int64_t r = (int64_t)blockIdx.x * rpb + (threadIdx.x >> tpr_log2); r < rows;
         r += (int64_t)gridDim.x * rpb) {
        const int64_t* a = r1 + r * ld;
        const int64_t* b = r2 + r * ld;
        int8_t* drow = planes + r * Kp;
        for (int64_t qd = lane_q; qd < quads; qd += tpr) {
            const int64_t k0 = qd << 2;
            int64_t v[4] = {0, 0, 0, 0};
            if (k0 + 4 <= n) {
                const longlong2 a0 = *reinterpret_cast<const longlong2*>(a + k0);
                const longlong2 a1 = *reinterpret_cast<const longlong2*>(a + k0 + 2);
                const longlong2 b0 = *reinterpret_cast<const longlong2*>(b + k0);
                const longlong2 b1 = *reinterpret_cast<const longlong2*>(b + k0 + 2);
                v[0] = (int64_t)((uint64_t)act_one<23, true>(a0.x, lut) * (uint64_t)b0.x) >> 23;
                v[1] = (int64_t)((uint64_t)act_one<23, true>(a0.y, lut) * (uint64_t)b0.y) >> 23;
                v[2] = (int64_t)((uint64_t)act_one<23, true>(a1.x, lut) * (uint64_t)b1.x) >> 23;
                v[3] = (int64_t)((uint64_t)act_one<23, true>(a1.y, lut) * (uint64_t)b1.y) >> 23;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (k0 + j < n)
                        v[j] = (int64_t)((uint64_t)act_one<23, true>(a[k0 + j], lut) * (uint64_t)b[k0 + j]) >> 23;
            }
            constexpr int LMAX = LL ? LL : 9;
            uint32_t w[LMAX];
            if (LL == 3) {
                // three limbs in 32-bit arithmetic: for -0x808080 <= v <= 0x7F7F7F the balanced digits of v are the
                // bytes of v + 0x808080 with their top bits flipped; anything outside takes the general path
                const uint64_t t0 = (uint64_t)v[0] + 0x808080ull, t1 = (uint64_t)v[1] + 0x808080ull,
                               t2 = (uint64_t)v[2] + 0x808080ull, t3 = (uint64_t)v[3] + 0x808080ull;
                if (((t0 | t1 | t2 | t3) >> 24) == 0) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int32_t x = (int32_t)v[j];
                        const uint32_t a32 = (uint32_t)(x ^ (x >> 31));
                        seen32 = a32 > seen32 ? a32 : seen32;
                    }
#pragma unroll
                    for (int l = 0; l < 3; ++l) {
                        const uint32_t sel = 0x0040u + 0x0011u * (uint32_t)l;
                        const uint32_t lo = __byte_perm((uint32_t)t0, (uint32_t)t1, sel),
                                       hi = __byte_perm((uint32_t)t2, (uint32_t)t3, sel);
                        *reinterpret_cast<uint32_t*>(drow + k0 + l * plane_stride) =
                            __byte_perm(lo, hi, 0x5410u) ^ 0x80808080u;
                    }
                    continue;
                }
            }
#pragma unroll
            for (int l = 0; l < LMAX; ++l) w[l] = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int64_t u = v[j];
                const uint64_t mag = (uint64_t)(u ^ (u >> 63));
                seen = mag > seen ? mag : seen;
#pragma unroll
                for (int l = 0; l < LMAX; ++l) {
                    if (LL || l < L) {
                        w[l] |= (uint32_t)(u & 0xFF) << (j * 8);
                        u = (u >> 8) + ((u >> 7) & 1);
                    }
                }
                ovf |= (u != 0);
            }
#pragma unroll
            for (int l = 0; l < LMAX; ++l)
                if (LL || l < L) *reinterpret_cast<uint32_t*>(drow + k0 + l * plane_stride) = w[l];
        }
    }
    seen = seen32 > seen ? seen32 : seen;
    if (ovf) *overflow = 1u;
    if (absmax_out) {
        seen = warp_max_u64(seen);
        if ((threadIdx.x & 31) == 0 && seen) atomicMax(absmax_out, (unsigned long long)seen);
    }
}

bool glu_planes_supported(const int64_t* r1, const int64_t* r2, int64_t ld, int64_t n)
{
    return n > 0 && (n & 1) == 0 && (ld & 1) == 0 && ((((uintptr_t)r1 | (uintptr_t)r2) & 15) == 0);
}

int launch_glu_planes(const int64_t* r1, const int64_t* r2, int64_t ld, const int64_t* lut, int8_t* planes, int L,
                      int64_t rows, int64_t n, int64_t Kp, int64_t plane_stride, unsigned* overflow,
                      unsigned long long* absmax_out, cudaStream_t st)
{
    if (rows == 0) return ZKDS_OK;
    if (!glu_planes_supported(r1, r2, ld, n) || L < 1 || L > 9 || (Kp & 3) || Kp < n) return ZKDS_ERR_UNSUPPORTED;
    int tl = 0;
    while (tl < 8 && (1 << tl) < (Kp >> 2)) ++tl;
    const int64_t rpb = kThreads >> tl;
    int64_t grid = (rows + rpb - 1) / rpb;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (grid > cap) grid = cap;
#define ZKDS_GP(LL)                                                                                         \
    glu_planes_kernel<LL><<<(unsigned)grid, kThreads, 0, st>>>(r1, r2, ld, lut, planes, L, rows, n, Kp,     \
                                                               plane_stride, overflow, absmax_out, tl)
    switch (L) {
    case 2: ZKDS_GP(2); break;
    case 3: ZKDS_GP(3); break;
    case 4: ZKDS_GP(4); break;
    case 5: ZKDS_GP(5); break;
    default: ZKDS_GP(0); break;
    }
#undef ZKDS_GP
    return check_launch();
}

// dst[r][:] = src[index[r]][:] for index[r] >= 0, zeros otherwise (token rows -> expert order)
__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(const longlong2* __restrict__ src, const int* __restrict__ index,
                   longlong2* __restrict__ dst, int64_t cols2)
{
    const int64_t r = blockIdx.x;
    const int i = index[r];
    longlong2* d = dst + r * cols2;
    if (i < 0) {
        for (int64_t c = threadIdx.x; c < cols2; c += kThreads) d[c] = make_longlong2(0, 0);
    } else {
        const longlong2* sp = src + (int64_t)i * cols2;
        for (int64_t c = threadIdx.x; c < cols2; c += kThreads) d[c] = sp[c];
    }
}

int launch_gather_rows(const int64_t* src, const int* index, int64_t* dst, int64_t rows, int64_t cols,
                       cudaStream_t st)
{
    if (rows == 0 || cols == 0) return ZKDS_OK;
    if ((cols & 1) || rows > 0x7fffffffll || ((((uintptr_t)src | (uintptr_t)dst) & 15) != 0))
        return ZKDS_ERR_ARG;
    gather_rows_kernel<<<(unsigned)rows, kThreads, 0, st>>>(
        reinterpret_cast<const longlong2*>(src), index, reinterpret_cast<longlong2*>(dst), cols / 2);
    return check_launch();
}

// y[t][:] = base[t][:] + sum_slot floor(out[pos[t][slot]][:] * w[t][slot] / 2^23)   (model.py:1379-1383:
// wrapping int64 product, floor division by 2^23, order-free integer sum); pos < 0 skips a slot
__global__ void __launch_bounds__(kThreads)
moe_combine_kernel(const longlong2* __restrict__ out, const int* __restrict__ pos,
                   const int64_t* __restrict__ w, const longlong2* __restrict__ base,
                   longlong2* __restrict__ y, int slots, int64_t cols2)
{
    const int64_t t = blockIdx.x;
    for (int64_t c = threadIdx.x; c < cols2; c += kThreads) {
        longlong2 acc = base ? base[t * cols2 + c] : make_longlong2(0, 0);
        for (int s = 0; s < slots; ++s) {
            const int r = pos[t * slots + s];
            if (r < 0) continue;
            const int64_t ws = w[t * slots + s];
            const longlong2 v = out[(int64_t)r * cols2 + c];
            acc.x = (int64_t)((uint64_t)acc.x + (uint64_t)((int64_t)((uint64_t)v.x * (uint64_t)ws) >> 23));
            acc.y = (int64_t)((uint64_t)acc.y + (uint64_t)((int64_t)((uint64_t)v.y * (uint64_t)ws) >> 23));
        }
        y[t * cols2 + c] = acc;
    }
}

int launch_moe_combine(const int64_t* out, const int* pos, const int64_t* w, const int64_t* base,
                       int64_t* y, int64_t tokens, int slots, int64_t cols, cudaStream_t st)
{
    if (tokens == 0 || cols == 0) return ZKDS_OK;
    if ((cols & 1) || tokens > 0x7fffffffll ||
        ((((uintptr_t)out | (uintptr_t)base | (uintptr_t)y) & 15) != 0))
        return ZKDS_ERR_ARG;
    moe_combine_kernel<<<(unsigned)tokens, kThreads, 0, st>>>(
        reinterpret_cast<const longlong2*>(out), pos, w, reinterpret_cast<const longlong2*>(base),
        reinterpret_cast<longlong2*>(y), slots, cols / 2);
    return check_launch();
}

// ------------------------------------------------------------------------------
// expert parallelism over peer memory: the owner of a token's experts writes the weighted sum of their outputs
// straight into the token's home GPU, one slot per (token, owner); the home GPU adds the slots it expects
// ------------------------------------------------------------------------------
struct PeerSlots {
    int64_t* base[kMaxRowParts];
};

// token g = part * tokens_per_part + t of the gathered batch; rows with no local expert are not touched.
// slot row of (t, my_part) on the home GPU: base[part] + (t * n_parts + my_part) * cols.
__global__ void __launch_bounds__(kThreads)
moe_combine_peer_kernel(const longlong2* __restrict__ out, const int* __restrict__ pos, const int64_t* __restrict__ w,
                        int slots, int64_t cols2, int64_t tokens_per_part, int n_parts, int my_part,
                        const PeerSlots peers)
{
    const int64_t g = blockIdx.x;
    __shared__ int s_any;
    if (threadIdx.x == 0) {
        int any = 0;
        for (int s = 0; s < slots; ++s) any |= pos[g * slots + s] >= 0;
        s_any = any;
    }
    __syncthreads();
    if (!s_any) return;
    const int64_t part = g / tokens_per_part, t = g - part * tokens_per_part;
    if (part >= n_parts) return;
    longlong2* dst = reinterpret_cast<longlong2*>(peers.base[part]) + (t * n_parts + my_part) * cols2;
    for (int64_t c = threadIdx.x; c < cols2; c += kThreads) {
        longlong2 acc = make_longlong2(0, 0);
        for (int s = 0; s < slots; ++s) {
            const int r = pos[g * slots + s];
            if (r < 0) continue;
            const int64_t ws = w[g * slots + s];
            const longlong2 v = out[(int64_t)r * cols2 + c];
            acc.x = (int64_t)((uint64_t)acc.x + (uint64_t)((int64_t)((uint64_t)v.x * (uint64_t)ws) >> 23));
            acc.y = (int64_t)((uint64_t)acc.y + (uint64_t)((int64_t)((uint64_t)v.y * (uint64_t)ws) >> 23));
        }
        dst[c] = acc;
    }
}

int launch_moe_combine_peer(const int64_t* out, const int* pos, const int64_t* w, int64_t tokens, int slots,
                            int64_t cols, int64_t tokens_per_part, int64_t* const* slot_bases, int n_parts,
                            int my_part, cudaStream_t st)
{
    if (tokens == 0 || cols == 0) return ZKDS_OK;
    if ((cols & 1) || tokens > 0x7fffffffll || n_parts < 1 || n_parts > kMaxRowParts || my_part < 0 ||
        my_part >= n_parts || tokens_per_part <= 0 || tokens > tokens_per_part * n_parts || slots < 1 ||
        (((uintptr_t)out) & 15) != 0)
        return ZKDS_ERR_ARG;
    PeerSlots peers{};
    for (int i = 0; i < n_parts; ++i) {
        if (!slot_bases[i] || (((uintptr_t)slot_bases[i]) & 15) != 0) return ZKDS_ERR_ARG;
        peers.base[i] = slot_bases[i];
    }
    moe_combine_peer_kernel<<<(unsigned)tokens, kThreads, 0, st>>>(
        reinterpret_cast<const longlong2*>(out), pos, w, slots, cols / 2, tokens_per_part, n_parts, my_part, peers);
    return check_launch();
}

// y[t] = base[t] + sum over the owners q of token t's experts (each owner once) of slot_rows[t][q]
__global__ void __launch_bounds__(kThreads)
moe_sum_slots_kernel(const longlong2* __restrict__ base, const longlong2* __restrict__ slot_rows,
                     const int64_t* __restrict__ indices, int slots, int64_t cols2, int n_parts,
                     int experts_per_part, longlong2* __restrict__ y)
{
    const int64_t t = blockIdx.x;
    __shared__ unsigned s_owners;
    if (threadIdx.x == 0) {
        unsigned m = 0;
        for (int s = 0; s < slots; ++s) {
            const int64_t e = indices[t * slots + s];
            const int64_t q = e >= 0 ? e / experts_per_part : -1;
            if (q >= 0 && q < n_parts) m |= 1u << q;
        }
        s_owners = m;
    }
    __syncthreads();
    const unsigned owners = s_owners;
    const longlong2* rows = slot_rows + t * n_parts * cols2;
    for (int64_t c = threadIdx.x; c < cols2; c += kThreads) {
        longlong2 acc = base ? base[t * cols2 + c] : make_longlong2(0, 0);
        for (int q = 0; q < n_parts; ++q) {
            if (!((owners >> q) & 1u)) continue;
            const longlong2 v = rows[q * cols2 + c];
            acc.x = (int64_t)((uint64_t)acc.x + (uint64_t)v.x);
            acc.y = (int64_t)((uint64_t)acc.y + (uint64_t)v.y);
        }
        y[t * cols2 + c] = acc;
    }
}

int launch_moe_sum_slots(const int64_t* base, const int64_t* slot_rows, const int64_t* indices, int64_t tokens,
                         int slots, int64_t cols, int n_parts, int experts_per_part, int64_t* y, cudaStream_t st)
{
    if (tokens == 0 || cols == 0) return ZKDS_OK;
    if ((cols & 1) || tokens > 0x7fffffffll || n_parts < 1 || n_parts > kMaxRowParts || experts_per_part < 1 ||
        slots < 1 || ((((uintptr_t)base | (uintptr_t)slot_rows | (uintptr_t)y) & 15) != 0))
        return ZKDS_ERR_ARG;
    moe_sum_slots_kernel<<<(unsigned)tokens, kThreads, 0, st>>>(
        reinterpret_cast<const longlong2*>(base), reinterpret_cast<const longlong2*>(slot_rows), indices, slots,
        cols / 2, n_parts, experts_per_part, reinterpret_cast<longlong2*>(y));
    return check_launch();
}

// Barrier between the GPUs of one node over peer-mapped flag words.  Every GPU owns n_parts 64-bit flags;
// GPU i announces epoch e by storing e into flag i of every GPU (its own included) and then waits until all
// of its own flags have reached e.  Epochs only grow, so a flag never has to be reset.  The wait is bounded
// (four seconds of the global timer): when it runs out the kernel sets *status and returns, the stream
// carries on with whatever data is there and the host reports the error from the status word.
struct PeerFlags {
    unsigned long long* base[kMaxRowParts];
};

__global__ void __launch_bounds__(32)
peer_barrier_kernel(const PeerFlags peers, int n_parts, int my_part, unsigned long long epoch, unsigned* status)
{
    const int i = threadIdx.x;
    if (i < n_parts) {
        // the writes of every earlier kernel of this stream are ordered before the announcement
        __threadfence_system();
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(peers.base[i] + my_part), "l"(epoch) : "memory");
        const unsigned long long* mine = peers.base[my_part] + i;
        unsigned long long t0, now, seen = 0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (;;) {
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(mine) : "memory");
            if (seen >= epoch) break;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - t0 > 4000000000ull) { atomicExch(status, 1u); break; }
            __nanosleep(200);
        }
        __threadfence_system();
    }
}

int launch_peer_barrier(unsigned long long* const* flag_bases, int n_parts, int my_part, unsigned long long epoch,
                        unsigned* status, cudaStream_t st)
{
    if (n_parts < 1 || n_parts > kMaxRowParts || my_part < 0 || my_part >= n_parts || !status) return ZKDS_ERR_ARG;
    PeerFlags peers{};
    for (int i = 0; i < n_parts; ++i) {
        if (!flag_bases[i] || (((uintptr_t)flag_bases[i]) & 7) != 0) return ZKDS_ERR_ARG;
        peers.base[i] = flag_bases[i];
    }
    peer_barrier_kernel<<<1, 32, 0, st>>>(peers, n_parts, my_part, epoch, status);
    return check_launch();
}

// ------------------------------------------------------------------------------
// gate: bias, grouped top-k selection, weights (Gate.forward, model.py:1140-1211), one warp per token
// ------------------------------------------------------------------------------
// scores = sigma + bias; per group the sum of its two largest scores (the largest when there is no bias);
// the topk_groups best groups stay, the others are out; the topk best remaining experts, in descending
// order of score; raw = sigma[idx]; w = ((raw * 2^23) // sum raw) * 5 // 2.  Ties go to the lower index
// (the set torch.topk's radix select takes; the order among equal scores is unspecified there).
namespace {

__device__ __forceinline__ int64_t floor_div_gate(int64_t a, int64_t b)
{
    if (b == 0) return 0;          // an all-zero weight row: torch would raise; defined as 0 here
    int64_t q = a / b, r = a % b;
    return (r != 0 && ((r < 0) != (b < 0))) ? q - 1 : q;
}

constexpr int kGateMaxE = 1024;          // experts per token held in shared memory per warp
constexpr int kGateWarps = 4;

struct Top2 { int64_t a, b; };           // a >= b

__device__ __forceinline__ Top2 top2_merge(Top2 x, Top2 y)
{
    Top2 r;
    if (x.a >= y.a) { r.a = x.a; r.b = x.b >= y.a ? x.b : y.a; }
    else { r.a = y.a; r.b = y.b >= x.a ? y.b : x.a; }
    return r;
}

__global__ void __launch_bounds__(32 * kGateWarps)
gate_select_kernel(const int64_t* __restrict__ sig, const int32_t* __restrict__ bias, int64_t T, int E, int n_groups,
                   int topk_groups, int topk, int64_t* __restrict__ indices, int64_t* __restrict__ raw_out,
                   int64_t* __restrict__ w_out)
{
    extern __shared__ int64_t gate_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * kGateWarps + warp;
    if (t >= T) return;
    int64_t* sc = gate_smem + (size_t)warp * E;
    const int64_t* srow = sig + t * E;
    for (int e = lane; e < E; e += 32) sc[e] = srow[e] + (bias ? (int64_t)bias[e] : 0);
    __syncwarp();
    const int gs = E / n_groups;
    if (n_groups > 1) {
        // group score in lane g (n_groups <= 32)
        int64_t gscore = INT64_MIN;
        for (int g = 0; g < n_groups; ++g) {
            Top2 m{INT64_MIN, INT64_MIN};
            for (int i = lane; i < gs; i += 32) m = top2_merge(m, Top2{sc[g * gs + i], INT64_MIN});
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                Top2 y{__shfl_xor_sync(0xffffffffu, m.a, o), __shfl_xor_sync(0xffffffffu, m.b, o)};
                m = top2_merge(m, y);
            }
            const int64_t v = bias ? (int64_t)((uint64_t)m.a + (uint64_t)m.b) : m.a;
            if (lane == g) gscore = v;
        }
        // keep the topk_groups best groups (lower index on ties), mask the rest
        unsigned kept = 0;
        for (int r = 0; r < topk_groups; ++r) {
            int64_t v = (lane < n_groups && !((kept >> lane) & 1u)) ? gscore : INT64_MIN;
            int idx = lane;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const int64_t ov = __shfl_xor_sync(0xffffffffu, v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
            }
            kept |= 1u << idx;
        }
        for (int e = lane; e < E; e += 32)
            if (!((kept >> (e / gs)) & 1u)) sc[e] = -(1ll << 42);           // model.py:1186
        __syncwarp();
    }
    // topk experts, descending; lower index on ties
    int64_t raw_sum = 0, my_raw = 0;
    int my_idx = 0;
    for (int r = 0; r < topk; ++r) {
        int64_t v = INT64_MIN;
        int idx = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const int64_t x = sc[e];
            if (x > v) { v = x; idx = e; }                                   // ascending e: first maximum kept
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const int64_t ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        const int64_t raw = srow[idx];
        raw_sum += raw;
        if (lane == r) { my_raw = raw; my_idx = idx; }
        if (lane == 0) sc[idx] = INT64_MIN;                                  // taken (below the group mask value)
        __syncwarp();
    }
    if (lane < topk) {
        indices[t * topk + lane] = my_idx;
        raw_out[t * topk + lane] = my_raw;
        // floor divisions of torch's `//` (model.py:1207, 1210); the wrapping products of int64 tensors
        int64_t w = floor_div_gate((int64_t)((uint64_t)my_raw << 23), raw_sum);
        w = floor_div_gate((int64_t)((uint64_t)w * 5ull), 2);
        w_out[t * topk + lane] = w;
    }
}

}  // namespace

int launch_gate_select(const int64_t* sig, const int32_t* bias, int64_t T, int E, int n_groups, int topk_groups,
                       int topk, int64_t* indices, int64_t* raw, int64_t* w, cudaStream_t st)
{
    if (T == 0) return ZKDS_OK;
    if (E <= 0 || E > kGateMaxE || n_groups < 1 || n_groups > 32 || E % n_groups || topk < 1 || topk > 32 ||
        topk_groups < 1 || topk_groups > n_groups || (int64_t)topk > (int64_t)topk_groups * (E / n_groups))
        return ZKDS_ERR_UNSUPPORTED;
    const int64_t blocks = (T + kGateWarps - 1) / kGateWarps;
    if (blocks > 0x7fffffffll) return ZKDS_ERR_RANGE;
    gate_select_kernel<<<(unsigned)blocks, 32 * kGateWarps, (size_t)kGateWarps * E * sizeof(int64_t), st>>>(
        sig, bias, T, E, n_groups, topk_groups, topk, indices, raw, w);
    return check_launch();
}

}  // namespace zkds
