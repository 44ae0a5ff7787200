// Exact int64 contraction on the 5th-generation tensor cores.
//
// Every operand element is written in balanced radix 256: v = sum_l d_l * 256^l with
// signed digits d_l in [-128, 127] ("limbs").  A pre-pass stores each limb of A and B as
// its own K-major int8 plane.  The product sum is then
//     sum_k a*b = sum_d 256^d * sum_{i+j=d} sum_k A_i[m,k] * B_j[n,k],
// i.e. one int8 GEMM per limb pair, accumulated per diagonal d = i + j.  The kernel keeps
// one int32 accumulator tile per diagonal in tensor memory.  The B limb planes of a tile
// are stacked along N in shared memory, so a single tcgen05.mma of A_i against the stack
// covers the diagonals i .. i+Lb-1 at once: the accumulators of consecutive diagonals are
// adjacent column ranges of tensor memory and the MMA for limb i simply starts NT columns
// further right.  The epilogue reads the diagonals back, recombines them in 128 bits, adds
// the rounding addend, shifts, and writes the int64 quotient (and remainder).
//
// One CTA computes a 128 x NT output tile: warp 0 issues plain per-CTA TMA loads,
// warp 1 owns tensor memory and issues the MMAs, warps 2-5 zero the accumulators, then
// run the epilogue.  Every wait is bounded; a wait that runs out raises a flag the host
// reads, and the CTA leaves through the normal exit path (tensor memory released).
//
// Exactness bound: a diagonal sums at most min(La, Lb) * K products of magnitude <= 2^14,
// which must stay below 2^31; the launcher refuses shapes beyond that.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace zkds {

namespace {

// ------------------------------------------------------------------------------------
// operand range and limb split
// ------------------------------------------------------------------------------------

template <typename T>
__global__ void __launch_bounds__(256)
absmax_kernel(const T* X, int64_t rows, int64_t cols, int64_t sz, int64_t sr, int64_t sc,
              int64_t div, uint64_t* out)
{
    const T* x = X + (int64_t)blockIdx.y * sz;
    uint64_t best = 0;
    const int64_t total = rows * cols;
    const bool row_major = (sc == 1);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r, c;
        if (row_major) { r = i / cols; c = i - r * cols; }
        else { c = i / rows; r = i - c * rows; }
        int64_t v = (int64_t)x[r * sr + c * sc];
        if (div != 1) v = v / div;
        uint64_t a = v < 0 ? (uint64_t)0 - (uint64_t)v : (uint64_t)v;
        // balanced digits reach one further down than up
        if (v < 0 && a) a -= 1;
        best = a > best ? a : best;
    }
    best = warp_max_u64(best);
    if ((threadIdx.x & 31) == 0 && best) atomicMax((unsigned long long*)out, (unsigned long long)best);
}

// planes[l][z][r][Kp] (int8) <- limb l of X[z*sz + r*sr + k*sk] / div.  One thread converts four
// consecutive k: with a k-contiguous source a warp reads 1 KB and writes 128 bytes per plane per
// instruction.  A value the L limbs cannot hold raises *overflow; absmax_out (optional) receives
// the largest magnitude seen.
template <typename T>
__global__ void __launch_bounds__(256)
split_kernel(const T* __restrict__ X, int8_t* __restrict__ planes, int L, int64_t rows, int64_t K,
             int64_t Kp, int64_t sz, int64_t sr, int64_t sk, int64_t div, int64_t plane_stride,
             unsigned* overflow, unsigned long long* absmax_out, int64_t dst_pitch, int64_t valid_H,
             int64_t valid_start)
{
    // valid_H > 0: row r = (s, h) only holds data in columns <= valid_start + s (causal attention
    // probabilities); the rest is written as zero without being read
    uint64_t seen = 0;
    bool ovf = false;
    const int64_t quads = Kp >> 2;
    const int64_t total = rows * quads;
    const int64_t z = blockIdx.y;
    const T* x = X + z * sz;
    const bool k_fast = (sk == 1);
    const bool vec = k_fast && sizeof(T) == 8 && ((((uintptr_t)X) & 15) == 0) && ((sr & 1) == 0) &&
                     ((sz & 1) == 0);
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        int64_t r, qd;
        if (k_fast) { r = t / quads; qd = t - r * quads; }
        else { qd = t / rows; r = t - qd * rows; }
        const int64_t k0 = qd << 2;
        int64_t v[4];
        const int64_t Kv = valid_H ? (valid_start + r / valid_H + 1 < K ? valid_start + r / valid_H + 1 : K) : K;
        if (k0 >= Kv) {
            v[0] = v[1] = v[2] = v[3] = 0;
        } else if (vec && k0 + 4 <= Kv) {
            const longlong2* src = reinterpret_cast<const longlong2*>(x + r * sr + k0);
            longlong2 a = src[0], b = src[1];
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = (k0 + j < Kv) ? (int64_t)x[r * sr + (k0 + j) * sk] : 0;
        }
        uint32_t w[9];
#pragma unroll
        for (int l = 0; l < 9; ++l) w[l] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int64_t u = v[j];
            if (div != 1) u = u / div;
            // |u| for u >= 0, |u| - 1 for u < 0: balanced digits reach one further down
            const uint64_t a = (uint64_t)(u ^ (u >> 63));
            seen = a > seen ? a : seen;
#pragma unroll
            for (int l = 0; l < 9; ++l) {
                if (l < L) {
                    w[l] |= (uint32_t)(u & 0xFF) << (j * 8);
                    u = (u >> 8) + ((u >> 7) & 1);
                }
            }
            ovf |= (u != 0);
        }
        int8_t* dst = planes + (z * rows + r) * dst_pitch + k0;
#pragma unroll
        for (int l = 0; l < 9; ++l)
            if (l < L) *reinterpret_cast<uint32_t*>(dst + l * plane_stride) = w[l];
    }
    if (ovf) *overflow = 1u;
    if (absmax_out) {
        seen = warp_max_u64(seen);
        if ((threadIdx.x & 31) == 0 && seen) atomicMax(absmax_out, (unsigned long long)seen);
    }
}

// The k-contiguous case of split_kernel without any integer division: a CTA of 256 threads is a
// (256 / tpr) x tpr grid, tpr = threads per row (a power of two), and walks whole rows; every
// thread converts four consecutive k per step, two steps in flight.
// source rows spread over several buffers (expert parallelism: the token rows of every rank, read in place over
// peer mappings): row g of the gathered matrix is row g % rows_per_part of base[g / rows_per_part]
struct RowParts {
    const void* base[kMaxRowParts];
    int n;
    int64_t rows_per_part;
};

template <typename T, int LL>     // LL: limb count known at compile time, 0 = use L
__global__ void __launch_bounds__(256)
split_rows_kernel(const T* __restrict__ X, int8_t* __restrict__ planes, int L, int64_t rows, int64_t K,
                  int64_t Kp, int64_t sz, int64_t sr, int64_t div, int64_t plane_stride,
                  unsigned* overflow, unsigned long long* absmax_out, int64_t dst_pitch, int64_t valid_H,
                  int64_t valid_start, int tpr_log2, unsigned nb, unsigned gx, int z_fast, int shl,
                  const int* __restrict__ row_index, unsigned kseg, int64_t seg_quads, const RowParts parts,
                  int group_box)
{
    uint64_t seen = 0;
    uint32_t seen32 = 0;          // largest magnitude met on the 32-bit path
    bool ovf = false;
    const int64_t quads = Kp >> 2;
    // Work items are (batch, row group) pairs, gx row groups per batch, walked grid-stride.  z_fast:
    // the batches are interleaved inside a source row (batch stride < row stride), so neighbouring
    // items take neighbouring batches of the same rows and read one contiguous stretch.
    const int tpr = 1 << tpr_log2;
    const int lane_q = threadIdx.x & (tpr - 1);
    const int64_t rpb = 256 >> tpr_log2;
    bool vec = sizeof(T) == 8 && ((((uintptr_t)X) & 15) == 0) && ((sr & 1) == 0) && ((sz & 1) == 0);
    for (int i = 0; i < parts.n; ++i) vec = vec && (((uintptr_t)parts.base[i]) & 15) == 0;
    // few rows (decode): a row is cut into kseg segments of seg_quads quads so that the launch still has
    // a CTA for every SM
    const unsigned items = nb * gx * kseg;
    for (unsigned it = blockIdx.x; it < items; it += gridDim.x) {
        const unsigned seg = it % kseg, item = it / kseg;
        const int64_t q_begin = (int64_t)seg * seg_quads;
        const int64_t q_end = q_begin + seg_quads < quads ? q_begin + seg_quads : quads;
        const unsigned zi = z_fast ? item % nb : item / gx;
        const unsigned bx = z_fast ? item / nb : item - zi * gx;
        const int64_t z = zi;
        const T* x = X + z * sz;
        const int64_t r = (int64_t)bx * rpb + (threadIdx.x >> tpr_log2);
        if (r >= rows) continue;
        int64_t Kv = K;
        if (valid_H) {
            const int64_t lim = valid_start + r / valid_H + 1;
            Kv = lim < K ? lim : K;
        }
        // row_index: plane row r is source row row_index[r] (a gather fused into the split); a negative
        // entry is a padding row of zeros
        int64_t rs = r;
        if (row_index) {
            rs = row_index[r];
            if (rs < 0) Kv = 0;
            // grouped tiles whose caller promised at most group_box rows per group: a row with data beyond the
            // box would be dropped by the GEMM, so it is reported like a limb bound that did not hold
            else if (group_box && (int)(r & 127) >= group_box) ovf = true;
        }
        const T* xr = x + (rs < 0 ? 0 : rs) * sr;
        if (parts.n && rs >= 0) {
            const int64_t part = rs / parts.rows_per_part;
            if (part < parts.n)
                xr = reinterpret_cast<const T*>(parts.base[part]) + (rs - part * parts.rows_per_part) * sr;
            else
                Kv = 0;             // an index beyond the pieces: zeros, never an address outside them
        }
        int8_t* drow = planes + (z * rows + r) * dst_pitch;
#pragma unroll 2
        for (int64_t qd = q_begin + lane_q; qd < q_end; qd += tpr) {
            const int64_t k0 = qd << 2;
            int64_t v[4];
            if (k0 >= Kv) {
                v[0] = v[1] = v[2] = v[3] = 0;
            } else if (vec && k0 + 4 <= Kv) {
                const longlong2* src = reinterpret_cast<const longlong2*>(xr + k0);
                longlong2 a = src[0], b = src[1];
                v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = (k0 + j < Kv) ? (int64_t)xr[k0 + j] : 0;
            }
            constexpr int LMAX = LL ? LL : 9;
            uint32_t w[LMAX];
            if (LL == 3 && div == 1 && !shl) {
                // Three limbs, the common case, in 32-bit arithmetic: for -0x808080 <= v <= 0x7F7F7F the balanced
                // digits of v are the bytes of v + 0x808080 with their top bits flipped (digit + 128 is what the
                // biased sum holds at every position).  Anything outside takes the general path below.
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
                        const uint32_t sel = 0x0040u + 0x0011u * (uint32_t)l;     // byte l of both operands
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
                if (div != 1) u = u / div;
                if (shl) {
                    const int64_t w2 = (int64_t)((uint64_t)u << shl);
                    ovf |= (w2 >> shl) != u;      // the scaled value must still be the value
                    u = w2;
                }
                const uint64_t a = (uint64_t)(u ^ (u >> 63));
                seen = a > seen ? a : seen;
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

// ------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

constexpr uint32_t kSpinLimit = 1u << 22;

// try_wait that lets the hardware park the thread for up to ~1 us instead of returning at once:
// a waiting producer or MMA warp then takes no issue slots from the epilogue warps of its scheduler
__device__ __forceinline__ bool mbar_try_parked(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000u)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the limit ran out or another role gave up.  backoff_ns > 0: sleep
// that long after a failed try, so a waiting warp leaves the issue slots of its scheduler to the
// warps that have work (the price is up to backoff_ns of extra latency on the wake-up).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned backoff_ns = 0)
{
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_parked(bar, parity)) return true;
        if ((it & 255u) == 255u && *abort_flag) return false;
        if (backoff_ns) __nanosleep(backoff_ns);
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// accumulate flag known at compile time: no predicate set-up in the instruction stream
__device__ __forceinline__ void umma_i8_acc(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.eq.u32 p, 1, 1;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int32_t (&v)[8])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, int32_t (&v)[4])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tmem_ldn(uint32_t taddr, int32_t (&v)[8]) { tmem_ld8(taddr, v); }
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, int32_t (&v)[4]) { tmem_ld4(taddr, v); }
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, int32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st8_zero(uint32_t taddr)
{
    const uint32_t z = 0;
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const int32_t (&v)[8])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(v[0]),
        "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
        : "memory");
}

__device__ __forceinline__ void tmem_st4_zero(uint32_t taddr)
{
    const uint32_t z = 0;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %1, %1, %1};" ::"r"(taddr), "r"(z) : "memory");
}

template <int CH>
__device__ __forceinline__ void tmem_stn_zero(uint32_t taddr)
{
    if (CH == 8) tmem_st8_zero(taddr);
    else tmem_st4_zero(taddr);
}

__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand tile, 128-byte rows, 128-byte swizzle: 8-row groups are 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;               // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;     // stride byte offset
    d |= (uint64_t)1 << 46;               // descriptor version
    d |= (uint64_t)2 << 61;               // SWIZZLE_128B
    return d;
}

// The MMAs of one K block (up to four K steps of 32 bytes, LA limb tiles of A against the stacked B
// tile), straight-line: the descriptors differ from the block's first one only in the 14-bit
// address field (units of 16 bytes), so each MMA costs one 32-bit add.  `first_accumulates` is 0 only
// for the K block that opens a set of accumulators (its very first MMA then overwrites).
template <int LA>
__device__ __forceinline__ void issue_k_block(uint32_t acc, uint32_t nt_cols, uint32_t sa, uint32_t sb,
                                              uint32_t idesc, uint32_t first_accumulates, int ks_n,
                                              uint32_t a_stride16 = (128 * 128) >> 4)
{
    const uint64_t hi = smem_desc_sw128(0) & 0xFFFFFFFF00000000ull;
    const uint32_t lo_fixed = (uint32_t)(smem_desc_sw128(0) & 0xFFFFC000ull);
    const uint32_t a_lo = lo_fixed | ((sa & 0x3FFFFu) >> 4);
    const uint32_t b_lo = lo_fixed | ((sb & 0x3FFFFu) >> 4);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        if (ks < ks_n) {
#pragma unroll
            for (int i = 0; i < LA; ++i) {
                const uint64_t adesc = hi | (uint64_t)(a_lo + (uint32_t)i * a_stride16 + (uint32_t)(ks * 2));
                const uint64_t bdesc = hi | (uint64_t)(b_lo + (uint32_t)(ks * 2));
                if (ks == 0 && i == 0) umma_i8(acc, adesc, bdesc, idesc, first_accumulates);
                else umma_i8_acc(acc + (uint32_t)i * nt_cols, adesc, bdesc, idesc);
            }
        }
    }
}

__device__ __forceinline__ void issue_k_block_n(int La, uint32_t acc, uint32_t nt_cols, uint32_t sa, uint32_t sb,
                                                uint32_t idesc, uint32_t first_accumulates, int ks_n,
                                                uint32_t a_stride16 = (128 * 128) >> 4)
{
    switch (La) {
    case 1: issue_k_block<1>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    case 2: issue_k_block<2>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    case 3: issue_k_block<3>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    case 4: issue_k_block<4>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    case 5: issue_k_block<5>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    case 6: issue_k_block<6>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    case 7: issue_k_block<7>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    case 8: issue_k_block<8>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    default: issue_k_block<9>(acc, nt_cols, sa, sb, idesc, first_accumulates, ks_n, a_stride16); break;
    }
}

// Merged dual accumulation, second part only: limb i of A against the lowest E - i limb tiles of the B
// stack lands on diagonals i .. E-1 of the extra set (a handful of MMAs per tile, so a plain loop).
__device__ __forceinline__ void issue_extra_block(int La, int E, uint32_t acc_extra, uint32_t nt_cols, uint32_t sa,
                                                  uint32_t sb, uint32_t idesc, bool opens_set, int ks_n)
{
    for (int ks = 0; ks < ks_n; ++ks) {
        for (int i = 0; i < La && i < E; ++i) {
            const uint32_t n_i = (uint32_t)(E - i) * nt_cols;
            const uint32_t idesc_i = (idesc & ~(0x3Fu << 17)) | ((n_i >> 3) << 17);
            const uint64_t adesc = smem_desc_sw128(sa + (uint32_t)i * (128u * 128u)) + (uint64_t)(ks * 2);
            const uint64_t bdesc = smem_desc_sw128(sb) + (uint64_t)(ks * 2);
            umma_i8(acc_extra + (uint32_t)i * nt_cols, adesc, bdesc, idesc_i, (opens_set && ks == 0 && i == 0) ? 0u : 1u);
        }
    }
}

// ------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------

constexpr int kTileM = 128;
constexpr int kBlockK = 128;   // bytes (= int8 elements) of K per pipeline stage
constexpr int kEpiWarps = 8;            // one-tile kernel: two warps per tensor-memory lane quarter, half the columns each
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kSplitTilesMax = 128;       // split-K: output tiles per launch (one arrival counter each)
constexpr size_t kSplitHeader = 1024;     // bytes reserved for the counters in front of the partial sums

struct LimbParams {
    int La, Lb, NT, stages;
    int kblocks;
    int64_t k_extent;         // K bytes per plane row (0 = unknown): a partial last K block issues fewer MMAs
    uint32_t tmem_cols;       // power of two >= (La + Lb - 1) * NT
    int64_t M, N, batches;
    int64_t a_rows_per_limb;  // batches * M
    int64_t b_rows_per_limb;  // nbB * b_batch_rows
    int64_t b_batch_rows;     // rows between the batches of B: N, or the capacity of resident cache planes
    int b_batched;            // 1: B differs per batch
    int64_t* C;
    int64_t* R;
    int64_t c_sz, c_sm;
    int64_t addend;
    int shift, r_legacy;
    int* error_flag;          // host-mapped
    int fits64;               // |addend + sum| < 2^62 proven on the host: one-word epilogue
    int64_t m_tiles, n_tiles, panel_m;   // tile raster (see the kernel)
    // dual accumulation (persistent kernel): K blocks from k_switch on feed a second set of
    // diagonals with its own addend and shift; the epilogue adds the two shifted sums
    int k_switch, shift2;
    int64_t addend2;
    int nbuf;                 // accumulator buffers in tensor memory: 2 (ping-pong) or 1
    // one buffer holding two sets: the epilogue hands the first set back as soon as it is drained,
    // so the next tile's first-set MMAs overlap the rest of the epilogue
    int split_release;
    // merged dual accumulation: the second part's operand A was scaled by 2^(shift - shift2) while it
    // was split, so both parts accumulate into ONE set of diagonals T = S1 + 2^(shift-shift2) S2; the
    // second part's lowest merged_E diagonals (all that matter modulo 2^shift) are accumulated once
    // more into a small extra set right of the main one, which yields the carry that separates
    // floor((S1+a1)/2^shift) + floor((S2+a2)/2^shift2) from floor((T+a1+2^(shift-shift2) a2)/2^shift)
    int merged_E;
    // the epilogue that folds the diagonals as they arrive, hands tensor memory back before its
    // arithmetic and stores from registers (epilogue_merged); set with the merged score mode.  (The same
    // epilogue on one plain set in a single 64-column buffer measured slower than the one-tile kernel
    // with 80-column tiles on P.KV: 8.6 against 8.0 ms.)
    int fold_epilogue;
    unsigned backoff;         // 1: waiting warps sleep between polls (see mbar_wait), 0: they poll back to back
    // optional wait accounting (null = off): [0] MMA warp cycles waiting for operand stages, [1] for
    // free accumulators, [2] MMA warp total, [3] first epilogue warp cycles waiting for accumulators,
    // [4] its total, summed over CTAs
    unsigned long long* wait_cycles;
    // causal skipping (optional): rows are (s, h) pairs with skip_H heads per sequence position s.
    //  skip_tiles: output tiles whose every column is beyond skip_start + s are not computed
    //              (the attention scores of masked positions are left unwritten);
    //  skip_k:     K blocks beyond skip_start + s_max + 1 are not accumulated (P . KV with P = 0 there)
    int skip_tiles, skip_k;
    int64_t skip_H, skip_start;
    // La is an upper bound when a_absmax is set: the kernel derives the limb count actually
    // needed from the range the split pass measured and skips the all-zero upper limbs
    const unsigned long long* a_absmax;
    unsigned* overflow_flag;
    // grouped mode: A is one flat [M, K] matrix whose 128-row tiles each belong to one group
    // (expert); tile_group[tile] selects the B batch, a negative entry skips the tile
    const int* tile_group;
    // grouped mode: per-group shift, group_shift[2g] for columns < n_split and [2g+1] from
    // n_split on (n_split a multiple of 8); null = the uniform shift above
    const int* group_shift;
    int64_t n_split;
    // epilogue extension: v = quotient; v += addin[m][n]; v = floor(v * ep_mul / ep_div);
    // rows are (s, h) pairs with causal_H heads: v += mask_value where n > causal_start + s
    const int64_t* addin;
    int64_t ep_mul, ep_div;
    int64_t causal_H, causal_start, mask_value;
    // split-K (one-tile kernel, few output tiles, deep K: the weight-streaming shapes of decode).
    // ksplit CTAs share an output tile, each accumulates kb_per_split K blocks; they add their shares of
    // the sums (integers: exact in any order) to partial[tile][word][column][row], and the CTA that
    // arrives last at tile_counter[tile] reads the totals back, shifts and stores them and leaves both
    // arrays zeroed for the next launch.
    int ksplit, kb_per_split;
    unsigned long long* partial;
    unsigned* tile_counter;
    // one-tile kernel, M <= 64 or grouped tiles with at most that many rows each: the A box holds only
    // a_box_rows (32 or 64) of the MMA's 128 rows, and the limb tiles lie that close together in shared
    // memory.  The MMA still reads 128 rows per limb; what it finds beyond the box (the next limb, the B stack)
    // lands in accumulator rows nobody stores (M <= 64) or that are zeroed before the epilogue reads them
    // (grouped tiles: their padding rows are stored, as the result of zero rows).  0 = 128.
    int a_box_rows;
};

__device__ __forceinline__ int limbs_needed_dev(unsigned long long maxabs)
{
    unsigned long long cover = 0;
    for (int L = 1; L <= 8; ++L) {
        cover = cover * 256ull + 127ull;
        if (maxabs <= cover) return L;
    }
    return 9;
}

__device__ __forceinline__ int64_t floor_div_i64(int64_t a, int64_t b)
{
    int64_t q = a / b, r = a % b;
    return (r != 0 && ((r < 0) != (b < 0))) ? q - 1 : q;
}

// a * b + c with 32-bit signed factors and a 64-bit accumulator in one instruction
__device__ __forceinline__ int64_t mad_wide(int32_t a, int32_t b, int64_t c)
{
    int64_t d;
    asm("mad.wide.s32 %0, %1, %2, %3;" : "=l"(d) : "r"(a), "r"(b), "l"(c));
    return d;
}

// four consecutive diagonals -> a0 + a1 * 2^8 + a2 * 2^16 + a3 * 2^24 (|a| < 2^31: fits 56 bits)
__device__ __forceinline__ int64_t four_diagonals(int32_t a0, int32_t a1, int32_t a2, int32_t a3)
{
    return mad_wide(a3, 1 << 24, mad_wide(a2, 1 << 16, mad_wide(a1, 1 << 8, (int64_t)a0)));
}

// One chunk (CH = 8 or 4 columns) of a tile whose sum fits 64 bits, diagonal count known at
// compile time: every diagonal is fetched before the single wait and no absent diagonal costs anything.
struct NoHook {
    __device__ __forceinline__ void operator()() const {}
};

// `after_loads` runs once the accumulators are in registers (before the arithmetic): the place to
// hand the tensor-memory columns back
template <int DD, int CH, typename Hook>
__device__ __forceinline__ void gather64_n(uint32_t taddr, int NT, int64_t addend, int64_t (&s)[CH],
                                           const Hook& after_loads)
{
    int32_t a[DD][CH];
#pragma unroll
    for (int d = 0; d < DD; ++d) tmem_ldn(taddr + (uint32_t)(d * NT), a[d]);
    tmem_ld_wait();
    after_loads();
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        int64_t lo = mad_wide(a[0][c], 1, addend);
        if (DD > 1) lo = mad_wide(a[DD > 1 ? 1 : 0][c], 1 << 8, lo);
        if (DD > 2) lo = mad_wide(a[DD > 2 ? 2 : 0][c], 1 << 16, lo);
        if (DD > 3) lo = mad_wide(a[DD > 3 ? 3 : 0][c], 1 << 24, lo);
        if (DD > 4) {
            // diagonals 4 and 5 only reach the upper word
            uint32_t hi = (uint32_t)a[DD > 4 ? 4 : 0][c];
            if (DD > 5) hi += (uint32_t)a[DD > 5 ? 5 : 0][c] << 8;
            lo = (int64_t)((uint64_t)lo + ((uint64_t)hi << 32));
        }
        s[c] = lo;
    }
}

// false when the diagonal count has no compiled specialisation (caller uses the generic loop)
template <int CH, typename Hook>
__device__ __forceinline__ bool gather64(int D, uint32_t taddr, int NT, int64_t addend, int64_t (&s)[CH],
                                         const Hook& h)
{
    switch (D) {
    case 1: gather64_n<1, CH>(taddr, NT, addend, s, h); return true;
    case 2: gather64_n<2, CH>(taddr, NT, addend, s, h); return true;
    case 3: gather64_n<3, CH>(taddr, NT, addend, s, h); return true;
    case 4: gather64_n<4, CH>(taddr, NT, addend, s, h); return true;
    case 5: gather64_n<5, CH>(taddr, NT, addend, s, h); return true;
    case 6: gather64_n<6, CH>(taddr, NT, addend, s, h); return true;
    default: return false;
    }
}

struct EpilogueCtx {
    uint32_t tq;
    int D, NT, group;
    int nc_begin, nc_end;     // columns of the tile this warp handles (multiples of 8)
    int64_t m, n0, z;
    int64_t* crow;
    int64_t* rrow;
    bool row_ok, vec_ok;
};

// floor(v * 94 / 695) for |v| < 2^42 (MLA's softmax scale, model.py:897): double estimate of the
// quotient (the product is below 2^49, exact in a double; the estimate is within one of the floor),
// exact remainder correction.  One straight-line path for every realistic score.
// the tier for |v| >= 2^31 (out of line: the epilogues that inline the 32-bit tier sixteen times per thread
// must stay small enough for the instruction cache)
__device__ __noinline__ int64_t scale_94_695_wide(int64_t v)
{
    const int64_t t = v * 94;
    int64_t q = __double2ll_rd((double)t * (1.0 / 695.0));
    int64_t r = t - q * 695;
    if (r < 0) { --q; r += 695; }
    if (r >= 695) ++q;
    return q;
}

__device__ __forceinline__ int64_t scale_94_695(int64_t v)
{
    if (v == (int64_t)(int32_t)v) {
        // 32-bit tier: q0 = floor(v * ceil(94 * 2^32 / 695) / 2^32) is the floor or one above it
        // (the constant errs by less than 1, so the product by less than |v| / 2^32 < 1/2); the
        // remainder, exact modulo 2^32 because it is small, tells which
        const int32_t x = (int32_t)v;
        int32_t q = __mulhi(x, 580902052);
        int32_t r = (int32_t)((uint32_t)x * 94u - (uint32_t)q * 695u);
        if (r < 0) { --q; r += 695; }
        if (r >= 695) ++q;
        return (int64_t)q;
    }
    return scale_94_695_wide(v);
}

// sequence position of row m when rows are (s, h) pairs with H heads per position; row counts are below
// 2^31 in practice, so the division runs in 32 bits (a 64-bit division costs a few hundred instructions
// per thread and tile)
__device__ __forceinline__ int64_t seq_row(int64_t m, int64_t H)
{
    if (((uint64_t)m | (uint64_t)H) >> 32) return m / H;
    return (int64_t)((uint32_t)m / (uint32_t)H);
}

// floor(v * mul / div) with a wrapping product, any operands (out of line: rare)
__device__ __noinline__ int64_t scale_general(int64_t v, int64_t mul, int64_t div)
{
    return floor_div_i64((int64_t)((uint64_t)v * (uint64_t)mul), div);
}

// element-wise tail of the attention scores: v += *arow (the addin element, if any);
// v = floor(v * mul / div); causal mask for column n of sequence row srow
__device__ __forceinline__ int64_t score_tail(const LimbParams& p, int64_t v, const int64_t* arow,
                                              int64_t n, int64_t srow)
{
    if (arow) v = (int64_t)((uint64_t)v + (uint64_t)*arow);
    if (p.ep_div) {
        if (p.ep_mul == 94 && p.ep_div == 695 && (uint64_t)(v + (1ll << 42)) < (uint64_t)(1ll << 43))
            v = scale_94_695(v);
        else
            v = scale_general(v, p.ep_mul, p.ep_div);
    }
    if (p.causal_H && n > p.causal_start + srow) v = (int64_t)((uint64_t)v + (uint64_t)p.mask_value);
    return v;
}

// shift, remainder, element-wise tail and store of one 8-column chunk whose sums are complete
template <bool FITS64>
__device__ __forceinline__ void finish_chunk(const LimbParams& p, const EpilogueCtx& e, int nc, const int64_t (&s64)[8],
                                             const i128w (&sum)[8], bool tail, const int64_t* arow, int64_t srow)
{
        int64_t cv[8], rv[8];
        const int64_t n = e.n0 + nc;
        const int shift = p.group_shift ? p.group_shift[2 * e.group + (n >= p.n_split ? 1 : 0)] : p.shift;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (FITS64) {
                cv[c] = shift >= 63 ? (s64[c] >> 63) : (s64[c] >> shift);
                if (e.rrow) rv[c] = gemm_remainder(make_i128(s64[c]), shift, p.r_legacy);
            } else {
                cv[c] = sar128_lo(sum[c], shift);
                if (e.rrow) rv[c] = gemm_remainder(sum[c], shift, p.r_legacy);
            }
        }
        if (tail) {
            int64_t av[8];
            if (arow) {
                if (e.vec_ok && n + 8 <= p.N && ((((uintptr_t)p.addin) & 15) == 0)) {
#pragma unroll
                    for (int c = 0; c < 8; c += 2) {
                        const longlong2 t = *reinterpret_cast<const longlong2*>(arow + n + c);
                        av[c] = t.x; av[c + 1] = t.y;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 8; ++c) av[c] = (n + c < p.N) ? arow[n + c] : 0;
                }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c)
                if (n + c < p.N) cv[c] = score_tail(p, cv[c], arow ? &av[c] : nullptr, n + c, srow);
        }
        if (e.vec_ok && n + 8 <= p.N) {
#pragma unroll
            for (int c = 0; c < 8; c += 2) {
                *reinterpret_cast<longlong2*>(e.crow + n + c) = make_longlong2(cv[c], cv[c + 1]);
                if (e.rrow) *reinterpret_cast<longlong2*>(e.rrow + n + c) = make_longlong2(rv[c], rv[c + 1]);
            }
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c)
                if (n + c < p.N) {
                    e.crow[n + c] = cv[c];
                    if (e.rrow) e.rrow[n + c] = rv[c];
                }
        }
}

// Reads the diagonals of one 128 x NT tile back from tensor memory, recombines them
// (sum_d acc_d * 2^(8 d)), shifts and stores.  FITS64: the launcher proved |sum| < 2^62, so the
// recombination runs in one 64-bit word instead of two.
// sum_d acc_d * 2^(8 d) + addend of one 8-column chunk, diagonals read back from tensor memory
template <bool FITS64>
__device__ __forceinline__ void gather_chunk(const EpilogueCtx& e, int nc, int64_t addend, int64_t (&s64)[8],
                                             i128w (&sum)[8])
{
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        if (FITS64) s64[c] = addend;
        else sum[c] = make_i128(addend);
    }
    for (int d0 = 0, g = 0; d0 < e.D; d0 += 4, ++g) {
        int32_t a[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (d0 + j < e.D) tmem_ld8(e.tq + (uint32_t)((d0 + j) * e.NT + nc), a[j]);
            else {
#pragma unroll
                for (int c = 0; c < 8; ++c) a[j][c] = 0;
            }
        }
        tmem_ld_wait();
        if (g >= 4) continue;         // diagonals from 16 on only reach bits beyond the 128 kept
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int64_t v = four_diagonals(a[0][c], a[1][c], a[2][c], a[3][c]);
            if (FITS64) {
                // the sum fits 62 bits, so it has at most 6 diagonals: g <= 1 here
                s64[c] += g ? (int64_t)((uint64_t)v << 32) : v;
            } else {
                i128w t;  // v * 2^(32 g)
                if (g == 0) { t.lo = (uint64_t)v; t.hi = v >> 63; }
                else if (g == 1) { t.lo = (uint64_t)v << 32; t.hi = v >> 32; }
                else if (g == 2) { t.lo = 0; t.hi = v; }
                else { t.lo = 0; t.hi = (int64_t)((uint64_t)v << 32); }
                sum[c] = add128(sum[c], t);
            }
        }
    }
}

template <bool FITS64>
__device__ __forceinline__ void epilogue_tile(const LimbParams& p, const EpilogueCtx& e)
{
    const bool tail = p.addin || p.ep_div || p.causal_H;
    const int64_t* arow = p.addin ? p.addin + e.z * p.c_sz + e.m * p.c_sm : nullptr;
    const int64_t srow = p.causal_H ? seq_row(e.m, p.causal_H) : 0;
    for (int nc = e.nc_begin; nc < e.nc_end; nc += 8) {
        i128w sum[8];
        int64_t s64[8];
        gather_chunk<FITS64>(e, nc, p.addend, s64, sum);
        if (!e.row_ok) continue;
        finish_chunk<FITS64>(p, e, nc, s64, sum, tail, arow, srow);
    }
}

// The same for sums that fit 62 bits with the diagonal count known at compile time (DD <= 6), software
// pipelined: the accumulators of the next CW columns are requested before the current ones are shifted and
// stored, so the tensor-memory round trip hides behind the arithmetic and the stores of the previous step.
template <int DD, int CW>
__device__ __forceinline__ void fetch_cols(const EpilogueCtx& e, int nc, int32_t (&a)[DD][CW])
{
#pragma unroll
    for (int d = 0; d < DD; ++d) tmem_ldn(e.tq + (uint32_t)(d * e.NT + nc), a[d]);
}

// tot != nullptr: split-K, the recombined sums (no addend) are added to the tile's totals instead
template <int DD, int CW>
__device__ __forceinline__ void finish_cols(const LimbParams& p, const EpilogueCtx& e, int nc, const int32_t (&a)[DD][CW],
                                            bool tail, const int64_t* arow, int64_t srow, unsigned long long* tot)
{
    if (!e.row_ok) return;
    const int64_t addend = tot ? 0 : p.addend;
#pragma unroll
    for (int h = 0; h < CW; h += 8) {
        int64_t s64[8];
        i128w unused[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            int64_t lo = mad_wide(a[0][h + c], 1, addend);
            if (DD > 1) lo = mad_wide(a[DD > 1 ? 1 : 0][h + c], 1 << 8, lo);
            if (DD > 2) lo = mad_wide(a[DD > 2 ? 2 : 0][h + c], 1 << 16, lo);
            if (DD > 3) lo = mad_wide(a[DD > 3 ? 3 : 0][h + c], 1 << 24, lo);
            if (DD > 4) {
                uint32_t hi = (uint32_t)a[DD > 4 ? 4 : 0][h + c];
                if (DD > 5) hi += (uint32_t)a[DD > 5 ? 5 : 0][h + c] << 8;
                lo = (int64_t)((uint64_t)lo + ((uint64_t)hi << 32));
            }
            s64[c] = lo;
        }
        if (tot) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
                if (s64[c]) atomicAdd(tot + (int64_t)(nc + h + c) * kTileM, (unsigned long long)s64[c]);
        } else
            finish_chunk<true>(p, e, nc + h, s64, unused, tail, arow, srow);
    }
}

template <int DD, int CW>
__device__ __forceinline__ void epilogue_tile_pipelined(const LimbParams& p, const EpilogueCtx& e, unsigned long long* tot)
{
    const bool tail = p.addin || p.ep_div || p.causal_H;
    const int64_t* arow = p.addin ? p.addin + e.z * p.c_sz + e.m * p.c_sm : nullptr;
    const int64_t srow = p.causal_H ? seq_row(e.m, p.causal_H) : 0;
    int32_t a0[DD][CW], a1[DD][CW];
    fetch_cols<DD, CW>(e, e.nc_begin, a0);
    for (int nc = e.nc_begin; nc < e.nc_end; nc += 2 * CW) {
        tmem_ld_wait();
        const bool more1 = nc + CW < e.nc_end;
        if (more1) fetch_cols<DD, CW>(e, nc + CW, a1);
        finish_cols<DD, CW>(p, e, nc, a0, tail, arow, srow, tot);
        if (more1) {
            tmem_ld_wait();
            if (nc + 2 * CW < e.nc_end) fetch_cols<DD, CW>(e, nc + 2 * CW, a0);
            finish_cols<DD, CW>(p, e, nc + CW, a1, tail, arow, srow, tot);
        }
    }
}

// false when the tile has no compiled pipelined epilogue (the caller then uses epilogue_tile)
__device__ __forceinline__ bool epilogue_tile_fast(const LimbParams& p, const EpilogueCtx& e, unsigned long long* tot = nullptr)
{
    if (!p.fits64) return false;
    switch (e.D) {
    case 2: epilogue_tile_pipelined<2, 8>(p, e, tot); return true;
    case 3: epilogue_tile_pipelined<3, 8>(p, e, tot); return true;
    case 4: epilogue_tile_pipelined<4, 8>(p, e, tot); return true;
    case 5: epilogue_tile_pipelined<5, 8>(p, e, tot); return true;
    case 6: epilogue_tile_pipelined<6, 8>(p, e, tot); return true;
    default: return false;
    }
}

// Split-K.  A CTA's share of a tile's sums, recombined from its diagonals, is added to the tile's totals in
// global memory, totals[word][column][row of the tile]: one 64-bit word when the sum fits 62 bits, else the low
// 55 bits and the rest (the launcher checked that the rest fits a word; sums of up to 256 shares of 55 bits
// stay below 2^63).  Integer sums: exact in any order.
constexpr int kSplitLowBits = 55;
template <bool FITS64>
__device__ __forceinline__ void add_partials_tile(const LimbParams& p, const EpilogueCtx& e, unsigned long long* tot)
{
    for (int nc = e.nc_begin; nc < e.nc_end; nc += 8) {
        i128w sum[8];
        int64_t s64[8];
        gather_chunk<FITS64>(e, nc, 0, s64, sum);
        if (!e.row_ok) continue;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            unsigned long long* w = tot + (int64_t)(nc + c) * kTileM;
            if (FITS64) {
                if (s64[c]) atomicAdd(w, (unsigned long long)s64[c]);
            } else {
                const unsigned long long lo = sum[c].lo & ((1ull << kSplitLowBits) - 1ull);
                const unsigned long long hi = (unsigned long long)sar128_lo(sum[c], kSplitLowBits);
                if (lo) atomicAdd(w, lo);
                if (hi) atomicAdd(w + (int64_t)e.NT * kTileM, hi);
            }
        }
    }
}

// The last CTA of a split-K tile: one 8-column chunk of one row from the totals.  Every word is requested
// before the first is used (one round trip to L2 per chunk) and written back as zero, the state the next
// launch expects.
template <bool FITS64>
__device__ __forceinline__ void epilogue_totals_chunk(const LimbParams& p, const EpilogueCtx& e, unsigned long long* col0,
                                                      int nc)
{
    if (!e.row_ok) return;
    unsigned long long lo[8], hi[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        lo[c] = __ldcg(col0 + (int64_t)(nc + c) * kTileM);
        hi[c] = FITS64 ? 0ull : __ldcg(col0 + (int64_t)(e.NT + nc + c) * kTileM);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        __stcg(col0 + (int64_t)(nc + c) * kTileM, 0ull);
        if (!FITS64) __stcg(col0 + (int64_t)(e.NT + nc + c) * kTileM, 0ull);
    }
    i128w sum[8];
    int64_t s64[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        if (FITS64) s64[c] = (int64_t)lo[c] + p.addend;
        else {
            i128w t;       // hi * 2^55 + lo + addend
            t.lo = hi[c] << kSplitLowBits;
            t.hi = (int64_t)hi[c] >> (64 - kSplitLowBits);
            i128w l;
            l.lo = lo[c]; l.hi = 0;
            sum[c] = add128(add128(t, l), make_i128(p.addend));
        }
    }
    const bool tail = p.addin || p.ep_div || p.causal_H;
    const int64_t* arow = p.addin ? p.addin + e.z * p.c_sz + e.m * p.c_sm : nullptr;
    const int64_t srow = p.causal_H ? seq_row(e.m, p.causal_H) : 0;
    finish_chunk<FITS64>(p, e, nc, s64, sum, tail, arow, srow);
}

__global__ void __launch_bounds__(kThreads, 1)
limb_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const LimbParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * 8 + 2];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_last;

    const long long t_cta0 = p.wait_cycles ? clock64() : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int group = 0;
    if (p.tile_group) {
        group = p.tile_group[blockIdx.x];
        if (group < 0) {
            // unused row tile (uniform for the CTA, before any barrier or allocation): its output
            // rows are defined as zero so that later passes over the whole buffer see clean data
            const int64_t r0 = (int64_t)blockIdx.x * kTileM, c0 = (int64_t)blockIdx.y * p.NT;
            for (int i = threadIdx.x; i < kTileM * p.NT; i += kThreads) {
                const int64_t r = r0 + i / p.NT, c = c0 + i % p.NT;
                if (r < p.M && c < p.N) p.C[r * p.c_sm + c] = 0;
            }
            return;
        }
    }
    int La = p.La;
    if (p.a_absmax) {
        const int need = limbs_needed_dev(*p.a_absmax);
        if (need > La) {
            if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) *p.overflow_flag = 1u;
        } else La = need;
    }
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_limb_bytes = (uint32_t)(p.a_box_rows ? p.a_box_rows : kTileM) * kBlockK;
    const uint32_t a_bytes = (uint32_t)p.La * a_limb_bytes;
    const uint32_t b_bytes = (uint32_t)p.Lb * p.NT * kBlockK;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    const uint32_t bar_full = smem_u32(&bars[0]);
    const uint32_t bar_empty = smem_u32(&bars[8]);
    const uint32_t bar_zeroed = smem_u32(&bars[16]);
    const uint32_t bar_accum = smem_u32(&bars[17]);

    // split-K: consecutive CTAs share an output tile and take consecutive K slices of it
    int64_t bx = blockIdx.x;
    int split = 0;
    if (p.ksplit > 1) { split = (int)(bx % p.ksplit); bx /= p.ksplit; }
    // tiles are walked panel by panel: panel_m row tiles x all column tiles, rows fastest, so the
    // A tiles of a panel and the B tile in flight stay in L2 while the panel is swept
    int64_t m_tile, n_tile;
    if (p.tile_group) { m_tile = blockIdx.x; n_tile = blockIdx.y; }
    else {
        const int64_t per_panel = p.panel_m * p.n_tiles;
        const int64_t panel = bx / per_panel;
        const int64_t within = bx - panel * per_panel;
        const int64_t rows_here = (p.m_tiles - panel * p.panel_m < p.panel_m) ? p.m_tiles - panel * p.panel_m
                                                                              : p.panel_m;
        n_tile = within / rows_here;
        m_tile = panel * p.panel_m + (within - n_tile * rows_here);
        if (n_tile >= p.n_tiles) return;   // cannot happen; keeps the indices in range
    }
    const int64_t m0 = m_tile * kTileM;
    const int64_t n0 = n_tile * p.NT;
    const int64_t z = blockIdx.z;
    int kb_end = p.kblocks;
    int kb_begin = 0;
    if (p.ksplit > 1) {
        kb_begin = split * p.kb_per_split;
        kb_end = kb_begin + p.kb_per_split < p.kblocks ? kb_begin + p.kb_per_split : p.kblocks;
    }
    if (p.skip_k) {
        // rows of this tile see nothing beyond column skip_start + s_max: later K blocks are all zero
        int64_t last_row = m0 + kTileM - 1;
        if (last_row > p.M - 1) last_row = p.M - 1;
        const int64_t need = (p.skip_start + last_row / p.skip_H + 1 + kBlockK - 1) / kBlockK;
        if (need < kb_end) kb_end = need < 1 ? 1 : (int)need;
    }
    const int D = La + p.Lb - 1;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_zeroed, kEpiWarps);
        mbar_init(bar_accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    volatile int* abort_flag = &s_abort;

    if (warp == 0) {
        // ---- TMA producer -------------------------------------------------------------
        if (lane == 0) {
            const int64_t zb = p.tile_group ? group : (p.b_batched ? z : 0);
            const uint32_t tx_bytes = (uint32_t)La * a_limb_bytes + b_bytes;
            int armed = 0;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                const int it = kb - kb_begin;
                const int s = it % p.stages;
                const uint32_t par = ((it / p.stages) & 1) ^ 1;
                if (!mbar_wait(bar_empty + 8 * s, par, abort_flag)) break;
                const uint32_t full = bar_full + 8 * s;
                mbar_expect_tx(full, tx_bytes);
                const uint32_t sa = smem_base + s * stage_bytes;
                const uint32_t sb = sa + a_bytes;
                for (int i = 0; i < La; ++i)
                    tma_load_2d(sa + i * a_limb_bytes, &tmA, kb * kBlockK,
                                (int)(i * p.a_rows_per_limb + z * p.M + m0), full);
                for (int j = 0; j < p.Lb; ++j)
                    tma_load_2d(sb + j * (p.NT * kBlockK), &tmB, kb * kBlockK,
                                (int)(j * p.b_rows_per_limb + zb * p.b_batch_rows + n0), full);
                armed = it + 1;
            }
            if (*abort_flag) {
                // leave no copy in flight: wait (bounded) for every stage that was armed and
                // that no consumer waited for
                for (int i = (armed > p.stages ? armed - p.stages : 0); i < armed; ++i)
                    for (uint32_t it = 0; it < kSpinLimit; ++it)
                        if (mbar_try(bar_full + 8 * (i % p.stages), (i / p.stages) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ---------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = (2u << 4)                               // int32 accumulators
                                   | (1u << 7) | (1u << 10)                 // signed 8-bit A and B
                                   | ((uint32_t)((p.Lb * p.NT) >> 3) << 17)  // N
                                   | ((uint32_t)(kTileM >> 4) << 24);        // M
            bool ok = mbar_wait(bar_zeroed, 0, abort_flag);
            tc_fence_after();
            for (int kb = kb_begin; ok && kb < kb_end; ++kb) {
                const int it = kb - kb_begin;
                const int s = it % p.stages;
                ok = mbar_wait(bar_full + 8 * s, (it / p.stages) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sa = smem_base + s * stage_bytes;
                issue_k_block_n(La, tmem, (uint32_t)p.NT, sa, sa + a_bytes, idesc, it ? 1u : 0u, kBlockK / 32,
                                a_limb_bytes >> 4);
                umma_commit(bar_empty + 8 * s);
            }
            umma_commit(bar_accum);
        }
    } else {
        // ---- accumulator zeroing, then epilogue -------------------------------------------
        const int q = warp & 3;  // tensor-memory lane quarter this warp may touch
        const int part = (warp - 2) >> 2;                 // which of the quarter's kEpiWarps / 4 warps
        constexpr int kParts = kEpiWarps / 4;
        const uint32_t tq = tmem + ((uint32_t)(q * 32) << 16);
        // the first MMA (limb 0, first K step) overwrites its Lb * NT columns; only the columns the
        // later limbs extend into must start at zero
        for (int c = p.Lb * p.NT + 8 * part; c < D * p.NT; c += 8 * kParts) tmem_st8_zero(tq + (uint32_t)c);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_zeroed);

        const bool prof = p.wait_cycles != nullptr && warp == 2 && lane == 0;
        long long ph0 = prof ? clock64() : 0, ph1 = 0, ph2 = 0, ph3 = 0;
        const bool ok = mbar_wait(bar_accum, 0, abort_flag);
        tc_fence_after();
        if (prof) ph1 = clock64();
        const int64_t m = m0 + q * 32 + lane;
        int64_t* crow = p.C + z * p.c_sz + m * p.c_sm;
        int64_t* rrow = p.R ? p.R + z * p.c_sz + m * p.c_sm : nullptr;
        const bool row_ok = ok && m < p.M;
        const bool beyond_box = p.tile_group && p.a_box_rows && q * 32 >= p.a_box_rows;
        const bool vec_ok = ((((uintptr_t)p.C | (uintptr_t)p.R) & 15) == 0) && ((p.c_sm & 1) == 0) &&
                            ((p.c_sz & 1) == 0);
        EpilogueCtx ec;
        ec.tq = tq; ec.D = D; ec.NT = p.NT; ec.m = m; ec.n0 = n0; ec.z = z; ec.group = group;
        {   // the quarter's warps take consecutive column ranges (multiples of 8)
            const int chunks = p.NT >> 3, per = (chunks + kParts - 1) / kParts;
            ec.nc_begin = 8 * per * part < p.NT ? 8 * per * part : p.NT;
            ec.nc_end = 8 * per * (part + 1) < p.NT ? 8 * per * (part + 1) : p.NT;
        }
        ec.crow = crow; ec.rrow = rrow; ec.row_ok = row_ok; ec.vec_ok = vec_ok;
        if (beyond_box && ok) {
            // padding rows of a grouped tile whose A box stops short of them: the MMAs summed whatever follows
            // the box in shared memory into these lanes.  Every warp clears the columns it is about to read.
            for (int d = 0; d < D; ++d)
                for (int c = ec.nc_begin; c < ec.nc_end; c += 8) tmem_st8_zero(tq + (uint32_t)(d * p.NT + c));
            tmem_st_wait();
        }
        bool finish = ok;
        if (p.ksplit > 1) {
            // add this CTA's share of the sums to the tile's totals (rows beyond M hold nothing)
            const int64_t tile_id = z * (p.m_tiles * p.n_tiles) + bx;
            unsigned long long* tile_tot = p.partial + tile_id * (2ll * p.NT * kTileM);
            if (ok && m0 + q * 32 < p.M) {
                if (!epilogue_tile_fast(p, ec, tile_tot + q * 32 + lane)) {
                    if (p.fits64) add_partials_tile<true>(p, ec, tile_tot + q * 32 + lane);
                    else add_partials_tile<false>(p, ec, tile_tot + q * 32 + lane);
                }
            }
            if (prof) ph2 = clock64();
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
            if (warp == 2 && lane == 0) {
                // a CTA that gave up a wait does not count: the tile then stays unfinished and the
                // error word tells the host
                s_last = 0;
                if (ok) s_last = atomicAdd(p.tile_counter + tile_id, 1u) == (unsigned)(p.ksplit - 1) ? 1 : 0;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
            finish = false;
            if (prof) ph3 = clock64();
            if (s_last) {
                // the last CTA of the tile: every (32-row group, 8-column chunk) of the totals is one unit
                // of work for any of the four warps (the totals are in global memory, not tied to lanes)
                __threadfence();
                if (warp == 2 && lane == 0) p.tile_counter[tile_id] = 0u;
                int64_t rows_here = p.M - m0;
                if (rows_here > kTileM) rows_here = kTileM;
                const int chunks = p.NT >> 3;
                const int units = (int)((rows_here + 31) >> 5) * chunks;
                for (int u = warp - 2; u < units; u += kEpiWarps) {
                    const int rg = u / chunks, nc = (u - rg * chunks) << 3;
                    EpilogueCtx eu = ec;
                    eu.m = m0 + rg * 32 + lane;
                    eu.row_ok = eu.m < p.M;
                    eu.crow = p.C + z * p.c_sz + eu.m * p.c_sm;
                    eu.rrow = p.R ? p.R + z * p.c_sz + eu.m * p.c_sm : nullptr;
                    unsigned long long* col0 = tile_tot + rg * 32 + lane;
                    if (p.fits64) epilogue_totals_chunk<true>(p, eu, col0, nc);
                    else epilogue_totals_chunk<false>(p, eu, col0, nc);
                }
            }
        }
        if (finish) {
            if (!epilogue_tile_fast(p, ec)) {
                if (p.fits64) epilogue_tile<true>(p, ec);
                else epilogue_tile<false>(p, ec);
            }
        }
        if (prof) {
            // longest phase over the CTAs: [8] start -> accumulators complete, [9] partials added, [10] fence and
            // arrival counter, [11] epilogue (last CTA of a tile), [12] CTA lifetime from its first instruction
            const long long ph4 = clock64();
            atomicMax(p.wait_cycles + 8, (unsigned long long)(ph1 - ph0));
            if (p.ksplit > 1) {
                atomicMax(p.wait_cycles + 9, (unsigned long long)(ph2 - ph1));
                atomicMax(p.wait_cycles + 10, (unsigned long long)(ph3 - ph2));
                if (s_last) atomicMax(p.wait_cycles + 11, (unsigned long long)(ph4 - ph3));
            } else
                atomicMax(p.wait_cycles + 11, (unsigned long long)(ph4 - ph1));
            atomicMax(p.wait_cycles + 12, (unsigned long long)(ph4 - t_cta0));
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem, p.tmem_cols);
    if (threadIdx.x == 0 && s_abort) *p.error_flag = 1;
}

// ------------------------------------------------------------------------------------
// persistent variant for shallow K
// ------------------------------------------------------------------------------------
// When K is small (attention scores, per-head projections) a tile's MMAs take a few thousand
// cycles and the prologue and epilogue of a one-tile CTA dominate.  Here one CTA per SM walks
// many tiles: the accumulators are double-buffered in tensor memory so the MMAs of tile t+1
// run while eight epilogue warps drain tile t, the TMA pipeline keeps streaming across tile
// boundaries, and the results leave through a shared-memory staging tile as whole rows
// (coalesced 16-byte stores) instead of one 64-byte fragment per thread.
// threads of the persistent kernel: warp 0 TMA, warp 1 MMA, then EW epilogue warps (8 or 16)
constexpr int persistent_threads(int ew) { return 64 + 32 * ew; }
// shared-memory staging of the epilogue warps for a tile NT columns wide
constexpr size_t persistent_staging(int ew, int nt) { return (size_t)ew * 32 * ((nt / (ew / 4)) * 8 + 16); }

struct TileCoord {
    int64_t z, m0, n0;
    int group;       // grouped mode: the B batch of this row tile (negative: unused tile), else 0
};

__device__ __forceinline__ TileCoord decode_tile(const LimbParams& p, int64_t tile)
{
    // every count here is below 2^31 (checked by the launcher): 32-bit divisions
    const uint32_t mt = (uint32_t)p.m_tiles, nt = (uint32_t)p.n_tiles, pm = (uint32_t)p.panel_m;
    const uint32_t per_batch = mt * nt;
    const uint32_t zz = (uint32_t)tile / per_batch;
    const uint32_t id = (uint32_t)tile - zz * per_batch;
    const uint32_t per_panel = pm * nt;
    const uint32_t panel = id / per_panel;
    const uint32_t within = id - panel * per_panel;
    const uint32_t left = mt - panel * pm;
    const uint32_t rows_here = left < pm ? left : pm;
    const uint32_t n_tile = within / rows_here;
    TileCoord c;
    c.z = zz;
    c.m0 = (int64_t)(panel * pm + (within - n_tile * rows_here)) * kTileM;
    c.n0 = (int64_t)n_tile * p.NT;
    c.group = p.tile_group ? p.tile_group[panel * pm + (within - n_tile * rows_here)] : 0;
    return c;
}

// every column of the tile lies beyond the last unmasked position of every row of the tile
__device__ __forceinline__ bool tile_masked(const LimbParams& p, const TileCoord& c)
{
    int64_t last_row = c.m0 + kTileM - 1;
    if (last_row > p.M - 1) last_row = p.M - 1;
    return c.n0 > p.skip_start + last_row / p.skip_H;
}

// quotients of one chunk of columns: (addend + sum_d acc_d * 2^(8 d)) >> shift, taddr = first column
// of diagonal 0 of the set
template <bool FITS64, int CH, typename Hook>
__device__ __forceinline__ void chunk_quotient(int D, uint32_t taddr, int NT, int64_t addend, int shift,
                                               int64_t (&cv)[CH], const Hook& after_loads)
{
    i128w sum[CH];
    int64_t s64[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        if (FITS64) s64[c] = addend;
        else sum[c] = make_i128(addend);
    }
    const bool done64 = FITS64 && gather64<CH>(D, taddr, NT, addend, s64, after_loads);
    for (int d0 = 0, g = 0; !done64 && d0 < D; d0 += 4, ++g) {
        int32_t a[4][CH];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (d0 + j < D) tmem_ldn(taddr + (uint32_t)((d0 + j) * NT), a[j]);
            else {
#pragma unroll
                for (int c = 0; c < CH; ++c) a[j][c] = 0;
            }
        }
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int64_t v = four_diagonals(a[0][c], a[1][c], a[2][c], a[3][c]);
            if (FITS64) {
                s64[c] += g ? (int64_t)((uint64_t)v << 32) : v;
            } else {
                i128w t;  // v * 2^(32 g)
                if (g == 0) { t.lo = (uint64_t)v; t.hi = v >> 63; }
                else if (g == 1) { t.lo = (uint64_t)v << 32; t.hi = v >> 32; }
                else if (g == 2) { t.lo = 0; t.hi = v; }
                else { t.lo = 0; t.hi = (int64_t)((uint64_t)v << 32); }
                sum[c] = add128(sum[c], t);
            }
        }
        if (d0 + 4 >= D) after_loads();
    }
    const int sh64 = shift >= 63 ? 63 : shift;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        if (FITS64) cv[c] = s64[c] >> sh64;
        else cv[c] = sar128_lo(sum[c], shift);
    }
}

// One epilogue warp: rows 32 q .. 32 q + 31 of the tile, columns [c0, c0 + CW) of it, CH columns per
// step.  With two sets of diagonals the first set is drained completely (its quotients parked in the
// staging rows) before the second is touched; release_bar != 0 hands the first set back to the MMA
// warp at that point, so the next tile's first-set MMAs run under the rest of this epilogue.
template <bool FITS64, int CH>
__device__ __forceinline__ void epilogue_part(const LimbParams& p, uint32_t tq, int D, const TileCoord& tc,
                                              int q, int lane, int c0, int CW, uint8_t* stage, int RS,
                                              int set_cols, uint32_t release_bar)
{
    const int64_t m = tc.m0 + q * 32 + lane;
    const bool tail = p.addin || p.ep_div || p.causal_H;
    const int64_t srow = p.causal_H ? seq_row(m, p.causal_H) : 0;
    const int64_t nbase = tc.n0 + c0;
    const bool vec_ok = ((((uintptr_t)p.C | (uintptr_t)p.addin) & 15) == 0) && ((p.c_sm & 1) == 0) &&
                        ((p.c_sz & 1) == 0);
    // lanes_per_row lanes move one staged row (16 bytes each); several rows per instruction
    int lanes_per_row = 1;
    while (lanes_per_row * 2 < CW) lanes_per_row <<= 1;
    const int rows_per_it = 32 / lanes_per_row;
    const int rl = lane / lanes_per_row, cl = (lane % lanes_per_row) * 2;
    const bool two = p.k_switch != 0;

    if (p.addin) {
        // bring this warp's part of the addin tile in as whole rows; the 16-byte copies are
        // asynchronous (all in flight together), one wait at the end
        for (int r0 = 0; r0 < 32; r0 += rows_per_it) {
            const int r = r0 + rl;
            const int64_t mr = tc.m0 + q * 32 + r;
            if (cl < CW && mr < p.M) {
                const int64_t* src = p.addin + tc.z * p.c_sz + mr * p.c_sm + nbase + cl;
                uint8_t* dst = stage + r * RS + cl * 8;
                if (vec_ok && nbase + cl + 2 <= p.N) {
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src)
                                 : "memory");
                } else {
                    int64_t v0 = 0, v1 = 0;
                    if (nbase + cl < p.N) v0 = src[0];
                    if (nbase + cl + 1 < p.N) v1 = src[1];
                    *reinterpret_cast<longlong2*>(dst) = make_longlong2(v0, v1);
                }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncwarp();
    }

    // hands the first set back: re-zero the columns no first-step MMA initialises, then arrive
    auto release_first = [&]() {
        for (int d = p.Lb; d < D; ++d)
            for (int c = 0; c < CW; c += 4) tmem_st4_zero(tq + (uint32_t)(d * p.NT + c0 + c));
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(release_bar);
    };
    // the first set can go back as soon as the accumulators of this warp's last chunk are in
    // registers, before the arithmetic on them
#pragma unroll 1
    for (int nc = 0; nc < CW; nc += CH) {
        const bool early = two && release_bar && nc + CH >= CW;
        int64_t cv[CH];
        // grouped mode: the shift belongs to the group and to the side of n_split the chunk lies on
        // (n_split and every chunk start are multiples of 4, a chunk never straddles it when CH <= 8)
        const int shift = p.group_shift ? p.group_shift[2 * tc.group + (nbase + nc >= p.n_split ? 1 : 0)] : p.shift;
        if (early) chunk_quotient<FITS64, CH>(D, tq + (uint32_t)(c0 + nc), p.NT, p.addend, shift, cv, release_first);
        else chunk_quotient<FITS64, CH>(D, tq + (uint32_t)(c0 + nc), p.NT, p.addend, shift, cv, NoHook());
        int64_t* srow_ptr = reinterpret_cast<int64_t*>(stage + lane * RS + nc * 8);
        if (tail && !two) {
#pragma unroll
            for (int c = 0; c < CH; ++c)
                cv[c] = score_tail(p, cv[c], p.addin ? srow_ptr + c : nullptr, nbase + nc + c, srow);
        }
#pragma unroll
        for (int c = 0; c < CH; c += 2)
            *reinterpret_cast<longlong2*>(srow_ptr + c) = make_longlong2(cv[c], cv[c + 1]);
    }
    if (two) {
        // second set of diagonals: its own addend and shift, then the two quotients add up
#pragma unroll 1
        for (int nc = 0; nc < CW; nc += CH) {
            int64_t v2[CH];
            int64_t* srow_ptr = reinterpret_cast<int64_t*>(stage + lane * RS + nc * 8);
            chunk_quotient<FITS64, CH>(D, tq + (uint32_t)(set_cols + c0 + nc), p.NT, p.addend2, p.shift2, v2, NoHook());
#pragma unroll
            for (int c = 0; c < CH; c += 2) {
                const longlong2 v1 = *reinterpret_cast<const longlong2*>(srow_ptr + c);
                v2[c] = (int64_t)((uint64_t)v2[c] + (uint64_t)v1.x);
                v2[c + 1] = (int64_t)((uint64_t)v2[c + 1] + (uint64_t)v1.y);
            }
            if (tail) {
#pragma unroll
                for (int c = 0; c < CH; ++c) v2[c] = score_tail(p, v2[c], nullptr, nbase + nc + c, srow);
            }
#pragma unroll
            for (int c = 0; c < CH; c += 2)
                *reinterpret_cast<longlong2*>(srow_ptr + c) = make_longlong2(v2[c], v2[c + 1]);
        }
    }
    __syncwarp();
    // write the staged rows out, whole rows at a time
    {
        int64_t mr = tc.m0 + q * 32 + rl;
        int64_t* dst = p.C + tc.z * p.c_sz + mr * p.c_sm + nbase + cl;
        const uint8_t* src = stage + rl * RS + cl * 8;
        const int64_t dstep = (int64_t)rows_per_it * p.c_sm;
        const int sstep = rows_per_it * RS;
        const bool full2 = vec_ok && nbase + cl + 2 <= p.N;
        for (int r0 = 0; r0 < 32; r0 += rows_per_it, mr += rows_per_it, dst += dstep, src += sstep) {
            if (cl < CW && mr < p.M) {
                const longlong2 v = *reinterpret_cast<const longlong2*>(src);
                if (full2) *reinterpret_cast<longlong2*>(dst) = v;
                else {
                    if (nbase + cl < p.N) dst[0] = v.x;
                    if (nbase + cl + 1 < p.N) dst[1] = v.y;
                }
            }
        }
    }
    __syncwarp();
}

// Epilogue of the merged dual accumulation (one warp: rows 32 q .. 32 q + 31, its CW columns of the
// tile, CW = 8 or 16).  The diagonals are folded into two running values per column as they arrive
// (T' = main sum + both addends in 64 bits, r2 = extra sum + scaled second addend modulo 2^32), one
// tensor-memory load per diagonal, so after D + E short waits everything this warp needs is in
// registers and both sets go straight back to the MMA warp; the quotients
// (T' >> shift) - [T' mod 2^shift < r2 mod 2^shift], the score tail and the stores (each thread writes its
// CW consecutive words of one row as full 32-byte sectors) then run while the next tile's MMAs are
// already under way.
template <int DD, int EE, int CW>
__device__ __forceinline__ void epilogue_merged(const LimbParams& p, uint32_t tq, const TileCoord& tc, int q,
                                                int lane, int c0, int set_cols, uint32_t release_main,
                                                uint32_t release_extra)
{
    int64_t T[CW];
    uint32_t R[EE ? CW : 1];
    // Fewer, fuller round trips to tensor memory while few values are live: the extra diagonals all at
    // once (nothing else is held yet), then main diagonals 0 and 1 together, then one per wait.
    if (EE) {
        int32_t e[EE ? EE : 1][CW];
#pragma unroll
        for (int d = 0; d < EE; ++d) tmem_ldn(tq + (uint32_t)(set_cols + d * p.NT + c0), e[d]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < CW; ++c) {
            uint32_t r = (uint32_t)e[0][c] + (uint32_t)p.addend2;
#pragma unroll
            for (int d = 1; d < EE; ++d) r += (uint32_t)e[d][c] << (8 * d);
            R[c] = r;
        }
    }
    {
        int32_t a0[CW], a1[CW];
        tmem_ldn(tq + (uint32_t)c0, a0);
        if (DD > 1) tmem_ldn(tq + (uint32_t)(p.NT + c0), a1);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < CW; ++c) {
            T[c] = mad_wide(a0[c], 1, p.addend);
            if (DD > 1) T[c] = mad_wide(a1[c], 1 << 8, T[c]);
        }
    }
#pragma unroll
    for (int d = 2; d < DD; ++d) {
        int32_t a[CW];
        tmem_ldn(tq + (uint32_t)(d * p.NT + c0), a);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < CW; ++c) {
            if (d < 4) T[c] = mad_wide(a[c], 1 << (8 * (d < 4 ? d : 0)), T[c]);
            else T[c] = (int64_t)((uint64_t)T[c] + ((uint64_t)(uint32_t)a[c] << (8 * d)));
        }
    }
    // re-zero the main columns no first-step MMA initialises, hand both sets back
    for (int d = p.Lb; d < DD; ++d)
        for (int c = 0; c < CW; c += 8) tmem_st8_zero(tq + (uint32_t)(d * p.NT + c0 + c));
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
        mbar_arrive(release_main);
        if (EE) mbar_arrive(release_extra);
    }

    const int64_t m = tc.m0 + q * 32 + lane;
    const int64_t srow = p.causal_H ? seq_row(m, p.causal_H) : 0;
    const int64_t nbase = tc.n0 + c0;
    const int sh = p.shift >= 63 ? 63 : p.shift;
    const uint32_t mask = EE ? (1u << p.shift) - 1u : 0u;
    const bool tail = p.ep_div || p.causal_H;
    // each thread owns CW consecutive words of one output row: 32-byte stores (one full sector each)
    int64_t* crow = p.C + tc.z * p.c_sz + m * p.c_sm + nbase;
    const bool wide_ok = ((((uintptr_t)p.C) & 31) == 0) && ((p.c_sm & 3) == 0) && ((p.c_sz & 3) == 0) &&
                         nbase + CW <= p.N;
    if (m < p.M) {
#pragma unroll
        for (int c = 0; c < CW; c += 4) {
            int64_t o[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const int64_t t = T[c + h];
                int64_t v = t >> sh;
                if (EE) v -= (((uint32_t)t & mask) < (R[EE ? c + h : 0] & mask) ? 1 : 0);
                o[h] = tail ? score_tail(p, v, nullptr, nbase + c + h, srow) : v;
            }
            if (wide_ok) {
                asm volatile("st.global.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(crow + c), "l"(o[0]), "l"(o[1]),
                             "l"(o[2]), "l"(o[3])
                             : "memory");
            } else {
#pragma unroll
                for (int h = 0; h < 4; ++h)
                    if (nbase + c + h < p.N) crow[c + h] = o[h];
            }
        }
    }
}

// false when the shape has no compiled specialisation
template <int CW>
__device__ __forceinline__ bool epilogue_merged_dispatch(const LimbParams& p, int D, uint32_t tq, const TileCoord& tc,
                                                         int q, int lane, int c0, int set_cols, uint32_t rel_main,
                                                         uint32_t rel_extra)
{
#define ZKDS_EM(DD, EE) epilogue_merged<DD, EE, CW>(p, tq, tc, q, lane, c0, set_cols, rel_main, rel_extra); return true
    if (p.merged_E == 3) {
        switch (D) {
        case 3: ZKDS_EM(3, 3);
        case 4: ZKDS_EM(4, 3);
        case 5: ZKDS_EM(5, 3);
        case 6: ZKDS_EM(6, 3);
        default: return false;
        }
    }
#undef ZKDS_EM
    return false;
}

template <int EW>
__global__ void __launch_bounds__(persistent_threads(EW), 1)
limb_gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                            const LimbParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * 8 + 4];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int La = p.La;
    if (p.a_absmax) {
        const int need = limbs_needed_dev(*p.a_absmax);
        if (need > La) {
            if (threadIdx.x == 0 && blockIdx.x == 0) *p.overflow_flag = 1u;
        } else La = need;
    }
    const int D = La + p.Lb - 1;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_bytes = (uint32_t)p.La * kTileM * kBlockK;
    const uint32_t b_bytes = (uint32_t)p.Lb * p.NT * kBlockK;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    const uint32_t bar_full = smem_u32(&bars[0]);
    const uint32_t bar_empty = smem_u32(&bars[8]);
    const uint32_t bar_tfull = smem_u32(&bars[16]);    // [2]: accumulators of a tile complete
    // [2]: buffer b drained and re-zeroed; with split_release (one buffer, two sets) [0] is the
    // first set and [1] the second
    const uint32_t bar_tempty = smem_u32(&bars[18]);
    const int set_cols = (p.La + p.Lb - 1) * p.NT;     // one set of diagonals
    const int nsets = p.k_switch ? 2 : 1;
    const int buf_cols = nsets * set_cols;             // spacing of the two accumulator buffers
    const int64_t n_tiles_total = p.batches * p.m_tiles * p.n_tiles;
    const bool split = p.split_release != 0;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, EW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    volatile int* abort_flag = &s_abort;

    if (warp == 0) {
        // ---- TMA producer: one continuous pipeline over all of this CTA's tiles ---------------
        if (lane == 0) {
            const uint32_t tx_bytes = (uint32_t)La * kTileM * kBlockK + b_bytes;
            int64_t it = 0, armed = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x) {
                const TileCoord tc = decode_tile(p, tile);
                if (p.skip_tiles && tile_masked(p, tc)) continue;
                if (tc.group < 0) continue;
                const int64_t zb = p.tile_group ? tc.group : (p.b_batched ? tc.z : 0);
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int s = (int)(it % p.stages);
                    const uint32_t par = (uint32_t)((it / p.stages) & 1) ^ 1u;
                    if (!mbar_wait(bar_empty + 8 * s, par, abort_flag, 96u * p.backoff)) { ok = false; break; }
                    const uint32_t full = bar_full + 8 * s;
                    mbar_expect_tx(full, tx_bytes);
                    const uint32_t sa = smem_base + s * stage_bytes;
                    const uint32_t sb = sa + a_bytes;
                    for (int i = 0; i < La; ++i)
                        tma_load_2d(sa + i * (kTileM * kBlockK), &tmA, kb * kBlockK,
                                    (int)(i * p.a_rows_per_limb + tc.z * p.M + tc.m0), full);
                    for (int j = 0; j < p.Lb; ++j)
                        tma_load_2d(sb + j * (p.NT * kBlockK), &tmB, kb * kBlockK,
                                    (int)(j * p.b_rows_per_limb + zb * p.b_batch_rows + tc.n0), full);
                    armed = it + 1;
                }
            }
            if (*abort_flag) {
                // leave no copy in flight: wait (bounded) for the stages armed last
                for (int64_t j = (armed > p.stages ? armed - p.stages : 0); j < armed; ++j)
                    for (uint32_t w = 0; w < kSpinLimit; ++w)
                        if (mbar_try(bar_full + 8 * (int)(j % p.stages), (uint32_t)((j / p.stages) & 1))) break;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ---------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) |
                                   ((uint32_t)((p.Lb * p.NT) >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            int64_t it = 0, t = 0;
            bool ok = true;
            const bool prof = p.wait_cycles != nullptr;
            long long w_full = 0, w_empty = 0, t_begin = prof ? clock64() : 0, t0 = 0;
            for (int64_t tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x) {
                if (p.skip_tiles || p.tile_group) {
                    const TileCoord tcm = decode_tile(p, tile);
                    if (tcm.group < 0 || (p.skip_tiles && tile_masked(p, tcm))) continue;
                }
                const int b = (int)(t % p.nbuf);
                const uint32_t tpar = (uint32_t)((t / p.nbuf) & 1);
                if (prof) t0 = clock64();
                ok = mbar_wait(bar_tempty + 8 * b, tpar, abort_flag, 24u * p.backoff);
                if (prof) w_empty += clock64() - t0;
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)(b * buf_cols);
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int s = (int)(it % p.stages);
                    const bool second = p.k_switch && kb >= p.k_switch;
                    if (split && kb == p.k_switch) {
                        // the second set is still being drained by the previous tile's epilogue
                        if (prof) t0 = clock64();
                        ok = mbar_wait(bar_tempty + 8, tpar, abort_flag, 24u * p.backoff);
                        if (prof) w_empty += clock64() - t0;
                        if (!ok) break;
                        tc_fence_after();
                    }
                    if (prof) t0 = clock64();
                    ok = mbar_wait(bar_full + 8 * s, (uint32_t)((it / p.stages) & 1), abort_flag, 24u * p.backoff);
                    if (prof) w_full += clock64() - t0;
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * stage_bytes;
                    const bool merged = p.merged_E != 0;
                    const uint32_t acc_set = acc + ((second && !merged) ? (uint32_t)set_cols : 0u);
                    const int kb_first = (second && !merged) ? p.k_switch : 0;     // first K block of this set
                    // a partial last K block: the copy zero-fills it, no need to multiply the zeros
                    int ks_n = kBlockK / 32;
                    if (p.k_extent) {
                        const int64_t left = p.k_extent - (int64_t)kb * kBlockK;
                        if (left < kBlockK) ks_n = (int)((left + 31) >> 5);
                    }
                    issue_k_block_n(La, acc_set, (uint32_t)p.NT, sa, sa + a_bytes, idesc,
                                    kb != kb_first ? 1u : 0u, ks_n);
                    if (merged && second)
                        issue_extra_block(La, p.merged_E, acc + (uint32_t)set_cols, (uint32_t)p.NT, sa, sa + a_bytes,
                                          idesc, kb == p.k_switch, ks_n);
                    umma_commit(bar_empty + 8 * s);
                }
                if (ok) umma_commit(bar_tfull + 8 * b);
                ++t;
            }
            if (prof) {
                atomicAdd(p.wait_cycles + 0, (unsigned long long)w_full);
                atomicAdd(p.wait_cycles + 1, (unsigned long long)w_empty);
                atomicAdd(p.wait_cycles + 2, (unsigned long long)(clock64() - t_begin));
            }
        }
    } else {
        // ---- epilogue warps: zero the buffers, then drain tile after tile -------------------------
        constexpr int NPART = EW / 4;           // warps sharing one lane quarter split the columns
        const int ew = warp - 2;
        const int q = warp & 3;                 // tensor-memory lane quarter of this warp
        const int part = ew >> 2;
        const int CW = p.NT / NPART, c0 = part * CW;
        const bool ch8 = (CW & 7) == 0;
        const int CH = ch8 ? 8 : 4;
        const int RS = CW * 8 + 16;             // staged row stride (padded against bank conflicts)
        uint8_t* stage = smem_raw + ((smem_base - smem_u32(smem_raw)) + (uint32_t)p.stages * stage_bytes) +
                         (size_t)ew * 32 * RS;
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
        // columns no first-step MMA initialises: [Lb * NT, D * NT) of each set, this warp's part
        auto zero_set = [&](uint32_t set_base) {
            for (int d = p.Lb; d < D; ++d)
                for (int c = 0; c < CW; c += CH) {
                    if (ch8) tmem_st8_zero(set_base + (uint32_t)(d * p.NT + c0 + c));
                    else tmem_st4_zero(set_base + (uint32_t)(d * p.NT + c0 + c));
                }
        };
        if (split) {
            for (int st = 0; st < 2; ++st) {
                // the extra set of the merged mode is written in full by its first MMA
                if (!(st == 1 && p.merged_E)) zero_set(lane_base + (uint32_t)(st * set_cols));
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * st);
            }
        } else {
            for (int b = 0; b < p.nbuf; ++b) {
                for (int st = 0; st < nsets; ++st) zero_set(lane_base + (uint32_t)(b * buf_cols + st * set_cols));
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
            }
        }
        int64_t t = 0;
        const bool prof = p.wait_cycles != nullptr && ew == 0 && lane == 0;
        long long w_acc = 0, t_begin = prof ? clock64() : 0, t0 = 0;
        for (int64_t tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x) {
            const TileCoord tc = decode_tile(p, tile);
            if (p.skip_tiles && tile_masked(p, tc)) continue;
            if (tc.group < 0) {
                // unused row tile: its output is defined as zero (later passes scan the whole buffer)
                for (int i = ew * 32 + lane; i < kTileM * p.NT; i += EW * 32) {
                    const int64_t r = tc.m0 + i / p.NT, c = tc.n0 + i % p.NT;
                    if (r < p.M && c < p.N) p.C[r * p.c_sm + c] = 0;
                }
                continue;
            }
            const int b = (int)(t % p.nbuf);
            if (prof) t0 = clock64();
            if (!mbar_wait(bar_tfull + 8 * b, (uint32_t)((t / p.nbuf) & 1), abort_flag, 48u * p.backoff)) break;
            if (prof) w_acc += clock64() - t0;
            tc_fence_after();
            const uint32_t tq = lane_base + (uint32_t)(b * buf_cols);
            const uint32_t rel = split ? bar_tempty : 0u;
            if (p.fold_epilogue) {
                // the launcher only asks for this epilogue on shapes it is compiled for
                bool done = false;
                const uint32_t rel_extra = p.merged_E ? bar_tempty + 8 : 0u;
                if (CW == 16)
                    done = epilogue_merged_dispatch<16>(p, D, tq, tc, q, lane, c0, set_cols, bar_tempty, rel_extra);
                else if (CW == 8)
                    done = epilogue_merged_dispatch<8>(p, D, tq, tc, q, lane, c0, set_cols, bar_tempty, rel_extra);
                if (!done) {
                    if (lane == 0) *abort_flag = 1;
                    break;
                }
                ++t;
                continue;
            }
            if (p.fits64) {
                if (ch8) epilogue_part<true, 8>(p, tq, D, tc, q, lane, c0, CW, stage, RS, set_cols, rel);
                else epilogue_part<true, 4>(p, tq, D, tc, q, lane, c0, CW, stage, RS, set_cols, rel);
            } else {
                if (ch8) epilogue_part<false, 8>(p, tq, D, tc, q, lane, c0, CW, stage, RS, set_cols, rel);
                else epilogue_part<false, 4>(p, tq, D, tc, q, lane, c0, CW, stage, RS, set_cols, rel);
            }
            // the set(s) this epilogue did not hand back itself
            for (int st = split ? 1 : 0; st < nsets; ++st)
                if (!(st == 1 && p.merged_E)) zero_set(tq + (uint32_t)(st * set_cols));
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * (split ? 1 : b));
            ++t;
        }
        if (prof) {
            atomicAdd(p.wait_cycles + 3, (unsigned long long)w_acc);
            atomicAdd(p.wait_cycles + 4, (unsigned long long)(clock64() - t_begin));
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem, p.tmem_cols);
    if (threadIdx.x == 0 && s_abort) *p.error_flag = 1;
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// planes seen as a 2-D uint8 tensor [rows_total][Kp], box = box_rows x 128 bytes, 128B swizzle
// pitch: bytes between rows when they are wider than the Kp columns in use (0 = Kp)
bool make_plane_map(CUtensorMap* map, void* base, int64_t rows_total, int64_t Kp, int box_rows, int64_t pitch = 0)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t gdim[2] = {(cuuint64_t)Kp, (cuuint64_t)rows_total};
    cuuint64_t gstride[1] = {(cuuint64_t)(pitch ? pitch : Kp)};
    cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, gdim, gstride, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct DeviceFlags {
    int* host = nullptr;      // mapped, host view
    int* dev = nullptr;       // device view of the same word
    unsigned* overflow = nullptr;  // second mapped word
    unsigned* overflow_dev = nullptr;
};
DeviceFlags g_flags[64];

DeviceFlags* flags_for_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    DeviceFlags& f = g_flags[dev];
    if (!f.host) {
        int* h = nullptr;
        if (cudaHostAlloc((void**)&h, 64, cudaHostAllocMapped) != cudaSuccess) return nullptr;
        h[0] = 0;
        h[1] = 0;
        int* d = nullptr;
        if (cudaHostGetDevicePointer((void**)&d, h, 0) != cudaSuccess) return nullptr;
        f.host = h;
        f.dev = d;
        f.overflow = (unsigned*)(h + 1);
        f.overflow_dev = (unsigned*)(d + 1);
    }
    return &f;
}

template <typename T>
int launch_split_t(const T* X, int8_t* planes, int L, int64_t nb, int64_t rows, int64_t K, int64_t Kp,
                   int64_t sz, int64_t sr, int64_t sk, int64_t div, unsigned* overflow, cudaStream_t st,
                   unsigned long long* absmax_out = nullptr, int64_t dst_pitch = 0, int64_t valid_H = 0,
                   int64_t valid_start = 0, int shl = 0, const int* row_index = nullptr,
                   const RowParts* row_parts = nullptr, int group_box = 0)
{
    if (dst_pitch == 0) dst_pitch = Kp;
    RowParts parts{};
    if (row_parts) parts = *row_parts;
    if (parts.n && (!row_index || sk != 1 || switches().split_generic)) return ZKDS_ERR_UNSUPPORTED;
    int64_t total = rows * (Kp >> 2);
    int64_t bx = (total + 255) / 256;
    int64_t cap = (int64_t)sm_count() * 32;
    if (bx > cap) bx = cap;
    if (nb > 65535) return ZKDS_ERR_RANGE;
    if (sk == 1 && !switches().split_generic) {
        int tl = 0;
        while (tl < 8 && (1 << tl) < (Kp >> 2)) ++tl;
        const int64_t rpb = 256 >> tl;
        const int64_t gx = (rows + rpb - 1) / rpb;        // row groups per batch
        if (gx * nb > 0x7fffffffll) return ZKDS_ERR_RANGE;   // the kernel's 32-bit item counter cannot wrap
        const int z_fast = (nb > 1 && sz < sr) ? 1 : 0;
        int64_t kseg = 1, seg_quads = Kp >> 2;
        const int64_t per_row = ((Kp >> 2) + (1 << tl) - 1) >> tl;      // quads each thread of a row walks
        if (gx * nb < 2 * (int64_t)sm_count() && per_row > 1) {
            kseg = (2 * (int64_t)sm_count() + gx * nb - 1) / (gx * nb);
            if (kseg > per_row) kseg = per_row;
            seg_quads = ((per_row + kseg - 1) / kseg) << tl;
            kseg = ((Kp >> 2) + seg_quads - 1) / seg_quads;
        }
        int64_t blocks = gx * nb * kseg;
        if (blocks > cap) blocks = cap;
        dim3 g2((unsigned)blocks);
#define ZKDS_SPLIT_ROWS(LL)                                                                              \
    split_rows_kernel<T, LL><<<g2, 256, 0, st>>>(X, planes, L, rows, K, Kp, sz, sr, div,                  \
                                                 nb * rows * dst_pitch, overflow, absmax_out, dst_pitch, \
                                                 valid_H, valid_start, tl, (unsigned)nb, (unsigned)gx, z_fast, shl, \
                                                 row_index, (unsigned)kseg, seg_quads, parts, group_box)
        switch (L) {
        case 2: ZKDS_SPLIT_ROWS(2); break;
        case 3: ZKDS_SPLIT_ROWS(3); break;
        case 4: ZKDS_SPLIT_ROWS(4); break;
        case 5: ZKDS_SPLIT_ROWS(5); break;
        default: ZKDS_SPLIT_ROWS(0); break;
        }
#undef ZKDS_SPLIT_ROWS
        return check_launch();
    }
    if (shl || row_index) return ZKDS_ERR_UNSUPPORTED;        // only the k-contiguous kernel scales or gathers
    dim3 grid((unsigned)bx, (unsigned)nb);
    split_kernel<T><<<grid, 256, 0, st>>>(X, planes, L, rows, K, Kp, sz, sr, sk, div, nb * rows * dst_pitch,
                                          overflow, absmax_out, dst_pitch, valid_H, valid_start);
    return check_launch();
}

}  // namespace

int launch_absmax(const void* X, int bits, int64_t batches, int64_t rows, int64_t cols, int64_t sz,
                  int64_t sr, int64_t sc, int64_t div, uint64_t* out_dev, cudaStream_t st)
{
    if (batches <= 0 || rows <= 0 || cols <= 0) return ZKDS_OK;
    if (batches > 65535) return ZKDS_ERR_RANGE;
    int64_t total = rows * cols;
    int64_t bx = (total + 255) / 256;
    int64_t cap = (int64_t)sm_count() * 8;
    if (bx > cap) bx = cap;
    dim3 grid((unsigned)bx, (unsigned)batches);
    if (bits == 64)
        absmax_kernel<int64_t><<<grid, 256, 0, st>>>((const int64_t*)X, rows, cols, sz, sr, sc, div, out_dev);
    else if (bits == 32)
        absmax_kernel<int32_t><<<grid, 256, 0, st>>>((const int32_t*)X, rows, cols, sz, sr, sc, div, out_dev);
    else return ZKDS_ERR_ARG;
    return check_launch();
}

int limb_device_status(int clear)
{
    DeviceFlags* f = flags_for_device();
    if (!f) return ZKDS_OK;
    int rc = ZKDS_OK;
    if (f->host[0]) rc = ZKDS_ERR_DEVICE;
    else if (*f->overflow) rc = ZKDS_ERR_RANGE;
    if (clear) { f->host[0] = 0; *f->overflow = 0; }
    return rc;
}

// ---- kernel timing hooks -------------------------------------------------------------
static bool g_timing = false;
static bool g_accumulate = false;
static cudaEvent_t g_ev[64][2];
static bool g_ev_made[64];
static bool g_ev_valid[64];

static double g_tot_ms = 0.0, g_tot_ops = 0.0;
static long long g_tot_launches = 0;
struct LaunchRecord { double v[8]; };
static LaunchRecord g_records[256];

int limb_timing_record(long long i, double* out8)
{
    if (i < 0 || i >= g_tot_launches || i >= 256) return 0;
    for (int j = 0; j < 8; ++j) out8[j] = g_records[i].v[j];
    return 1;
}

void limb_timing_enable(int on)
{
    g_timing = on != 0;
    if (on == 2) { g_tot_ms = 0.0; g_tot_ops = 0.0; g_tot_launches = 0; }
    g_accumulate = (on == 2);
}

void limb_timing_totals(double* ms, double* int8_ops, long long* launches)
{
    if (ms) *ms = g_tot_ms;
    if (int8_ops) *int8_ops = g_tot_ops;
    if (launches) *launches = g_tot_launches;
}

float limb_last_kernel_ms()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_ev_valid[dev]) return -1.f;
    float ms = -1.f;
    if (cudaEventSynchronize(g_ev[dev][1]) != cudaSuccess) return -1.f;
    if (cudaEventElapsedTime(&ms, g_ev[dev][0], g_ev[dev][1]) != cudaSuccess) return -1.f;
    return ms;
}

// Share of a launch's (row tile x column tile x K block) work that is issued under causal skipping
// (LimbParams::skip_tiles / skip_k): what the timing records count as int8 operations.
static double issued_share(int64_t M, int64_t N, int64_t K, int NT, int skip_tiles, int skip_k, int64_t H,
                           int64_t start)
{
    if ((!skip_tiles && !skip_k) || H <= 0) return 1.0;
    const int64_t mt = (M + kTileM - 1) / kTileM, nt = (N + NT - 1) / NT, kb = (K + kBlockK - 1) / kBlockK;
    double issued = 0.0;
    for (int64_t t = 0; t < mt; ++t) {
        int64_t last = t * kTileM + kTileM - 1;
        if (last > M - 1) last = M - 1;
        const int64_t s_max = last / H;
        int64_t cols = nt, blocks = kb;
        if (skip_tiles) { cols = (start + s_max) / NT + 1; if (cols > nt) cols = nt; }
        if (skip_k) { blocks = (start + s_max + 1 + kBlockK - 1) / kBlockK; if (blocks > kb) blocks = kb; if (blocks < 1) blocks = 1; }
        issued += (double)cols * (double)blocks;
    }
    return issued / ((double)mt * (double)nt * (double)kb);
}

// The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel: set once.
template <typename K>
static int allow_big_smem(K kernel, bool (&done)[64])
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!done[dev]) {
        ZKDS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024 - 3072)));
        done[dev] = true;
    }
    return ZKDS_OK;
}
static bool g_attr_onetile[64], g_attr_p16[64], g_attr_p8[64];

static cudaEvent_t* timing_events()
{
    int dev = 0;
    if (!g_timing || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!g_ev_made[dev]) {
        if (cudaEventCreate(&g_ev[dev][0]) != cudaSuccess || cudaEventCreate(&g_ev[dev][1]) != cudaSuccess)
            return nullptr;
        g_ev_made[dev] = true;
    }
    g_ev_valid[dev] = true;
    return g_ev[dev];
}

// |addend + sum_k a*b| < 2^62 for every operand the limb counts admit?  |a| <= 2^(8 La - 1) * 1.004
static int sum_fits64(int La, int Lb, int64_t K, int64_t addend)
{
    int kbits = 0;
    while (((int64_t)1 << kbits) < K) ++kbits;
    const int bits = (8 * La - 1) + (8 * Lb - 1) + kbits + 1;
    const int64_t lim = (int64_t)1 << 61;
    return bits <= 61 && addend < lim && addend > -lim;
}

int limbs_needed(uint64_t maxabs)
{
    unsigned __int128 cover = 0, w = 1;
    for (int L = 1; L <= 9; ++L) {
        cover += (unsigned __int128)127 * w;
        w <<= 8;
        if ((unsigned __int128)maxabs <= cover) return L;
    }
    return 10;
}

namespace {
// New rows of the MLA latent cache (kv [B][S][C1], rope part [B][S][C2]) as balanced 8-bit limb planes, in the
// two layouts the attention contractions read them in and at their place in buffers that hold `cap` positions:
//   score planes [L][B][cap][C1 + C2r]: position t is a row, the latent and the rope part side by side
//                                       (the B operand of the fused score kernel, K = C1 + C2);
//   value planes [L][B][C1][cap]:       position t is a column (the B operand of P . KV, K = positions).
// One thread per (b, s, column).
__global__ void __launch_bounds__(256)
cache_planes_append_kernel(const int64_t* __restrict__ kv_new, const int64_t* __restrict__ pe_new,
                           int8_t* __restrict__ sp, int8_t* __restrict__ vp, int64_t B, int64_t S, int C1, int C2,
                           int64_t start, int64_t cap, int L, int64_t pitch, unsigned* overflow)
{
    const int C = C1 + C2;
    const int64_t total = B * S * C;
    bool ovf = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int64_t bs = i / C, s = bs % S, b = bs / S;
        int64_t u = c < C1 ? kv_new[bs * C1 + c] : pe_new[bs * C2 + (c - C1)];
        const int64_t t = start + s;
        for (int l = 0; l < L; ++l) {
            const int8_t digit = (int8_t)(u & 0xFF);
            u = (u >> 8) + ((u >> 7) & 1);
            sp[(((int64_t)l * B + b) * cap + t) * pitch + c] = digit;
            if (c < C1) vp[(((int64_t)l * B + b) * C1 + c) * cap + t] = digit;
        }
        ovf |= (u != 0);
    }
    if (ovf) *overflow = 1u;
}
}  // namespace

int launch_cache_planes_append(const int64_t* kv_new, const int64_t* pe_new, int8_t* score_planes,
                               int8_t* value_planes, int64_t B, int64_t S, int64_t C1, int64_t C2,
                               int64_t start_pos, int64_t cap, int L, cudaStream_t st)
{
    if (B <= 0 || S <= 0) return ZKDS_OK;
    if (C1 <= 0 || C2 <= 0 || C1 > 65536 || C2 > 65536 || (C1 & 15) || L < 1 || L > 9 || start_pos < 0 ||
        start_pos + S > cap || (cap & 15))
        return ZKDS_ERR_ARG;
    DeviceFlags* fl = flags_for_device();
    if (!fl) return ZKDS_ERR_WORKSPACE;
    const int64_t pitch = C1 + ((C2 + 15) & ~(int64_t)15);
    const int64_t total = B * S * (C1 + C2);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap_blocks = (int64_t)sm_count() * 16;
    if (blocks > cap_blocks) blocks = cap_blocks;
    cache_planes_append_kernel<<<(unsigned)blocks, 256, 0, st>>>(kv_new, pe_new, score_planes, value_planes, B, S,
                                                                 (int)C1, (int)C2, start_pos, cap, L, pitch,
                                                                 fl->overflow_dev);
    return check_launch();
}

int planes_split(const void* X, int bits, int64_t nb, int64_t rows, int64_t K, int64_t sz, int64_t sr,
                 int64_t sk, int64_t div, int L, int8_t* dst, cudaStream_t st)
{
    DeviceFlags* fl = flags_for_device();
    if (!fl) return ZKDS_ERR_WORKSPACE;
    const int64_t Kp = (K + 15) & ~(int64_t)15;
    if (bits == 32)
        return launch_split_t<int32_t>((const int32_t*)X, dst, L, nb, rows, K, Kp, sz, sr, sk, div,
                                       fl->overflow_dev, st);
    if (bits == 64)
        return launch_split_t<int64_t>((const int64_t*)X, dst, L, nb, rows, K, Kp, sz, sr, sk, div,
                                       fl->overflow_dev, st);
    return ZKDS_ERR_ARG;
}

// Epilogue warps of the persistent kernel.  Measured on a B200: the fused attention scores run best with 16
// (four per tensor-memory lane quarter), plain contractions show no gain beyond 8, which also keeps 168
// registers per thread.  ZKDS_EPI_WARPS = 8 | 16 overrides for experiments.
static int persistent_epilogue_warps(bool fused_scores)
{
    const int v = switches().epi_warps;
    if (v == 8 || v == 16) return v;
    return fused_scores ? 16 : 8;
}

static int launch_persistent(int ew, int ctas, size_t smem, cudaStream_t st, const CUtensorMap& tmA,
                             const CUtensorMap& tmB, const LimbParams& lp_in)
{
    LimbParams lp = lp_in;
    lp.backoff = switches().no_backoff ? 0u : 1u;
    // ZKDS_WAIT_PROFILE=1: a synchronous diagnostic run that prints where the MMA warp and the first
    // epilogue warp spent their cycles (share of their lifetime spent waiting)
    unsigned long long* prof = nullptr;
    if (switches().wait_profile) {
        prof = (unsigned long long*)workspace(8 * sizeof(unsigned long long), 4);
        if (prof) ZKDS_CUDA(cudaMemsetAsync(prof, 0, 8 * sizeof(unsigned long long), st));
        lp.wait_cycles = prof;
    }
    struct Report {
        unsigned long long* d; cudaStream_t st; const LimbParams* lp;
        ~Report()
        {
            if (!d) return;
            unsigned long long h[8];
            if (cudaStreamSynchronize(st) != cudaSuccess) return;
            if (cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return;
            fprintf(stderr, "persistent M=%lld N=%lld kblocks=%d NT=%d nbuf=%d split=%d: MMA warp waits operands "
                            "%.1f%% accumulators %.1f%%; epilogue warp waits accumulators %.1f%%\n",
                    (long long)lp->M, (long long)lp->N, lp->kblocks, lp->NT, lp->nbuf, lp->split_release,
                    100.0 * h[0] / (h[2] ? h[2] : 1), 100.0 * h[1] / (h[2] ? h[2] : 1),
                    100.0 * h[3] / (h[4] ? h[4] : 1));
        }
    } report{prof, st, &lp};
    if (ew == 16) {
        { int rc_a = allow_big_smem(limb_gemm_persistent_kernel<16>, g_attr_p16); if (rc_a != ZKDS_OK) return rc_a; }
        limb_gemm_persistent_kernel<16><<<ctas, persistent_threads(16), smem, st>>>(tmA, tmB, lp);
    } else {
        { int rc_a = allow_big_smem(limb_gemm_persistent_kernel<8>, g_attr_p8); if (rc_a != ZKDS_OK) return rc_a; }
        limb_gemm_persistent_kernel<8><<<ctas, persistent_threads(8), smem, st>>>(tmA, tmB, lp);
    }
    return check_launch();
}

int launch_contraction_limb(const Contraction& p, int La, int Lb, const Planes* pre_b, cudaStream_t st)
{
    if (pre_b) Lb = pre_b->L;
    if (La < 1 || Lb < 1 || La > 9 || Lb > 9) return ZKDS_ERR_UNSUPPORTED;
    if (p.K <= 0) return ZKDS_ERR_UNSUPPORTED;
    const int D = La + Lb - 1;
    const int pairs = La < Lb ? La : Lb;
    if ((int64_t)pairs * p.K >= 131072) return ZKDS_ERR_UNSUPPORTED;  // int32 diagonal bound
    // tile width: the B stack must fit one MMA (<= 256 columns), the diagonals tensor memory
    // (<= 512 columns), and two pipeline stages shared memory
    const size_t smem_max = 227 * 1024 - 4096;  // static barriers + alignment slack stay below the opt-in limit
    // An MMA of M = 128 takes as long as one 256 columns wide, so the B stack (Lb * NT columns) should
    // come close to 256; among the widths that fit, take the one that wastes the least of that time
    // (narrow stack) and of the last column tile (padding).
    int NT = 0;
    double best = 0.0;
    for (int cand : {16, 32, 48, 64, 80, 96, 112, 128}) {     // ties go to the narrower tile
        if (Lb * cand > 256 || D * cand > 512) continue;
        size_t stage = (size_t)La * kTileM * kBlockK + (size_t)Lb * cand * kBlockK;
        if (smem_max / stage < 2) continue;
        const int64_t tiles = (p.N + cand - 1) / cand;
        double score = ((double)p.N / (double)(tiles * cand)) * ((double)(Lb * cand) / 256.0);
        if (smem_max / stage < 3) score *= 0.97;      // prefer three pipeline stages when it is close
        if (score > best * 1.02) { best = score; NT = cand; }
    }
    if (switches().tile_nt) {       // experiments: force a width that fits
        const int want = switches().tile_nt;
        if (want >= 16 && want % 16 == 0 && Lb * want <= 256 && D * want <= 512 &&
            smem_max / ((size_t)La * kTileM * kBlockK + (size_t)Lb * want * kBlockK) >= 2)
            NT = want;
    }
    if (!NT) return ZKDS_ERR_UNSUPPORTED;
    const size_t stage = (size_t)La * kTileM * kBlockK + (size_t)Lb * NT * kBlockK;
    int stages = (int)(smem_max / stage);
    if (stages > 8) stages = 8;
    const int64_t Kp = (p.K + 15) & ~(int64_t)15;
    const int64_t nbB = p.tile_group ? (pre_b ? pre_b->nb : 0) : (p.b_sz ? p.batches : 1);
    if (p.tile_group && (!pre_b || p.batches != 1)) return ZKDS_ERR_ARG;
    const int64_t a_rows = p.batches * p.M, b_rows = nbB * p.N;
    if (a_rows * La > 0x7fffff00ll || b_rows * Lb > 0x7fffff00ll || Kp > 0x7fffff00ll) return ZKDS_ERR_UNSUPPORTED;
    const int64_t mt = (p.M + kTileM - 1) / kTileM, nt = (p.N + NT - 1) / NT;
    if (mt > 0x7fffffffll || nt > 65535 || p.batches > 65535) return ZKDS_ERR_UNSUPPORTED;
    if (pre_b && (pre_b->nb != nbB || pre_b->rows != p.N || pre_b->K != p.K)) return ZKDS_ERR_ARG;

    // shallow K, plain output: the persistent double-buffered kernel (see above)
    bool persistent = false;
    int pNT = 0, pstages = 0;
    size_t psmem = 0;
    int ew = persistent_epilogue_warps(false);
    // up to 8 K blocks (K <= 1024); measured: from 12 blocks on the one-tile kernel with its wider tile
    // (a full 256-column B stack for two-limb weights) wins although it overlaps nothing
    // (wq_b, K = 1536: 0.70 against 0.85 ms; w2 of the shared expert, K = 2048: 0.68 against 0.93 ms)
    int64_t max_kb = 8;
    if (switches().persistent_max_kb >= 0) max_kb = switches().persistent_max_kb;
    if (!p.R && !p.skip_k && (Kp + kBlockK - 1) / kBlockK <= max_kb && !switches().no_persistent &&
        !(p.tile_group && switches().no_persistent_grouped)) {
        for (int cand : {64, 48, 32, 16}) {
            if (Lb * cand > 256 || 2 * D * cand > 512) continue;
            size_t st_b = (size_t)La * kTileM * kBlockK + (size_t)Lb * cand * kBlockK;
            size_t staging = persistent_staging(ew, cand);
            if (smem_max < staging + 1024) continue;
            int ns = (int)((smem_max - staging - 1024) / st_b);
            if (ns < 2) continue;
            pNT = cand;
            pstages = ns > 8 ? 8 : ns;
            psmem = st_b * pstages + staging + 1024;
            persistent = true;
            break;
        }
        // narrow outputs: the smallest valid width (16, 32, 48, 64) that still covers N
        if (persistent) {
            int want = pNT;
            for (int cand : {48, 32, 16})
                if (cand < pNT && p.N <= cand) want = cand;
            if (want != pNT) {
                pNT = want;
                size_t st_b = (size_t)La * kTileM * kBlockK + (size_t)Lb * pNT * kBlockK;
                size_t staging = persistent_staging(ew, pNT);
                int ns = (int)((smem_max - staging - 1024) / st_b);
                pstages = ns > 8 ? 8 : ns;
                psmem = st_b * pstages + staging + 1024;
            }
        }
    }
    if (persistent) NT = pNT;
    const int64_t nt_eff = (p.N + NT - 1) / NT;

    DeviceFlags* fl = flags_for_device();
    if (!fl) return ZKDS_ERR_WORKSPACE;
    int8_t* pa = (int8_t*)workspace((size_t)La * a_rows * Kp + 1024, 0);
    if (!pa) return ZKDS_ERR_WORKSPACE;
    unsigned long long* d_absmax = nullptr;
    if (p.dynamic_a) {
        unsigned long long* words = (unsigned long long*)workspace(8 * sizeof(uint64_t), 5);
        if (!words) return ZKDS_ERR_WORKSPACE;
        d_absmax = words + 2;
        ZKDS_CUDA(cudaMemsetAsync(d_absmax, 0, sizeof(uint64_t), st));
    }
    const int64_t Kp16 = Kp;
    int rc;
    if (p.softmax_lut) {
        if (p.a_sm != p.K || p.a_sz != p.M * p.K || p.a_div != 1) return ZKDS_ERR_ARG;
        rc = launch_softmax_planes(p.A, p.softmax_lut, pa, La, a_rows, p.K, Kp, a_rows * Kp, fl->overflow_dev,
                                   d_absmax, p.skip_k ? p.skip_H : 0, p.softmax_S, p.skip_start, st);
    } else if (p.glu_lut) {
        if (p.batches != 1 || p.a_div != 1 || p.a_row_index || !p.glu_r2) return ZKDS_ERR_ARG;
        rc = launch_glu_planes(p.A, p.glu_r2, p.a_sm, p.glu_lut, pa, La, a_rows, p.K, Kp, a_rows * Kp,
                               fl->overflow_dev, d_absmax, st);
    } else {
        RowParts parts{};
        if (p.a_n_parts > 0) {
            if (p.a_n_parts > kMaxRowParts || p.a_rows_per_part <= 0 || !p.a_row_index) return ZKDS_ERR_ARG;
            parts.n = p.a_n_parts;
            parts.rows_per_part = p.a_rows_per_part;
            for (int i = 0; i < parts.n; ++i) parts.base[i] = p.a_parts[i];
        }
        rc = launch_split_t<int64_t>(p.A, pa, La, p.batches, p.M, p.K, Kp16, p.a_sz, p.a_sm, 1, p.a_div,
                                     fl->overflow_dev, st, d_absmax, 0, p.skip_k ? p.skip_H : 0, p.skip_start, 0,
                                     p.a_row_index, parts.n ? &parts : nullptr,
                                     (p.tile_group && p.a_row_index) ? p.group_rows : 0);
    }
    if (rc != ZKDS_OK) return rc;
    int8_t* pb;
    if (pre_b) pb = pre_b->data;
    else {
        pb = (int8_t*)workspace((size_t)Lb * b_rows * Kp + 1024, 1);
        if (!pb) return ZKDS_ERR_WORKSPACE;
        rc = planes_split(p.B, p.b_bits, nbB, p.N, p.K, p.b_sz, p.b_sn, p.b_sk, p.b_div, Lb, pb, st);
        if (rc != ZKDS_OK) return rc;
    }

    // few rows (decode, the small-M GEMM): a smaller A box, more pipeline stages
    int a_box = kTileM;
    if (!persistent && (p.tile_group ? p.group_rows != 0 : p.M <= 64)) {
        const int want = p.tile_group ? p.group_rows : p.M <= 32 ? 32 : 64;
        // the MMA of the last limb reads 128 rows from its tile's start: that must stay inside the stage
        if ((size_t)(kTileM - want) * kBlockK <= (size_t)Lb * NT * kBlockK) a_box = want;
    }
    size_t stage_bytes = stage;
    if (a_box != kTileM) {
        stage_bytes = (size_t)La * a_box * kBlockK + (size_t)Lb * NT * kBlockK;
        stages = (int)(smem_max / stage_bytes);
        if (stages > 8) stages = 8;
    }
    CUtensorMap tmA, tmB;
    if (!make_plane_map(&tmA, pa, (int64_t)La * a_rows, Kp, a_box)) return ZKDS_ERR_UNSUPPORTED;
    const int64_t b_pitch = (pre_b && pre_b->pitch) ? pre_b->pitch : Kp;
    if (b_pitch < Kp || (b_pitch & 15)) return ZKDS_ERR_ARG;
    if (!make_plane_map(&tmB, pb, (int64_t)Lb * b_rows, Kp, NT, b_pitch)) return ZKDS_ERR_UNSUPPORTED;

    LimbParams lp{};
    lp.La = La; lp.Lb = Lb; lp.NT = NT; lp.stages = stages;
    lp.a_box_rows = a_box == kTileM ? 0 : a_box;
    lp.kblocks = (int)((Kp + kBlockK - 1) / kBlockK);
    lp.k_extent = Kp;
    uint32_t cols = 32;
    while (cols < (uint32_t)((persistent ? 2 : 1) * D * NT)) cols <<= 1;
    lp.tmem_cols = cols;
    if (persistent) lp.stages = pstages;
    lp.nbuf = 2;
    lp.M = p.M; lp.N = p.N; lp.batches = p.batches;
    lp.a_rows_per_limb = a_rows; lp.b_rows_per_limb = b_rows; lp.b_batch_rows = p.N;
    lp.b_batched = p.b_sz ? 1 : 0;
    lp.C = p.C; lp.R = p.R; lp.c_sz = p.c_sz; lp.c_sm = p.c_sm;
    lp.addend = p.addend; lp.shift = p.shift; lp.r_legacy = p.r_legacy;
    lp.error_flag = fl->dev;
    lp.fits64 = sum_fits64(La, Lb, p.K, p.addend);
    lp.a_absmax = d_absmax;
    lp.overflow_flag = fl->overflow_dev;
    lp.skip_tiles = p.skip_tiles; lp.skip_k = p.skip_k; lp.skip_H = p.skip_H; lp.skip_start = p.skip_start;
    lp.tile_group = p.tile_group;
    lp.group_shift = p.group_shift; lp.n_split = p.n_split;
    lp.addin = p.addin; lp.ep_mul = p.ep_mul; lp.ep_div = p.ep_div;
    lp.causal_H = p.causal_H; lp.causal_start = p.causal_start; lp.mask_value = p.mask_value;

    // split-K for the weight-streaming shapes (few output tiles, deep K): see LimbParams::ksplit
    lp.ksplit = 1;
    const int64_t tiles_total = p.batches * mt * nt_eff;
    if (!persistent && !p.tile_group && !p.skip_k && !p.skip_tiles && lp.kblocks >= 2 && !switches().no_split_k &&
        tiles_total * 2 <= sm_count() && tiles_total <= kSplitTilesMax && 8 * (La + Lb) + 18 <= 116) {
        int want = (int)(sm_count() / tiles_total);
        if (want > lp.kblocks) want = lp.kblocks;
        const int per = (lp.kblocks + want - 1) / want;
        const int ks = (lp.kblocks + per - 1) / per;
        if (ks > 1) {
            const size_t words = (size_t)tiles_total * 2 * NT * kTileM;
            size_t fresh = 0;
            uint8_t* ws = (uint8_t*)workspace_fresh(kSplitHeader + words * sizeof(uint64_t), 6, &fresh);
            if (!ws) return ZKDS_ERR_WORKSPACE;
            // the kernel leaves the block zeroed; it has to be cleared when it is new, and after a launch
            // that gave up a wait (its tiles were never finished)
            if (fresh) ZKDS_CUDA(cudaMemsetAsync(ws, 0, fresh, st));
            else if (fl->host[0]) ZKDS_CUDA(cudaMemsetAsync(ws, 0, kSplitHeader + words * sizeof(uint64_t), st));
            lp.ksplit = ks;
            lp.kb_per_split = per;
            lp.tile_counter = (unsigned*)ws;
            lp.partial = (unsigned long long*)(ws + kSplitHeader);
        }
    }

    size_t smem = stage_bytes * stages + 1024;
    // more than half the shared memory per CTA keeps one CTA per SM, so its tensor-memory
    // allocation can never wait for a co-resident CTA
    if (smem < 120 * 1024) smem = 120 * 1024;
    { int rc_a = allow_big_smem(limb_gemm_kernel, g_attr_onetile); if (rc_a != ZKDS_OK) return rc_a; }
    // panel height: the A limb tiles of one panel should stay L2 resident (~32 MB)
    int64_t panel = (32ll << 20) / ((int64_t)La * kTileM * Kp);
    if (panel < 1) panel = 1;
    if (panel > mt) panel = mt;
    lp.m_tiles = mt; lp.n_tiles = nt_eff; lp.panel_m = panel;
    if (mt * nt_eff > 0x7fffffffll) return ZKDS_ERR_UNSUPPORTED;
    dim3 grid = p.tile_group ? dim3((unsigned)mt, (unsigned)nt_eff, 1)
                             : dim3((unsigned)(mt * nt_eff * lp.ksplit), 1, (unsigned)p.batches);
    cudaEvent_t* ev = timing_events();
    if (ev) ZKDS_CUDA(cudaEventRecord(ev[0], st));
    if (persistent) {
        if (psmem < 120 * 1024) psmem = 120 * 1024;
        int64_t total_tiles = p.batches * mt * nt_eff;
        if (total_tiles > 0x7fffffffll) return ZKDS_ERR_UNSUPPORTED;
        int ctas = sm_count();
        if (total_tiles < ctas) ctas = (int)total_tiles;
        rc = launch_persistent(ew, ctas, psmem, st, tmA, tmB, lp);
    } else {
        unsigned long long* prof = nullptr;
        if (switches().wait_profile) {
            prof = (unsigned long long*)workspace(32 * sizeof(unsigned long long), 4);
            if (prof) ZKDS_CUDA(cudaMemsetAsync(prof, 0, 32 * sizeof(unsigned long long), st));
            lp.wait_cycles = prof;
        }
        limb_gemm_kernel<<<grid, kThreads, smem, st>>>(tmA, tmB, lp);
        rc = check_launch();
        if (prof && rc == ZKDS_OK) {
            unsigned long long h[32];
            ZKDS_CUDA(cudaStreamSynchronize(st));
            ZKDS_CUDA(cudaMemcpy(h, prof, sizeof(h), cudaMemcpyDeviceToHost));
            fprintf(stderr, "one-tile M=%lld N=%lld kblocks=%d NT=%d stages=%d ksplit=%d ctas=%u: longest phase in cycles: "
                            "accumulate %llu, add partials %llu, fence+counter %llu, epilogue %llu, CTA lifetime %llu\n",
                    (long long)lp.M, (long long)lp.N, lp.kblocks, lp.NT, lp.stages, lp.ksplit, grid.x * grid.z, h[8], h[9],
                    h[10], h[11], h[12]);
        }
    }
    if (ev) ZKDS_CUDA(cudaEventRecord(ev[1], st));
    if (ev && g_accumulate && rc == ZKDS_OK) {
        // profiling pass: wait for the kernel, add its duration and the int8 work it issued
        float ms = 0.f;
        ZKDS_CUDA(cudaEventSynchronize(ev[1]));
        ZKDS_CUDA(cudaEventElapsedTime(&ms, ev[0], ev[1]));
        int la_used = La;
        if (d_absmax) {
            unsigned long long h = 0;
            ZKDS_CUDA(cudaMemcpy(&h, d_absmax, sizeof(h), cudaMemcpyDeviceToHost));
            int need = limbs_needed(h);
            if (need < la_used) la_used = need;
        }
        if (switches().trace)
            fprintf(stderr, "limb_gemm batches=%lld M=%lld N=%lld K=%lld La=%d(%d) Lb=%d NT=%d stages=%d fits64=%d tail=%d: %.3f ms\n",
                    (long long)p.batches, (long long)p.M, (long long)p.N, (long long)p.K, la_used, La, Lb, NT,
                    stages, lp.fits64, (p.addin || p.ep_div || p.causal_H) ? 1 : 0, ms);
        if (g_tot_launches < 256) {
            LaunchRecord& r = g_records[g_tot_launches];
            r.v[0] = (double)p.batches; r.v[1] = (double)p.M; r.v[2] = (double)p.N; r.v[3] = (double)p.K;
            r.v[4] = la_used; r.v[5] = Lb; r.v[6] = ms; r.v[7] = (p.tile_group ? 1.0 : 0.0) + (p.b_sz ? 2.0 : 0.0);
        }
        g_tot_ms += ms;
        g_tot_ops += 2.0 * (double)la_used * Lb * (double)p.batches * (double)p.M * (double)p.N * (double)p.K *
                     issued_share(p.M, p.N, p.K, NT, p.skip_tiles, p.skip_k, p.skip_H, p.skip_start);
        g_tot_launches += 1;
    }
    return rc;
}

// ------------------------------------------------------------------------------------
// MLA attention scores in one pass
// ------------------------------------------------------------------------------------
// scores[b,m,n] = tail( ((add1 + A1[b,m,:] . B1[b,n,:]) >> s1) + ((add2 + A2[b,m,:] . B2[b,n,:]) >> s2) )
// The limb planes of A1|A2 and of B1|B2 are laid side by side along K, so the whole thing is one
// contraction over K1 + K2 whose K blocks from K1 on accumulate into a second set of diagonals;
// neither partial score tensor is ever written to memory.
int launch_scores_fused(const FusedScores& f, int La, int Lb, cudaStream_t st)
{
    if (La < 1 || Lb < 1 || La > 9 || Lb > 9) return ZKDS_ERR_UNSUPPORTED;
    if (f.K1 <= 0 || f.K2 <= 0 || (f.K1 % kBlockK) != 0) return ZKDS_ERR_UNSUPPORTED;
    if (switches().no_persistent) return ZKDS_ERR_UNSUPPORTED;
    const int D = La + Lb - 1;
    const int pairs = La < Lb ? La : Lb;
    const int64_t Kmax = f.K1 > f.K2 ? f.K1 : f.K2;
    if ((int64_t)pairs * Kmax >= 131072) return ZKDS_ERR_UNSUPPORTED;
    const size_t smem_max = 227 * 1024 - 4096;
    // Two sets of diagonals per buffer.  A wide tile matters more than the ping-pong: every
    // output tile re-reads its A limb tiles, so narrow tiles are bound by L2 traffic.  Take two
    // buffers only if the tile can still be 32 columns wide, else one buffer with the widest tile.
    int NT = 0, stages = 0, nbuf = 0;
    size_t smem = 0;
    const int ew_pref = persistent_epilogue_warps(true);
    int ew = ew_pref;
    // Merged mode (see LimbParams::merged_E): one set of D diagonals plus E low diagonals of the
    // second part instead of two full sets, so the tile can be wider (8 x 64 instead of 10 x 48 columns
    // of tensor memory for 3 x 3 limbs): fewer, wider MMAs and less operand traffic per output.
    const int delta = f.shift1 - f.shift2;
    int E = 0;
    const int64_t Kp2m = (f.K2 + 15) & ~(int64_t)15;
    if (delta >= 0 && delta <= 8 && f.shift1 >= 1 && f.shift1 <= 31 && !switches().no_merged) {
        const int e = (f.shift1 + 7) / 8;
        const int64_t a12 = f.addend1 + (int64_t)((uint64_t)f.addend2 << delta);
        // the one-pass epilogue is compiled for three extra diagonals and up to six main ones
        if (e == 3 && e <= Lb && D <= 6 && f.addend1 >= 0 && f.addend2 >= 0 && f.addend2 < (1ll << 40) &&
            (int64_t)pairs * (f.K1 + Kp2m) < 131072 && sum_fits64(La, Lb, f.K1 + f.K2, a12))
            E = e;
    }
    for (int bufs : {2, 1}) {
        for (int cand : {64, 48, 32, 16}) {
            if (bufs == 2 && cand < 32) continue;
            if (E && (bufs == 2 || cand == 48 || cand == 16)) continue;   // merged: one buffer, 8 or 16 columns per warp
            if (Lb * cand > 256 || (E ? (D + E) : 2 * bufs * D) * cand > 512) continue;
            const int ew_c = E ? 16 : ew_pref;        // the one-pass merged epilogue is written for 16 warps
            size_t st_b = (size_t)La * kTileM * kBlockK + (size_t)Lb * cand * kBlockK;
            // the merged epilogue stores straight from registers: no staging tile
            size_t staging = E ? 0 : persistent_staging(ew_c, cand);
            int ns = (int)((smem_max - staging - 1024) / st_b);
            if (ns < 2) continue;
            NT = cand;
            ew = ew_c;
            nbuf = bufs;
            stages = ns > 8 ? 8 : ns;
            smem = st_b * stages + staging + 1024;
            break;
        }
        if (NT) break;
    }
    if (!NT) return ZKDS_ERR_UNSUPPORTED;
    const int64_t Kp2 = (f.K2 + 15) & ~(int64_t)15;
    const int64_t pitch = f.K1 + Kp2;
    if (f.b_planes && (f.b_batch_rows < f.N || (((uintptr_t)f.b_planes) & 15))) return ZKDS_ERR_ARG;
    const int64_t a_rows = f.batches * f.M, b_rows = f.batches * (f.b_planes ? f.b_batch_rows : f.N);
    if (a_rows * La > 0x7fffff00ll || b_rows * Lb > 0x7fffff00ll) return ZKDS_ERR_UNSUPPORTED;
    const int64_t mt = (f.M + kTileM - 1) / kTileM, nt = (f.N + NT - 1) / NT;
    if (f.batches * mt * nt > 0x7fffffffll) return ZKDS_ERR_UNSUPPORTED;

    DeviceFlags* fl = flags_for_device();
    if (!fl) return ZKDS_ERR_WORKSPACE;
    int8_t* pa = (int8_t*)workspace((size_t)La * a_rows * pitch + 1024, 0);
    int8_t* pb = f.b_planes ? const_cast<int8_t*>(f.b_planes)
                            : (int8_t*)workspace((size_t)Lb * b_rows * pitch + 1024, 1);
    if (!pa || !pb) return ZKDS_ERR_WORKSPACE;
    unsigned long long* d_absmax = nullptr;
    if (f.dynamic_a) {
        unsigned long long* words = (unsigned long long*)workspace(8 * sizeof(uint64_t), 5);
        if (!words) return ZKDS_ERR_WORKSPACE;
        d_absmax = words + 2;
        ZKDS_CUDA(cudaMemsetAsync(d_absmax, 0, sizeof(uint64_t), st));
    }
    int rc = launch_split_t<int64_t>(f.A1, pa, La, f.batches, f.M, f.K1, f.K1, f.M * f.K1, f.K1, 1, 1,
                                     fl->overflow_dev, st, d_absmax, pitch);
    if (rc == ZKDS_OK)
        rc = launch_split_t<int64_t>(f.A2, pa + f.K1, La, f.batches, f.M, f.K2, Kp2, f.M * f.K2, f.K2, 1, 1,
                                     fl->overflow_dev, st, d_absmax, pitch, 0, 0, E ? delta : 0);
    if (rc == ZKDS_OK && !f.b_planes)
        rc = launch_split_t<int64_t>(f.B1, pb, Lb, f.batches, f.N, f.K1, f.K1, f.N * f.K1, f.K1, 1, 1,
                                     fl->overflow_dev, st, nullptr, pitch);
    if (rc == ZKDS_OK && !f.b_planes)
        rc = launch_split_t<int64_t>(f.B2, pb + f.K1, Lb, f.batches, f.N, f.K2, Kp2, f.N * f.K2, f.K2, 1, 1,
                                     fl->overflow_dev, st, nullptr, pitch);
    if (rc != ZKDS_OK) return rc;

    CUtensorMap tmA, tmB;
    if (!make_plane_map(&tmA, pa, (int64_t)La * a_rows, pitch, kTileM)) return ZKDS_ERR_UNSUPPORTED;
    if (!make_plane_map(&tmB, pb, (int64_t)Lb * b_rows, pitch, NT)) return ZKDS_ERR_UNSUPPORTED;

    LimbParams lp{};
    lp.La = La; lp.Lb = Lb; lp.NT = NT; lp.stages = stages;
    lp.k_switch = (int)(f.K1 / kBlockK);
    lp.kblocks = lp.k_switch + (int)((Kp2 + kBlockK - 1) / kBlockK);
    lp.k_extent = pitch;
    uint32_t cols = 32;
    while (cols < (uint32_t)((E ? (D + E) : 2 * nbuf * D) * NT)) cols <<= 1;
    lp.tmem_cols = cols;
    lp.nbuf = nbuf;
    lp.split_release = (nbuf == 1 && (E || !switches().no_split_release)) ? 1 : 0;
    lp.merged_E = E;
    lp.fold_epilogue = E ? 1 : 0;
    lp.M = f.M; lp.N = f.N; lp.batches = f.batches;
    lp.a_rows_per_limb = a_rows; lp.b_rows_per_limb = b_rows; lp.b_batch_rows = f.b_planes ? f.b_batch_rows : f.N;
    lp.b_batched = 1;
    lp.C = f.out; lp.R = nullptr; lp.c_sz = f.M * f.N; lp.c_sm = f.N;
    lp.addend = f.addend1; lp.shift = f.shift1; lp.addend2 = f.addend2; lp.shift2 = f.shift2;
    lp.r_legacy = 0;
    lp.error_flag = fl->dev;
    lp.fits64 = sum_fits64(La, Lb, Kmax, f.addend1) && sum_fits64(La, Lb, Kmax, f.addend2);
    if (E) {
        // the parked total carries both addends; the extra set only the scaled second one
        lp.addend2 = (int64_t)((uint64_t)f.addend2 << delta);
        lp.addend = f.addend1 + lp.addend2;
        lp.fits64 = 1;
    }
    lp.a_absmax = d_absmax;
    lp.overflow_flag = fl->overflow_dev;
    lp.ep_mul = f.ep_mul; lp.ep_div = f.ep_div;
    lp.causal_H = f.causal_H; lp.causal_start = f.causal_start; lp.mask_value = f.mask_value;
    lp.skip_tiles = (f.skip_tiles && f.causal_H) ? 1 : 0; lp.skip_H = f.causal_H; lp.skip_start = f.causal_start;
    int64_t panel = (32ll << 20) / ((int64_t)La * kTileM * pitch);
    if (panel < 1) panel = 1;
    if (panel > mt) panel = mt;
    lp.m_tiles = mt; lp.n_tiles = nt; lp.panel_m = panel;

    if (smem < 120 * 1024) smem = 120 * 1024;
    const int64_t total_tiles = f.batches * mt * nt;
    int ctas = sm_count();
    if (total_tiles < ctas) ctas = (int)total_tiles;
    cudaEvent_t* ev = timing_events();
    if (ev) ZKDS_CUDA(cudaEventRecord(ev[0], st));
    rc = launch_persistent(ew, ctas, smem, st, tmA, tmB, lp);
    if (ev) ZKDS_CUDA(cudaEventRecord(ev[1], st));
    if (ev && g_accumulate && rc == ZKDS_OK) {
        float ms = 0.f;
        ZKDS_CUDA(cudaEventSynchronize(ev[1]));
        ZKDS_CUDA(cudaEventElapsedTime(&ms, ev[0], ev[1]));
        int la_used = La;
        if (d_absmax) {
            unsigned long long h = 0;
            ZKDS_CUDA(cudaMemcpy(&h, d_absmax, sizeof(h), cudaMemcpyDeviceToHost));
            int need = limbs_needed(h);
            if (need < la_used) la_used = need;
        }
        if (switches().trace)
            fprintf(stderr, "scores_fused batches=%lld M=%lld N=%lld K=%lld+%lld La=%d(%d) Lb=%d NT=%d stages=%d fits64=%d: %.3f ms\n",
                    (long long)f.batches, (long long)f.M, (long long)f.N, (long long)f.K1, (long long)f.K2,
                    la_used, La, Lb, NT, stages, lp.fits64, ms);
        if (g_tot_launches < 256) {
            LaunchRecord& r = g_records[g_tot_launches];
            r.v[0] = (double)f.batches; r.v[1] = (double)f.M; r.v[2] = (double)f.N; r.v[3] = (double)(f.K1 + f.K2);
            r.v[4] = la_used; r.v[5] = Lb; r.v[6] = ms; r.v[7] = 2.0;
        }
        g_tot_ms += ms;
        g_tot_ops += 2.0 * (double)la_used * Lb * (double)f.batches * (double)f.M * (double)f.N * (double)(f.K1 + f.K2) *
                     issued_share(f.M, f.N, f.K1 + f.K2, NT, f.skip_tiles, 0, f.causal_H, f.causal_start);
        g_tot_launches += 1;
    }
    return rc;
}

// ------------------------------------------------------------------------------------
// GEMM for callers that must not allocate
// ------------------------------------------------------------------------------------
// Some hosts of this library cannot tolerate a memory allocation inside a call: a serving
// loop that has handed every byte of the GPU to its own pool (so a cudaMalloc here would
// fail or fragment it), or a latency-critical section where the implicit device
// synchronisation of cudaMalloc / cudaFree is not acceptable.  For them the limb planes and
// the status words live in the fixed array below, which is part of the loaded module: every
// GPU that loads the library holds kNoAllocBytes of it until the process exits.
//
// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a
// kernel could use; the device address is fetched once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the kernels
// receive.
constexpr size_t kNoAllocBytes = (size_t)64 << 20;   // 64 MiB
constexpr size_t kNoAllocHeader = 256;               // status words live in front of the planes
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
static unsigned char* g_noalloc_ptr[64];

size_t gemm_noalloc_capacity() { return kNoAllocBytes - kNoAllocHeader; }

size_t gemm_noalloc_bytes(int64_t Bdim, int64_t M, int64_t K, int64_t N, int a_limbs, int b_limbs)
{
    const int64_t Kp = (K + 15) & ~(int64_t)15;
    size_t a = ((size_t)a_limbs * Bdim * M * Kp + 1023) & ~(size_t)1023;
    size_t b = ((size_t)b_limbs * N * Kp + 1023) & ~(size_t)1023;
    return a + b;
}

int launch_gemm_noalloc(const Contraction& p, int La, int Lb, cudaStream_t st)
{
    int dev = 0;
    ZKDS_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return ZKDS_ERR_ARG;
    if (!g_noalloc_ptr[dev]) {
        // first call on this device: resolve the device address of the static array
        void* sym = nullptr;
        ZKDS_CUDA(cudaGetSymbolAddress(&sym, g_noalloc_scratch));
        if (!sym) return ZKDS_ERR_WORKSPACE;
        g_noalloc_ptr[dev] = (unsigned char*)sym;
    }
    unsigned char* base = g_noalloc_ptr[dev];
    // header: [0] device error word, [1] limb overflow word, [2..5] two 64-bit range words
    int* d_err = (int*)base;
    unsigned* d_ovf = (unsigned*)(base + 4);
    uint64_t* d_range = (uint64_t*)(base + 8);
    // the array keeps what the previous call left: the status words must start at zero
    ZKDS_CUDA(cudaMemsetAsync(base, 0, kNoAllocHeader, st));

    if (p.K <= 0) return ZKDS_ERR_UNSUPPORTED;
    if (La <= 0 || Lb <= 0) {
        int rc = launch_absmax(p.A, 64, p.batches, p.M, p.K, p.a_sz, p.a_sm, 1, p.a_div, d_range, st);
        if (rc != ZKDS_OK) return rc;
        rc = launch_absmax(p.B, p.b_bits, 1, p.N, p.K, 0, p.b_sn, p.b_sk, p.b_div, d_range + 1, st);
        if (rc != ZKDS_OK) return rc;
        uint64_t h[2] = {0, 0};
        ZKDS_CUDA(cudaMemcpyAsync(h, d_range, sizeof(h), cudaMemcpyDeviceToHost, st));
        ZKDS_CUDA(cudaStreamSynchronize(st));
        if (La <= 0) La = limbs_needed(h[0]);
        if (Lb <= 0) Lb = limbs_needed(h[1]);
    }
    if (La > 9 || Lb > 9) return ZKDS_ERR_UNSUPPORTED;
    const int D = La + Lb - 1;
    const int pairs = La < Lb ? La : Lb;
    if ((int64_t)pairs * p.K >= 131072) return ZKDS_ERR_UNSUPPORTED;
    const size_t smem_max = 227 * 1024 - 4096;
    int NT = 0;
    for (int cand : {128, 64, 32, 16}) {
        if (Lb * cand > 256 || D * cand > 512) continue;
        size_t stage = (size_t)La * kTileM * kBlockK + (size_t)Lb * cand * kBlockK;
        if (smem_max / stage < 2) continue;
        NT = cand;
        break;
    }
    if (!NT) return ZKDS_ERR_UNSUPPORTED;
    while (NT > 16 && p.N <= NT / 2) NT /= 2;
    const size_t stage = (size_t)La * kTileM * kBlockK + (size_t)Lb * NT * kBlockK;
    int stages = (int)(smem_max / stage);
    if (stages > 8) stages = 8;
    const int64_t Kp = (p.K + 15) & ~(int64_t)15;
    const int64_t a_rows = p.batches * p.M, b_rows = p.N;
    const int64_t mt = (p.M + kTileM - 1) / kTileM, nt = (p.N + NT - 1) / NT;
    if (mt > 0x7fffffffll || nt > 65535 || p.batches > 65535) return ZKDS_ERR_UNSUPPORTED;
    if (gemm_noalloc_bytes(p.batches, p.M, p.K, p.N, La, Lb) > gemm_noalloc_capacity())
        return ZKDS_ERR_RANGE;

    int8_t* pa = (int8_t*)(base + kNoAllocHeader);
    int8_t* pb = pa + (((size_t)La * a_rows * Kp + 1023) & ~(size_t)1023);
    int rc = launch_split_t<int64_t>(p.A, pa, La, p.batches, p.M, p.K, Kp, p.a_sz, p.a_sm, 1, p.a_div,
                                     d_ovf, st);
    if (rc != ZKDS_OK) return rc;
    if (p.b_bits == 32)
        rc = launch_split_t<int32_t>((const int32_t*)p.B, pb, Lb, 1, p.N, p.K, Kp, 0, p.b_sn, p.b_sk,
                                     p.b_div, d_ovf, st);
    else
        rc = launch_split_t<int64_t>((const int64_t*)p.B, pb, Lb, 1, p.N, p.K, Kp, 0, p.b_sn, p.b_sk,
                                     p.b_div, d_ovf, st);
    if (rc != ZKDS_OK) return rc;

    CUtensorMap tmA, tmB;
    if (!make_plane_map(&tmA, pa, (int64_t)La * a_rows, Kp, kTileM)) return ZKDS_ERR_UNSUPPORTED;
    if (!make_plane_map(&tmB, pb, (int64_t)Lb * b_rows, Kp, NT)) return ZKDS_ERR_UNSUPPORTED;

    LimbParams lp{};
    lp.La = La; lp.Lb = Lb; lp.NT = NT; lp.stages = stages;
    lp.kblocks = (int)((Kp + kBlockK - 1) / kBlockK);
    uint32_t cols = 32;
    while (cols < (uint32_t)(D * NT)) cols <<= 1;
    lp.tmem_cols = cols;
    lp.M = p.M; lp.N = p.N; lp.batches = p.batches;
    lp.a_rows_per_limb = a_rows; lp.b_rows_per_limb = b_rows;
    lp.b_batched = 0;
    lp.C = p.C; lp.R = p.R; lp.c_sz = p.c_sz; lp.c_sm = p.c_sm;
    lp.addend = p.addend; lp.shift = p.shift; lp.r_legacy = p.r_legacy;
    lp.error_flag = d_err;
    lp.fits64 = sum_fits64(La, Lb, p.K, p.addend);

    size_t smem = stage * stages + 1024;
    if (smem < 120 * 1024) smem = 120 * 1024;
    { int rc_a = allow_big_smem(limb_gemm_kernel, g_attr_onetile); if (rc_a != ZKDS_OK) return rc_a; }
    lp.m_tiles = mt; lp.n_tiles = nt; lp.panel_m = mt;
    if (mt * nt > 0x7fffffffll) return ZKDS_ERR_UNSUPPORTED;
    dim3 grid((unsigned)(mt * nt), 1, (unsigned)p.batches);
    limb_gemm_kernel<<<grid, kThreads, smem, st>>>(tmA, tmB, lp);
    rc = check_launch();
    if (rc != ZKDS_OK) return rc;
    // the status words are device memory: read them back (this waits for the kernels)
    int hs[2] = {0, 0};
    ZKDS_CUDA(cudaMemcpyAsync(hs, base, sizeof(hs), cudaMemcpyDeviceToHost, st));
    ZKDS_CUDA(cudaStreamSynchronize(st));
    if (hs[0]) return ZKDS_ERR_DEVICE;
    if (hs[1]) return ZKDS_ERR_RANGE;
    return ZKDS_OK;
}

}  // namespace zkds
