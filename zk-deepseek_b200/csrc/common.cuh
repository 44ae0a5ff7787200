// Shared helpers for the int64 fixed-point kernels: status codes, launch checks,
// two-word 128-bit integer arithmetic and warp/block reductions.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// Status codes returned by every *_v2 / zkds_* entry point.
#define ZKDS_OK 0
#define ZKDS_ERR_ARG 1        // null pointer, negative or unsupported size, bad flag
#define ZKDS_ERR_RANGE 2      // extent does not fit the entry point's index type
#define ZKDS_ERR_CUDA 3       // a CUDA runtime call or launch failed (see zkds_last_cuda_error)
#define ZKDS_ERR_WORKSPACE 4  // scratch memory could not be provided
#define ZKDS_ERR_DEVICE 5     // a kernel reported a bounded wait that ran out
#define ZKDS_ERR_UNSUPPORTED 6

namespace zkds {

int set_cuda_error(cudaError_t e);           // records e, returns ZKDS_ERR_CUDA (or OK)
int check_launch();                          // cudaGetLastError -> status

#define ZKDS_CUDA(expr)                                   \
    do {                                                  \
        cudaError_t _e = (expr);                          \
        if (_e != cudaSuccess) return zkds::set_cuda_error(_e); \
    } while (0)

// ---- 128-bit two's complement value as two 64-bit words -----------------
struct i128w {
    uint64_t lo;
    int64_t hi;
};

__device__ __forceinline__ i128w make_i128(int64_t v) { return {(uint64_t)v, v >> 63}; }

__device__ __forceinline__ i128w add128(i128w a, i128w b)
{
    i128w r;
    r.lo = a.lo + b.lo;
    r.hi = (int64_t)((uint64_t)a.hi + (uint64_t)b.hi + (r.lo < a.lo ? 1ull : 0ull));
    return r;
}

__device__ __forceinline__ i128w sub128(i128w a, i128w b)
{
    i128w r;
    r.lo = a.lo - b.lo;
    r.hi = (int64_t)((uint64_t)a.hi - (uint64_t)b.hi - (a.lo < b.lo ? 1ull : 0ull));
    return r;
}

// signed 64 x 64 -> 128
__device__ __forceinline__ i128w mul64x64(int64_t a, int64_t b)
{
    i128w r;
    r.lo = (uint64_t)a * (uint64_t)b;
    r.hi = __mul64hi(a, b);
    return r;
}

// acc += a * b (signed, 128-bit accumulate)
__device__ __forceinline__ void mac128(i128w& acc, int64_t a, int64_t b)
{
    uint64_t lo = (uint64_t)a * (uint64_t)b;
    int64_t hi = __mul64hi(a, b);
    uint64_t nlo = acc.lo + lo;
    acc.hi = (int64_t)((uint64_t)acc.hi + (uint64_t)hi + (nlo < lo ? 1ull : 0ull));
    acc.lo = nlo;
}

// low 64 bits of (v >> s), arithmetic, 0 <= s <= 127
__device__ __forceinline__ int64_t sar128_lo(i128w v, int s)
{
    if (s == 0) return (int64_t)v.lo;
    if (s < 64) return (int64_t)((v.lo >> s) | ((uint64_t)v.hi << (64 - s)));
    if (s == 64) return v.hi;
    return v.hi >> (s - 64);
}

// remainder written next to a GEMM quotient.
//   legacy = 0: sum mod 2^s, truncated to 64 bits
//   legacy = 1: what the reference binary returns for "sum & ((1 << s) - 1)" with a 32-bit
//               "1" (int64_gemm.cu:22): 2^s-1 as mask for s <= 31, the low 32 bits of the
//               sum for every s >= 32 (observed on a B200, nvcc 12.9 build)
__device__ __forceinline__ int64_t gemm_remainder(i128w v, int s, int legacy)
{
    if (legacy) {
        uint64_t m = (s >= 0 && s <= 31) ? ((1ull << s) - 1ull) : 0xFFFFFFFFull;
        return (int64_t)(v.lo & m);
    }
    if (s <= 0) return 0;
    if (s >= 64) return (int64_t)v.lo;
    return (int64_t)(v.lo & ((1ull << s) - 1ull));
}

// ---- reductions --------------------------------------------------------------
__device__ __forceinline__ int64_t warp_max_i64(int64_t v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        int64_t t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    return v;
}

__device__ __forceinline__ int64_t warp_sum_i64(int64_t v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint64_t warp_max_u64(uint64_t v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        uint64_t t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    return v;
}

}  // namespace zkds
