// Tensor-core contraction on signed 8-bit limbs (placeholder translation unit: the
// operand range reduction lives here; the tcgen05 kernel follows).
#include "common.cuh"
#include "kernels.h"

namespace zkds {

namespace {

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
        // balanced digits reach further down than up: -128 * 256^k needs no extra limb
        if (v < 0 && a) a -= 1;
        best = a > best ? a : best;
    }
    best = warp_max_u64(best);
    if ((threadIdx.x & 31) == 0 && best) atomicMax((unsigned long long*)out, (unsigned long long)best);
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

int launch_contraction_limb(const Contraction&, int, int, cudaStream_t) { return ZKDS_ERR_UNSUPPORTED; }

}  // namespace zkds
