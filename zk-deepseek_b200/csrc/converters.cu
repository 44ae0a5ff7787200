// Float bit-pattern -> fixed-point integer converters.  The reference exports
// these three entry points (inference/int64_gemm.cu:92-221) but nothing calls
// them; they are kept so that the library exports the same symbol set.
// "1 << n" is evaluated the way the reference's device code does: in 32-bit int
// with the shift count clamped, so n >= 32 gives 0; a zero divisor (undefined in
// the reference) yields 0 here.
#include "common.cuh"
#include "kernels.h"

namespace zkds {

namespace {

__device__ __forceinline__ int32_t pow2_i32(int n) { return n < 32 ? (int32_t)(1u << n) : 0; }

__global__ void bf16_kernel(const uint16_t* in, int32_t* out, int64_t n, int rescale, int wkv_b)
{
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int bits = in[i];
    const int ex = ((bits >> 7) & 0xFF) - 127;
    const int frac = bits & 0x7F;
    if (ex == -127 && frac == 0) { out[i] = 0; return; }
    if (wkv_b && ex >= -1) { out[i] = 0x7FFFFFFF; return; }
    const int e2 = ex + (wkv_b ? 25 : rescale);
    const int mant = frac + 128;
    uint32_t v;
    if (e2 >= 0) v = (uint32_t)(mant * pow2_i32(e2));
    else {
        int32_t d = pow2_i32(-e2);
        v = d ? (uint32_t)(mant / d) : 0u;
    }
    if (bits & 0x8000) v = 0u - v;
    out[i] = (int32_t)v;
}

__global__ void f32_kernel(const uint32_t* in, int64_t* out, int64_t n, int rescale)
{
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t bits = in[i];
    const int ex = (int)((bits >> 23) & 0xFF) - 127;
    const int frac = (int)(bits & 0x7FFFFF);
    if (ex == -127 && frac == 0) { out[i] = 0; return; }
    const int e2 = ex + rescale;
    const int64_t mant = (int64_t)frac + 8388608;
    int64_t v;
    if (e2 >= 0) v = (int64_t)((uint64_t)mant * (uint64_t)(int64_t)pow2_i32(e2));
    else {
        int32_t d = pow2_i32(-e2);
        v = d ? mant / (int64_t)d : 0;
    }
    if (bits & 0x80000000u) v = (int64_t)(0 - (uint64_t)v);
    out[i] = v;
}

}  // namespace

int launch_bf16_to_int32(const uint16_t* in, int32_t* out, int rows, int cols, int rescale,
                         int wkv_b_variant, cudaStream_t st)
{
    int64_t n = (int64_t)rows * cols;
    if (n <= 0) return ZKDS_OK;
    bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(in, out, n, rescale, wkv_b_variant);
    return check_launch();
}

int launch_f32_to_int64(const uint32_t* in, int64_t* out, int rows, int cols, int rescale,
                        cudaStream_t st)
{
    int64_t n = (int64_t)rows * cols;
    if (n <= 0) return ZKDS_OK;
    f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(in, out, n, rescale);
    return check_launch();
}

}  // namespace zkds
