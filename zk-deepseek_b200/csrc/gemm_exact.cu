// CUDA-core contraction with a 128-bit accumulator per output: exact for every
// int64 input, any shape and any stride.  This is the path for shapes and operand
// ranges the tensor-core limb kernel does not take, and the in-library cross-check
// for it.  Semantics: inference/int64_gemm.cu:20-33 (GEMM) and :401-413, :442-455,
// :483-496, :525-536 (the four MLA einsums).
#include "common.cuh"
#include "kernels.h"

namespace zkds {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;
constexpr int THREADS = 256;

template <typename BT>
__global__ void __launch_bounds__(THREADS) exact_kernel(Contraction p)
{
    __shared__ int64_t As[TK][TM + 1];
    __shared__ int64_t Bs[TK][TN + 1];
    const int64_t z = blockIdx.z;
    const int64_t m0 = (int64_t)blockIdx.x * TM;
    const int64_t n0 = (int64_t)blockIdx.y * TN;
    const int64_t* A = p.A + z * p.a_sz;
    const BT* B = reinterpret_cast<const BT*>(p.B) + z * p.b_sz;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    const bool b_kmajor = (p.b_sk == 1);

    i128w acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = make_i128(p.addend);

    for (int64_t k0 = 0; k0 < p.K; k0 += TK) {
        // A tile: 64 rows x 16 k, k fastest
#pragma unroll
        for (int e = 0; e < (TM * TK) / THREADS; ++e) {
            int idx = e * THREADS + threadIdx.x;
            int kk = idx & (TK - 1), mm = idx >> 4;
            int64_t m = m0 + mm, k = k0 + kk;
            int64_t v = 0;
            if (m < p.M && k < p.K) {
                v = A[m * p.a_sm + k];
                if (p.a_div != 1) v = v / p.a_div;
            }
            As[kk][mm] = v;
        }
        // B tile: walk the contiguous direction fastest
#pragma unroll
        for (int e = 0; e < (TN * TK) / THREADS; ++e) {
            int idx = e * THREADS + threadIdx.x;
            int kk, nn;
            if (b_kmajor) { kk = idx & (TK - 1); nn = idx >> 4; }
            else { nn = idx & (TN - 1); kk = idx >> 6; }
            int64_t n = n0 + nn, k = k0 + kk;
            int64_t v = 0;
            if (n < p.N && k < p.K) {
                v = (int64_t)B[n * p.b_sn + k * p.b_sk];
                if (p.b_div != 1) v = v / p.b_div;
            }
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            int64_t a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mac128(acc[i][j], a[i], b[j]);
        }
        __syncthreads();
    }

    int64_t* C = p.C + z * p.c_sz;
    int64_t* R = p.R ? p.R + z * p.c_sz : nullptr;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int64_t m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int64_t n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            int64_t v = sar128_lo(acc[i][j], p.shift);
            if (p.addin) v = (int64_t)((uint64_t)v + (uint64_t)p.addin[z * p.c_sz + m * p.c_sm + n]);
            if (p.ep_div) {
                int64_t t = (int64_t)((uint64_t)v * (uint64_t)p.ep_mul);
                int64_t qd = t / p.ep_div, rd = t % p.ep_div;
                v = (rd != 0 && ((rd < 0) != (p.ep_div < 0))) ? qd - 1 : qd;
            }
            if (p.causal_H && n > p.causal_start + m / p.causal_H)
                v = (int64_t)((uint64_t)v + (uint64_t)p.mask_value);
            C[m * p.c_sm + n] = v;
            if (R) R[m * p.c_sm + n] = gemm_remainder(acc[i][j], p.shift, p.r_legacy);
        }
    }
}

}  // namespace

int launch_contraction_exact(const Contraction& p, cudaStream_t st)
{
    if (p.batches == 0 || p.M == 0 || p.N == 0) return ZKDS_OK;
    if (p.tile_group) return ZKDS_ERR_UNSUPPORTED;
    int64_t gx = (p.M + TM - 1) / TM, gy = (p.N + TN - 1) / TN;
    if (gx > 0x7fffffffll || gy > 65535) return ZKDS_ERR_RANGE;
    if (p.batches > 65535) {
        // grid.z is 16-bit: walk the batch dimension in slabs
        for (int64_t z0 = 0; z0 < p.batches; z0 += 65535) {
            Contraction q = p;
            q.batches = (p.batches - z0 < 65535) ? p.batches - z0 : 65535;
            q.A = p.A + z0 * p.a_sz;
            q.B = (const char*)p.B + z0 * p.b_sz * (p.b_bits / 8);
            q.C = p.C + z0 * p.c_sz;
            q.R = p.R ? p.R + z0 * p.c_sz : nullptr;
            q.addin = p.addin ? p.addin + z0 * p.c_sz : nullptr;     // same layout as C
            int rc = launch_contraction_exact(q, st);
            if (rc != ZKDS_OK) return rc;
        }
        return ZKDS_OK;
    }
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)p.batches);
    if (p.b_bits == 32) exact_kernel<int32_t><<<grid, THREADS, 0, st>>>(p);
    else if (p.b_bits == 64) exact_kernel<int64_t><<<grid, THREADS, 0, st>>>(p);
    else return ZKDS_ERR_ARG;
    return check_launch();
}

}  // namespace zkds
