// extern "C" surface of libint64gemm.so: argument checks, dispatch between the
// tensor-core limb kernel and the exact CUDA-core kernel, the library-owned scratch
// arenas, and the 21 entry points of the reference library with their original
// names and argument lists (declared and documented in include/zkds_int64.h).
#include <math.h>
#include <stdio.h>
#include <mutex>
#include <stdlib.h>

#include "../../include/zkds_int64.h"
#include "common.cuh"
#include "kernels.h"

namespace zkds {

static thread_local int t_status = ZKDS_OK;
static thread_local int t_cuda_error = 0;

int set_cuda_error(cudaError_t e)
{
    if (e == cudaSuccess) return ZKDS_OK;
    t_cuda_error = (int)e;
    return ZKDS_ERR_CUDA;
}

int check_launch() { return set_cuda_error(cudaGetLastError()); }

static constexpr int kMaxDevices = 64;
static constexpr int kSlots = 8;

struct Arena {
    void* ptr[kSlots] = {};
    size_t cap[kSlots] = {};
    int sms = 0;
};
static Arena g_arena[kMaxDevices];
static std::mutex g_mu;

const Switches& switches()
{
    static const Switches sw = [] {
        Switches v{};
        auto on = [](const char* n) { return getenv(n) != nullptr; };
        auto num = [](const char* n, int dflt) { const char* e = getenv(n); return e ? atoi(e) : dflt; };
        v.wait_profile = on("ZKDS_WAIT_PROFILE");
        v.trace = on("ZKDS_TRACE");
        v.no_persistent = on("ZKDS_NO_PERSISTENT");
        v.no_persistent_grouped = on("ZKDS_NO_PERSISTENT_GROUPED");
        v.no_merged = on("ZKDS_NO_MERGED");
        v.no_split_release = on("ZKDS_NO_SPLIT_RELEASE");
        v.no_backoff = on("ZKDS_NO_BACKOFF");
        v.no_split_k = on("ZKDS_NO_SPLIT_K");
        v.split_generic = on("ZKDS_SPLIT_GENERIC");
        v.softmax_generic = on("ZKDS_SOFTMAX_GENERIC");
        v.rms_staged = on("ZKDS_RMS_STAGED");
        v.rms_nostage = on("ZKDS_RMS_NOSTAGE");
        v.epi_warps = num("ZKDS_EPI_WARPS", 0);
        v.tile_nt = num("ZKDS_TILE_NT", 0);
        v.persistent_max_kb = num("ZKDS_PERSISTENT_MAX_KB", -1);
        return v;
    }();
    return sw;
}

int sm_count()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (g_arena[dev].sms == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_arena[dev].sms = n;
    }
    return g_arena[dev].sms;
}

void* workspace(size_t bytes, int slot) { return workspace_fresh(bytes, slot, nullptr); }

void* workspace_fresh(size_t bytes, int slot, size_t* fresh_bytes)
{
    if (fresh_bytes) *fresh_bytes = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (slot < 0 || slot >= kSlots) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    Arena& a = g_arena[dev];
    if (a.cap[slot] >= bytes && a.ptr[slot]) return a.ptr[slot];
    if (a.ptr[slot]) {
        // earlier launches may still read the old block
        if (cudaDeviceSynchronize() != cudaSuccess) return nullptr;
        cudaFree(a.ptr[slot]);
        a.ptr[slot] = nullptr;
        a.cap[slot] = 0;
    }
    size_t want = bytes + bytes / 4;
    want = (want + 255) & ~(size_t)255;
    void* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) {
        cudaGetLastError();
        want = (bytes + 255) & ~(size_t)255;
        if (cudaMalloc(&p, want) != cudaSuccess) {
            set_cuda_error(cudaGetLastError());
            return nullptr;
        }
    }
    a.ptr[slot] = p;
    a.cap[slot] = want;
    if (fresh_bytes) *fresh_bytes = want;
    return p;
}

static void free_arenas()
{
    std::lock_guard<std::mutex> lk(g_mu);
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) return;
    for (int d = 0; d < kMaxDevices; ++d) {
        bool any = false;
        for (int s = 0; s < kSlots; ++s) any |= g_arena[d].ptr[s] != nullptr;
        if (!any) continue;
        if (cudaSetDevice(d) != cudaSuccess) continue;
        cudaDeviceSynchronize();
        for (int s = 0; s < kSlots; ++s) {
            if (g_arena[d].ptr[s]) cudaFree(g_arena[d].ptr[s]);
            g_arena[d].ptr[s] = nullptr;
            g_arena[d].cap[s] = 0;
        }
    }
    cudaSetDevice(cur);
}

struct PlanesHandle {
    Planes pl;
    int device;
    int b_bits;
};

static int run_contraction(const Contraction& p, int a_limbs, int b_limbs, int flags,
                           cudaStream_t st, const Planes* pre_b = nullptr)
{
    const int algo = flags & ZKDS_ALGO_MASK;
    if (algo == 3) return ZKDS_ERR_ARG;
    if (p.batches < 0 || p.M < 0 || p.N < 0 || p.K < 0) return ZKDS_ERR_ARG;
    if (p.batches == 0 || p.M == 0 || p.N == 0) return ZKDS_OK;
    if (!p.C || (p.K > 0 && (!p.A || (!p.B && !pre_b)))) return ZKDS_ERR_ARG;
    if (p.a_div == 0 || p.b_div == 0) return ZKDS_ERR_ARG;
    if (p.shift < 0 || p.shift > 127) return ZKDS_ERR_ARG;
    if (p.b_bits != 32 && p.b_bits != 64) return ZKDS_ERR_ARG;
    if (algo == ZKDS_ALGO_EXACT) return pre_b ? ZKDS_ERR_ARG : launch_contraction_exact(p, st);
    if (pre_b) b_limbs = pre_b->L;
    Contraction pd = p;
    pd.dynamic_a = ((flags & ZKDS_LIMBS_DYNAMIC) && a_limbs > 0) ? 1 : 0;

    if (p.skip_k && a_limbs <= 0) return ZKDS_ERR_ARG;   // the unread part of A may hold anything
    if (a_limbs <= 0 || b_limbs <= 0) {
        uint64_t* d = (uint64_t*)workspace(2 * sizeof(uint64_t), 5);
        if (!d) return ZKDS_ERR_WORKSPACE;
        ZKDS_CUDA(cudaMemsetAsync(d, 0, 2 * sizeof(uint64_t), st));
        int rc = launch_absmax(p.A, 64, p.batches, p.M, p.K, p.a_sz, p.a_sm, 1, p.a_div, d, st);
        if (rc != ZKDS_OK) return rc;
        // B may be shared by every batch (b_sz == 0)
        if (b_limbs <= 0) {
            rc = launch_absmax(p.B, p.b_bits, p.b_sz ? p.batches : 1, p.N, p.K, p.b_sz, p.b_sn, p.b_sk,
                               p.b_div, d + 1, st);
            if (rc != ZKDS_OK) return rc;
        }
        uint64_t h[2];
        ZKDS_CUDA(cudaMemcpyAsync(h, d, sizeof(h), cudaMemcpyDeviceToHost, st));
        ZKDS_CUDA(cudaStreamSynchronize(st));
        if (a_limbs <= 0) a_limbs = limbs_needed(h[0]);
        if (b_limbs <= 0) b_limbs = limbs_needed(h[1]);
    }
    int rc = launch_contraction_limb(pd, a_limbs, b_limbs, pre_b, st);
    if (rc == ZKDS_ERR_UNSUPPORTED && algo == ZKDS_ALGO_AUTO && !pre_b) rc = launch_contraction_exact(p, st);
    return rc;
}

static Contraction gemm_problem(const int64_t* A, const void* B, int b_bits, int64_t* C, int64_t* R,
                                int64_t a_r, int64_t b_r, int64_t s, int64_t Bdim, int64_t M,
                                int64_t K, int64_t N, int legacy_r)
{
    Contraction p{};
    p.A = A; p.B = B; p.b_bits = b_bits; p.C = C; p.R = R;
    p.batches = Bdim; p.M = M; p.N = N; p.K = K;
    p.a_sz = M * K; p.a_sm = K;
    p.b_sz = 0; p.b_sn = K; p.b_sk = 1;
    p.c_sz = M * N; p.c_sm = N;
    p.a_div = a_r; p.b_div = b_r;
    p.addend = 0;
    p.shift = (s < 0 || s > 127) ? -1 : (int)s;
    p.r_legacy = legacy_r;
    return p;
}

// which: 0 bshd,hdc->bshc  1 bshc,btc->bsht  2 bsht,btc->bshc  3 bshc,hdc->bshd
static Contraction einsum_problem(int which, const int64_t* A, const void* B, int64_t* out,
                                  int64_t r, int64_t Bn, int64_t S, int64_t H, int64_t X, int64_t Y)
{
    Contraction p{};
    p.A = A; p.B = B; p.C = out; p.R = nullptr;
    p.a_div = 1; p.b_div = 1;
    p.shift = (r < 0 || r > 127) ? -1 : (int)r;
    p.addend = (which == 3) ? 0 : r / 2;
    p.r_legacy = 0;
    switch (which) {
    case 0: {  // X = D (contracted), Y = C
        p.b_bits = 32; p.batches = H; p.M = Bn * S; p.K = X; p.N = Y;
        p.a_sz = X; p.a_sm = H * X;
        p.b_sz = X * Y; p.b_sn = 1; p.b_sk = Y;
        p.c_sz = Y; p.c_sm = H * Y;
        break;
    }
    case 1: {  // X = T, Y = C (contracted)
        p.b_bits = 64; p.batches = Bn; p.M = S * H; p.K = Y; p.N = X;
        p.a_sz = S * H * Y; p.a_sm = Y;
        p.b_sz = X * Y; p.b_sn = Y; p.b_sk = 1;
        p.c_sz = S * H * X; p.c_sm = X;
        break;
    }
    case 2: {  // X = T (contracted), Y = C
        p.b_bits = 64; p.batches = Bn; p.M = S * H; p.K = X; p.N = Y;
        p.a_sz = S * H * X; p.a_sm = X;
        p.b_sz = X * Y; p.b_sn = 1; p.b_sk = Y;
        p.c_sz = S * H * Y; p.c_sm = Y;
        break;
    }
    default: {  // X = D, Y = C (contracted)
        p.b_bits = 32; p.batches = H; p.M = Bn * S; p.K = Y; p.N = X;
        p.a_sz = Y; p.a_sm = H * Y;
        p.b_sz = X * Y; p.b_sn = Y; p.b_sk = 1;
        p.c_sz = X; p.c_sm = H * X;
        break;
    }
    }
    return p;
}

static int finish(int rc, const char* who)
{
    t_status = rc;
    if (rc != ZKDS_OK)
        fprintf(stderr, "libint64gemm: %s failed: %s%s%s\n", who, zkds_status_string(rc),
                rc == ZKDS_ERR_CUDA ? ": " : "",
                rc == ZKDS_ERR_CUDA ? cudaGetErrorString((cudaError_t)t_cuda_error) : "");
    return rc;
}

static int make_lut(int64_t* lut, int kind)
{
    if (!lut) return ZKDS_ERR_ARG;
    // the exponent is formed in float and widened, as the reference's host code does
    for (int i = 0; i < 256; ++i) {
        float e = (kind <= 1) ? i * (-1.0f) / 256 : i * 1.0f / 256;
        double scale = kind == 0 ? 524288.0 : kind == 1 ? 2097152.0 : kind == 2 ? 8388608.0
                                                                                : 33554432.0;
        lut[i] = (int64_t)(pow(2.0, (double)e) * scale);
    }
    return (kind >= 0 && kind <= 3) ? ZKDS_OK : ZKDS_ERR_ARG;
}

}  // namespace zkds

using namespace zkds;

#define ST(s) ((cudaStream_t)(s))

extern "C" {

int zkds_last_status(void) { return t_status; }
int zkds_last_cuda_error(void) { return t_cuda_error; }
const char* zkds_version(void) { return "zkds-int64 0.1 (sm_100a)"; }
void zkds_shutdown(void) { free_arenas(); }

const char* zkds_status_string(int s)
{
    switch (s) {
    case ZKDS_OK: return "ok";
    case ZKDS_ERR_ARG: return "invalid argument";
    case ZKDS_ERR_RANGE: return "extent out of range";
    case ZKDS_ERR_CUDA: return "CUDA error";
    case ZKDS_ERR_WORKSPACE: return "scratch memory unavailable";
    case ZKDS_ERR_DEVICE: return "device-side wait ran out";
    case ZKDS_ERR_UNSUPPORTED: return "not supported by the selected algorithm";
    default: return "unknown status";
    }
}

int zkds_gemm(const int64_t* A, const void* B, int b_bits, int64_t* C, int64_t* R, int64_t a_rescale,
              int64_t b_rescale, int64_t c_rescale, int64_t Bdim, int64_t M, int64_t K, int64_t N,
              int a_limbs, int b_limbs, int flags, void* stream)
{
    Contraction p = gemm_problem(A, B, b_bits, C, R, a_rescale, b_rescale, c_rescale, Bdim, M, K, N,
                                 (flags & ZKDS_REMAINDER_LEGACY) ? 1 : 0);
    return finish(run_contraction(p, a_limbs, b_limbs, flags, ST(stream)), "zkds_gemm");
}

int zkds_gemm_noalloc(const int64_t* A, const void* B, int b_bits, int64_t* C, int64_t* R,
                      int64_t a_rescale, int64_t b_rescale, int64_t c_rescale, int64_t Bdim, int64_t M,
                      int64_t K, int64_t N, int a_limbs, int b_limbs, int flags, void* stream)
{
    Contraction p = gemm_problem(A, B, b_bits, C, R, a_rescale, b_rescale, c_rescale, Bdim, M, K, N,
                                 (flags & ZKDS_REMAINDER_LEGACY) ? 1 : 0);
    int rc;
    if (Bdim < 0 || M < 0 || K < 0 || N < 0 || a_limbs < 0 || b_limbs < 0) rc = ZKDS_ERR_ARG;
    else if (Bdim == 0 || M == 0 || N == 0) rc = ZKDS_OK;
    else if (!A || !B || !C || a_rescale == 0 || b_rescale == 0 || p.shift < 0 ||
             (b_bits != 32 && b_bits != 64))
        rc = ZKDS_ERR_ARG;
    else if (a_limbs > 0 && b_limbs > 0 &&
             gemm_noalloc_bytes(Bdim, M, K, N, a_limbs, b_limbs) > gemm_noalloc_capacity()) {
        fprintf(stderr,
                "libint64gemm: zkds_gemm_noalloc: this shape needs %zu bytes of limb planes, the fixed "
                "scratch array holds %zu\n",
                gemm_noalloc_bytes(Bdim, M, K, N, a_limbs, b_limbs), gemm_noalloc_capacity());
        rc = ZKDS_ERR_RANGE;
    } else
        rc = launch_gemm_noalloc(p, a_limbs, b_limbs, ST(stream));
    return finish(rc, "zkds_gemm_noalloc");
}

unsigned long long zkds_gemm_noalloc_capacity(void) { return (unsigned long long)gemm_noalloc_capacity(); }

unsigned long long zkds_gemm_noalloc_bytes(int64_t Bdim, int64_t M, int64_t K, int64_t N, int a_limbs,
                                           int b_limbs)
{
    return (unsigned long long)gemm_noalloc_bytes(Bdim, M, K, N, a_limbs, b_limbs);
}

int zkds_einsum_bshd_hdc_bshc(const int64_t* q, const int32_t* W, int64_t* out, int64_t rescale,
                              int64_t B, int64_t S, int64_t H, int64_t D, int64_t C, int a_limbs,
                              int b_limbs, int flags, void* stream)
{
    Contraction p = einsum_problem(0, q, W, out, rescale, B, S, H, D, C);
    return finish(run_contraction(p, a_limbs, b_limbs, flags, ST(stream)),
                  "zkds_einsum_bshd_hdc_bshc");
}

int zkds_einsum_bshc_btc_bsht(const int64_t* A, const int64_t* KV, int64_t* out, int64_t rescale,
                              int64_t B, int64_t S, int64_t H, int64_t T, int64_t C, int a_limbs,
                              int b_limbs, int flags, void* stream)
{
    Contraction p = einsum_problem(1, A, KV, out, rescale, B, S, H, T, C);
    return finish(run_contraction(p, a_limbs, b_limbs, flags, ST(stream)),
                  "zkds_einsum_bshc_btc_bsht");
}

int zkds_einsum_bsht_btc_bshc(const int64_t* P, const int64_t* KV, int64_t* out, int64_t rescale,
                              int64_t B, int64_t S, int64_t H, int64_t T, int64_t C, int a_limbs,
                              int b_limbs, int flags, void* stream)
{
    Contraction p = einsum_problem(2, P, KV, out, rescale, B, S, H, T, C);
    return finish(run_contraction(p, a_limbs, b_limbs, flags, ST(stream)),
                  "zkds_einsum_bsht_btc_bshc");
}

int zkds_einsum_bshc_hdc_bshd(const int64_t* A, const int32_t* W, int64_t* out, int64_t rescale,
                              int64_t B, int64_t S, int64_t H, int64_t D, int64_t C, int a_limbs,
                              int b_limbs, int flags, void* stream)
{
    Contraction p = einsum_problem(3, A, W, out, rescale, B, S, H, D, C);
    return finish(run_contraction(p, a_limbs, b_limbs, flags, ST(stream)),
                  "zkds_einsum_bshc_hdc_bshd");
}

int zkds_einsum_bshc_btc_bsht_ex(const int64_t* A, const int64_t* KV, int64_t* out, int64_t rescale,
                                 int64_t B, int64_t S, int64_t H, int64_t T, int64_t C,
                                 const int64_t* addin, int64_t ep_mul, int64_t ep_div, int causal,
                                 int64_t start_pos, int64_t mask_value, int a_limbs, int b_limbs,
                                 int flags, void* stream)
{
    Contraction p = einsum_problem(1, A, KV, out, rescale, B, S, H, T, C);
    p.addin = addin; p.ep_mul = ep_mul; p.ep_div = ep_div;
    p.causal_H = causal ? H : 0; p.causal_start = start_pos; p.mask_value = mask_value;
    if (causal && (flags & ZKDS_CAUSAL_SKIP)) { p.skip_tiles = 1; p.skip_H = H; p.skip_start = start_pos; }
    return finish(run_contraction(p, a_limbs, b_limbs, flags, ST(stream)),
                  "zkds_einsum_bshc_btc_bsht_ex");
}

int zkds_mla_scores(const int64_t* q_abs, const int64_t* kv, const int64_t* q_pe, const int64_t* pe,
                    int64_t* out, int64_t B, int64_t S, int64_t H, int64_t T, int64_t C1, int64_t C2,
                    int64_t rescale1, int64_t rescale2, int64_t ep_mul, int64_t ep_div, int causal,
                    int64_t start_pos, int64_t mask_value, int a_limbs, int b_limbs, int flags, void* stream)
{
    if (B < 0 || S < 0 || H < 0 || T < 0 || C1 <= 0 || C2 <= 0 || rescale1 < 0 || rescale1 > 127 ||
        rescale2 < 0 || rescale2 > 127)
        return finish(ZKDS_ERR_ARG, "zkds_mla_scores");
    if (B == 0 || S == 0 || H == 0 || T == 0) return finish(ZKDS_OK, "zkds_mla_scores");
    if (!q_abs || !kv || !q_pe || !pe || !out) return finish(ZKDS_ERR_ARG, "zkds_mla_scores");
    cudaStream_t st = ST(stream);
    if (a_limbs <= 0 || b_limbs <= 0) {
        uint64_t* d = (uint64_t*)workspace(8 * sizeof(uint64_t), 5);
        if (!d) return finish(ZKDS_ERR_WORKSPACE, "zkds_mla_scores");
        int rc = set_cuda_error(cudaMemsetAsync(d, 0, 3 * sizeof(uint64_t), st));
        if (rc == ZKDS_OK) rc = launch_absmax(q_abs, 64, B, S * H, C1, S * H * C1, C1, 1, 1, d, st);
        if (rc == ZKDS_OK) rc = launch_absmax(q_pe, 64, B, S * H, C2, S * H * C2, C2, 1, 1, d + 2, st);
        if (rc == ZKDS_OK) rc = launch_absmax(kv, 64, B, T, C1, T * C1, C1, 1, 1, d + 1, st);
        if (rc == ZKDS_OK) rc = launch_absmax(pe, 64, B, T, C2, T * C2, C2, 1, 1, d + 1, st);
        uint64_t h[3] = {0, 0, 0};
        if (rc == ZKDS_OK) rc = set_cuda_error(cudaMemcpyAsync(h, d, sizeof(h), cudaMemcpyDeviceToHost, st));
        if (rc == ZKDS_OK) rc = set_cuda_error(cudaStreamSynchronize(st));
        if (rc != ZKDS_OK) return finish(rc, "zkds_mla_scores");
        // the kernel may scale q_pe by 2^(rescale1 - rescale2) while splitting it (one shared set of
        // accumulators): the limbs have to hold the scaled values
        const int64_t dl = rescale1 - rescale2;
        uint64_t pe_max = h[2];
        if (dl > 0 && dl <= 8) pe_max = (pe_max >> (63 - dl)) ? ~0ull : ((pe_max + 1) << dl);
        if (pe_max > h[0]) h[0] = pe_max;
        if (a_limbs <= 0) { a_limbs = limbs_needed(h[0]); flags &= ~ZKDS_LIMBS_DYNAMIC; }
        if (b_limbs <= 0) b_limbs = limbs_needed(h[1]);
    }
    FusedScores f{};
    f.A1 = q_abs; f.A2 = q_pe; f.B1 = kv; f.B2 = pe; f.out = out;
    f.batches = B; f.M = S * H; f.N = T; f.K1 = C1; f.K2 = C2;
    f.addend1 = rescale1 / 2; f.addend2 = rescale2 / 2;       // int64_gemm.cu:442
    f.shift1 = (int)rescale1; f.shift2 = (int)rescale2;
    f.ep_mul = ep_mul; f.ep_div = ep_div;
    f.causal_H = causal ? H : 0; f.causal_start = start_pos; f.mask_value = mask_value;
    f.dynamic_a = (flags & ZKDS_LIMBS_DYNAMIC) ? 1 : 0;
    f.skip_tiles = (flags & ZKDS_CAUSAL_SKIP) ? 1 : 0;
    // ZKDS_ERR_UNSUPPORTED is an expected answer here (the caller then runs the two contractions
    // separately), so it is returned without the stderr line
    int rc = launch_scores_fused(f, a_limbs, b_limbs, st);
    if (rc == ZKDS_ERR_UNSUPPORTED) { t_status = rc; return rc; }
    return finish(rc, "zkds_mla_scores");
}

static int grouped_prepared(const int64_t* A, const int* row_index, const void* planes, const int* tile_group,
                            int64_t n_tiles, int64_t* C, int64_t a_rescale, int64_t addend, int64_t shift,
                            const int* group_shift, int64_t n_split, int a_limbs, int flags, void* stream);

int zkds_glu_prepared(const int64_t* r1, const int64_t* r2, int64_t ld, const int64_t* lut, int64_t rows,
                      const void* planes, const int* tile_group, int64_t* C, int64_t shift,
                      const int* group_shift, int64_t n_split, int a_limbs, int flags, void* stream)
{
    if (!planes || rows < 0 || a_limbs <= 0 || (group_shift && (n_split & 7)) || (tile_group && (rows & 127)))
        return finish(ZKDS_ERR_ARG, "zkds_glu_prepared");
    if (rows == 0) return finish(ZKDS_OK, "zkds_glu_prepared");
    if (!r1 || !r2 || !lut || !C) return finish(ZKDS_ERR_ARG, "zkds_glu_prepared");
    const PlanesHandle* hd = (const PlanesHandle*)planes;
    if (!glu_planes_supported(r1, r2, ld, hd->pl.K)) { t_status = ZKDS_ERR_UNSUPPORTED; return t_status; }
    Contraction p{};
    p.A = r1; p.B = nullptr; p.b_bits = hd->b_bits; p.C = C; p.R = nullptr;
    p.batches = 1; p.M = rows; p.N = hd->pl.rows; p.K = hd->pl.K;
    p.a_sz = 0; p.a_sm = ld;
    p.b_sz = tile_group ? 1 : 0; p.b_sn = 0; p.b_sk = 0;
    p.c_sz = 0; p.c_sm = hd->pl.rows;
    p.a_div = 1; p.b_div = 1;
    p.addend = 0;
    p.shift = (shift < 0 || shift > 127) ? -1 : (int)shift;
    p.tile_group = tile_group;
    p.group_shift = group_shift; p.n_split = n_split;
    p.glu_r2 = r2; p.glu_lut = lut;
    p.dynamic_a = (flags & ZKDS_LIMBS_DYNAMIC) ? 1 : 0;
    p.group_rows = !tile_group ? 0 : (flags & ZKDS_GROUP_ROWS_32) ? 32 : (flags & ZKDS_GROUP_ROWS_64) ? 64 : 0;
    if (p.shift < 0) return finish(ZKDS_ERR_ARG, "zkds_glu_prepared");
    int rc = launch_contraction_limb(p, a_limbs, 0, &hd->pl, ST(stream));
    if (rc == ZKDS_ERR_UNSUPPORTED) { t_status = rc; return rc; }
    return finish(rc, "zkds_glu_prepared");
}

int zkds_grouped_prepared(const int64_t* A, const void* planes, const int* tile_group, int64_t n_tiles,
                          int64_t* C, int64_t a_rescale, int64_t addend, int64_t shift,
                          const int* group_shift, int64_t n_split, int a_limbs, int flags, void* stream)
{
    return grouped_prepared(A, nullptr, planes, tile_group, n_tiles, C, a_rescale, addend, shift, group_shift,
                            n_split, a_limbs, flags, stream);
}

int zkds_grouped_gather_prepared(const int64_t* A, const int* row_index, const void* planes, const int* tile_group,
                                 int64_t n_tiles, int64_t* C, int64_t a_rescale, int64_t addend, int64_t shift,
                                 const int* group_shift, int64_t n_split, int a_limbs, int flags, void* stream)
{
    if (!row_index) return finish(ZKDS_ERR_ARG, "zkds_grouped_gather_prepared");
    return grouped_prepared(A, row_index, planes, tile_group, n_tiles, C, a_rescale, addend, shift, group_shift,
                            n_split, a_limbs, flags, stream);
}

static int grouped_prepared(const int64_t* A, const int* row_index, const void* planes, const int* tile_group,
                            int64_t n_tiles, int64_t* C, int64_t a_rescale, int64_t addend, int64_t shift,
                            const int* group_shift, int64_t n_split, int a_limbs, int flags, void* stream)
{
    if (!planes || !tile_group || n_tiles < 0 || (group_shift && (n_split & 7)))
        return finish(ZKDS_ERR_ARG, "zkds_grouped_prepared");
    if (row_index && a_limbs <= 0)      // measuring the range would have to follow the index too
        return finish(ZKDS_ERR_ARG, "zkds_grouped_gather_prepared");
    const PlanesHandle* hd = (const PlanesHandle*)planes;
    Contraction p{};
    p.A = A; p.B = nullptr; p.b_bits = hd->b_bits; p.C = C; p.R = nullptr;
    p.batches = 1; p.M = n_tiles * 128; p.N = hd->pl.rows; p.K = hd->pl.K;
    p.a_sz = 0; p.a_sm = hd->pl.K;
    p.b_sz = 1; p.b_sn = 0; p.b_sk = 0;
    p.c_sz = 0; p.c_sm = hd->pl.rows;
    p.a_div = a_rescale; p.b_div = 1;
    p.addend = addend;
    p.shift = (shift < 0 || shift > 127) ? -1 : (int)shift;
    p.tile_group = tile_group;
    p.a_row_index = row_index;
    p.group_shift = group_shift; p.n_split = n_split;
    p.group_rows = (flags & ZKDS_GROUP_ROWS_32) ? 32 : (flags & ZKDS_GROUP_ROWS_64) ? 64 : 0;
    int f = (flags & ~ZKDS_ALGO_MASK) | ZKDS_ALGO_LIMB;
    return finish(run_contraction(p, a_limbs, 0, f, ST(stream), &hd->pl), "zkds_grouped_prepared");
}

int zkds_einsum_bsht_btc_bshc_causal(const int64_t* P, const int64_t* KV, int64_t* out, int64_t rescale,
                                     int64_t B, int64_t S, int64_t H, int64_t T, int64_t C, int64_t start_pos,
                                     int a_limbs, int b_limbs, int flags, void* stream)
{
    Contraction p = einsum_problem(2, P, KV, out, rescale, B, S, H, T, C);
    p.skip_k = 1; p.skip_H = H; p.skip_start = start_pos;
    int f = (flags & ~ZKDS_ALGO_MASK) | ZKDS_ALGO_LIMB;     // only the limb kernel knows the causal layout
    return finish(run_contraction(p, a_limbs, b_limbs, f, ST(stream)), "zkds_einsum_bsht_btc_bshc_causal");
}

int zkds_softmax_pv(const int64_t* scores, const int64_t* KV, int64_t* out, const int64_t* lut,
                    int64_t rescale, int64_t B, int64_t S, int64_t H, int64_t T, int64_t C, int causal_skip,
                    int64_t start_pos, int a_limbs, int b_limbs, int flags, void* stream)
{
    if (B < 0 || S < 0 || H < 0 || T < 0 || C < 0 || rescale < 0 || rescale > 127 || start_pos < 0)
        return finish(ZKDS_ERR_ARG, "zkds_softmax_pv");
    if (B == 0 || S == 0 || H == 0 || C == 0) return finish(ZKDS_OK, "zkds_softmax_pv");
    if (T == 0 || !scores || !KV || !out || !lut) return finish(ZKDS_ERR_ARG, "zkds_softmax_pv");
    const int64_t Kp = (T + 15) & ~(int64_t)15;
    if (!softmax_planes_supported(scores, B * S * H, T, Kp)) { t_status = ZKDS_ERR_UNSUPPORTED; return t_status; }
    cudaStream_t st = ST(stream);
    Contraction p = einsum_problem(2, scores, KV, out, rescale, B, S, H, T, C);
    p.softmax_lut = lut; p.softmax_S = S;
    if (causal_skip) { p.skip_k = 1; p.skip_H = H; p.skip_start = start_pos; }
    p.dynamic_a = ((flags & ZKDS_LIMBS_DYNAMIC) && a_limbs > 0) ? 1 : 0;
    if (a_limbs <= 0) a_limbs = 3;
    if (b_limbs <= 0) {
        uint64_t* d = (uint64_t*)workspace(2 * sizeof(uint64_t), 5);
        if (!d) return finish(ZKDS_ERR_WORKSPACE, "zkds_softmax_pv");
        int rc = set_cuda_error(cudaMemsetAsync(d, 0, 2 * sizeof(uint64_t), st));
        if (rc == ZKDS_OK) rc = launch_absmax(KV, 64, B, C, T, T * C, 1, C, 1, d + 1, st);
        uint64_t h = 0;
        if (rc == ZKDS_OK) rc = set_cuda_error(cudaMemcpyAsync(&h, d + 1, sizeof(h), cudaMemcpyDeviceToHost, st));
        if (rc == ZKDS_OK) rc = set_cuda_error(cudaStreamSynchronize(st));
        if (rc != ZKDS_OK) return finish(rc, "zkds_softmax_pv");
        b_limbs = limbs_needed(h);
    }
    int rc = launch_contraction_limb(p, a_limbs, b_limbs, nullptr, st);
    if (rc == ZKDS_ERR_UNSUPPORTED) { t_status = rc; return rc; }
    return finish(rc, "zkds_softmax_pv");
}

int zkds_cache_planes_append(const int64_t* kv_new, const int64_t* pe_new, int8_t* score_planes,
                             int8_t* value_planes, int64_t B, int64_t S, int64_t C1, int64_t C2,
                             int64_t start_pos, int64_t capacity, int limbs, void* stream)
{
    if (B < 0 || S < 0 || (B && S && (!kv_new || !pe_new || !score_planes || !value_planes)))
        return finish(ZKDS_ERR_ARG, "zkds_cache_planes_append");
    return finish(launch_cache_planes_append(kv_new, pe_new, score_planes, value_planes, B, S, C1, C2, start_pos,
                                             capacity, limbs, ST(stream)),
                  "zkds_cache_planes_append");
}

int zkds_mla_scores_cached(const int64_t* q_abs, const int64_t* q_pe, const int8_t* score_planes,
                           int64_t capacity, int64_t* out, int64_t B, int64_t S, int64_t H, int64_t T,
                           int64_t C1, int64_t C2, int64_t rescale1, int64_t rescale2, int64_t ep_mul,
                           int64_t ep_div, int causal, int64_t start_pos, int64_t mask_value, int a_limbs,
                           int b_limbs, int flags, void* stream)
{
    if (B < 0 || S < 0 || H < 0 || T < 0 || C1 <= 0 || C2 <= 0 || rescale1 < 0 || rescale1 > 127 ||
        rescale2 < 0 || rescale2 > 127 || a_limbs <= 0 || b_limbs <= 0 || T > capacity)
        return finish(ZKDS_ERR_ARG, "zkds_mla_scores_cached");
    if (B == 0 || S == 0 || H == 0 || T == 0) return finish(ZKDS_OK, "zkds_mla_scores_cached");
    if (!q_abs || !q_pe || !score_planes || !out) return finish(ZKDS_ERR_ARG, "zkds_mla_scores_cached");
    FusedScores f{};
    f.A1 = q_abs; f.A2 = q_pe; f.B1 = nullptr; f.B2 = nullptr; f.out = out;
    f.b_planes = score_planes; f.b_batch_rows = capacity;
    f.batches = B; f.M = S * H; f.N = T; f.K1 = C1; f.K2 = C2;
    f.addend1 = rescale1 / 2; f.addend2 = rescale2 / 2;
    f.shift1 = (int)rescale1; f.shift2 = (int)rescale2;
    f.ep_mul = ep_mul; f.ep_div = ep_div;
    f.causal_H = causal ? H : 0; f.causal_start = start_pos; f.mask_value = mask_value;
    f.dynamic_a = (flags & ZKDS_LIMBS_DYNAMIC) ? 1 : 0;
    f.skip_tiles = (flags & ZKDS_CAUSAL_SKIP) ? 1 : 0;
    int rc = launch_scores_fused(f, a_limbs, b_limbs, ST(stream));
    if (rc == ZKDS_ERR_UNSUPPORTED) { t_status = rc; return rc; }
    return finish(rc, "zkds_mla_scores_cached");
}

int zkds_softmax_pv_cached(const int64_t* scores, const int8_t* value_planes, int64_t capacity, int64_t* out,
                           const int64_t* lut, int64_t rescale, int64_t B, int64_t S, int64_t H, int64_t T,
                           int64_t C, int causal_skip, int64_t start_pos, int a_limbs, int b_limbs, int flags,
                           void* stream)
{
    if (B < 0 || S < 0 || H < 0 || T < 0 || C < 0 || rescale < 0 || rescale > 127 || start_pos < 0 ||
        b_limbs <= 0 || T > capacity || (capacity & 15))
        return finish(ZKDS_ERR_ARG, "zkds_softmax_pv_cached");
    if (B == 0 || S == 0 || H == 0 || C == 0) return finish(ZKDS_OK, "zkds_softmax_pv_cached");
    if (T == 0 || !scores || !value_planes || !out || !lut) return finish(ZKDS_ERR_ARG, "zkds_softmax_pv_cached");
    const int64_t Kp = (T + 15) & ~(int64_t)15;
    if (!softmax_planes_supported(scores, B * S * H, T, Kp)) { t_status = ZKDS_ERR_UNSUPPORTED; return t_status; }
    Contraction p = einsum_problem(2, scores, nullptr, out, rescale, B, S, H, T, C);
    p.softmax_lut = lut; p.softmax_S = S;
    if (causal_skip) { p.skip_k = 1; p.skip_H = H; p.skip_start = start_pos; }
    p.dynamic_a = ((flags & ZKDS_LIMBS_DYNAMIC) && a_limbs > 0) ? 1 : 0;
    if (a_limbs <= 0) a_limbs = 3;
    Planes pl{};
    pl.data = const_cast<int8_t*>(value_planes); pl.L = b_limbs; pl.nb = B; pl.rows = C; pl.K = T;
    pl.pitch = capacity;
    int rc = launch_contraction_limb(p, a_limbs, b_limbs, &pl, ST(stream));
    if (rc == ZKDS_ERR_UNSUPPORTED) { t_status = rc; return rc; }
    return finish(rc, "zkds_softmax_pv_cached");
}

int zkds_softmax_causal(const int64_t* X, int64_t* C, const int64_t* lut, int64_t B, int64_t S, int64_t H,
                        int64_t T, int64_t start_pos, void* stream)
{
    int rc;
    if (B < 0 || S < 0 || H < 0 || T < 0) rc = ZKDS_ERR_ARG;
    else if (B && S && H && T && (!X || !C || !lut)) rc = ZKDS_ERR_ARG;
    else rc = launch_softmax_causal(X, C, lut, B, S, H, T, start_pos, ST(stream));
    if (rc == ZKDS_ERR_UNSUPPORTED) { t_status = rc; return rc; }
    return finish(rc, "zkds_softmax_causal");
}

int zkds_rope(const int64_t* A, const int64_t* table, int64_t* C, int64_t batch, int64_t seq,
              int64_t heads, int64_t pairs, int shift, void* stream)
{
    int rc;
    if (batch < 0 || seq < 0 || heads < 0 || pairs < 0) rc = ZKDS_ERR_ARG;
    else if (batch && seq && heads && pairs && (!A || !table || !C)) rc = ZKDS_ERR_ARG;
    else rc = launch_rope(A, table, C, batch, seq, heads, pairs, shift, ST(stream));
    return finish(rc, "zkds_rope");
}

int zkds_rms_norm(const int64_t* A, const void* W, int w_bits, int64_t* C, int64_t* rms_out,
                  int64_t M, int64_t N, int64_t eps, int64_t dim, void* stream)
{
    int rc;
    if (M < 0 || N < 0 || dim <= 0) rc = ZKDS_ERR_ARG;
    else if (M && N && (!A || !W || !C)) rc = ZKDS_ERR_ARG;
    else rc = launch_rmsnorm(A, W, w_bits, nullptr, rms_out, C, M, N, eps, dim, 1, ST(stream));
    return finish(rc, "zkds_rms_norm");
}

int zkds_rms_norm_apply(const int64_t* A, const void* W, int w_bits, const int64_t* rms, int64_t* C,
                        int64_t M, int64_t N, void* stream)
{
    int rc;
    if (M < 0 || N < 0) rc = ZKDS_ERR_ARG;
    else if (M && N && (!A || !W || !C || !rms)) rc = ZKDS_ERR_ARG;
    else rc = launch_rmsnorm(A, W, w_bits, rms, nullptr, C, M, N, 0, 1, 0, ST(stream));
    return finish(rc, "zkds_rms_norm_apply");
}

int zkds_softmax(const int64_t* X, int64_t* weights_out, int64_t* C, const int64_t* lut,
                 int64_t rows, int64_t T, int frac, void* stream)
{
    int rc;
    if (rows < 0 || T < 0) rc = ZKDS_ERR_ARG;
    else if (rows && T && (!X || !C || !lut)) rc = ZKDS_ERR_ARG;
    else rc = launch_softmax(X, weights_out, C, lut, rows, T, frac, ST(stream));
    return finish(rc, "zkds_softmax");
}

int zkds_act(const int64_t* X, int64_t* C, const int64_t* lut, int64_t n, int frac, int silu,
             void* stream)
{
    int rc;
    if (n < 0) rc = ZKDS_ERR_ARG;
    else if (n && (!X || !C || !lut)) rc = ZKDS_ERR_ARG;
    else rc = launch_act(X, C, lut, n, frac, silu, ST(stream));
    return finish(rc, "zkds_act");
}

int zkds_device_status(int clear) { return limb_device_status(clear); }
void zkds_timing(int enable) { limb_timing_enable(enable); }
float zkds_last_kernel_ms(void) { return limb_last_kernel_ms(); }
int zkds_timing_record(long long i, double* out8) { return limb_timing_record(i, out8); }
void zkds_timing_totals(double* ms, double* int8_ops, long long* launches)
{
    limb_timing_totals(ms, int8_ops, launches);
}

int zkds_planes_create(const void* W, int bits, int64_t nb, int64_t rows, int64_t K, int64_t s_batch,
                       int64_t s_row, int64_t s_k, int64_t div, int limbs, void** out, void* stream)
{
    if (!out) return finish(ZKDS_ERR_ARG, "zkds_planes_create");
    *out = nullptr;
    if (!W || (bits != 32 && bits != 64) || nb <= 0 || rows <= 0 || K <= 0 || div == 0 || limbs < 0 ||
        limbs > 9)
        return finish(ZKDS_ERR_ARG, "zkds_planes_create");
    cudaStream_t st = ST(stream);
    int rc = ZKDS_OK;
    if (limbs == 0) {
        uint64_t* d = (uint64_t*)workspace(2 * sizeof(uint64_t), 5);
        if (!d) return finish(ZKDS_ERR_WORKSPACE, "zkds_planes_create");
        uint64_t h = 0;
        rc = set_cuda_error(cudaMemsetAsync(d, 0, sizeof(uint64_t), st));
        if (rc == ZKDS_OK) rc = launch_absmax(W, bits, nb, rows, K, s_batch, s_row, s_k, div, d, st);
        if (rc == ZKDS_OK) rc = set_cuda_error(cudaMemcpyAsync(&h, d, sizeof(h), cudaMemcpyDeviceToHost, st));
        if (rc == ZKDS_OK) rc = set_cuda_error(cudaStreamSynchronize(st));
        if (rc != ZKDS_OK) return finish(rc, "zkds_planes_create");
        limbs = limbs_needed(h);
        if (limbs > 9) return finish(ZKDS_ERR_UNSUPPORTED, "zkds_planes_create");
    }
    const int64_t Kp = (K + 15) & ~(int64_t)15;
    PlanesHandle* hd = new PlanesHandle();
    hd->pl.L = limbs; hd->pl.nb = nb; hd->pl.rows = rows; hd->pl.K = K;
    hd->b_bits = bits;
    cudaGetDevice(&hd->device);
    void* mem = nullptr;
    rc = set_cuda_error(cudaMalloc(&mem, (size_t)limbs * nb * rows * Kp + 1024));
    if (rc == ZKDS_OK) {
        hd->pl.data = (int8_t*)mem;
        rc = planes_split(W, bits, nb, rows, K, s_batch, s_row, s_k, div, limbs, hd->pl.data, st);
    }
    if (rc != ZKDS_OK) {
        if (mem) cudaFree(mem);
        delete hd;
        return finish(rc, "zkds_planes_create");
    }
    *out = hd;
    return finish(ZKDS_OK, "zkds_planes_create");
}

int zkds_planes_limbs(const void* planes) { return planes ? ((const PlanesHandle*)planes)->pl.L : 0; }

int zkds_planes_destroy(void* planes)
{
    if (!planes) return ZKDS_OK;
    PlanesHandle* hd = (PlanesHandle*)planes;
    int rc = set_cuda_error(cudaFree(hd->pl.data));
    delete hd;
    return finish(rc, "zkds_planes_destroy");
}

int zkds_contraction_prepared(const int64_t* A, int64_t a_s_batch, int64_t a_s_row, const void* planes,
                              int b_batched, int64_t* C, int64_t* R, int64_t c_s_batch, int64_t c_s_row,
                              int64_t batches, int64_t M, int64_t a_rescale, int64_t addend, int64_t shift,
                              int a_limbs, int flags, void* stream)
{
    if (!planes) return finish(ZKDS_ERR_ARG, "zkds_contraction_prepared");
    const PlanesHandle* hd = (const PlanesHandle*)planes;
    Contraction p{};
    p.A = A; p.B = nullptr; p.b_bits = hd->b_bits; p.C = C; p.R = R;
    p.batches = batches; p.M = M; p.N = hd->pl.rows; p.K = hd->pl.K;
    p.a_sz = a_s_batch; p.a_sm = a_s_row;
    p.b_sz = b_batched ? 1 : 0; p.b_sn = 0; p.b_sk = 0;
    p.c_sz = c_s_batch; p.c_sm = c_s_row;
    p.a_div = a_rescale; p.b_div = 1;
    p.addend = addend;
    p.shift = (shift < 0 || shift > 127) ? -1 : (int)shift;
    p.r_legacy = (flags & ZKDS_REMAINDER_LEGACY) ? 1 : 0;
    int f = (flags & ~ZKDS_ALGO_MASK) | ZKDS_ALGO_LIMB;
    return finish(run_contraction(p, a_limbs, 0, f, ST(stream), &hd->pl), "zkds_contraction_prepared");
}

int zkds_glu_q23(const int64_t* r1, const int64_t* r2, int64_t ld, int64_t* h, int64_t* s1_out,
                 const int64_t* lut, int64_t rows, int64_t n, void* stream)
{
    int rc = (rows < 0 || n < 0 || (rows && n && (!r1 || !r2 || !h || !lut)))
                 ? ZKDS_ERR_ARG
                 : launch_glu(r1, r2, ld, h, s1_out, lut, rows, n, ST(stream));
    return finish(rc, "zkds_glu_q23");
}

int zkds_gather_rows(const int64_t* src, const int* index, int64_t* dst, int64_t rows, int64_t cols,
                     void* stream)
{
    int rc = (rows < 0 || cols < 0 || (rows && cols && (!src || !index || !dst)))
                 ? ZKDS_ERR_ARG
                 : launch_gather_rows(src, index, dst, rows, cols, ST(stream));
    return finish(rc, "zkds_gather_rows");
}

int zkds_moe_combine(const int64_t* out, const int* pos, const int64_t* w, const int64_t* base,
                     int64_t* y, int64_t tokens, int slots, int64_t cols, void* stream)
{
    int rc = (tokens < 0 || cols < 0 || slots < 0 || (tokens && cols && (!out || !pos || !w || !y)))
                 ? ZKDS_ERR_ARG
                 : launch_moe_combine(out, pos, w, base, y, tokens, slots, cols, ST(stream));
    return finish(rc, "zkds_moe_combine");
}

int zkds_grouped_gather_parts_prepared(const int64_t* const* parts, int n_parts, int64_t rows_per_part,
                                       const int* row_index, const void* planes, const int* tile_group,
                                       int64_t n_tiles, int64_t* C, int64_t shift, const int* group_shift,
                                       int64_t n_split, int a_limbs, int flags, void* stream)
{
    if (!parts || n_parts < 1 || n_parts > kMaxRowParts || rows_per_part <= 0 || !row_index || !planes ||
        !tile_group || n_tiles < 0 || a_limbs <= 0 || (group_shift && (n_split & 7)))
        return finish(ZKDS_ERR_ARG, "zkds_grouped_gather_parts_prepared");
    const PlanesHandle* hd = (const PlanesHandle*)planes;
    Contraction p{};
    p.A = parts[0]; p.B = nullptr; p.b_bits = hd->b_bits; p.C = C; p.R = nullptr;
    p.batches = 1; p.M = n_tiles * 128; p.N = hd->pl.rows; p.K = hd->pl.K;
    p.a_sz = 0; p.a_sm = hd->pl.K;
    p.b_sz = 1; p.b_sn = 0; p.b_sk = 0;
    p.c_sz = 0; p.c_sm = hd->pl.rows;
    p.a_div = 1; p.b_div = 1;
    p.addend = 0;
    p.shift = (shift < 0 || shift > 127) ? -1 : (int)shift;
    p.tile_group = tile_group;
    p.a_row_index = row_index;
    p.a_n_parts = n_parts; p.a_rows_per_part = rows_per_part;
    for (int i = 0; i < n_parts; ++i) {
        if (!parts[i]) return finish(ZKDS_ERR_ARG, "zkds_grouped_gather_parts_prepared");
        p.a_parts[i] = parts[i];
    }
    p.group_shift = group_shift; p.n_split = n_split;
    p.group_rows = (flags & ZKDS_GROUP_ROWS_32) ? 32 : (flags & ZKDS_GROUP_ROWS_64) ? 64 : 0;
    int f = (flags & ~ZKDS_ALGO_MASK) | ZKDS_ALGO_LIMB;
    return finish(run_contraction(p, a_limbs, 0, f, ST(stream), &hd->pl), "zkds_grouped_gather_parts_prepared");
}

int zkds_moe_combine_peer(const int64_t* out, const int* pos, const int64_t* w, int64_t tokens, int slots,
                          int64_t cols, int64_t tokens_per_part, int64_t* const* slot_bases, int n_parts,
                          int my_part, void* stream)
{
    int rc = (tokens < 0 || cols < 0 || !slot_bases || (tokens && cols && (!out || !pos || !w)))
                 ? ZKDS_ERR_ARG
                 : launch_moe_combine_peer(out, pos, w, tokens, slots, cols, tokens_per_part, slot_bases, n_parts,
                                           my_part, ST(stream));
    return finish(rc, "zkds_moe_combine_peer");
}

int zkds_moe_sum_slots(const int64_t* base, const int64_t* slot_rows, const int64_t* indices, int64_t tokens,
                       int slots, int64_t cols, int n_parts, int experts_per_part, int64_t* y, void* stream)
{
    int rc = (tokens < 0 || cols < 0 || (tokens && cols && (!slot_rows || !indices || !y)))
                 ? ZKDS_ERR_ARG
                 : launch_moe_sum_slots(base, slot_rows, indices, tokens, slots, cols, n_parts, experts_per_part, y,
                                        ST(stream));
    return finish(rc, "zkds_moe_sum_slots");
}

int zkds_peer_barrier(uint64_t* const* flag_bases, int n_parts, int my_part, uint64_t epoch, uint32_t* status,
                      void* stream)
{
    int rc = !flag_bases ? ZKDS_ERR_ARG
                         : launch_peer_barrier((unsigned long long* const*)flag_bases, n_parts, my_part,
                                               (unsigned long long)epoch, (unsigned*)status, ST(stream));
    return finish(rc, "zkds_peer_barrier");
}

int zkds_gate_select(const int64_t* sigma, const int32_t* bias, int64_t tokens, int experts, int n_groups,
                     int topk_groups, int topk, int64_t* indices, int64_t* raw_weights, int64_t* weights, void* stream)
{
    int rc = (tokens < 0 || (tokens && (!sigma || !indices || !raw_weights || !weights)))
                 ? ZKDS_ERR_ARG
                 : launch_gate_select(sigma, bias, tokens, experts, n_groups, topk_groups, topk, indices, raw_weights,
                                      weights, ST(stream));
    if (rc == ZKDS_ERR_UNSUPPORTED) { t_status = rc; return rc; }       // silent: the caller falls back
    return finish(rc, "zkds_gate_select");
}

int zkds_lut(int64_t* host_lut, int kind) { return finish(make_lut(host_lut, kind), "zkds_lut"); }

// ---- the reference's 21 symbols ---------------------------------------------------

static bool nonneg(int a, int b, int c, int d) { return a >= 0 && b >= 0 && c >= 0 && d >= 0; }

void int64_32_bmm_broadcast_launcher(const int64_t* A, const int32_t* B, int64_t* C, int64_t* R,
                                     const int64_t a_rescale, const int64_t b_rescale,
                                     const int64_t c_rescale, int Bdim, int M, int K, int N)
{
    if (!nonneg(Bdim, M, K, N)) { finish(ZKDS_ERR_ARG, "int64_32_bmm_broadcast_launcher"); return; }
    Contraction p = gemm_problem(A, B, 32, C, R, a_rescale, b_rescale, c_rescale, Bdim, M, K, N, 1);
    finish(run_contraction(p, 0, 0, ZKDS_ALGO_AUTO, 0), "int64_32_bmm_broadcast_launcher");
}

void int64_64_bmm_broadcast_launcher(const int64_t* A, const int64_t* B, int64_t* C, int64_t* R,
                                     const int64_t a_rescale, const int64_t b_rescale,
                                     const int64_t c_rescale, int Bdim, int M, int K, int N)
{
    if (!nonneg(Bdim, M, K, N)) { finish(ZKDS_ERR_ARG, "int64_64_bmm_broadcast_launcher"); return; }
    Contraction p = gemm_problem(A, B, 64, C, R, a_rescale, b_rescale, c_rescale, Bdim, M, K, N, 1);
    finish(run_contraction(p, 0, 0, ZKDS_ALGO_AUTO, 0), "int64_64_bmm_broadcast_launcher");
}

void bf16_to_int32_2d(const uint16_t* input, int32_t* output, int rows, int cols, int rescale)
{
    finish(launch_bf16_to_int32(input, output, rows, cols, rescale, 0, 0), "bf16_to_int32_2d");
}

void wkv_b_bf16_to_int32(const uint16_t* input, int32_t* output, int rows, int cols)
{
    finish(launch_bf16_to_int32(input, output, rows, cols, 0, 1, 0), "wkv_b_bf16_to_int32");
}

void float32_to_int64_2d(const uint32_t* input, int64_t* output, int rows, int cols, int rescale)
{
    finish(launch_f32_to_int64(input, output, rows, cols, rescale, 0), "float32_to_int64_2d");
}

void complex_int64_mul(const int64_t* A, const int64_t* B, int64_t* C, int batchSize, int seqLen,
                       int headCount, int headDim)
{
    if (!nonneg(batchSize, seqLen, headCount, headDim)) { finish(ZKDS_ERR_ARG, "complex_int64_mul"); return; }
    finish(launch_rope(A, B, C, batchSize, seqLen, headCount, headDim, 42, 0), "complex_int64_mul");
}

void rms_norm_32(const int64_t* A, const int32_t* W, const int64_t* rms, int64_t* C, int seqLen,
                 int Dim)
{
    if (seqLen < 0 || Dim < 0) { finish(ZKDS_ERR_ARG, "rms_norm_32"); return; }
    finish(launch_rmsnorm(A, W, 32, rms, nullptr, C, seqLen, Dim, 0, 1, 0, 0), "rms_norm_32");
}

void rms_norm_64(const int64_t* A, const int64_t* W, const int64_t* rms, int64_t* C, int seqLen,
                 int Dim)
{
    if (seqLen < 0 || Dim < 0) { finish(ZKDS_ERR_ARG, "rms_norm_64"); return; }
    finish(launch_rmsnorm(A, W, 64, rms, nullptr, C, seqLen, Dim, 0, 1, 0, 0), "rms_norm_64");
}

void einsum_bshd_hdc_bshc(const int64_t* q_nope, const int32_t* wkv_b_1, int64_t* out,
                          int64_t rescale, int B, int S, int H, int D, int C)
{
    if (!nonneg(B, S, H, D) || C < 0) { finish(ZKDS_ERR_ARG, "einsum_bshd_hdc_bshc"); return; }
    Contraction p = einsum_problem(0, q_nope, wkv_b_1, out, rescale, B, S, H, D, C);
    finish(run_contraction(p, 0, 0, ZKDS_ALGO_AUTO, 0), "einsum_bshd_hdc_bshc");
}

void einsum_bshc_btc_bsht(const int64_t* A, const int64_t* B, int64_t* C, int64_t rescale, int Bsz,
                          int S, int H, int T, int Cdim)
{
    if (!nonneg(Bsz, S, H, T) || Cdim < 0) { finish(ZKDS_ERR_ARG, "einsum_bshc_btc_bsht"); return; }
    Contraction p = einsum_problem(1, A, B, C, rescale, Bsz, S, H, T, Cdim);
    finish(run_contraction(p, 0, 0, ZKDS_ALGO_AUTO, 0), "einsum_bshc_btc_bsht");
}

void einsum_bsht_btc_bshc(const int64_t* A, const int64_t* B, int64_t* C, int64_t rescale, int Bsz,
                          int S, int H, int T, int Cdim)
{
    if (!nonneg(Bsz, S, H, T) || Cdim < 0) { finish(ZKDS_ERR_ARG, "einsum_bsht_btc_bshc"); return; }
    Contraction p = einsum_problem(2, A, B, C, rescale, Bsz, S, H, T, Cdim);
    finish(run_contraction(p, 0, 0, ZKDS_ALGO_AUTO, 0), "einsum_bsht_btc_bshc");
}

void einsum_bshc_hdc_bshd(const int64_t* A, const int32_t* B, int64_t* C, int64_t rescale, int Bsz,
                          int S, int H, int D, int Cdim)
{
    if (!nonneg(Bsz, S, H, D) || Cdim < 0) { finish(ZKDS_ERR_ARG, "einsum_bshc_hdc_bshd"); return; }
    Contraction p = einsum_problem(3, A, B, C, rescale, Bsz, S, H, D, Cdim);
    finish(run_contraction(p, 0, 0, ZKDS_ALGO_AUTO, 0), "einsum_bshc_hdc_bshd");
}

static void legacy_softmax(int64_t* R, int64_t* C, int64_t* lut, int Bsz, int S, int H, int T,
                           int frac, const char* who)
{
    if (!nonneg(Bsz, S, H, T)) { finish(ZKDS_ERR_ARG, who); return; }
    int64_t rows = (int64_t)Bsz * S * H;
    // the reference leaves the unnormalised weights in its input buffer
    finish(launch_softmax(R, R, C, lut, rows, T, frac, 0), who);
}

void softmax_q21(int64_t* R, int64_t* C, int64_t* EXP2_FRAC_LUT, int Bsz, int S, int H, int T)
{
    legacy_softmax(R, C, EXP2_FRAC_LUT, Bsz, S, H, T, 21, "softmax_q21");
}

void softmax_q19(int64_t* R, int64_t* C, int64_t* EXP2_FRAC_LUT, int Bsz, int S, int H, int T)
{
    legacy_softmax(R, C, EXP2_FRAC_LUT, Bsz, S, H, T, 19, "softmax_q19");
}

void softmax_init_q21(int64_t* EXP2_FRAC_LUT) { finish(make_lut(EXP2_FRAC_LUT, 1), "softmax_init_q21"); }
void softmax_init_q19(int64_t* EXP2_FRAC_LUT) { finish(make_lut(EXP2_FRAC_LUT, 0), "softmax_init_q19"); }
void silu_init_q25(int64_t* EXP2_FRAC_LUT) { finish(make_lut(EXP2_FRAC_LUT, 3), "silu_init_q25"); }
void silu_init_q23(int64_t* EXP2_FRAC_LUT) { finish(make_lut(EXP2_FRAC_LUT, 2), "silu_init_q23"); }

static void legacy_act(int64_t* R, int64_t* C, int64_t* lut, int Bsz, int S, int Dim, int frac,
                       int silu, const char* who)
{
    if (Bsz < 0 || S < 0 || Dim < 0) { finish(ZKDS_ERR_ARG, who); return; }
    finish(launch_act(R, C, lut, (int64_t)Bsz * S * Dim, frac, silu, 0), who);
}

void silu_q25(int64_t* R, int64_t* C, int64_t* L, int Bsz, int S, int Dim) { legacy_act(R, C, L, Bsz, S, Dim, 25, 1, "silu_q25"); }
void sigmoid_q25(int64_t* R, int64_t* C, int64_t* L, int Bsz, int S, int Dim) { legacy_act(R, C, L, Bsz, S, Dim, 25, 0, "sigmoid_q25"); }
void silu_q23(int64_t* R, int64_t* C, int64_t* L, int Bsz, int S, int Dim) { legacy_act(R, C, L, Bsz, S, Dim, 23, 1, "silu_q23"); }
void sigmoid_q23(int64_t* R, int64_t* C, int64_t* L, int Bsz, int S, int Dim) { legacy_act(R, C, L, Bsz, S, Dim, 23, 0, "sigmoid_q23"); }

}  // extern "C"
