// The float32 path's matrix product: y[M, N] = x[M, K] w[N, K]^T (+ bias[N]), every product and
// sum a float32 FMA on the CUDA cores (no tensor cores, no reduced-precision mode of any kind).
//
// The reference's engine uses the library product here (nn.Linear,
// somi_inference/models/qwen2.py:221-222,268-271).  This engine does not, for two reasons.  The
// float32 path exists to show faults that bfloat16 hides, so its arithmetic must be beyond doubt:
// on the software stack this engine was developed on (cuBLAS 12.8, B200) the library's float32
// product with TF32 switched off returned, in some processes, pairs of wrong output columns for
// products of a few rows (16 x 320 x 192 and the like).  And an output element here is the sum of
// its K terms in ascending order, whatever M and N are: the same token gives the same bits in a
// step of one token and in a step of a thousand, which the library does not promise.
//
// One CTA computes a BM x 128 tile with 256 threads (a 16 x 16 grid of threads, BM/16 x 8 outputs
// each); K goes through shared memory in slices of 8, both operands transposed there so that a
// thread reads its BM/16 + 8 values of a slice as vectors.  BM is 128, or 32 for steps of few
// rows.  Any M, N, K; rows are read as float4 where K is a multiple of 4.
#include "common.cuh"

namespace somi {

constexpr int kSgBN = 128;
constexpr int kSgBK = 8;
constexpr int kSgThreads = 256;

template <int BM>
__global__ void __launch_bounds__(kSgThreads)
sgemm_nt_kernel(const float* __restrict__ x, const float* __restrict__ w,
                const float* __restrict__ bias, float* __restrict__ y, int M, int N, int K) {
    constexpr int TM = BM / 16;          // rows per thread
    constexpr int TN = kSgBN / 16;       // columns per thread (8)
    __shared__ __align__(16) float xs[kSgBK][BM];
    __shared__ __align__(16) float ws[kSgBK][kSgBN];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * kSgBN;
    const int tr = tid / 16, tc = tid % 16;       // this thread's rows tr*TM.., columns tc*TN..
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    const bool vec = (K & 3) == 0;
    // loading: a slice is BM (or 128) rows of 8 floats = two float4 per row
    for (int k0 = 0; k0 < K; k0 += kSgBK) {
        for (int idx = tid; idx < BM * 2; idx += kSgThreads) {
            const int r = idx >> 1, h = (idx & 1) * 4;
            const int gm = m0 + r, gk = k0 + h;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gm < M) {
                const float* p = x + static_cast<size_t>(gm) * K + gk;
                if (vec && gk + 3 < K) v = *reinterpret_cast<const float4*>(p);
                else {
                    if (gk < K) v.x = p[0];
                    if (gk + 1 < K) v.y = p[1];
                    if (gk + 2 < K) v.z = p[2];
                    if (gk + 3 < K) v.w = p[3];
                }
            }
            xs[h][r] = v.x; xs[h + 1][r] = v.y; xs[h + 2][r] = v.z; xs[h + 3][r] = v.w;
        }
        for (int idx = tid; idx < kSgBN * 2; idx += kSgThreads) {
            const int r = idx >> 1, h = (idx & 1) * 4;
            const int gn = n0 + r, gk = k0 + h;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gn < N) {
                const float* p = w + static_cast<size_t>(gn) * K + gk;
                if (vec && gk + 3 < K) v = *reinterpret_cast<const float4*>(p);
                else {
                    if (gk < K) v.x = p[0];
                    if (gk + 1 < K) v.y = p[1];
                    if (gk + 2 < K) v.z = p[2];
                    if (gk + 3 < K) v.w = p[3];
                }
            }
            ws[h][r] = v.x; ws[h + 1][r] = v.y; ws[h + 2][r] = v.z; ws[h + 3][r] = v.w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kSgBK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][tr * TM + i];
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const float4 t = *reinterpret_cast<const float4*>(&ws[kk][tc * TN + j]);
                b[j] = t.x; b[j + 1] = t.y; b[j + 2] = t.z; b[j + 3] = t.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + tr * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tc * TN + j;
            if (gn < N) y[static_cast<size_t>(gm) * N + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
        }
    }
}

}  // namespace somi

using namespace somi;

// y[M, N] = x[M, K] w[N, K]^T (+ bias), all float32, row-major.
SOMI_API int somi_gemm_f32(const float* x, const float* w, const float* bias, float* y, int M, int N,
                           int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return SOMI_ERR_UNSUPPORTED;
    const unsigned tiles_n = static_cast<unsigned>((N + kSgBN - 1) / kSgBN);
    if (M <= 32) {
        launch_pdl(sgemm_nt_kernel<32>, dim3(tiles_n, (M + 31) / 32), dim3(kSgThreads), 0, stream, x, w,
                   bias, y, M, N, K);
    } else {
        const unsigned tiles_m = static_cast<unsigned>((M + 127) / 128);
        if (tiles_m > 65535u) return SOMI_ERR_UNSUPPORTED;
        launch_pdl(sgemm_nt_kernel<128>, dim3(tiles_n, tiles_m), dim3(kSgThreads), 0, stream, x, w,
                   bias, y, M, N, K);
    }
    return launch_status();
}
