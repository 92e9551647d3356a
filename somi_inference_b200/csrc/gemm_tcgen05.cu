// Weight-streaming matrix product for few tokens (decode steps): Y[M, N] = X[M, K] W[N, K]^T,
// M <= 64, on the 5th-generation tensor cores.
//
// With few tokens the product is bound by reading W once.  The roles are swapped so that the
// weight rows fill the 128 rows of the MMA and the tokens sit on its N side (16, 32 or 64):
// D[n, m] = sum_k W[n, k] X[m, k], accumulated in tensor memory (128 lanes x M columns, float32).
// One CTA owns 128 output features and a range of K (split-K fills the SMs when N is small).
// Warp roles: warp 0 = TMA producer (one thread issues `cp.async.bulk.tensor` loads of W and X
// tiles, 128-byte swizzle, into a ring of shared-memory stages), warp 1 = MMA issuer (one thread
// issues `tcgen05.mma`, `tcgen05.commit` hands stages back and finally signals the accumulator),
// warp 6 = a second MMA issuer: the two take the K blocks in turn, each into an accumulator of
// its own (the thread that issues MMAs has no queue in front of the tensor pipe, so the pipe
// idles for the ~220 cycles that thread spends on each barrier test; with two threads one
// thread's test runs under the other's MMAs), the epilogue adds the two accumulators;
// warps 2-5 = epilogue (`tcgen05.ld` of their 32 lanes, then bias / SiLU(gate)*up / float32
// output and coalesced stores).  All waits on mbarriers are bounded; a wait that runs out sets
// an error word, and the CTA still frees its tensor memory and returns.
//
// The reference computes these products with nn.Linear (somi_inference/models/qwen2.py:221-222,
// 268-271) or a plain Triton matmul without any fused epilogue (somi_inference/core/mlp_triton.py:51-108).
#include "mma.cuh"
#include "tma.cuh"

namespace somi {

constexpr int kGemmBN = 128;              // output features per CTA (MMA M)
constexpr int kGemmBK = 64;               // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 224;
constexpr int kGemmWBytes = kGemmBN * kGemmBK * 2;      // 16 KiB

enum GemmMode { kGemmBf16 = 0, kGemmF32 = 1, kGemmPartialF32 = 2, kGemmSwiGLU = 3 };

__device__ int g_gemm_error = 0;

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
    // K-major operand, 128-byte swizzle: 8-row groups are 1024 bytes apart
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);          // start address
    d |= static_cast<uint64_t>(1) << 16;                              // leading byte offset (unused)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                      // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                              // descriptor version
    d |= static_cast<uint64_t>(2) << 61;                              // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}

// TOK: tokens padded to the MMA's N (16, 32, 64).  STAGES: depth of the shared-memory ring.
template <int TOK, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, (STAGES <= 6 ? 2 : 1))
skinny_gemm_kernel(const __grid_constant__ CUtensorMap w_map,
                   const __grid_constant__ CUtensorMap x_map, int M, int N, int K,
                   int kb_per_split, int mode, const void* __restrict__ bias, int bias_dtype,
                   void* __restrict__ out, long long out_split_stride) {
    // The two MMA threads take the K blocks in turn.  With an even number of stages each stage
    // belongs to one of them for good, and that thread sees every phase of the stage's barrier in
    // order.  With an odd number a stage would alternate between the threads: a thread could meet
    // a barrier for the first time in its second phase, before the first has completed, and a
    // parity wait cannot tell "not yet" from "done" then (it passed at once, the thread multiplied
    // the wrong tile and released the stage under the other thread: wrong sums, run-out waits,
    // once a launch failure, until this was found).
    static_assert(STAGES % 2 == 0, "the ring depth must be even: see the comment");
    constexpr int XBytes = TOK * kGemmBK * 2;
    constexpr int StageBytes = kGemmWBytes + XBytes;
    constexpr int TmemCols = 2 * TOK < 32 ? 32 : 2 * TOK;     // one accumulator per MMA thread
    extern __shared__ unsigned char smem_raw[];
    unsigned char* stages = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], accum_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed_s;

    pdl_launch_dependents();      // the next kernel may be scheduled; it waits for this one itself
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kGemmBN;
    const int split = blockIdx.y;
    const int nkb_total = (K + kGemmBK - 1) / kGemmBK;
    const int kb0 = split * kb_per_split;
    const int nkb = min(kb_per_split, nkb_total - kb0);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&accum_bar), 2);         // one arrival per MMA thread
        mbar_fence_init();
        failed_s = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(&tmem_base_s)),
                     "r"(TmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_d = tmem_base_s;
    // Barriers and tensor memory are set up.  The weights are written by no kernel [constant],
    // so the producer fills the ring's first stages with W tiles before it waits for that kernel;
    // the activation tiles, and everything any other thread reads or writes, come after the wait.
    const int n_pre = min(nkb, STAGES);
    if (warp == 0 && lane == 0) {
        for (int kb = 0; kb < n_pre; ++kb) {
            const uint32_t fb = smem_u32(&full_bar[kb]);
            mbar_expect_tx(fb, StageBytes);
            tma_load_2d(smem_u32(stages + kb * StageBytes), &w_map, (kb0 + kb) * kGemmBK, n0, fb);
        }
    }
    // The barriers of those stages are armed with their byte counts now.  Other warps will issue
    // copies that complete on them: a copy must not complete on a barrier before its bytes have
    // been announced (the count would pass below zero), so everyone meets here first.
    __syncthreads();
    pdl_wait();

    // The activation tiles of the stages that already hold their weights: a thread issues a copy
    // every hundred-odd cycles, so the epilogue warps, idle until the accumulator is complete,
    // share them with the producer.
    if (lane == 0 && (warp == 0 || warp >= 2) && warp != 6) {
        const int w5 = warp == 0 ? 0 : warp - 1;           // 0..4
        for (int kb = w5; kb < n_pre; kb += 5)
            tma_load_2d(smem_u32(stages + kb * StageBytes + kGemmWBytes), &x_map,
                        (kb0 + kb) * kGemmBK, 0, smem_u32(&full_bar[kb]));
    }
    __syncwarp();
    if (warp == 0) {
        if (lane == 0) {
            for (int kb = n_pre; kb < nkb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1)) { failed_s = 1; break; }
                const uint32_t fb = smem_u32(&full_bar[s]);
                mbar_expect_tx(fb, StageBytes);
                unsigned char* st = stages + s * StageBytes;
                tma_load_2d(smem_u32(st), &w_map, (kb0 + kb) * kGemmBK, n0, fb);
                tma_load_2d(smem_u32(st + kGemmWBytes), &x_map, (kb0 + kb) * kGemmBK, 0, fb);
            }
        }
    } else if (warp == 1 || warp == 6) {
        if (lane == 0) {
            const int par = warp == 1 ? 0 : 1;       // this thread's K blocks: par, par + 2, ...
            const uint32_t tmem_acc = tmem_d + par * TOK;
            // instruction descriptor: float32 accumulator, bf16 x bf16, both K-major, N = TOK, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                   (static_cast<uint32_t>(TOK >> 3) << 17) |
                                   (static_cast<uint32_t>(kGemmBN >> 4) << 24);
            bool ok = true;
            for (int kb = par; kb < nkb && ok; kb += 2) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(smem_u32(&full_bar[s]), ph)) { failed_s = 1; ok = false; break; }
                tcgen05_fence_after();
                const uint32_t wa = smem_u32(stages + s * StageBytes);
                const uint32_t xa = wa + kGemmWBytes;
#pragma unroll
                for (int k16 = 0; k16 < kGemmBK / 16; ++k16)
                    umma_bf16(tmem_acc, umma_smem_desc(wa + k16 * 32), umma_smem_desc(xa + k16 * 32),
                              idesc, (kb > par || k16 > 0) ? 1u : 0u);
                // the stage is free once these MMAs have read it; nobody waits for a stage that
                // is not filled again
                if (kb + STAGES < nkb) umma_commit(smem_u32(&empty_bar[s]));
            }
            umma_commit(smem_u32(&accum_bar));                 // accumulator complete
        }
    } else {
        // ---- epilogue: warp w reads TMEM lanes 32 * (w % 4) ..; its lane is one output feature
        const int q = warp & 3;
        const int n = n0 + q * 32 + lane;
        const bool ok = mbar_wait(smem_u32(&accum_bar), 0, 2000000);
        if (!ok) failed_s = 1;
        tcgen05_fence_after();
        float acc[TOK];
        if (nkb > 0) {
#pragma unroll
            for (int c = 0; c < TOK / 16; ++c) {
                uint32_t r[16];
                tmem_load_16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + c * 16, r);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c * 16 + j] = __uint_as_float(r[j]);
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (nkb > 1) {          // the second thread's accumulator holds the odd K blocks
#pragma unroll
                for (int c = 0; c < TOK / 16; ++c) {
                    uint32_t r[16];
                    tmem_load_16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + TOK + c * 16, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[c * 16 + j] += __uint_as_float(r[j]);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < TOK; ++j) acc[j] = 0.f;
        }
        if (ok) {
            float b = 0.f;
            if (bias != nullptr && n < N && (mode != kGemmPartialF32 || split == 0))
                b = load_as_float(bias, bias_dtype, n);
            if (mode == kGemmBf16) {
                __nv_bfloat16* y = static_cast<__nv_bfloat16*>(out);
                if (n < N)
#pragma unroll
                    for (int m = 0; m < TOK; ++m)
                        if (m < M) y[static_cast<size_t>(m) * N + n] = __float2bfloat16_rn(acc[m] + b);
            } else if (mode == kGemmF32 || mode == kGemmPartialF32) {
                float* y = static_cast<float*>(out) + static_cast<size_t>(split) * out_split_stride;
                if (n < N)
#pragma unroll
                    for (int m = 0; m < TOK; ++m)
                        if (m < M) y[static_cast<size_t>(m) * N + n] = acc[m] + b;
            } else {   // kGemmSwiGLU: even rows of W are gate rows, odd rows the matching up rows
                __nv_bfloat16* y = static_cast<__nv_bfloat16*>(out);
                const int half_n = N >> 1;
#pragma unroll
                for (int m = 0; m < TOK; ++m) {
                    if (m >= M) break;                      // uniform: M is a kernel argument
                    const float other = __shfl_xor_sync(0xffffffffu, acc[m], 1);
                    if ((lane & 1) == 0 && n < N) {
                        const float g = acc[m];
                        y[static_cast<size_t>(m) * half_n + (n >> 1)] =
                            __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * other);
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d),
                     "r"(TmemCols)
                     : "memory");
    }
    if (tid == 0 && failed_s) atomicExch(&g_gemm_error, 1);
}

template <int TOK, int STAGES>
int launch_skinny(const CUtensorMap* w_map, const CUtensorMap* x_map, int M, int N, int K,
                  int splits, int mode, const void* bias, int bias_dtype, void* out,
                  long long out_split_stride, cudaStream_t stream) {
    constexpr int StageBytes = kGemmWBytes + TOK * kGemmBK * 2;
    const size_t smem = static_cast<size_t>(STAGES) * StageBytes + 1024;
    cudaFuncSetAttribute(skinny_gemm_kernel<TOK, STAGES>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int nkb = (K + kGemmBK - 1) / kGemmBK;
    const int kbps = (nkb + splits - 1) / splits;
    dim3 grid((N + kGemmBN - 1) / kGemmBN, (nkb + kbps - 1) / kbps);
    launch_pdl(skinny_gemm_kernel<TOK, STAGES>, dim3(grid), dim3(kGemmThreads), smem, stream, 
        *w_map, *x_map, M, N, K, kbps, mode, bias, bias_dtype, out, out_split_stride);
    return launch_status();
}

}  // namespace somi

using namespace somi;

// A tensor map over a row-major bfloat16 matrix [rows, cols] with boxes [box_rows, 64] and the
// 128-byte swizzle; `map_out` is 128 bytes, 64-byte aligned.  cols must be a multiple of 8.
SOMI_API int somi_make_gemm_tensor_map(void* map_out, const void* base, long long rows,
                                       long long cols, int box_rows) {
    if (cols % 8 != 0 || box_rows <= 0 || box_rows > 256) return SOMI_ERR_UNSUPPORTED;
    return make_tensor_map_bf16_2d(static_cast<CUtensorMap*>(map_out), base,
                                   static_cast<uint64_t>(rows), static_cast<uint64_t>(cols),
                                   static_cast<uint32_t>(box_rows), kGemmBK, CU_TENSOR_MAP_SWIZZLE_128B);
}

SOMI_API int somi_skinny_gemm_max_tokens() { return 64; }

// Number of K splits actually launched for a request of `splits` (a split never is empty).
SOMI_API int somi_skinny_gemm_splits(int K, int splits) {
    const int nkb = (K + kGemmBK - 1) / kGemmBK;
    if (splits < 1) splits = 1;
    const int kbps = (nkb + splits - 1) / splits;
    return (nkb + kbps - 1) / kbps;
}

SOMI_API int somi_gemm_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

// mode: 0 bf16 [M, N]; 1 float32 [M, N]; 2 float32 partial sums [splits, M, N] (bias in split 0);
// 3 SwiGLU over interleaved gate/up rows, bf16 [M, N / 2].  `x_box_rows` is the box height the
// x tensor map was made with (16, 32 or 64) and must be >= M.
SOMI_API int somi_skinny_gemm(const void* w_map, const void* x_map, int x_box_rows, int M, int N,
                              int K, int splits, int mode, const void* bias, int bias_dtype,
                              void* out, int deep_ring, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > x_box_rows || K % 8 != 0 || K <= 0 || mode < 0 || mode > 3) return SOMI_ERR_UNSUPPORTED;
    if (mode == kGemmSwiGLU && (N & 1)) return SOMI_ERR_UNSUPPORTED;
    if (mode != kGemmPartialF32) splits = 1;
    const CUtensorMap* wm = static_cast<const CUtensorMap*>(w_map);
    const CUtensorMap* xm = static_cast<const CUtensorMap*>(x_map);
    const long long stride = static_cast<long long>(M) * N;
    // deep_ring: one CTA per SM with an 8-stage ring; otherwise two CTAs per SM with 4 or 6
    // stages each (an even number that fits twice into shared memory), so that one CTA's prologue
    // and epilogue overlap the other's main loop.
#define SOMI_SKINNY(TOK, ST) \
    return launch_skinny<TOK, ST>(wm, xm, M, N, K, splits, mode, bias, bias_dtype, out, stride, stream)
    switch (x_box_rows) {
        case 16: if (deep_ring) SOMI_SKINNY(16, 8); else SOMI_SKINNY(16, 6);
        case 32: if (deep_ring) SOMI_SKINNY(32, 8); else SOMI_SKINNY(32, 4);
        case 64: if (deep_ring) SOMI_SKINNY(64, 8); else SOMI_SKINNY(64, 4);
        default: return SOMI_ERR_UNSUPPORTED;
    }
#undef SOMI_SKINNY
}
