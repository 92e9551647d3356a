// Causal grouped-query attention over the paged cache, any dtype, any head size
// (multiple of 16 up to 256), any page size: the reference kernel of the library.
// It is the float32 path's attention and the fallback of the bfloat16 path for
// sizes that the tensor-core kernels refuse.  Products are accumulated with
// float32 FMAs, softmax is float32 and online, key tiles are aligned to
// multiples of BN from position 0, so the arithmetic on one query row does not
// depend on how its request was cut into steps or on what else is in the batch.
//
// One CTA = one q tile (<= BM consecutive tokens of one request) x one query head.
// Tiles [0, n_tiles) come from the tile list (request, first row, rows); CTAs
// beyond them are the single-token requests: request n_prefill_req + i, row
// n_prefill_tok + i.
#include "common.cuh"

namespace somi {

constexpr int kBM = 16;        // query rows per CTA
constexpr int kBN = 32;        // keys per iteration
constexpr int kThreads = 128;
constexpr int kMaxHd = 256;
constexpr int kAccPerThread = kBM * kMaxHd / kThreads;   // 32

template <typename T>
__global__ void __launch_bounds__(kThreads)
paged_attention_generic_kernel(const T* __restrict__ qkv, int row_stride,
                               const T* __restrict__ kcache, const T* __restrict__ vcache,
                               const int* __restrict__ block_table, int bt_stride,
                               const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                               const int* __restrict__ tiles, int n_tiles, int n_prefill_req,
                               int n_prefill_tok, int nq, int nkv, int hd, int page_size,
                               float scale, int window, T* __restrict__ out) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    float* Qs = smem;                           // [kBM][hd]
    float* Ks = Qs + kBM * hd;                  // [kBN][hd + 1]
    float* Vs = Ks + kBN * (hd + 1);            // [kBN][hd]
    float* Ss = Vs + kBN * hd;                  // [kBM][kBN + 1]
    float* m_s = Ss + kBM * (kBN + 1);          // [kBM]
    float* l_s = m_s + kBM;                     // [kBM]
    float* a_s = l_s + kBM;                     // [kBM]

    int req, row0, rows;
    if (static_cast<int>(blockIdx.x) < n_tiles) {
        req = tiles[3 * blockIdx.x];
        row0 = tiles[3 * blockIdx.x + 1];
        rows = tiles[3 * blockIdx.x + 2];
    } else {
        const int i = blockIdx.x - n_tiles;
        req = n_prefill_req + i;
        row0 = n_prefill_tok + i;
        rows = 1;
    }
    const int head = blockIdx.y;
    const int kvh = head / (nq / nkv);
    const int tid = threadIdx.x;
    const int q_pos0 = ctx_len[req] + (row0 - cu_q[req]);
    const int kv_end = q_pos0 + rows;                                   // exclusive
    const int kv_first = window > 0 ? max(0, q_pos0 - window + 1) : 0;   // first key any row reads
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;

    for (int idx = tid; idx < kBM * hd; idx += kThreads) {
        const int m = idx / hd, d = idx - m * hd;
        Qs[idx] = m < rows ? to_float(qkv[static_cast<size_t>(row0 + m) * row_stride + head * hd + d]) * scale
                           : 0.f;
    }
    if (tid < kBM) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
    float acc[kAccPerThread];
#pragma unroll
    for (int i = 0; i < kAccPerThread; ++i) acc[i] = 0.f;
    __syncthreads();

    for (int kb = (kv_first / kBN) * kBN; kb < kv_end; kb += kBN) {
        for (int idx = tid; idx < kBN * hd; idx += kThreads) {
            const int n = idx / hd, d = idx - n * hd;
            const int j = kb + n;
            float kval = 0.f, vval = 0.f;
            if (j >= kv_first && j < kv_end) {
                const int page = bt[j / page_size];
                const size_t base = ((static_cast<size_t>(page) * nkv + kvh) * page_size + j % page_size) * hd + d;
                kval = to_float(kcache[base]);
                vval = to_float(vcache[base]);
            }
            Ks[n * (hd + 1) + d] = kval;
            Vs[n * hd + d] = vval;
        }
        __syncthreads();
        for (int idx = tid; idx < kBM * kBN; idx += kThreads) {
            const int m = idx / kBN, n = idx - m * kBN;
            const int j = kb + n, qp = q_pos0 + m;
            float s = -INFINITY;
            if (m < rows && j <= qp && j >= kv_first && (window <= 0 || j > qp - window)) {
                s = 0.f;
                const float* q = Qs + m * hd;
                const float* k = Ks + n * (hd + 1);
                for (int d = 0; d < hd; ++d) s = fmaf(q[d], k[d], s);
            }
            Ss[m * (kBN + 1) + n] = s;
        }
        __syncthreads();
        {   // online softmax: one warp per row, one key per lane (kBN == 32)
            const int warp = tid >> 5, lane = tid & 31;
            for (int m = warp; m < kBM; m += kThreads / 32) {
                const float s = Ss[m * (kBN + 1) + lane];
                const float m_old = m_s[m];
                const float m_new = fmaxf(m_old, warp_max(s));
                float p = 0.f, alpha = 1.f;
                if (m_new != -INFINITY) {
                    alpha = expf(m_old - m_new);          // m_old = -inf gives 0
                    p = expf(s - m_new);                   // s = -inf gives 0
                }
                const float psum = warp_sum(p);
                Ss[m * (kBN + 1) + lane] = p;
                if (lane == 0) {
                    m_s[m] = m_new;
                    l_s[m] = l_s[m] * alpha + psum;
                    a_s[m] = alpha;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kAccPerThread; ++i) {
            const int idx = tid + i * kThreads;
            if (idx < kBM * hd) {
                const int m = idx / hd, d = idx - m * hd;
                float o = acc[i] * a_s[m];
                const float* p = Ss + m * (kBN + 1);
                for (int n = 0; n < kBN; ++n) o = fmaf(p[n], Vs[n * hd + d], o);
                acc[i] = o;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < kAccPerThread; ++i) {
        const int idx = tid + i * kThreads;
        if (idx < kBM * hd) {
            const int m = idx / hd, d = idx - m * hd;
            if (m < rows)
                out[static_cast<size_t>(row0 + m) * (nq * hd) + head * hd + d] =
                    from_float<T>(acc[i] / l_s[m]);
        }
    }
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_attention_generic_q_tile() { return kBM; }

SOMI_API int somi_paged_attention_generic(
    const void* qkv, int dtype, int row_stride, const void* kcache, const void* vcache,
    const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len, const int* tiles,
    int n_tiles, int n_prefill_req, int n_prefill_tok, int n_decode, int nq, int nkv, int hd,
    int page_size, float scale, int window, void* out, cudaStream_t stream) {
    if (n_tiles + n_decode <= 0) return 0;
    if (hd <= 0 || hd > kMaxHd || hd % 16 || nkv <= 0 || nq % nkv || page_size <= 0)
        return SOMI_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * (static_cast<size_t>(kBM) * hd + kBN * (hd + 1) + kBN * hd +
                                         kBM * (kBN + 1) + 3 * kBM);
    dim3 grid(n_tiles + n_decode, nq);
#define SOMI_LAUNCH_ATT(T)                                                                      \
    do {                                                                                        \
        if (smem > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(paged_attention_generic_kernel<T>,                             \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        launch_pdl(paged_attention_generic_kernel<T>, dim3(grid), dim3(kThreads), smem, stream,                     \
            static_cast<const T*>(qkv), row_stride, static_cast<const T*>(kcache),              \
            static_cast<const T*>(vcache), block_table, bt_stride, cu_q, ctx_len, tiles,        \
            n_tiles, n_prefill_req, n_prefill_tok, nq, nkv, hd, page_size, scale, window,       \
            static_cast<T*>(out));                                                              \
    } while (0)
    if (dtype == SOMI_F32) SOMI_LAUNCH_ATT(float);
    else SOMI_LAUNCH_ATT(__nv_bfloat16);
#undef SOMI_LAUNCH_ATT
    return launch_status();
}
