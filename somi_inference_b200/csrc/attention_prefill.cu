// Causal grouped-query attention for portions of prompts over the paged bfloat16 cache.
//
// A portion of q_len tokens of one request sits at positions ctx .. ctx + q_len - 1; its keys
// and values, like those of everything before it, are already in the cache, so one kernel
// serves a whole prompt, a later portion of it, or a portion of two tokens.  One CTA = one
// tile of up to 64 consecutive query rows of one request x one query head; each of its four
// warps owns 16 rows.  Key/value tiles of 64 positions are gathered page by page with
// asynchronous copies into double-buffered, swizzled shared memory; S = Q K^T and O += P V run
// on tensor cores (m16n8k16, float32 accumulation); the softmax is online, in float32, base 2.
// Key tiles are aligned to multiples of 64 from position 0, so the sequence of operations on a
// query row does not depend on where its portion was cut.
//
// The reference's prefill kernel (somi_inference/core/flash_attention_triton.py:31-194) is a
// FlashAttention-2 loop over a dense [B, heads, T, d] tensor without cached context; formulas
// in somi_inference/models/qwen2.py:158-186.
#include "mma.cuh"

namespace somi {

constexpr int kPfBM = 64;
constexpr int kPfBN = 64;
constexpr int kPfThreads = 128;

template <int HD>
__device__ __forceinline__ void load_kv_tile(unsigned char* Kd, unsigned char* Vd,
                                             const __nv_bfloat16* __restrict__ kcache,
                                             const __nv_bfloat16* __restrict__ vcache,
                                             const int* __restrict__ bt, int kb, int kv_first,
                                             int kv_end, int nkv, int kvh, int page_size, int tid) {
    constexpr int CPR = HD / 8;
    for (int c = tid; c < kPfBN * CPR; c += kPfThreads) {
        const int r = c / CPR, ch = c - r * CPR;
        const int j = kb + r;
        const bool ok = j >= kv_first && j < kv_end;
        size_t off = 0;
        if (ok) {
            const int page = bt[j / page_size];
            off = ((static_cast<size_t>(page) * nkv + kvh) * page_size + j % page_size) * HD + ch * 8;
        }
        const int so = swizzled_offset<HD>(r, ch);
        cp_async_16(smem_u32(Kd + so), kcache + off, ok ? 16 : 0);
        cp_async_16(smem_u32(Vd + so), vcache + off, ok ? 16 : 0);
    }
}

template <int HD>
__global__ void __launch_bounds__(kPfThreads)
paged_prefill_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride,
                     const __nv_bfloat16* __restrict__ kcache,
                     const __nv_bfloat16* __restrict__ vcache,
                     const int* __restrict__ block_table, int bt_stride,
                     const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                     const int* __restrict__ tiles, int nq, int nkv, int page_size,
                     float scale_log2e, int window, __nv_bfloat16* __restrict__ out) {
    constexpr int CPR = HD / 8;
    constexpr int TILE = kPfBN * HD * 2;                       // bytes of one K or V tile
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* Qs = smem_raw;                               // [64][HD]
    unsigned char* Ks = Qs + kPfBM * HD * 2;                    // 2 x [64][HD]
    unsigned char* Vs = Ks + 2 * TILE;                          // 2 x [64][HD]
    pdl_launch_dependents();
    pdl_wait();

    // later tiles of a prompt see more keys: they are started first so that the last CTAs
    // to run are the short ones
    const int tile = gridDim.x - 1 - blockIdx.x;
    const int req = tiles[3 * tile], row0 = tiles[3 * tile + 1];
    const int rows = tiles[3 * tile + 2];
    const int head = blockIdx.y, kvh = head / (nq / nkv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q_pos0 = ctx_len[req] + (row0 - cu_q[req]);
    const int kv_end = q_pos0 + rows;
    const int kv_first = window > 0 ? max(0, q_pos0 - window + 1) : 0;
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;

    for (int c = tid; c < kPfBM * CPR; c += kPfThreads) {
        const int r = c / CPR, ch = c - r * CPR;
        const bool ok = r < rows;
        const __nv_bfloat16* src = qkv + static_cast<size_t>(row0 + (ok ? r : 0)) * row_stride + head * HD + ch * 8;
        cp_async_16(smem_u32(Qs + swizzled_offset<HD>(r, ch)), src, ok ? 16 : 0);
    }
    const int kb0 = (kv_first / kPfBN) * kPfBN;
    const int n_tiles = (kv_end - kb0 + kPfBN - 1) / kPfBN;
    load_kv_tile<HD>(Ks, Vs, kcache, vcache, bt, kb0, kv_first, kv_end, nkv, kvh, page_size, tid);
    cp_async_commit();

    float o[HD / 8][4];
#pragma unroll
    for (int a = 0; a < HD / 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) o[a][b] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const int qr = warp * 16;                                   // this warp's first row in the tile
    const int pos_lo = q_pos0 + qr + (lane >> 2), pos_hi = pos_lo + 8;

    for (int t = 0; t < n_tiles; ++t) {
        const int kb = kb0 + t * kPfBN;
        const int buf = t & 1;
        if (t + 1 < n_tiles)
            load_kv_tile<HD>(Ks + (buf ^ 1) * TILE, Vs + (buf ^ 1) * TILE, kcache, vcache, bt,
                             kb + kPfBN, kv_first, kv_end, nkv, kvh, page_size, tid);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* Kt = Ks + buf * TILE;
        const unsigned char* Vt = Vs + buf * TILE;

        // a warp whose rows all lie before this tile's first key has nothing to do in it
        if (kb <= q_pos0 + qr + 15) {
            float s[8][4];
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, smem_u32(Qs + swizzled_offset<HD>(qr + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                                2 * ks + (lane >> 4))));
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, smem_u32(Kt + swizzled_offset<HD>(np * 16 + (lane & 7) + (lane >> 4) * 8,
                                                                    2 * ks + ((lane >> 3) & 1))));
                    mma_bf16_16816(s[2 * np], a, b[0], b[1]);
                    mma_bf16_16816(s[2 * np + 1], a, b[2], b[3]);
                }
            }
            // mask (causal, window, end of the cache) and row maxima
            float t_lo = -INFINITY, t_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = kb + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = e < 2 ? pos_lo : pos_hi;
                    const bool ok = key <= pos && key >= kv_first && (window <= 0 || key > pos - window);
                    const float v = ok ? s[nt][e] * scale_log2e : -INFINITY;
                    s[nt][e] = v;
                    if (e < 2) t_lo = fmaxf(t_lo, v); else t_hi = fmaxf(t_hi, v);
                }
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1));
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
            const float n_lo = fmaxf(m_lo, t_lo), n_hi = fmaxf(m_hi, t_hi);
            const float b_lo = n_lo == -INFINITY ? 0.f : n_lo, b_hi = n_hi == -INFINITY ? 0.f : n_hi;
            const float a_lo = exp2f(m_lo - b_lo), a_hi = exp2f(m_hi - b_hi);
            m_lo = n_lo;
            m_hi = n_hi;
            float r_lo = 0.f, r_hi = 0.f;
            uint32_t pa[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const uint32_t lo = pack_bf16(exp2f(s[nt][0] - b_lo), exp2f(s[nt][1] - b_lo));
                const uint32_t hi = pack_bf16(exp2f(s[nt][2] - b_hi), exp2f(s[nt][3] - b_hi));
                const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&lo);
                const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&hi);
                r_lo += __low2float(lo2) + __high2float(lo2);
                r_hi += __low2float(hi2) + __high2float(hi2);
                pa[nt >> 1][(nt & 1) * 2] = lo;
                pa[nt >> 1][(nt & 1) * 2 + 1] = hi;
            }
            r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 1);
            r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 2);
            r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 1);
            r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 2);
            l_lo = l_lo * a_lo + r_lo;
            l_hi = l_hi * a_hi + r_hi;
#pragma unroll
            for (int nt = 0; nt < HD / 8; ++nt) {
                o[nt][0] *= a_lo; o[nt][1] *= a_lo;
                o[nt][2] *= a_hi; o[nt][3] *= a_hi;
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                for (int dc = 0; dc < HD / 16; ++dc) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, smem_u32(Vt + swizzled_offset<HD>(
                                             kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                             2 * dc + (lane >> 4))));
                    mma_bf16_16816(o[2 * dc], pa[kk], b[0], b[1]);
                    mma_bf16_16816(o[2 * dc + 1], pa[kk], b[2], b[3]);
                }
        }
        __syncthreads();     // everyone is done with this buffer before it is filled again
    }

    const int r_lo = qr + (lane >> 2), r_hi = r_lo + 8;
    const float i_lo = 1.0f / l_lo, i_hi = 1.0f / l_hi;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        const int d = nt * 8 + (lane & 3) * 2;
        if (r_lo < rows)
            *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(row0 + r_lo) * nq * HD + head * HD + d) =
                pack_bf16(o[nt][0] * i_lo, o[nt][1] * i_lo);
        if (r_hi < rows)
            *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(row0 + r_hi) * nq * HD + head * HD + d) =
                pack_bf16(o[nt][2] * i_hi, o[nt][3] * i_hi);
    }
}

template <int HD>
int launch_prefill(const void* qkv, int row_stride, const void* kcache, const void* vcache,
                   const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len,
                   const int* tiles, int n_tiles, int nq, int nkv, int page_size, float scale,
                   int window, void* out, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(kPfBM + 4 * kPfBN) * HD * 2;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(paged_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    dim3 grid(n_tiles, nq);
    launch_pdl(paged_prefill_kernel<HD>, dim3(grid), dim3(kPfThreads), smem, stream, 
        static_cast<const __nv_bfloat16*>(qkv), row_stride,
        static_cast<const __nv_bfloat16*>(kcache), static_cast<const __nv_bfloat16*>(vcache),
        block_table, bt_stride, cu_q, ctx_len, tiles, nq, nkv, page_size,
        scale * 1.4426950408889634f, window, static_cast<__nv_bfloat16*>(out));
    return launch_status();
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_prefill_q_tile() { return kPfBM; }

SOMI_API int somi_prefill_supported(int nq, int nkv, int hd) {
    if (nkv <= 0 || nq % nkv) return 0;
    return hd == 32 || hd == 64 || hd == 128;
}

// `tiles`: int32 [n_tiles, 3] = (request, first row, rows <= 64) over the multi-token requests.
SOMI_API int somi_paged_attention_prefill(
    const void* qkv, int row_stride, const void* kcache, const void* vcache,
    const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len, const int* tiles,
    int n_tiles, int nq, int nkv, int hd, int page_size, float scale, int window, void* out,
    cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!somi_prefill_supported(nq, nkv, hd) || page_size <= 0 || nq > 65535)
        return SOMI_ERR_UNSUPPORTED;
#define SOMI_PF(HD)                                                                             \
    return launch_prefill<HD>(qkv, row_stride, kcache, vcache, block_table, bt_stride, cu_q,    \
                              ctx_len, tiles, n_tiles, nq, nkv, page_size, scale, window, out,  \
                              stream)
    if (hd == 32) SOMI_PF(32);
    if (hd == 64) SOMI_PF(64);
    SOMI_PF(128);
#undef SOMI_PF
}
