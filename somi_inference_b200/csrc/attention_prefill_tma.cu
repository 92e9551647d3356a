// Prompt-portion attention whose keys and values arrive by TMA.
//
// Same tiling and arithmetic as attention_prefill.cu (one CTA = up to 64 query rows of one
// request x one query head, four warps of 16 rows, key tiles of 64 positions aligned to
// multiples of 64, online float32 softmax, m16n8k16 MMAs), but the key/value tiles are fetched
// page by page with `cp.async.bulk.tensor.2d` into a two-stage ring of hardware-swizzled
// shared memory, signalled by mbarriers; one thread looks the pages up and issues the copies,
// so no thread computes per-element cache addresses.  Tiles that lie wholly inside every
// row's visible range skip the mask, and exponentials use the hardware approximation.
//
// Needs head_dim 64 or 128 and a page size that is a multiple of 8 and divides 64.
#include "mma.cuh"
#include "tma.cuh"

namespace somi {

constexpr int kTpBM = 64;
constexpr int kTpBN = 64;
constexpr int kTpThreads = 128;
constexpr int kTpHalfBytes = kTpBN * 128;        // one 64-element half of a 64-key tile

__device__ int g_prefill_tma_error = 0;

__device__ __forceinline__ int tp_tile_offset(int key, int chunk) {
    return (chunk >> 3) * kTpHalfBytes + key * 128 + (((chunk & 7) ^ (key & 7)) << 4);
}

template <int HD>
__global__ void __launch_bounds__(kTpThreads)
paged_prefill_tma_kernel(const __grid_constant__ CUtensorMap kv_map,
                         const __nv_bfloat16* __restrict__ qkv, int row_stride, long long k_row0,
                         long long v_row0, const int* __restrict__ block_table, int bt_stride,
                         const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                         const int* __restrict__ tiles, int nq, int nkv, int page_size,
                         float scale_log2e, int window, __nv_bfloat16* __restrict__ out) {
    constexpr int CPR = HD / 8;
    constexpr int HALVES = HD / 64;
    constexpr int TILE = HALVES * kTpHalfBytes;                 // bytes of one K or V tile
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* Ks = base;                                   // 2 stages x HALVES x [64][64]
    unsigned char* Vs = Ks + 2 * TILE;
    unsigned char* Qs = Vs + 2 * TILE;                          // [64][HD], software swizzle
    __shared__ __align__(8) unsigned long long full_bar[2];

    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        mbar_init(smem_u32(&full_bar[0]), 1);
        mbar_init(smem_u32(&full_bar[1]), 1);
        mbar_fence_init();
    }
    // value rows that no copy ever fills (pages outside the request's range in the first and
    // last tile) must hold finite numbers: they are multiplied by probabilities that are zero
    for (int c = tid; c < 2 * TILE / 16; c += kTpThreads)
        reinterpret_cast<uint4*>(Vs)[c] = make_uint4(0, 0, 0, 0);
    pdl_wait();

    // later tiles of a prompt see more keys: they are started first so that the last CTAs
    // to run are the short ones
    const int tile = gridDim.x - 1 - blockIdx.x;
    const int req = tiles[3 * tile], row0 = tiles[3 * tile + 1];
    const int rows = tiles[3 * tile + 2];
    const int head = blockIdx.y, kvh = head / (nq / nkv);
    const int q_pos0 = ctx_len[req] + (row0 - cu_q[req]);
    const int kv_end = q_pos0 + rows;
    const int kv_first = window > 0 ? max(0, q_pos0 - window + 1) : 0;
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;

    for (int c = tid; c < kTpBM * CPR; c += kTpThreads) {
        const int r = c / CPR, ch = c - r * CPR;
        const bool ok = r < rows;
        const __nv_bfloat16* src = qkv + static_cast<size_t>(row0 + (ok ? r : 0)) * row_stride + head * HD + ch * 8;
        cp_async_16(smem_u32(Qs + swizzled_offset<HD>(r, ch)), src, ok ? 16 : 0);
    }
    cp_async_commit();
    const int kb0 = (kv_first / kTpBN) * kTpBN;
    const int n_tiles = (kv_end - kb0 + kTpBN - 1) / kTpBN;

    // one thread issues, for a tile, the copies of every page that holds keys the tile's rows
    // may read, keys and values on the stage's barrier
    auto issue_tile = [&](int t) {
        const int kb = kb0 + t * kTpBN;
        const int stage = t & 1;
        const int p_lo = max(kb, kv_first) / page_size;
        const int p_hi = (min(kb + kTpBN, kv_end) - 1) / page_size;
        const uint32_t bar = smem_u32(&full_bar[stage]);
        mbar_expect_tx(bar, static_cast<uint32_t>(p_hi - p_lo + 1) * page_size * HD * 2 * 2);
        for (int ap = p_lo; ap <= p_hi; ++ap) {
            const long long prow = (static_cast<long long>(bt[ap]) * nkv + kvh) * page_size;
            const int r = ap * page_size - kb;                 // the page's first row in the tile
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
                tma_load_2d(smem_u32(Ks + stage * TILE + h * kTpHalfBytes + r * 128), &kv_map,
                            h * 64, static_cast<int>(k_row0 + prow), bar);
                tma_load_2d(smem_u32(Vs + stage * TILE + h * kTpHalfBytes + r * 128), &kv_map,
                            h * 64, static_cast<int>(v_row0 + prow), bar);
            }
        }
    };
    fence_proxy_async();       // the zero fill is ordered before the copies into the same bytes
    cp_async_wait<0>();
    __syncthreads();
    if (tid == 0) issue_tile(0);

    float o[HD / 8][4];
#pragma unroll
    for (int a = 0; a < HD / 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) o[a][b] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const int qr = warp * 16;                                   // this warp's first row in the tile
    const int pos_lo = q_pos0 + qr + (lane >> 2), pos_hi = pos_lo + 8;

    bool copies_ok = true;
    for (int t = 0; t < n_tiles; ++t) {
        const int kb = kb0 + t * kTpBN;
        const int buf = t & 1;
        // the other stage was released by the barrier that ended the previous iteration
        if (tid == 0 && t + 1 < n_tiles) issue_tile(t + 1);
        copies_ok = mbar_wait(smem_u32(&full_bar[buf]), (t >> 1) & 1) && copies_ok;
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
                    ldmatrix_x4(b, smem_u32(Kt + tp_tile_offset(np * 16 + (lane & 7) + (lane >> 4) * 8,
                                                               2 * ks + ((lane >> 3) & 1))));
                    mma_bf16_16816(s[2 * np], a, b[0], b[1]);
                    mma_bf16_16816(s[2 * np + 1], a, b[2], b[3]);
                }
            }
            // mask (causal, window) where this tile can hold hidden keys for this warp's rows;
            // tiles that lie wholly inside every row's visible range skip the comparisons
            float t_lo = -INFINITY, t_hi = -INFINITY;
            const bool edge = kb + kTpBN - 1 > q_pos0 + qr || kb < kv_first ||
                              (window > 0 && kb <= q_pos0 + qr + 15 - window);
            if (edge) {
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
            } else {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float v = s[nt][e] * scale_log2e;
                        s[nt][e] = v;
                        if (e < 2) t_lo = fmaxf(t_lo, v); else t_hi = fmaxf(t_hi, v);
                    }
            }
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1));
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
            const float n_lo = fmaxf(m_lo, t_lo), n_hi = fmaxf(m_hi, t_hi);
            const float b_lo = n_lo == -INFINITY ? 0.f : n_lo, b_hi = n_hi == -INFINITY ? 0.f : n_hi;
            const float a_lo = fast_exp2(m_lo - b_lo), a_hi = fast_exp2(m_hi - b_hi);
            m_lo = n_lo;
            m_hi = n_hi;
            float r_lo = 0.f, r_hi = 0.f;
            uint32_t pa[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const uint32_t lo = pack_bf16(fast_exp2(s[nt][0] - b_lo), fast_exp2(s[nt][1] - b_lo));
                const uint32_t hi = pack_bf16(fast_exp2(s[nt][2] - b_hi), fast_exp2(s[nt][3] - b_hi));
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
                    ldmatrix_x4_trans(b, smem_u32(Vt + tp_tile_offset(
                                             kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                             2 * dc + (lane >> 4))));
                    mma_bf16_16816(o[2 * dc], pa[kk], b[0], b[1]);
                    mma_bf16_16816(o[2 * dc + 1], pa[kk], b[2], b[3]);
                }
        }
        __syncthreads();     // everyone is done with this buffer before it is filled again
    }

    if (!copies_ok && lane == 0) atomicExch(&g_prefill_tma_error, 1);
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
int launch_prefill_tma(const CUtensorMap* map, const void* qkv, int row_stride, long long k_row0,
                       long long v_row0, const int* block_table, int bt_stride, const int* cu_q,
                       const int* ctx_len, const int* tiles, int n_tiles, int nq, int nkv,
                       int page_size, float scale, int window, void* out, cudaStream_t stream) {
    constexpr int TILE = (HD / 64) * kTpHalfBytes;
    const size_t smem = 4 * TILE + kTpBM * HD * 2 + 1024;
    cudaFuncSetAttribute(paged_prefill_tma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
    dim3 grid(n_tiles, nq);
    launch_pdl(paged_prefill_tma_kernel<HD>, grid, dim3(kTpThreads), smem, stream, *map,
               static_cast<const __nv_bfloat16*>(qkv), row_stride, k_row0, v_row0, block_table,
               bt_stride, cu_q, ctx_len, tiles, nq, nkv, page_size,
               scale * 1.4426950408889634f, window, static_cast<__nv_bfloat16*>(out));
    return launch_status();
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_prefill_tma_supported(int nq, int nkv, int hd, int page_size) {
    if (nkv <= 0 || nq % nkv) return 0;
    if (hd != 64 && hd != 128) return 0;
    return page_size >= 8 && page_size % 8 == 0 && kTpBN % page_size == 0;
}

SOMI_API int somi_prefill_tma_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_prefill_tma_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_prefill_tma_error, &zero, sizeof(int));
    return v;
}

// `tensor_map`: the cache storage's map as made by somi_make_kv_tensor_map (boxes of one page).
SOMI_API int somi_paged_attention_prefill_tma(
    const void* tensor_map, const void* qkv, int row_stride, long long k_row0, long long v_row0,
    const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len, const int* tiles,
    int n_tiles, int nq, int nkv, int hd, int page_size, float scale, int window, void* out,
    cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!somi_prefill_tma_supported(nq, nkv, hd, page_size) || nq > 65535) return SOMI_ERR_UNSUPPORTED;
    const CUtensorMap* map = static_cast<const CUtensorMap*>(tensor_map);
    if (hd == 64)
        return launch_prefill_tma<64>(map, qkv, row_stride, k_row0, v_row0, block_table, bt_stride,
                                      cu_q, ctx_len, tiles, n_tiles, nq, nkv, page_size, scale,
                                      window, out, stream);
    return launch_prefill_tma<128>(map, qkv, row_stride, k_row0, v_row0, block_table, bt_stride,
                                   cu_q, ctx_len, tiles, n_tiles, nq, nkv, page_size, scale, window,
                                   out, stream);
}
