// Split-KV grouped-query decode attention whose keys and values arrive by TMA.
//
// Same decomposition and arithmetic as attention_decode.cu (one CTA = request x kv head x
// 128 keys, all query heads of the group as MMA rows, partial results merged by a second
// kernel), but the cache pages are fetched by bulk tensor copies: one thread issues, per page,
// one `cp.async.bulk.tensor.2d` per 64-element half of the head for keys and one for values;
// the 128-byte hardware swizzle lays the rows out conflict-free for ldmatrix, and two
// mbarriers tell the warps when the keys and when the values have landed.  No thread computes
// a per-element address.  The cache group's whole storage is one 2-D tensor map
// [rows = runs * 2 * pages * kv_heads * page_size, head_dim]; a page of one kv head is
// page_size consecutive rows.
//
// Needs head_dim 64 or 128 and a page size that is a multiple of 8 and divides 128.
#include <algorithm>

#include "attention_merge.cuh"
#include "mma.cuh"
#include "tma.cuh"

namespace somi {

constexpr int kTdChunk = 128;
constexpr int kTdThreads = 128;     // 4 warps: 32 keys each for the scores, HD/4 columns each for P.V
constexpr int kTdWarps = kTdThreads / 32;
constexpr int kTdRows = 16;
constexpr int kHalfBytes = kTdChunk * 128;     // one 64-element half of a 128-key tile

__device__ int g_decode_tma_error = 0;          // set when a bounded wait ran out

// byte offset of 16-byte chunk `chunk` (0 .. HD/8) of key `key` in a tile made of HD/64 halves
__device__ __forceinline__ int tma_tile_offset(int key, int chunk) {
    return (chunk >> 3) * kHalfBytes + key * 128 + (((chunk & 7) ^ (key & 7)) << 4);
}

struct TdRange {
    int kv_len, first_key, first_split, n_splits;
};
__device__ __forceinline__ TdRange td_range(int ctx_len, int window) {
    TdRange r;
    r.kv_len = ctx_len + 1;
    r.first_key = window > 0 ? max(0, ctx_len - window + 1) : 0;
    r.first_split = r.first_key / kTdChunk;
    r.n_splits = (r.kv_len + kTdChunk - 1) / kTdChunk;
    return r;
}

template <int HD>
__global__ void __launch_bounds__(kTdThreads, 3)
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap kv_map,
                        const __nv_bfloat16* __restrict__ qkv, int row_stride, int row_base,
                        int req_base, long long k_row0, long long v_row0,
                        const int* __restrict__ block_table, int bt_stride,
                        const int* __restrict__ ctx_len, int nq, int nkv, int page_size,
                        float scale_log2e, int window, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int max_splits,
                        __nv_bfloat16* __restrict__ out) {
    constexpr int CPR = HD / 8;
    constexpr int HALVES = HD / 64;
    constexpr int TILE = HALVES * kHalfBytes;
    constexpr int DW = HD / kTdWarps;             // output columns owned by one warp in P.V
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* Ks = base;                     // HALVES x [128][64] bf16, hardware swizzle
    unsigned char* Vs = Ks + TILE;
    unsigned char* Qs = Vs + TILE;                // [16][HD] bf16, software swizzle
    unsigned char* Ps = Qs + kTdRows * HD * 2;    // [16][128 keys] bf16, software swizzle
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ float m_s[kTdWarps][kTdRows], l_s[kTdWarps][kTdRows];
    pdl_launch_dependents();
    // A kernel of this step wrote the step's own keys and values (one position per request
    // here) and the queries.  Lengths and block tables [descriptor] and the cache pages of older
    // positions [old-cache] are written by no kernel of this step, so their copies are issued
    // before the dependency wait and fly while the predecessor finishes; only the page of the
    // newest position and Q come after the wait.

    const int split = blockIdx.x, kvh = blockIdx.y, i = blockIdx.z;
    const int req = req_base + i, row = row_base + i;
    const int G = nq / nkv;
    const TdRange rg = td_range(ld_step(ctx_len + req), window);      // before the wait
    if (split < rg.first_split || split >= rg.n_splits) {
        pdl_wait();
        return;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k0 = split * kTdChunk;
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;
    const uint32_t bar_k = smem_u32(&bars[0]), bar_v = smem_u32(&bars[1]);

    // pages of this chunk that hold keys the request reads
    const int pages_in_chunk = kTdChunk / page_size;
    const int first_page = max(k0, rg.first_key) / page_size;             // absolute index
    const int last_page = (min(k0 + kTdChunk, rg.kv_len) - 1) / page_size;
    const int chunk_page0 = k0 / page_size;
    const int newest_page = (rg.kv_len - 1) / page_size;                  // written by the predecessor

    // Warp 0 starts the copies before anything else: lane 0 arms both barriers with the byte
    // counts, then one lane per page looks its page up and issues that page's copies, so the
    // page-table reads run side by side instead of one after another.
    if (warp == 0) {
        if (lane == 0) {
            mbar_init(bar_k, 1);
            mbar_init(bar_v, 1);
            mbar_fence_init();
            const uint32_t bytes = static_cast<uint32_t>(last_page - first_page + 1) * page_size * HD * 2;
            mbar_expect_tx(bar_k, bytes);
            mbar_expect_tx(bar_v, bytes);
        }
        __syncwarp();
        for (int p = lane; p < pages_in_chunk; p += 32) {
            const int ap = chunk_page0 + p;
            if (ap < first_page || ap > last_page || ap == newest_page) continue;
            const long long prow = (static_cast<long long>(ld_step(bt + ap)) * nkv + kvh) * page_size;
            const int r = p * page_size;
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
                tma_load_2d(smem_u32(Ks + h * kHalfBytes + r * 128), &kv_map, h * 64,
                            static_cast<int>(k_row0 + prow), bar_k);
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
                tma_load_2d(smem_u32(Vs + h * kHalfBytes + r * 128), &kv_map, h * 64,
                            static_cast<int>(v_row0 + prow), bar_v);
        }
    }
    // V rows of pages that are not loaded must not hold stale non-finite bit patterns
    for (int p = 0; p < pages_in_chunk; ++p) {
        const int ap = chunk_page0 + p;
        if (ap >= first_page && ap <= last_page) continue;
        for (int c = tid; c < page_size * CPR; c += kTdThreads) {
            const int r = p * page_size + c / CPR, ch = c % CPR;
            *reinterpret_cast<uint4*>(Vs + tma_tile_offset(r, ch)) = make_uint4(0, 0, 0, 0);
        }
    }
    pdl_wait();
    if (warp == 0 && newest_page >= max(first_page, chunk_page0) &&
        newest_page <= last_page && lane == (newest_page - chunk_page0) % 32) {
        const int p = newest_page - chunk_page0;
        const long long prow = (static_cast<long long>(ld_step(bt + newest_page)) * nkv + kvh) * page_size;
        const int r = p * page_size;
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
            tma_load_2d(smem_u32(Ks + h * kHalfBytes + r * 128), &kv_map, h * 64,
                        static_cast<int>(k_row0 + prow), bar_k);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
            tma_load_2d(smem_u32(Vs + h * kHalfBytes + r * 128), &kv_map, h * 64,
                        static_cast<int>(v_row0 + prow), bar_v);
    }
    // Q: rows of the group's heads, zero rows up to 16
    const __nv_bfloat16* qrow = qkv + static_cast<size_t>(row) * row_stride + static_cast<size_t>(kvh) * G * HD;
    for (int c = tid; c < kTdRows * CPR; c += kTdThreads) {
        const int r = c / CPR, ch = c - r * CPR;
        const bool ok = r < G;
        cp_async_16(smem_u32(Qs + swizzled_offset<HD>(r, ch)), ok ? qrow + r * HD + ch * 8 : qrow,
                    ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();      // Q is in place; the barriers' initialisation is visible to all warps

    bool ok_wait = mbar_wait(bar_k, 0);
    // ---- S = Q K^T for this warp's 32 keys
    float s[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
    const int kw = warp * 32;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, smem_u32(Qs + swizzled_offset<HD>((lane & 7) + ((lane >> 3) & 1) * 8,
                                                        2 * ks + (lane >> 4))));
#pragma unroll
        for (int np = 0; np < 2; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, smem_u32(Ks + tma_tile_offset(kw + np * 16 + (lane & 7) + (lane >> 4) * 8,
                                                         2 * ks + ((lane >> 3) & 1))));
            mma_bf16_16816(s[2 * np], a, b[0], b[1]);
            mma_bf16_16816(s[2 * np + 1], a, b[2], b[3]);
        }
    }
    // ---- mask; the row maximum is taken over the whole chunk (all four warps)
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    float m_lo = -INFINITY, m_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = k0 + kw + nt * 8 + (lane & 3) * 2 + (e & 1);
            const bool ok = key < rg.kv_len && key >= rg.first_key;
            const float v = ok ? s[nt][e] * scale_log2e : -INFINITY;
            s[nt][e] = v;
            if (e < 2) m_lo = fmaxf(m_lo, v); else m_hi = fmaxf(m_hi, v);
        }
    m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 1));
    m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 2));
    m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 1));
    m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 2));
    if ((lane & 3) == 0) { m_s[warp][r_lo] = m_lo; m_s[warp][r_hi] = m_hi; }
    __syncthreads();
    float M_lo = fmaxf(fmaxf(m_s[0][r_lo], m_s[1][r_lo]), fmaxf(m_s[2][r_lo], m_s[3][r_lo]));
    float M_hi = fmaxf(fmaxf(m_s[0][r_hi], m_s[1][r_hi]), fmaxf(m_s[2][r_hi], m_s[3][r_hi]));
    // a valid chunk has at least one visible key, so the maxima of real rows are finite
    const float b_lo = M_lo == -INFINITY ? 0.f : M_lo, b_hi = M_hi == -INFINITY ? 0.f : M_hi;
    float l_lo = 0.f, l_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const uint32_t lo = pack_bf16(fast_exp2(s[nt][0] - b_lo), fast_exp2(s[nt][1] - b_lo));
        const uint32_t hi = pack_bf16(fast_exp2(s[nt][2] - b_hi), fast_exp2(s[nt][3] - b_hi));
        const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&lo);
        const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&hi);
        l_lo += __low2float(lo2) + __high2float(lo2);
        l_hi += __low2float(hi2) + __high2float(hi2);
        // P goes to shared memory: every warp needs all 128 keys of it for its output columns
        const int chunk = warp * 4 + nt;
        *reinterpret_cast<uint32_t*>(Ps + swizzled_offset<128>(r_lo, chunk) + (lane & 3) * 4) = lo;
        *reinterpret_cast<uint32_t*>(Ps + swizzled_offset<128>(r_hi, chunk) + (lane & 3) * 4) = hi;
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if ((lane & 3) == 0) { l_s[warp][r_lo] = l_lo; l_s[warp][r_hi] = l_hi; }

    ok_wait = mbar_wait(bar_v, 0) && ok_wait;
    if (!ok_wait) {
        // a copy did not complete within the limit: record it; the values written below are
        // not to be trusted and the host raises when it reads the error word
        if (lane == 0) atomicExch(&g_decode_tma_error, 1);
    }
    __syncthreads();       // P and the row sums of all warps are in shared memory

    // ---- O[:, warp's DW columns] = P V over all 128 keys: no reduction across warps
    float o[DW / 8][4];
#pragma unroll
    for (int a = 0; a < DW / 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) o[a][b] = 0.f;
    const int c0 = warp * (DW / 8);               // first 16-byte chunk of this warp's columns
#pragma unroll
    for (int kk = 0; kk < kTdChunk / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, smem_u32(Ps + swizzled_offset<128>((lane & 7) + ((lane >> 3) & 1) * 8,
                                                         2 * kk + (lane >> 4))));
#pragma unroll
        for (int dc = 0; dc < DW / 16; ++dc) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, smem_u32(Vs + tma_tile_offset(
                                     kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                     c0 + 2 * dc + (lane >> 4))));
            mma_bf16_16816(o[2 * dc], a, b[0], b[1]);
            mma_bf16_16816(o[2 * dc + 1], a, b[2], b[3]);
        }
    }
    const float L_lo = l_s[0][r_lo] + l_s[1][r_lo] + l_s[2][r_lo] + l_s[3][r_lo];
    const float L_hi = l_s[0][r_hi] + l_s[1][r_hi] + l_s[2][r_hi] + l_s[3][r_hi];
    const bool single = rg.n_splits - rg.first_split == 1;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int g = half ? r_hi : r_lo;
        if (g >= G) continue;
        const int head = kvh * G + g;
        const float L = half ? L_hi : L_lo, M = half ? M_hi : M_lo;
        if (single) {
            const float inv = 1.0f / L;
            __nv_bfloat16* dst = out + static_cast<size_t>(row) * nq * HD + head * HD + warp * DW;
#pragma unroll
            for (int nt = 0; nt < DW / 8; ++nt)
                *reinterpret_cast<uint32_t*>(dst + nt * 8 + (lane & 3) * 2) =
                    pack_bf16(o[nt][half * 2] * inv, o[nt][half * 2 + 1] * inv);
        } else {
            const size_t p = (static_cast<size_t>(i) * nq + head) * max_splits + split;
            float* dst = part_o + p * HD + warp * DW;
#pragma unroll
            for (int nt = 0; nt < DW / 8; ++nt)
                *reinterpret_cast<float2*>(dst + nt * 8 + (lane & 3) * 2) =
                    make_float2(o[nt][half * 2], o[nt][half * 2 + 1]);
            if (warp == 0 && (lane & 3) == 0) { part_ml[2 * p] = M; part_ml[2 * p + 1] = L; }
        }
    }
}

// ---------------------------------------------------------------------------------------
// The same attention for steps with many chunks (large batches, long contexts): a CTA takes
// `cpc` consecutive chunks of one (request, kv head).  Q and the barriers are set up once, the
// running maximum, sum and output stay in registers from chunk to chunk (one partial result
// per CTA, `cpc` times fewer for the merge), and the next chunk's values and, as soon as the
// scores are taken, its keys are copied while a chunk is computed.  Two further warps issue
// the copies, one the keys' and one the values': what bounds a warp that issues 2 KB copies
// is their number, and the computing warps should not pay for it.  One key tile and two value
// tiles: at head size 128 that leaves room for two CTAs per SM, whose phases overlap; two and
// three tiles with one CTA per SM were slower than the one-chunk kernel.
constexpr int kRingK = 1, kRingV = 2;
constexpr int kRingThreads = kTdThreads + 64;    // four computing warps, two producer warps
__device__ __forceinline__ void ring_compute_sync() {         // the four computing warps only
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
}
constexpr int kRingMaxCpc = 8;
static int g_ring_chunks = 0;           // chunks per CTA; 0: chosen from the step's size

template <int HD>
__global__ void __launch_bounds__(kRingThreads)
paged_decode_ring_kernel(const __grid_constant__ CUtensorMap kv_map,
                         const __nv_bfloat16* __restrict__ qkv, int row_stride, int row_base,
                         int req_base, long long k_row0, long long v_row0,
                         const int* __restrict__ block_table, int bt_stride,
                         const int* __restrict__ ctx_len, int nq, int nkv, int page_size,
                         float scale_log2e, int window, float* __restrict__ part_o,
                         float* __restrict__ part_ml, int max_splits, int cpc,
                         __nv_bfloat16* __restrict__ out) {
    constexpr int CPR = HD / 8;
    constexpr int HALVES = HD / 64;
    constexpr int TILE = HALVES * kHalfBytes;
    constexpr int DW = HD / kTdWarps;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* Ks = base;                              // kRingK tiles
    unsigned char* Vs = Ks + kRingK * TILE;                // kRingV tiles
    unsigned char* Qs = Vs + kRingV * TILE;                // [16][HD] bf16, software swizzle
    unsigned char* Ps = Qs + kTdRows * HD * 2;             // [16][128 keys] bf16, software swizzle
    __shared__ __align__(8) unsigned long long k_full[kRingK], k_empty[kRingK], v_full[kRingV], v_empty[kRingV];
    __shared__ float m_s[kTdWarps][kTdRows], l_s[kTdWarps][kTdRows];
    pdl_launch_dependents();

    const int group = blockIdx.x, kvh = blockIdx.y, i = blockIdx.z;
    const int req = req_base + i, row = row_base + i;
    const int G = nq / nkv;
    const TdRange rg = td_range(ld_step(ctx_len + req), window);      // before the wait
    const int c_begin = max(group * cpc, rg.first_split);
    const int c_end = min((group + 1) * cpc, rg.n_splits);
    if (c_begin >= c_end) {
        pdl_wait();
        return;
    }
    const int n_chunks = c_end - c_begin;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;
    const int pages_in_chunk = kTdChunk / page_size;
    const int newest_page = (rg.kv_len - 1) / page_size;   // written by the kernel before this one

    // pages of chunk c (counted from c_begin) that hold keys the request reads
    auto first_page_of = [&](int c) { return max((c_begin + c) * kTdChunk, rg.first_key) / page_size; };
    auto last_page_of = [&](int c) {
        return (min((c_begin + c + 1) * kTdChunk, rg.kv_len) - 1) / page_size;
    };
    if (tid == 0) {
        for (int x = 0; x < kRingK; ++x) {
            mbar_init(smem_u32(&k_full[x]), 1);
            mbar_init(smem_u32(&k_empty[x]), kTdWarps);     // one arrival per computing warp
        }
        for (int x = 0; x < kRingV; ++x) {
            mbar_init(smem_u32(&v_full[x]), 1);
            mbar_init(smem_u32(&v_empty[x]), kTdWarps);
        }
        mbar_fence_init();
    }
    // When a value tile of the ring is used for the first time, the rows of pages that are not
    // copied must not hold stale non-finite bit patterns (later they hold an older chunk's values,
    // which meet probabilities of zero).
    for (int c = 0; c < min(n_chunks, kRingV); ++c) {
        const int fp = first_page_of(c), lp = last_page_of(c);
        for (int pg = 0; pg < pages_in_chunk; ++pg) {
            const int ap = (c_begin + c) * pages_in_chunk + pg;
            if (ap >= fp && ap <= lp) continue;
            for (int x = tid; x < page_size * CPR; x += kRingThreads) {
                const int r = pg * page_size + x / CPR, ch = x % CPR;
                *reinterpret_cast<uint4*>(Vs + c * TILE + tma_tile_offset(r, ch)) = make_uint4(0, 0, 0, 0);
            }
        }
    }
    fence_proxy_async();       // those rows are overwritten by bulk copies of later chunks
    __syncthreads();           // the barriers are initialised

    if (warp >= kTdWarps) {
        // ---- producer warps: warp 4 the keys, warp 5 the values.  Lane 0 keeps the barriers,
        // one lane per page looks its page up and issues that page's copies.  Older cache pages,
        // lengths and block tables were complete before the kernel before this one started, so
        // their copies fly while it finishes; only the newest position's page waits for it.
        const bool values = warp == kTdWarps + 1;
        const int depth = values ? kRingV : kRingK;
        unsigned long long* full = values ? v_full : k_full;
        unsigned long long* empty = values ? v_empty : k_empty;
        unsigned char* tiles = values ? Vs : Ks;
        const long long row0 = values ? v_row0 : k_row0;
        bool waited = false;
        for (int c = 0; c < n_chunks; ++c) {
            const int st = c % depth;
            if (c >= depth && !mbar_wait(smem_u32(&empty[st]), (c / depth - 1) & 1)) {
                if (lane == 0) atomicExch(&g_decode_tma_error, 1);
                break;
            }
            const int fp = first_page_of(c), lp = last_page_of(c);
            if (lane == 0)
                mbar_expect_tx(smem_u32(&full[st]), static_cast<uint32_t>(lp - fp + 1) * page_size * HD * 2);
            __syncwarp();
            const int ap = (c_begin + c) * pages_in_chunk + lane;
            const bool mine = lane < pages_in_chunk && ap >= fp && ap <= lp;
            const bool has_newest = newest_page >= fp && newest_page <= lp;
            auto copy = [&]() {
                const long long prow = (static_cast<long long>(ld_step(bt + ap)) * nkv + kvh) * page_size;
                unsigned char* dst = tiles + st * TILE + lane * page_size * 128;
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(smem_u32(dst + h * kHalfBytes), &kv_map, h * 64,
                                static_cast<int>(row0 + prow), smem_u32(&full[st]));
            };
            if (mine && (waited || ap != newest_page)) copy();
            if (has_newest && !waited) {
                pdl_wait();
                waited = true;
                if (mine && ap == newest_page) copy();
            }
        }
        return;
    }

    // ---- computing warps
    pdl_wait();
    const __nv_bfloat16* qrow = qkv + static_cast<size_t>(row) * row_stride + static_cast<size_t>(kvh) * G * HD;
    for (int c = tid; c < kTdRows * CPR; c += kTdThreads) {
        const int r = c / CPR, ch = c - r * CPR;
        const bool ok = r < G;
        cp_async_16(smem_u32(Qs + swizzled_offset<HD>(r, ch)), ok ? qrow + r * HD + ch * 8 : qrow,
                    ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    ring_compute_sync();

    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const int kw = warp * 32;
    const int c0 = warp * (DW / 8);               // first 16-byte chunk of this warp's columns
    float o[DW / 8][4];
#pragma unroll
    for (int a = 0; a < DW / 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) o[a][b] = 0.f;
    float M_lo = -INFINITY, M_hi = -INFINITY;     // running maxima of the rows (all warps agree)
    float l_lo = 0.f, l_hi = 0.f;                 // this warp's 32 keys of every chunk so far
    bool ok_wait = true;
    for (int c = 0; c < n_chunks; ++c) {
        const unsigned char* Kt = Ks + (c % kRingK) * TILE;
        const unsigned char* Vt = Vs + (c % kRingV) * TILE;
        const int k0 = (c_begin + c) * kTdChunk;
        ok_wait = mbar_wait(smem_u32(&k_full[c % kRingK]), (c / kRingK) & 1) && ok_wait;
        // ---- S = Q K^T for this warp's 32 keys
        float s[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, smem_u32(Qs + swizzled_offset<HD>((lane & 7) + ((lane >> 3) & 1) * 8,
                                                            2 * ks + (lane >> 4))));
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, smem_u32(Kt + tma_tile_offset(kw + np * 16 + (lane & 7) + (lane >> 4) * 8,
                                                             2 * ks + ((lane >> 3) & 1))));
                mma_bf16_16816(s[2 * np], a, b[0], b[1]);
                mma_bf16_16816(s[2 * np + 1], a, b[2], b[3]);
            }
        }
        // ---- mask; the chunk's row maximum over all four warps
        float m_lo = -INFINITY, m_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = k0 + kw + nt * 8 + (lane & 3) * 2 + (e & 1);
                const bool ok = key < rg.kv_len && key >= rg.first_key;
                const float v = ok ? s[nt][e] * scale_log2e : -INFINITY;
                s[nt][e] = v;
                if (e < 2) m_lo = fmaxf(m_lo, v); else m_hi = fmaxf(m_hi, v);
            }
        m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 1));
        m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 2));
        m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 1));
        m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 2));
        if ((lane & 3) == 0) { m_s[warp][r_lo] = m_lo; m_s[warp][r_hi] = m_hi; }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&k_empty[c % kRingK]));      // this warp has read the keys
        ring_compute_sync();
        // every chunk a CTA takes has a visible key, so the new maxima of real rows are finite
        const float n_lo = fmaxf(M_lo, fmaxf(fmaxf(m_s[0][r_lo], m_s[1][r_lo]), fmaxf(m_s[2][r_lo], m_s[3][r_lo])));
        const float n_hi = fmaxf(M_hi, fmaxf(fmaxf(m_s[0][r_hi], m_s[1][r_hi]), fmaxf(m_s[2][r_hi], m_s[3][r_hi])));
        const float a_lo = M_lo == -INFINITY ? 0.f : fast_exp2(M_lo - n_lo);
        const float a_hi = M_hi == -INFINITY ? 0.f : fast_exp2(M_hi - n_hi);
        M_lo = n_lo;
        M_hi = n_hi;
        const float b_lo = n_lo == -INFINITY ? 0.f : n_lo, b_hi = n_hi == -INFINITY ? 0.f : n_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const uint32_t lo = pack_bf16(fast_exp2(s[nt][0] - b_lo), fast_exp2(s[nt][1] - b_lo));
            const uint32_t hi = pack_bf16(fast_exp2(s[nt][2] - b_hi), fast_exp2(s[nt][3] - b_hi));
            const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&lo);
            const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&hi);
            sum_lo += __low2float(lo2) + __high2float(lo2);
            sum_hi += __low2float(hi2) + __high2float(hi2);
            const int chunk = warp * 4 + nt;
            *reinterpret_cast<uint32_t*>(Ps + swizzled_offset<128>(r_lo, chunk) + (lane & 3) * 4) = lo;
            *reinterpret_cast<uint32_t*>(Ps + swizzled_offset<128>(r_hi, chunk) + (lane & 3) * 4) = hi;
        }
        l_lo = l_lo * a_lo + sum_lo;              // the four lanes of a row are added up at the end
        l_hi = l_hi * a_hi + sum_hi;
        ok_wait = mbar_wait(smem_u32(&v_full[c % kRingV]), (c / kRingV) & 1) && ok_wait;
        ring_compute_sync();   // P is in shared memory
        // ---- O[:, warp's DW columns] = a * O + P V over the chunk's 128 keys
#pragma unroll
        for (int nt = 0; nt < DW / 8; ++nt) {
            o[nt][0] *= a_lo;
            o[nt][1] *= a_lo;
            o[nt][2] *= a_hi;
            o[nt][3] *= a_hi;
        }
#pragma unroll
        for (int kk = 0; kk < kTdChunk / 16; ++kk) {
            uint32_t a[4];
            ldmatrix_x4(a, smem_u32(Ps + swizzled_offset<128>((lane & 7) + ((lane >> 3) & 1) * 8,
                                                             2 * kk + (lane >> 4))));
#pragma unroll
            for (int dc = 0; dc < DW / 16; ++dc) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, smem_u32(Vt + tma_tile_offset(
                                         kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                         c0 + 2 * dc + (lane >> 4))));
                mma_bf16_16816(o[2 * dc], a, b[0], b[1]);
                mma_bf16_16816(o[2 * dc + 1], a, b[2], b[3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&v_empty[c % kRingV]));      // and the values
    }
    if (!ok_wait && lane == 0) atomicExch(&g_decode_tma_error, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if ((lane & 3) == 0) { l_s[warp][r_lo] = l_lo; l_s[warp][r_hi] = l_hi; }
    ring_compute_sync();
    const float L_lo = l_s[0][r_lo] + l_s[1][r_lo] + l_s[2][r_lo] + l_s[3][r_lo];
    const float L_hi = l_s[0][r_hi] + l_s[1][r_hi] + l_s[2][r_hi] + l_s[3][r_hi];
    const bool single = rg.first_split / cpc == (rg.n_splits - 1) / cpc;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int g = half ? r_hi : r_lo;
        if (g >= G) continue;
        const int head = kvh * G + g;
        const float L = half ? L_hi : L_lo, M = half ? M_hi : M_lo;
        if (single) {
            const float inv = 1.0f / L;
            __nv_bfloat16* dst = out + static_cast<size_t>(row) * nq * HD + head * HD + warp * DW;
#pragma unroll
            for (int nt = 0; nt < DW / 8; ++nt)
                *reinterpret_cast<uint32_t*>(dst + nt * 8 + (lane & 3) * 2) =
                    pack_bf16(o[nt][half * 2] * inv, o[nt][half * 2 + 1] * inv);
        } else {
            const size_t p = (static_cast<size_t>(i) * nq + head) * max_splits + group;
            float* dst = part_o + p * HD + warp * DW;
#pragma unroll
            for (int nt = 0; nt < DW / 8; ++nt)
                *reinterpret_cast<float2*>(dst + nt * 8 + (lane & 3) * 2) =
                    make_float2(o[nt][half * 2], o[nt][half * 2 + 1]);
            if (warp == 0 && (lane & 3) == 0) { part_ml[2 * p] = M; part_ml[2 * p + 1] = L; }
        }
    }
}
template <int HD>
int launch_tma_decode(const CUtensorMap* map, const void* qkv, int row_stride, int row_base,
                      int req_base, int n_decode, long long k_row0, long long v_row0,
                      const int* block_table, int bt_stride, const int* ctx_len, int nq, int nkv,
                      int page_size, float scale, int window, float* part_o, float* part_ml,
                      int max_splits, void* out, cudaStream_t stream) {
    constexpr int TILE = (HD / 64) * kHalfBytes;
    const size_t smem = 2 * TILE + kTdRows * HD * 2 + kTdRows * kTdChunk * 2 + 1024;
    cudaFuncSetAttribute(paged_decode_tma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
    // Many chunks per SM: CTAs that walk through several chunks each (see the ring kernel).
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            sm_count <= 0)
            sm_count = 148;
    }
    const long long units = static_cast<long long>(max_splits) * nkv * n_decode;
    const int cpc = g_ring_chunks > 0
                        ? std::min(g_ring_chunks, kRingMaxCpc)
                        : static_cast<int>(std::min<long long>(kRingMaxCpc, units / (8LL * sm_count)));
    if (cpc >= 2) {
        const size_t ring_smem = (kRingK + kRingV) * TILE + kTdRows * HD * 2 + kTdRows * kTdChunk * 2 + 1024;
        cudaFuncSetAttribute(paged_decode_ring_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)ring_smem);
        const int groups = (max_splits + cpc - 1) / cpc;
        launch_pdl(paged_decode_ring_kernel<HD>, dim3(groups, nkv, n_decode), dim3(kRingThreads),
                   ring_smem, stream, *map, static_cast<const __nv_bfloat16*>(qkv), row_stride,
                   row_base, req_base, k_row0, v_row0, block_table, bt_stride, ctx_len, nq, nkv,
                   page_size, scale * 1.4426950408889634f, window, part_o, part_ml, max_splits, cpc,
                   static_cast<__nv_bfloat16*>(out));
        int rc = launch_status();
        if (rc != 0 || groups == 1) return rc;
        return launch_decode_merge<HD>(part_o, part_ml, max_splits, kTdChunk * cpc, ctx_len, row_base,
                                       req_base, n_decode, nq, window,
                                       static_cast<__nv_bfloat16*>(out), stream);
    }
    dim3 grid(max_splits, nkv, n_decode);
    launch_pdl(paged_decode_tma_kernel<HD>, dim3(grid), dim3(kTdThreads), smem, stream, 
        *map, static_cast<const __nv_bfloat16*>(qkv), row_stride, row_base, req_base, k_row0,
        v_row0, block_table, bt_stride, ctx_len, nq, nkv, page_size,
        scale * 1.4426950408889634f, window, part_o, part_ml, max_splits,
        static_cast<__nv_bfloat16*>(out));
    int rc = launch_status();
    if (rc != 0 || max_splits == 1) return rc;
    return launch_decode_merge<HD>(part_o, part_ml, max_splits, kTdChunk, ctx_len, row_base, req_base,
                                   n_decode, nq, window, static_cast<__nv_bfloat16*>(out), stream);
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_decode_tma_supported(int nq, int nkv, int hd, int page_size) {
    if (nkv <= 0 || nq % nkv || nq / nkv > kTdRows) return 0;
    if (hd != 64 && hd != 128) return 0;
    return page_size >= 8 && page_size % 8 == 0 && kTdChunk % page_size == 0;
}

// Chunks per CTA of the decode kernel: 1 = always the one-chunk kernel, 2..8 = always the ring
// kernel with that many, 0 = chosen from the number of chunks in the step (the default).
SOMI_API void somi_decode_ring_chunks(int chunks) { g_ring_chunks = chunks < 0 ? 0 : chunks; }

// Fills `map_out` (128 bytes, 64-byte aligned) for a cache storage of `rows` x `hd` bfloat16.
SOMI_API int somi_make_kv_tensor_map(void* map_out, const void* storage, long long rows, int hd,
                                     int page_size) {
    return make_tensor_map_bf16_2d(static_cast<CUtensorMap*>(map_out), storage,
                                   static_cast<uint64_t>(rows), static_cast<uint64_t>(hd),
                                   static_cast<uint32_t>(page_size), 64, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Reads and clears the error word of the TMA decode kernel (synchronises the device).
SOMI_API int somi_decode_tma_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_decode_tma_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_decode_tma_error, &zero, sizeof(int));
    return v;
}

// k_row0 / v_row0: first row, in the tensor map, of this run's key and value planes.
SOMI_API int somi_paged_attention_decode_tma(
    const void* tensor_map, const void* qkv, int row_stride, int row_base, int req_base,
    int n_decode, long long k_row0, long long v_row0, const int* block_table, int bt_stride,
    const int* ctx_len, int nq, int nkv, int hd, int page_size, float scale, int window,
    float* part_o, float* part_ml, int max_splits, void* out, cudaStream_t stream) {
    if (n_decode <= 0) return 0;
    if (!somi_decode_tma_supported(nq, nkv, hd, page_size) || max_splits <= 0 ||
        n_decode > 65535 || nkv > 65535)
        return SOMI_ERR_UNSUPPORTED;
    const CUtensorMap* map = static_cast<const CUtensorMap*>(tensor_map);
    if (hd == 64)
        return launch_tma_decode<64>(map, qkv, row_stride, row_base, req_base, n_decode, k_row0,
                                     v_row0, block_table, bt_stride, ctx_len, nq, nkv, page_size,
                                     scale, window, part_o, part_ml, max_splits, out, stream);
    return launch_tma_decode<128>(map, qkv, row_stride, row_base, req_base, n_decode, k_row0,
                                  v_row0, block_table, bt_stride, ctx_len, nq, nkv, page_size,
                                  scale, window, part_o, part_ml, max_splits, out, stream);
}
