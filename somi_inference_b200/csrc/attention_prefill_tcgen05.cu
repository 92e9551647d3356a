// Prompt-portion attention over the paged cache on the 5th-generation tensor cores.
//
// One CTA = up to 128 consecutive query rows of one request x one query head; key tiles of 128
// positions aligned to multiples of 128.  Both products run as `tcgen05.mma` with accumulators
// in tensor memory: S = Q K^T (128 x 128, two buffers, issued two tiles ahead of the softmax)
// and O += P V (128 x head_dim).  Operands come from shared memory in the 128-byte-swizzle
// layout: Q and the K/V pages by `cp.async.bulk.tensor.2d` (V is the MN-major operand of the
// second product, so the cache's [key][dim] rows are used as they are), P written by the
// softmax warps.  Keys and values have rings of their own: a key tile is free again as soon as
// its scores are computed, a value tile only after the second product, so the keys can be
// fetched two tiles ahead with two stages.  Warp roles: warp 0 key producer (TMA), warp 1 MMA
// issuer, warps 2-9 softmax, warp 10 value producer.  A query row is one lane of tensor memory
// and is served by two threads, one per 64 of a tile's 128 keys; each half keeps its own
// maximum and sum and has its own output accumulator in tensor memory (O_lo += P_lo V_lo,
// O_hi += P_hi V_hi), and the two are added at the end like the parts of a split over the keys,
// so the halves exchange nothing per tile.  An accumulator is rescaled in tensor memory
// (tcgen05.ld / tcgen05.st) only when its row maximum grows by more than 2^8, otherwise the old
// maximum keeps serving as the reference (probabilities up to 256 are harmless in float32 sums
// and bfloat16 operands), so most tiles cost the softmax warps one pass over S and one over P.
// A tile's fixed costs (barrier tests, tensor-memory load latency, the proxy fence) are paid
// once per 128 keys: with 64-key tiles the same kernel took 1.5 times as long.  Softmax is
// float32, base 2.  Every wait on an mbarrier is bounded and failure is recorded in an error
// word.
//
// The reference's prefill kernel (somi_inference/core/flash_attention_triton.py:31-194) is a
// FlashAttention-2 loop on `tl.dot`; formulas in somi_inference/models/qwen2.py:158-186.
#include "mma.cuh"
#include "tma.cuh"

namespace somi {

constexpr int kFaBM = 128;               // query rows per CTA
constexpr int kFaBN = 128;               // keys per tile
// Key and value tiles in flight, as many as shared memory holds beside Q and the two P buffers.
constexpr int kFaMaxStages = 4;
__host__ __device__ constexpr int fa_stages(int hd) { return hd == 128 ? 2 : 4; }
constexpr int kFaThreads = 352;          // K producer warp, MMA warp, 8 softmax warps, V producer warp
constexpr int kFaHalf = kFaBM * 128;     // bytes of one [128 rows][64 elements] swizzled block (Q, P)
constexpr int kFaKvHalf = kFaBN * 128;   // bytes of one [128 keys][64 elements] block (K, V)

__device__ int g_prefill_tc_error = 0;

__device__ __forceinline__ uint64_t fa_desc_kmajor(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// MN-major operand: 64 elements (128 bytes) contiguous along N, 8 K-rows form a 1024-byte
// group; the leading byte offset steps to the next 64-element block along N, the stride byte
// offset to the next group of 8 rows along K.
__device__ __forceinline__ uint64_t fa_desc_mnmajor(uint32_t addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__device__ __forceinline__ void fa_umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void fa_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fa_tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}
// The same without waiting: several loads may be in flight before one fa_tmem_wait_ld().
__device__ __forceinline__ void fa_tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void fa_tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void fa_pair_sync(int id) {          // the two warps that share rows
    asm volatile("bar.sync %0, 64;\n" ::"r"(id) : "memory");
}
__device__ __forceinline__ void fa_tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]),
        "f"(v[8]), "f"(v[9]), "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]),
        "f"(v[16]), "f"(v[17]), "f"(v[18]), "f"(v[19]), "f"(v[20]), "f"(v[21]), "f"(v[22]),
        "f"(v[23]), "f"(v[24]), "f"(v[25]), "f"(v[26]), "f"(v[27]), "f"(v[28]), "f"(v[29]),
        "f"(v[30]), "f"(v[31])
        : "memory");
}
__device__ __forceinline__ void fa_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void fa_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}

template <int HD>
__global__ void __launch_bounds__(kFaThreads, 1)
paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map,
                        const __grid_constant__ CUtensorMap kv_map, long long k_row0,
                        long long v_row0, const int* __restrict__ block_table, int bt_stride,
                        const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                        const int* __restrict__ tiles, int nq, int nkv, int page_size,
                        float scale_log2e, int window, __nv_bfloat16* __restrict__ out,
                        int n_q_tiles) {
    constexpr int HALVES = HD / 64;
    constexpr int QTILE = HALVES * kFaHalf;              // bytes of the Q tile
    constexpr int TILE = HALVES * kFaKvHalf;             // bytes of a K or V tile
    constexpr uint32_t TmemCols = 512;                   // S0 | S1 (128 each) | PV (up to 128)
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* Qs = base;
    constexpr int STAGES = fa_stages(HD);
    unsigned char* Ks = Qs + QTILE;                      // STAGES tiles
    unsigned char* Vs = Ks + STAGES * TILE;           // STAGES tiles
    unsigned char* Ps = Vs + STAGES * TILE;           // two buffers of two [128 rows][64 keys] blocks
    __shared__ __align__(8) unsigned long long q_full, k_full[kFaMaxStages], k_empty[kFaMaxStages],
        v_full[kFaMaxStages], v_empty[kFaMaxStages], s_full[2], p_full[2][2], pv_full[2][2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed_s;

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(smem_u32(&q_full), 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            for (int h = 0; h < 2; ++h) {
                mbar_init(smem_u32(&p_full[h][s]), 4);   // one arrival per softmax warp of the half
                mbar_init(smem_u32(&pv_full[h][s]), 1);
            }
        }
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
    // value rows that no copy fills (pages outside the request's range) must be finite numbers
    for (int c = tid; c < STAGES * TILE / 16; c += kFaThreads)
        reinterpret_cast<uint4*>(Vs)[c] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
    fa_fence_before();
    __syncthreads();
    fa_fence_after();
    pdl_wait();
    const uint32_t tmem_s = tmem_base_s;                 // S buffers at columns 0 and 128
    const uint32_t tmem_pv = tmem_base_s + 2 * kFaBN;    // O of key half 0, then O of key half 1

    // Later tiles of a prompt see more keys.  Blocks are handed out longest first (heads
    // first, last tile first), so that the short ones fill the end.
    const int rank = blockIdx.x;
    const int tile = n_q_tiles - 1 - rank / nq;
    const int req = tiles[3 * tile], row0 = tiles[3 * tile + 1];
    const int rows = tiles[3 * tile + 2];
    const int head = rank % nq, kvh = head / (nq / nkv);
    const int q_pos0 = ctx_len[req] + (row0 - cu_q[req]);
    const int kv_end = q_pos0 + rows;
    const int kv_first = window > 0 ? max(0, q_pos0 - window + 1) : 0;
    const int kb0 = (kv_first / kFaBN) * kFaBN;
    const int n_tiles = (kv_end - kb0 + kFaBN - 1) / kFaBN;
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;

    if (warp == 0 || warp == 10) {
        // producer warps, one for the keys (and Q) and one for the values: a copy of a 16-token
        // page is a small box, and what bounds a warp is the number of copies it issues.
        // Lane 0 keeps the barriers, one lane per page looks its page up and issues that
        // page's copies, so the page-table reads of a tile run side by side.
        if (warp == 0 && lane == 0) {
            mbar_expect_tx(smem_u32(&q_full), kFaBM * HD * 2);
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
                tma_load_2d(smem_u32(Qs + h * kFaHalf), &q_map, head * HD + h * 64, row0,
                            smem_u32(&q_full));
        }
        const int pages_per_tile = kFaBN / page_size;
        // one tile's keys (which = 0) or values (which = 1) into stage t % STAGES of their ring
        auto load_tile = [&](int t, int which) -> bool {
            const int st = t % STAGES;
            const int kb = kb0 + t * kFaBN;
            const int p_lo = max(kb, kv_first) / page_size;
            const int p_hi = (min(kb + kFaBN, kv_end) - 1) / page_size;
            // the table entries do not depend on the stage being free: read them first
            int my_page = -1;
            const int ap = kb / page_size + lane;
            if (lane < pages_per_tile && ap >= p_lo && ap <= p_hi) my_page = bt[ap];
            const uint32_t bar = smem_u32(which ? &v_full[st] : &k_full[st]);
            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait(smem_u32(which ? &v_empty[st] : &k_empty[st]), ((t / STAGES) & 1) ^ 1) ? 1 : 0;
                if (ok) mbar_expect_tx(bar, static_cast<uint32_t>(p_hi - p_lo + 1) * page_size * HD * 2);
                else failed_s = 1;
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) return false;
            if (my_page >= 0) {
                const long long prow = (static_cast<long long>(my_page) * nkv + kvh) * page_size;
                const int r = lane * page_size;
                unsigned char* dst = (which ? Vs : Ks) + st * TILE + r * 128;
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(smem_u32(dst + h * kFaKvHalf), &kv_map, h * 64,
                                static_cast<int>((which ? v_row0 : k_row0) + prow), bar);
            }
            return true;
        };
        const int which = warp == 0 ? 0 : 1;
        for (int t = 0; t < n_tiles; ++t)
            if (!load_tile(t, which)) break;
    } else if (warp == 1) {
        if (lane == 0) {
            // float32 accumulators, bf16 operands; scores: both K-major, N = 128 keys;
            // P.V: A (P) K-major, B (V) MN-major, N = head_dim
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) |
                                      (static_cast<uint32_t>(kFaBN >> 3) << 17) |
                                      (static_cast<uint32_t>(kFaBM >> 4) << 24);
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      (static_cast<uint32_t>(HD >> 3) << 17) |
                                      (static_cast<uint32_t>(kFaBM >> 4) << 24);
            bool ok = mbar_wait(smem_u32(&q_full), 0);
            // descriptors differ only in their start address field (units of 16 bytes), so they
            // are built once and advanced by additions while MMAs are issued
            const uint64_t q_desc = fa_desc_kmajor(smem_u32(Qs));
            const uint64_t k_desc = fa_desc_kmajor(smem_u32(Ks));
            const uint64_t p_desc = fa_desc_kmajor(smem_u32(Ps));
            const uint64_t v_desc = fa_desc_mnmajor(smem_u32(Vs), kFaKvHalf);
            auto issue_scores = [&](int t) {
                const int st = t % STAGES;
                if (!mbar_wait(smem_u32(&k_full[st]), (t / STAGES) & 1)) { ok = false; return; }
                fa_fence_after();
                const uint64_t kd = k_desc + ((st * TILE) >> 4);
#pragma unroll
                for (int k16 = 0; k16 < HD / 16; ++k16)
                    fa_umma(tmem_s + (t & 1) * kFaBN,
                            q_desc + (((k16 >> 2) * kFaHalf + (k16 & 3) * 32) >> 4),
                            kd + (((k16 >> 2) * kFaKvHalf + (k16 & 3) * 32) >> 4),
                            idesc_qk, k16 > 0 ? 1u : 0u);
                fa_commit(smem_u32(&s_full[t & 1]));
                fa_commit(smem_u32(&k_empty[st]));             // the key tile is free once these ran
            };
            // scores run two tiles ahead of the softmax: S(t + 2) is issued as soon as the
            // softmax warps have read S(t), so they never wait for the tensor core
            if (ok) issue_scores(0);
            if (ok && n_tiles > 1) issue_scores(1);
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int st = t % STAGES;
                if (!mbar_wait(smem_u32(&v_full[st]), (t / STAGES) & 1)) { ok = false; break; }
                // each half of the tile's keys has its own probabilities, its own output
                // accumulator and its own pace
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (!mbar_wait(smem_u32(&p_full[h][t & 1]), (t >> 1) & 1)) { ok = false; break; }
                    fa_fence_after();
                    const uint64_t pd = p_desc + (((t & 1) * 2 * kFaHalf + h * kFaHalf) >> 4);
                    const uint64_t vd = v_desc + ((st * TILE + h * 64 * 128) >> 4);
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)
                        fa_umma(tmem_pv + h * HD, pd + ((k16 * 32) >> 4), vd + ((k16 * 16 * 128) >> 4),
                                idesc_pv, (t > 0 || k16 > 0) ? 1u : 0u);   // accumulates over the tiles
                    fa_commit(smem_u32(&pv_full[h][t & 1]));
                }
                if (!ok) break;
                fa_commit(smem_u32(&v_empty[st]));
                if (t + 2 < n_tiles) issue_scores(t + 2);      // S buffer t & 1 has been read
            }
            if (!ok) {
                failed_s = 1;
                // let the softmax warps run out of their bounded waits instead of hanging
            }
        }
    } else if (warp < 10) {
        // ---- softmax warps: a query row (one lane of tensor memory) is served by two threads, one
        // per half of the tile's 128 keys.  The halves are independent: each keeps its own
        // maximum and sum and feeds its own output accumulator, and the two results are added
        // at the end like the partial results of a split over the keys.  So the halves do not
        // meet in every tile.  (Starting them half a tile apart, so that one half's exp2 phase
        // would run beside the other's loads, changed nothing: both wait for the same scores,
        // which are issued when the later half is done with a tile.)
        const int q = warp & 3;                                  // lane quarter this warp may access
        const int half = (warp - 2) >> 2;                        // which 64 keys of a tile
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const int pos = q_pos0 + row;
        const int lo = window > 0 ? max(kv_first, pos - window + 1) : kv_first;
        // the highest first visible key among the block's rows, and this row's visible span
        const int lo_max = window > 0 ? max(kv_first, q_pos0 + kFaBM - 1 - window + 1) : kv_first;
        const unsigned span = static_cast<unsigned>(pos - lo);
        float m = -INFINITY, l = 0.f;        // m: the reference maximum in use (log2 units)
        bool ok = true;
        const uint32_t tmem_o = tmem_pv + half * HD;         // this half's output accumulator
        for (int t = 0; t < n_tiles; ++t) {
            ok = mbar_wait(smem_u32(&s_full[t & 1]), (t >> 1) & 1, ok ? 400000 : 1) && ok;
            fa_fence_after();
            uint32_t ra[32], rb[32];
            const uint32_t s_addr = tmem_s + (t & 1) * kFaBN + half * 64 + lane_addr;
            fa_tmem_ld32_nowait(s_addr, ra);
            fa_tmem_ld32_nowait(s_addr + 32, rb);
            fa_tmem_wait_ld();
            const int kb = kb0 + t * kFaBN + half * 64;
            float sv[64];
            // a tile in which no row of this block has a hidden key takes the short way
            const bool tile_inner = kb0 + t * kFaBN + kFaBN - 1 <= q_pos0 && kb0 + t * kFaBN >= lo_max;
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains, not one
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                float x = __uint_as_float(j < 32 ? ra[j] : rb[j - 32]);
                if (!tile_inner) {
                    // key in [lo, pos] as one unsigned comparison
                    const unsigned d = static_cast<unsigned>(kb + j - lo);
                    x = d <= span ? x : -INFINITY;
                }
                sv[j] = x;
                mx[j & 3] = fmaxf(mx[j & 3], x);
            }
            // the scale is positive, so the maximum is taken over the raw scores and scaled once
            const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2e;
            // This tile's P buffer was last read by the products of tile t - 2.  They were
            // issued before the scores of tile t, and a commit covers everything issued before
            // it, so the wait for S(t) has covered them already.
            // keep the old reference maximum unless the new one is more than 2^8 above it
            float alpha = 1.f;
            bool rescale = false;
            if (m == -INFINITY) {
                m = tmax;                                   // nothing accumulated yet for this row
            } else if (tmax > m + 8.0f) {
                alpha = fast_exp2(m - tmax);
                m = tmax;
                rescale = true;
            }
            if (__any_sync(0xffffffffu, rescale)) {
                // this half's O of the tiles so far must be complete before it is rescaled in
                // tensor memory
                if (t >= 1) ok = mbar_wait(smem_u32(&pv_full[half][(t - 1) & 1]), ((t - 1) >> 1) & 1, ok ? 400000 : 1) && ok;
                fa_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    float v[32];
                    const uint32_t a = tmem_o + lane_addr + c * 32;
                    fa_tmem_ld32(a, v);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] *= alpha;
                    fa_tmem_st32(a, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                l *= alpha;
            }
            const float neg_m = m == -INFINITY ? 0.f : -m;
            float ps[2] = {0.f, 0.f};
            // this thread's 64 keys are one 128-byte line of its [128 rows][64 keys] block
            unsigned char* prow = Ps + (t & 1) * 2 * kFaHalf + half * kFaHalf + row * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                uint32_t pk[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p0 = fast_exp2(fmaf(sv[ch * 8 + 2 * j], scale_log2e, neg_m));
                    const float p1 = fast_exp2(fmaf(sv[ch * 8 + 2 * j + 1], scale_log2e, neg_m));
                    ps[0] += p0;
                    ps[1] += p1;
                    pk[j] = pack_bf16(p0, p1);
                }
                *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) =
                    make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
            l += ps[0] + ps[1];
            fa_fence_before();
            fence_proxy_async();                // P is read by the tensor core (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[half][t & 1]));
        }
        // ---- the output: the two halves' results added up; each thread writes half of its row
        const int last = n_tiles - 1;
        ok = mbar_wait(smem_u32(&pv_full[half][last & 1]), (last >> 1) & 1, ok ? 400000 : 1) && ok;
        // (maximum, sum) of the two halves meet in the Q tile's place: every product that reads Q
        // was issued, and has completed, before the last product of either half
        float2* ml_s = reinterpret_cast<float2*>(Qs);
        ml_s[half * kFaBM + row] = make_float2(m, l);
        // the partner's accumulator is complete, and its maximum and sum are in shared memory
        fa_fence_before();
        fa_pair_sync(1 + q);
        fa_fence_after();
        if (!ok) failed_s = 1;
        const float2 other = ml_s[(half ^ 1) * kFaBM + row];
        const float m_o = other.x, l_o = other.y;
        // a half in which the row saw no key has maximum -inf and sum 0
        const float mm = fmaxf(m, m_o);
        const float w_me = m == -INFINITY ? 0.f : fast_exp2(m - mm);
        const float w_ot = m_o == -INFINITY ? 0.f : fast_exp2(m_o - mm);
        const float inv = 1.0f / (w_me * l + w_ot * l_o);
        const float a_me = w_me * inv, a_ot = w_ot * inv;
        __nv_bfloat16* dst = out + static_cast<size_t>(row0 + row) * nq * HD + head * HD + half * (HD / 2);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
            float v[32], u[32];
            fa_tmem_ld32(tmem_o + lane_addr + half * (HD / 2) + c * 32, v);
            fa_tmem_ld32(tmem_pv + (half ^ 1) * HD + lane_addr + half * (HD / 2) + c * 32, u);
            if (row < rows) {
#pragma unroll
                for (int d = 0; d < 32; d += 8) {
                    uint4 w;
                    w.x = pack_bf16(v[d] * a_me + u[d] * a_ot, v[d + 1] * a_me + u[d + 1] * a_ot);
                    w.y = pack_bf16(v[d + 2] * a_me + u[d + 2] * a_ot, v[d + 3] * a_me + u[d + 3] * a_ot);
                    w.z = pack_bf16(v[d + 4] * a_me + u[d + 4] * a_ot, v[d + 5] * a_me + u[d + 5] * a_ot);
                    w.w = pack_bf16(v[d + 6] * a_me + u[d + 6] * a_ot, v[d + 7] * a_me + u[d + 7] * a_ot);
                    *reinterpret_cast<uint4*>(dst + c * 32 + d) = w;
                }
            }
        }
    }
    fa_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base_s),
                     "r"(TmemCols)
                     : "memory");
    }
    if (tid == 0 && failed_s) atomicExch(&g_prefill_tc_error, 1);
}

template <int HD>
int launch_prefill_tc(const CUtensorMap* q_map, const CUtensorMap* kv_map, long long k_row0,
                      long long v_row0, const int* block_table, int bt_stride, const int* cu_q,
                      const int* ctx_len, const int* tiles, int n_tiles, int nq, int nkv,
                      int page_size, float scale, int window, void* out, cudaStream_t stream) {
    const size_t smem = (HD / 64) * kFaHalf + 2 * fa_stages(HD) * (HD / 64) * kFaKvHalf + 4 * kFaHalf + 1024;
    cudaFuncSetAttribute(paged_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
    dim3 grid(static_cast<unsigned>(nq) * n_tiles);
    launch_pdl(paged_prefill_tc_kernel<HD>, grid, dim3(kFaThreads), smem, stream, *q_map, *kv_map,
               k_row0, v_row0, block_table, bt_stride, cu_q, ctx_len, tiles, nq, nkv, page_size,
               scale * 1.4426950408889634f, window, static_cast<__nv_bfloat16*>(out), n_tiles);
    return launch_status();
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_prefill_tc_q_tile() { return kFaBM; }

SOMI_API int somi_prefill_tc_supported(int nq, int nkv, int hd, int page_size) {
    if (nkv <= 0 || nq % nkv) return 0;
    if (hd != 64 && hd != 128) return 0;
    return page_size >= 8 && page_size % 8 == 0 && kFaBN % page_size == 0;
}

SOMI_API int somi_prefill_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_prefill_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_prefill_tc_error, &zero, sizeof(int));
    return v;
}

// A tensor map over the step's projection buffer [tokens, width] (bfloat16, row-major) with
// boxes of 128 rows x 64 columns, from which the query tiles are fetched.
SOMI_API int somi_make_q_tensor_map(void* map_out, const void* qkv, long long tokens,
                                    long long width) {
    if (width % 8 != 0) return SOMI_ERR_UNSUPPORTED;
    return make_tensor_map_bf16_2d(static_cast<CUtensorMap*>(map_out), qkv,
                                   static_cast<uint64_t>(tokens), static_cast<uint64_t>(width),
                                   kFaBM, 64, CU_TENSOR_MAP_SWIZZLE_128B);
}

// `tiles`: int32 [n_tiles, 3] = (request, first row, rows <= 128) over the multi-token requests.
SOMI_API int somi_paged_attention_prefill_tc(
    const void* q_map, const void* kv_map, long long k_row0, long long v_row0,
    const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len, const int* tiles,
    int n_tiles, int nq, int nkv, int hd, int page_size, float scale, int window, void* out,
    cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!somi_prefill_tc_supported(nq, nkv, hd, page_size) ) return SOMI_ERR_UNSUPPORTED;
    const CUtensorMap* qm = static_cast<const CUtensorMap*>(q_map);
    const CUtensorMap* km = static_cast<const CUtensorMap*>(kv_map);
    if (hd == 64)
        return launch_prefill_tc<64>(qm, km, k_row0, v_row0, block_table, bt_stride, cu_q, ctx_len,
                                     tiles, n_tiles, nq, nkv, page_size, scale, window, out, stream);
    return launch_prefill_tc<128>(qm, km, k_row0, v_row0, block_table, bt_stride, cu_q, ctx_len, tiles,
                                  n_tiles, nq, nkv, page_size, scale, window, out, stream);
}
