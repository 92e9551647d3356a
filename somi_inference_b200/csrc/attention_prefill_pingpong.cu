// Prompt-portion attention over the paged cache on the 5th-generation tensor cores, two query
// tiles per CTA in ping-pong.
//
// One CTA = up to 256 consecutive query rows of one request x one query head, as two tiles A and
// B of 128 rows; key tiles of 128 positions aligned to multiples of 128, fetched once for both
// query tiles.  Tensor memory holds S_A, S_B (128 columns each) and O_A, O_B (head_dim columns
// each).  A softmax warp group of 128 threads serves each query tile, one thread per row (one
// lane of tensor memory): it reads its row of S, writes the probabilities back over the same
// columns as packed bfloat16 pairs, and the second product takes them from there as its A
// operand (`tcgen05.mma` with A in tensor memory), so P never passes through shared memory.
// One thread issues the products in the order
//     S_A(0) S_B(0) | PV_A(t) S_A(t+1) PV_B(t) S_B(t+1) | ...
// so that while warp group A works on tile t's scores the tensor core runs B's products of
// tile t-1 and B's scores of tile t, and the other way round.  The pipe executes in issue order,
// which is what makes the aliasing of P over S safe: S_X(t+1) is issued after PV_X(t).
// An accumulator is rescaled in tensor memory only when its row maximum grows by more than 2^8
// (probabilities up to 256 are harmless in float32 sums and bfloat16 operands).  Because tile B's
// rows come later in the sequence, tile A runs out of key tiles first and writes its output
// while B goes on.  Softmax is float32, base 2.  Every wait on an mbarrier is bounded and failure
// is recorded in an error word.
//
// Warp roles: warps 0-3 softmax of tile A, 4-7 softmax of tile B, warp 8 key (and Q) producer,
// warp 9 MMA issuer and owner of tensor memory, warp 10 value producer, warp 11 idle.
//
// The reference's prefill kernel (somi_inference/core/flash_attention_triton.py:31-194) is a
// FlashAttention-2 loop on `tl.dot`; formulas in somi_inference/models/qwen2.py:158-186.
#include "tcgen05.cuh"

namespace somi {

constexpr int kPpBM = 128;               // rows of one query tile
constexpr int kPpRows = 2 * kPpBM;       // rows of a CTA
constexpr int kPpBN = 128;               // keys per tile
constexpr int kPpThreads = 384;
constexpr int kPpMaxStages = 4;
__host__ __device__ constexpr int pp_stages(int hd) { return hd == 128 ? 2 : 4; }
constexpr int kPpQHalf = kPpBM * 128;    // bytes of one [128 rows][64 elements] swizzled block
constexpr int kPpKvHalf = kPpBN * 128;

__device__ int g_prefill_pp_error = 0;

template <int HD>
__global__ void __launch_bounds__(kPpThreads, 1)
paged_prefill_pp_kernel(const __grid_constant__ CUtensorMap q_map,
                        const __grid_constant__ CUtensorMap kv_map, long long k_row0,
                        long long v_row0, const int* __restrict__ block_table, int bt_stride,
                        const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                        const int* __restrict__ tiles, int nq, int nkv, int page_size,
                        float scale_log2e, int window, __nv_bfloat16* __restrict__ out,
                        int n_q_tiles) {
    constexpr int HALVES = HD / 64;
    constexpr int QTILE = HALVES * kPpQHalf;
    constexpr int TILE = HALVES * kPpKvHalf;
    constexpr int STAGES = pp_stages(HD);
    constexpr uint32_t TmemCols = 512;                   // S_A | S_B | O_A | O_B, 128 columns each
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* Qs = base;                            // two query tiles
    unsigned char* Ks = Qs + 2 * QTILE;                  // STAGES tiles
    unsigned char* Vs = Ks + STAGES * TILE;              // STAGES tiles
    __shared__ __align__(8) unsigned long long q_full[2], k_full[kPpMaxStages], k_empty[kPpMaxStages],
        v_full[kPpMaxStages], v_empty[kPpMaxStages], s_full[2], p_full[2], o_done[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed_s;

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int x = 0; x < 2; ++x) {
            mbar_init(smem_u32(&q_full[x]), 1);
            mbar_init(smem_u32(&s_full[x]), 1);
            mbar_init(smem_u32(&p_full[x]), 4);          // one arrival per warp of the group
            mbar_init(smem_u32(&o_done[x]), 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        mbar_fence_init();
        failed_s = 0;
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(&tmem_base_s)),
                     "r"(TmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    // value rows that no copy fills (pages outside the request's range) must be finite numbers
    for (int c = tid; c < STAGES * TILE / 16; c += kPpThreads)
        reinterpret_cast<uint4*>(Vs)[c] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
    t5::fence_before();
    __syncthreads();
    t5::fence_after();
    pdl_wait();
    const uint32_t tmem_s = tmem_base_s;                 // S_A at column 0, S_B at 128
    const uint32_t tmem_o = tmem_base_s + 2 * kPpBN;     // O_A at 256, O_B at 384

    // Later tiles of a prompt see more keys.  Blocks are handed out longest first (heads
    // first, last tile first), so that the short ones fill the end.
    const int rank = blockIdx.x;
    const int tile = n_q_tiles - 1 - rank / nq;
    const int req = tiles[3 * tile], row0 = tiles[3 * tile + 1];
    const int rows = tiles[3 * tile + 2];
    const int head = rank % nq, kvh = head / (nq / nkv);
    const bool has_b = rows > kPpBM;
    const int q_pos0 = ctx_len[req] + (row0 - cu_q[req]);
    const int kv_first = window > 0 ? max(0, q_pos0 - window + 1) : 0;
    const int kb0 = (kv_first / kPpBN) * kPpBN;
    const int end_a = q_pos0 + min(rows, kPpBM), end_all = q_pos0 + rows;
    const int n_a = (end_a - kb0 + kPpBN - 1) / kPpBN;            // key tiles that tile A reads
    const int n_t = (end_all - kb0 + kPpBN - 1) / kPpBN;          // key tiles of the CTA
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;

    // The softmax threads hold a row of 128 scores in registers; the producer and issuing warps
    // need few.  Warps 8-11 give registers back and the softmax warp groups take them.
    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
      if (warp == 8 || warp == 10) {
        // ---- producer warps, one for the keys (and Q) and one for the values.  Lane 0 keeps the
        // barriers, one lane per page looks its page up and issues that page's copies.
        if (warp == 8 && lane == 0) {
            for (int x = 0; x < (has_b ? 2 : 1); ++x) {
                mbar_expect_tx(smem_u32(&q_full[x]), kPpBM * HD * 2);
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(smem_u32(Qs + x * QTILE + h * kPpQHalf), &q_map, head * HD + h * 64,
                                row0 + x * kPpBM, smem_u32(&q_full[x]));
            }
        }
        const int pages_per_tile = kPpBN / page_size;
        const int which = warp == 8 ? 0 : 1;
        for (int t = 0; t < n_t; ++t) {
            const int st = t % STAGES;
            const int kb = kb0 + t * kPpBN;
            const int p_lo = max(kb, kv_first) / page_size;
            const int p_hi = (min(kb + kPpBN, end_all) - 1) / page_size;
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
            if (!ok) break;
            if (my_page >= 0) {
                const long long prow = (static_cast<long long>(my_page) * nkv + kvh) * page_size;
                unsigned char* dst = (which ? Vs : Ks) + st * TILE + lane * page_size * 128;
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(smem_u32(dst + h * kPpKvHalf), &kv_map, h * 64,
                                static_cast<int>((which ? v_row0 : k_row0) + prow), bar);
            }
        }
      } else if (warp == 9) {
        if (lane == 0) {
            // float32 accumulators, bf16 operands.  Scores: A and B K-major, N = 128 keys.
            // P.V: A (P) from tensor memory, B (V) MN-major, N = head_dim.
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) |
                                      (static_cast<uint32_t>(kPpBN >> 3) << 17) |
                                      (static_cast<uint32_t>(kPpBM >> 4) << 24);
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      (static_cast<uint32_t>(HD >> 3) << 17) |
                                      (static_cast<uint32_t>(kPpBM >> 4) << 24);
            const uint64_t q_desc = t5::desc_kmajor(smem_u32(Qs));
            const uint64_t k_desc = t5::desc_kmajor(smem_u32(Ks));
            const uint64_t v_desc = t5::desc_mnmajor(smem_u32(Vs), kPpKvHalf);
            bool ok = true;
            auto wait = [&](unsigned long long* bar, int parity) {
                if (ok && !mbar_wait(smem_u32(bar), parity)) ok = false;
                t5::fence_after();
            };
            auto scores = [&](int x, int t) {            // S_x(t) = Q_x K(t)^T
                const uint64_t kd = k_desc + (((t % STAGES) * TILE) >> 4);
                const uint64_t qd = q_desc + ((x * QTILE) >> 4);
#pragma unroll
                for (int k16 = 0; k16 < HD / 16; ++k16)
                    t5::mma_ss(tmem_s + x * kPpBN,
                               qd + (((k16 >> 2) * kPpQHalf + (k16 & 3) * 32) >> 4),
                               kd + (((k16 >> 2) * kPpKvHalf + (k16 & 3) * 32) >> 4), idesc_qk,
                               k16 > 0 ? 1u : 0u);
                t5::commit(smem_u32(&s_full[x]));
            };
            auto outputs = [&](int x, int t) {           // O_x += P_x(t) V(t)
                const uint64_t vd = v_desc + (((t % STAGES) * TILE) >> 4);
#pragma unroll
                for (int k16 = 0; k16 < kPpBN / 16; ++k16)
                    t5::mma_ts(tmem_o + x * kPpBN, tmem_s + x * kPpBN + 8 * k16,
                               vd + ((k16 * 16 * 128) >> 4), idesc_pv, (t > 0 || k16 > 0) ? 1u : 0u);
                t5::commit(smem_u32(&o_done[x]));
            };
            wait(&q_full[0], 0);
            wait(&k_full[0], 0);
            if (ok) scores(0, 0);
            if (has_b) {
                wait(&q_full[1], 0);
                if (ok) scores(1, 0);
            }
            if (ok) t5::commit(smem_u32(&k_empty[0]));
            for (int t = 0; t < n_t && ok; ++t) {
                const int st = t % STAGES;
                // the tiles this iteration reads arrived long ago: their barriers are tested
                // before the wait for the probabilities, so that no test (a couple of hundred
                // cycles even on a completed barrier) sits between the products of a query tile
                wait(&v_full[st], (t / STAGES) & 1);
                if (t + 1 < n_t) wait(&k_full[(t + 1) % STAGES], ((t + 1) / STAGES) & 1);
                if (t < n_a) {
                    wait(&p_full[0], t & 1);
                    if (!ok) break;
                    outputs(0, t);
                    if (t + 1 < n_a) scores(0, t + 1);
                }
                if (has_b) {
                    wait(&p_full[1], t & 1);
                    if (!ok) break;
                    outputs(1, t);
                }
                t5::commit(smem_u32(&v_empty[st]));
                if (t + 1 < n_t) {
                    if (has_b) scores(1, t + 1);
                    t5::commit(smem_u32(&k_empty[(t + 1) % STAGES]));
                }
            }
            if (!ok) failed_s = 1;       // the softmax warps run out of their bounded waits
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;\n");
        // ---- softmax: warp group x serves query tile x, one thread per row
        const int x = warp >> 2;
        if (x == 0 || has_b) {
            const int q = warp & 3;                                  // lane quarter this warp may access
            const int row = q * 32 + lane;                           // row within the query tile
            const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
            const int tile_pos0 = q_pos0 + x * kPpBM;                // position of the tile's first row
            const int pos = tile_pos0 + row;
            const int lo = window > 0 ? max(0, pos - window + 1) : 0;
            // the highest first visible key among the tile's rows
            const int lo_max = window > 0 ? max(0, tile_pos0 + kPpBM - 1 - window + 1) : 0;
            const unsigned span = static_cast<unsigned>(pos - lo);
            const int n_x = x == 0 ? n_a : n_t;
            const uint32_t s_addr = tmem_s + x * kPpBN + lane_addr;
            const uint32_t o_addr = tmem_o + x * kPpBN + lane_addr;
            float m = -INFINITY, l = 0.f;        // m: the reference maximum in use (log2 units)
            bool ok = true;
            for (int t = 0; t < n_x; ++t) {
                ok = mbar_wait(smem_u32(&s_full[x]), t & 1, ok ? 400000 : 1) && ok;
                t5::fence_after();
                const int kb = kb0 + t * kPpBN;
                // a tile in which no row of this query tile has a hidden key takes the short way
                const bool tile_inner = kb + kPpBN - 1 <= tile_pos0 && kb >= lo_max;
                // ---- the row's 128 scores into registers: four loads in flight, one wait
                uint32_t sv[128];
#pragma unroll
                for (int c = 0; c < 4; ++c) t5::ld32_nowait(s_addr + c * 32, sv + c * 32);
                t5::wait_ld();
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                if (tile_inner) {
#pragma unroll
                    for (int j = 0; j < 128; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(sv[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 128; ++j) {
                        // key in [lo, pos] as one unsigned comparison
                        const unsigned d = static_cast<unsigned>(kb + j - lo);
                        const float v = d <= span ? __uint_as_float(sv[j]) : -INFINITY;
                        sv[j] = __float_as_uint(v);
                        mx[j & 3] = fmaxf(mx[j & 3], v);
                    }
                }
                // the scale is positive: the maximum is taken over the raw scores and scaled once
                const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2e;
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
                    // O of the tiles so far must be complete before it is rescaled in tensor memory
                    if (t >= 1) ok = mbar_wait(smem_u32(&o_done[x]), (t - 1) & 1, ok ? 400000 : 1) && ok;
                    t5::fence_after();
#pragma unroll
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t ov[32];
                        t5::ld32_nowait(o_addr + c * 32, ov);
                        t5::wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
                        t5::st32(o_addr + c * 32, ov);
                    }
                    t5::wait_st();
                    l *= alpha;
                }
                const float neg_m = m == -INFINITY ? 0.f : -m;
                // ---- probabilities, written over the scores as bfloat16 pairs: chunk c's 32 keys
                // become 16 columns at 16 c (every score is in registers by now)
                float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(sv[c * 32 + 2 * j]), scale_log2e, neg_m));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(sv[c * 32 + 2 * j + 1]), scale_log2e, neg_m));
                        ps[(2 * j) & 3] += p0;
                        ps[(2 * j + 1) & 3] += p1;
                        pk[j] = pack_bf16(p0, p1);
                    }
                    t5::st16(s_addr + c * 16, pk);
                }
                ps[0] += ps[2];
                ps[1] += ps[3];
                l += ps[0] + ps[1];
                t5::wait_st();
                t5::fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&p_full[x]));
            }
            // ---- the output of this row
            ok = mbar_wait(smem_u32(&o_done[x]), (n_x - 1) & 1, ok ? 400000 : 1) && ok;
            t5::fence_after();
            if (!ok) failed_s = 1;
            const float inv = 1.0f / l;
            const int r = x * kPpBM + row;
            __nv_bfloat16* dst = out + static_cast<size_t>(row0 + r) * nq * HD + head * HD;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t v[32];
                t5::ld32_nowait(o_addr + c * 32, v);
                t5::wait_ld();
                if (r < rows) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[d]) * inv, __uint_as_float(v[d + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[d + 2]) * inv, __uint_as_float(v[d + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[d + 4]) * inv, __uint_as_float(v[d + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[d + 6]) * inv, __uint_as_float(v[d + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + d) = w;
                    }
                }
            }
        }
    }
    t5::fence_before();
    __syncthreads();
    if (warp == 9) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base_s),
                     "r"(TmemCols)
                     : "memory");
    }
    if (tid == 0 && failed_s) atomicExch(&g_prefill_pp_error, 1);
}

template <int HD>
int launch_prefill_pp(const CUtensorMap* q_map, const CUtensorMap* kv_map, long long k_row0,
                      long long v_row0, const int* block_table, int bt_stride, const int* cu_q,
                      const int* ctx_len, const int* tiles, int n_tiles, int nq, int nkv,
                      int page_size, float scale, int window, void* out, cudaStream_t stream) {
    const size_t smem = 2 * (HD / 64) * kPpQHalf + 2 * pp_stages(HD) * (HD / 64) * kPpKvHalf + 1024;
    cudaFuncSetAttribute(paged_prefill_pp_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
    dim3 grid(static_cast<unsigned>(nq) * n_tiles);
    launch_pdl(paged_prefill_pp_kernel<HD>, grid, dim3(kPpThreads), smem, stream, *q_map, *kv_map,
               k_row0, v_row0, block_table, bt_stride, cu_q, ctx_len, tiles, nq, nkv, page_size,
               scale * 1.4426950408889634f, window, static_cast<__nv_bfloat16*>(out), n_tiles);
    return launch_status();
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_prefill_pp_q_tile() { return kPpRows; }

SOMI_API int somi_prefill_pp_supported(int nq, int nkv, int hd, int page_size) {
    if (nkv <= 0 || nq % nkv) return 0;
    if (hd != 64 && hd != 128) return 0;
    return page_size >= 8 && page_size % 8 == 0 && kPpBN % page_size == 0;
}

SOMI_API int somi_prefill_pp_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_prefill_pp_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_prefill_pp_error, &zero, sizeof(int));
    return v;
}

// `tiles`: int32 [n_tiles, 3] = (request, first row, rows <= 256) over the multi-token requests;
// `q_map`: the projection buffer's map with boxes of 128 rows x 64 columns (as the one-tile kernel's).
SOMI_API int somi_paged_attention_prefill_pp(
    const void* q_map, const void* kv_map, long long k_row0, long long v_row0,
    const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len, const int* tiles,
    int n_tiles, int nq, int nkv, int hd, int page_size, float scale, int window, void* out,
    cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!somi_prefill_pp_supported(nq, nkv, hd, page_size)) return SOMI_ERR_UNSUPPORTED;
    const CUtensorMap* qm = static_cast<const CUtensorMap*>(q_map);
    const CUtensorMap* km = static_cast<const CUtensorMap*>(kv_map);
    if (hd == 64)
        return launch_prefill_pp<64>(qm, km, k_row0, v_row0, block_table, bt_stride, cu_q, ctx_len,
                                     tiles, n_tiles, nq, nkv, page_size, scale, window, out, stream);
    return launch_prefill_pp<128>(qm, km, k_row0, v_row0, block_table, bt_stride, cu_q, ctx_len, tiles,
                                  n_tiles, nq, nkv, page_size, scale, window, out, stream);
}
