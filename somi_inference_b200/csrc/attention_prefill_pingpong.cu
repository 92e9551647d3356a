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
// (Two issuing threads, one per query tile, fall into step with each other: both softmax warp
// groups then want the exponential unit at the same time and a round takes a third longer.)
// What the issuing thread does between products costs a hundred cycles and more apiece (a
// barrier test, a fence, a commit), during which the pipe runs dry, so it does as little of
// it as possible: it tests only the two p_full barriers in a round (the softmax warp group that
// announces P has seen the value tile and the next key tile arrive, before it waits for the
// scores, where it has time), it commits o_done only after a query tile's last key tile (the
// commit behind s_full covers the output products issued before it), and it hands both stages
// back at the end of a round.
// An accumulator is rescaled in tensor memory only when its row maximum grows by more than 2^8
// (probabilities up to 256 are harmless in float32 sums and bfloat16 operands).  Because tile B's
// rows come later in the sequence, tile A runs out of key tiles first and writes its output
// while B goes on.  Softmax is float32, base 2; scaling, subtraction and the row sum work on
// pairs of keys (`fma.rn.f32x2`, `add.rn.f32x2`), the maximum on three values at a time.  Every
// wait on an mbarrier is bounded and failure is recorded in an error word.
//
// Warp roles: warps 0-3 softmax of tile A, 4-7 softmax of tile B (both clear the value stages
// first), warp 8 key (and Q) producer, warp 9 MMA issuer and owner of tensor memory, warp 10
// value producer, warp 11 idle.  Two key stages and three value stages at head size 128 (a value
// tile is read a round later than the key tile that came with it), four and four at 64.
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
// A value tile is read one key tile later than the key tile that arrived with it (its products
// wait for the softmax in between), so at the same distance of prefetch it needs a stage more.
__host__ __device__ constexpr int pp_k_stages(int hd) { return hd == 128 ? 2 : 4; }
__host__ __device__ constexpr int pp_v_stages(int hd) { return hd == 128 ? 3 : 4; }
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
    constexpr int KST = pp_k_stages(HD), VST = pp_v_stages(HD);
    constexpr uint32_t TmemCols = 512;                   // S_A | S_B | O_A | O_B, 128 columns each
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* Qs = base;                            // two query tiles
    unsigned char* Ks = Qs + 2 * QTILE;                  // KST tiles
    unsigned char* Vs = Ks + KST * TILE;                 // VST tiles
    __shared__ __align__(8) unsigned long long q_full[2], k_full[kPpMaxStages], k_empty[kPpMaxStages],
        v_full[kPpMaxStages], v_empty[kPpMaxStages], s_full[2], p_full[2], o_done[2], v_zeroed;
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
        for (int s = 0; s < kPpMaxStages; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        mbar_init(smem_u32(&v_zeroed), 8);               // one arrival per softmax warp
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
    // need few.  Warps 8-11 give registers back and the softmax warp groups take them.  The
    // pool is what the CTA was given at launch, 12 warps x 168 registers a thread: 8 x 216 +
    // 4 x 72 uses exactly that.  `setmaxnreg.inc` waits, without a limit, until the pool has what
    // it asks for, so the two figures must never add up to more.
    static_assert(8 * 216 + 4 * 72 <= 12 * 168, "setmaxnreg would wait for registers that never come");
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
        const int n_st = which ? VST : KST;
        // no value copy before the softmax warps have cleared the value stages
        if (which && !mbar_wait(smem_u32(&v_zeroed), 0)) failed_s = 1;
        __syncwarp();
        for (int t = 0; t < n_t; ++t) {
            const int st = t % n_st;
            const int kb = kb0 + t * kPpBN;
            const int p_lo = max(kb, kv_first) / page_size;
            const int p_hi = (min(kb + kPpBN, end_all) - 1) / page_size;
            int my_page = -1;
            const int ap = kb / page_size + lane;
            if (lane < pages_per_tile && ap >= p_lo && ap <= p_hi) my_page = bt[ap];
            const uint32_t bar = smem_u32(which ? &v_full[st] : &k_full[st]);
            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait(smem_u32(which ? &v_empty[st] : &k_empty[st]), ((t / n_st) & 1) ^ 1) ? 1 : 0;
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
            // the same with the test that returns at once: this thread has nothing else to do,
            // and wakes up sooner than from the test that may suspend it
            auto spin = [&](unsigned long long* bar, int parity) {
                if (ok) {
                    int i = 0;
                    while (!mbar_test_now(smem_u32(bar), parity))
                        if (++i > 8000000) { ok = false; break; }
                }
                t5::fence_after();
            };
            auto scores = [&](int x, int t) {            // S_x(t) = Q_x K(t)^T
                const uint64_t kd = k_desc + (((t % KST) * TILE) >> 4);
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
                const uint64_t vd = v_desc + (((t % VST) * TILE) >> 4);
#pragma unroll
                for (int k16 = 0; k16 < kPpBN / 16; ++k16)
                    t5::mma_ts(tmem_o + x * kPpBN, tmem_s + x * kPpBN + 8 * k16,
                               vd + ((k16 * 16 * 128) >> 4), idesc_pv, (t > 0 || k16 > 0) ? 1u : 0u);
                // A commit covers every product issued so far: s_full of tile t + 1 also says
                // that O holds tile t, so o_done is only needed after a query tile's last.
                if (t + 1 == (x == 0 ? n_a : n_t)) t5::commit(smem_u32(&o_done[x]));
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
                // The key and value tiles these products read have been seen by the softmax
                // warp group that announces P (it waits for them before it arrives), so this
                // thread tests nothing but the two p_full barriers in an iteration: every test
                // and every commit is time in which this thread issues no product.
                if (t < n_a) {
                    spin(&p_full[0], t & 1);
                    if (!ok) break;
                    outputs(0, t);
                    if (t + 1 < n_a) scores(0, t + 1);
                }
                if (has_b) {
                    spin(&p_full[1], t & 1);
                    if (!ok) break;
                    outputs(1, t);
                    if (t + 1 < n_t) scores(1, t + 1);
                }
                // both stages are handed back at the end, so that no commit sits between the
                // products of a query tile
                t5::commit(smem_u32(&v_empty[t % VST]));
                if (t + 1 < n_t) t5::commit(smem_u32(&k_empty[(t + 1) % KST]));
            }
            if (!ok) failed_s = 1;       // the softmax warps run out of their bounded waits
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;\n");
        // Value rows that no copy fills (pages outside the request's range) must be finite
        // numbers, whatever the shared memory held before.  These warps have nothing to do
        // until the first scores are there, so they clear the value stages while the keys and
        // queries are on their way; the value producer waits for them.
        for (int c = tid; c < VST * TILE / 16; c += 8 * 32)
            reinterpret_cast<uint4*>(Vs)[c] = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&v_zeroed));
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
                // On behalf of the issuing thread: the values of this tile and the keys of the
                // next have arrived before this warp group announces P(t).  They are tested
                // here, where the warp would wait for the scores anyway (a test costs a few
                // hundred cycles even on a completed barrier), by the whole warp, so that it
                // stays converged for the aligned instructions.
                if (q == 0) {
                    ok = mbar_wait(smem_u32(&v_full[t % VST]), (t / VST) & 1, ok ? 400000 : 1) && ok;
                    if (t + 1 < n_x)
                        ok = mbar_wait(smem_u32(&k_full[(t + 1) % KST]), ((t + 1) / KST) & 1,
                                       ok ? 400000 : 1) && ok;
                }
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
                    for (int j = 0; j < 128; j += 2)
                        mx[(j >> 1) & 3] = fmax3(mx[(j >> 1) & 3], __uint_as_float(sv[j]), __uint_as_float(sv[j + 1]));
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
                    // O holds the tiles so far: the commit behind s_full covered the products
                    // of tile t - 1 as well (issued before S(t) by the same thread)
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
                // (scaling, subtraction and the row sum on pairs of keys: one instruction for two)
                const uint64_t scale2 = pair_f32(scale_log2e, scale_log2e), neg_m2 = pair_f32(neg_m, neg_m);
                uint64_t ps2[2] = {pair_f32(0.f, 0.f), pair_f32(0.f, 0.f)};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float a0, a1;
                        unpair_f32(fma_f32x2(pair_f32(__uint_as_float(sv[c * 32 + 2 * j]),
                                                      __uint_as_float(sv[c * 32 + 2 * j + 1])),
                                             scale2, neg_m2), a0, a1);
                        const float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
                        ps2[j & 1] = add_f32x2(ps2[j & 1], pair_f32(p0, p1));
                        pk[j] = pack_bf16(p0, p1);
                    }
                    t5::st16(s_addr + c * 16, pk);
                }
                {
                    float s0, s1, s2, s3;
                    unpair_f32(ps2[0], s0, s1);
                    unpair_f32(ps2[1], s2, s3);
                    l += (s0 + s2) + (s1 + s3);
                }
                t5::wait_st();
                t5::fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&p_full[x]));
            }
            // ---- the output of this row
            ok = mbar_wait(smem_u32(&o_done[x]), 0, ok ? 400000 : 1) && ok;
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
    const size_t smem = 2 * (HD / 64) * kPpQHalf +
                        (pp_k_stages(HD) + pp_v_stages(HD)) * (HD / 64) * kPpKvHalf + 1024;
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
