// Split-KV grouped-query attention for single-token requests over the paged bfloat16 cache.
//
// One CTA = one request x one kv head x one chunk of 128 keys; it serves all query heads of
// the group at once (they become the rows of the MMA tile), so keys and values are read once.
// Scores and P.V run on tensor cores (m16n8k16, float32 accumulation), softmax in float32 with
// base-2 exponentials.  The chunk size is fixed, so what a request computes does not depend on
// the rest of the batch.  A request whose keys span several chunks leaves per-chunk partial
// results (un-normalised output, running maximum, sum) in scratch memory, which a second
// kernel merges; a request with a single chunk is written directly.
//
// What the reference does here: one program per (sequence, query head) that walks all pages
// of the sequence with an online softmax, re-reading keys and values for every query head of
// a group (somi_inference/core/paged_attention_triton.py:29-150); formulas in
// somi_inference/core/paged_attention.py:352-413.
#include "attention_merge.cuh"
#include "mma.cuh"

namespace somi {

constexpr int kDecChunk = 128;     // keys per CTA
constexpr int kDecThreads = 128;   // 4 warps, 32 keys each
constexpr int kDecRows = 16;       // query heads per group, padded to the MMA's 16 rows

struct DecodeRange {
    int kv_len, first_key, first_split, n_splits;
};

__device__ __forceinline__ DecodeRange decode_range(int ctx_len, int window) {
    DecodeRange r;
    r.kv_len = ctx_len + 1;                      // the new token's key is already in the cache
    const int pos = ctx_len;
    r.first_key = window > 0 ? max(0, pos - window + 1) : 0;
    r.first_split = r.first_key / kDecChunk;
    r.n_splits = (r.kv_len + kDecChunk - 1) / kDecChunk;
    return r;
}

template <int HD>
__global__ void __launch_bounds__(kDecThreads)
paged_decode_split_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride, int row_base,
                          int req_base, const __nv_bfloat16* __restrict__ kcache,
                          const __nv_bfloat16* __restrict__ vcache,
                          const int* __restrict__ block_table, int bt_stride,
                          const int* __restrict__ ctx_len, int nq, int nkv, int page_size,
                          float scale_log2e, int window, float* __restrict__ part_o,
                          float* __restrict__ part_ml, int max_splits,
                          __nv_bfloat16* __restrict__ out) {
    constexpr int CPR = HD / 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* Qs = smem_raw;                               // [16][HD] bf16
    unsigned char* Ks = Qs + kDecRows * HD * 2;                 // [128][HD] bf16
    unsigned char* Vs = Ks + kDecChunk * HD * 2;                // [128][HD] bf16
    __shared__ float m_s[4][kDecRows], l_s[4][kDecRows];
    pdl_launch_dependents();
    pdl_wait();

    const int split = blockIdx.x, kvh = blockIdx.y, i = blockIdx.z;
    const int req = req_base + i, row = row_base + i;
    const int G = nq / nkv;
    const DecodeRange rg = decode_range(ctx_len[req], window);
    if (split < rg.first_split || split >= rg.n_splits) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k0 = split * kDecChunk;
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;

    // ---- asynchronous loads: Q and K in the first group, V in the second
    const __nv_bfloat16* qrow = qkv + static_cast<size_t>(row) * row_stride + static_cast<size_t>(kvh) * G * HD;
    for (int c = tid; c < kDecRows * CPR; c += kDecThreads) {
        const int r = c / CPR, ch = c - r * CPR;
        const bool ok = r < G;
        cp_async_16(smem_u32(Qs + swizzled_offset<HD>(r, ch)), ok ? qrow + r * HD + ch * 8 : qrow,
                    ok ? 16 : 0);
    }
    for (int c = tid; c < kDecChunk * CPR; c += kDecThreads) {
        const int r = c / CPR, ch = c - r * CPR;
        const int j = k0 + r;
        const bool ok = j < rg.kv_len && j >= rg.first_key;
        const __nv_bfloat16* src = kcache;
        if (ok) {
            const int page = bt[j / page_size];
            src = kcache + ((static_cast<size_t>(page) * nkv + kvh) * page_size + j % page_size) * HD + ch * 8;
        }
        cp_async_16(smem_u32(Ks + swizzled_offset<HD>(r, ch)), src, ok ? 16 : 0);
    }
    cp_async_commit();
    for (int c = tid; c < kDecChunk * CPR; c += kDecThreads) {
        const int r = c / CPR, ch = c - r * CPR;
        const int j = k0 + r;
        const bool ok = j < rg.kv_len && j >= rg.first_key;
        const __nv_bfloat16* src = vcache;
        if (ok) {
            const int page = bt[j / page_size];
            src = vcache + ((static_cast<size_t>(page) * nkv + kvh) * page_size + j % page_size) * HD + ch * 8;
        }
        cp_async_16(smem_u32(Vs + swizzled_offset<HD>(r, ch)), src, ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // ---- S = Q K^T for this warp's 32 keys
    float s[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
    const int kw = warp * 32;       // this warp's first key within the chunk
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, smem_u32(Qs + swizzled_offset<HD>((lane & 7) + ((lane >> 3) & 1) * 8,
                                                        2 * ks + (lane >> 4))));
#pragma unroll
        for (int np = 0; np < 2; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, smem_u32(Ks + swizzled_offset<HD>(kw + np * 16 + (lane & 7) + (lane >> 4) * 8,
                                                            2 * ks + ((lane >> 3) & 1))));
            mma_bf16_16816(s[2 * np], a, b[0], b[1]);
            mma_bf16_16816(s[2 * np + 1], a, b[2], b[3]);
        }
    }
    // ---- mask, softmax over the warp's keys (rows: lane/4 and lane/4 + 8)
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
    const float ms_lo = m_lo == -INFINITY ? 0.f : m_lo, ms_hi = m_hi == -INFINITY ? 0.f : m_hi;
    float l_lo = 0.f, l_hi = 0.f;
    uint32_t pa[2][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const float p0 = exp2f(s[nt][0] - ms_lo), p1 = exp2f(s[nt][1] - ms_lo);
        const float p2 = exp2f(s[nt][2] - ms_hi), p3 = exp2f(s[nt][3] - ms_hi);
        // the probabilities enter P.V rounded to bfloat16; the sum uses the same rounded values
        const uint32_t lo = pack_bf16(p0, p1), hi = pack_bf16(p2, p3);
        const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&lo);
        const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&hi);
        l_lo += __low2float(lo2) + __high2float(lo2);
        l_hi += __low2float(hi2) + __high2float(hi2);
        pa[nt >> 1][(nt & 1) * 2] = lo;
        pa[nt >> 1][(nt & 1) * 2 + 1] = hi;
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    cp_async_wait<0>();
    __syncthreads();       // V has arrived; nobody reads K any more

    // ---- O = P V for this warp's 32 keys
    float o[HD / 8][4];
#pragma unroll
    for (int a = 0; a < HD / 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) o[a][b] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk)
#pragma unroll
        for (int dc = 0; dc < HD / 16; ++dc) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, smem_u32(Vs + swizzled_offset<HD>(
                                     kw + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                     2 * dc + (lane >> 4))));
            mma_bf16_16816(o[2 * dc], pa[kk], b[0], b[1]);
            mma_bf16_16816(o[2 * dc + 1], pa[kk], b[2], b[3]);
        }

    // ---- merge the four warps through shared memory (the K tile's space is free now)
    float* obuf = reinterpret_cast<float*>(Ks);          // [4][16][HD]
    {
        const int r_lo = lane >> 2, r_hi = r_lo + 8;
        float* ob = obuf + static_cast<size_t>(warp) * kDecRows * HD;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
            const int d = nt * 8 + (lane & 3) * 2;
            ob[r_lo * HD + d] = o[nt][0];
            ob[r_lo * HD + d + 1] = o[nt][1];
            ob[r_hi * HD + d] = o[nt][2];
            ob[r_hi * HD + d + 1] = o[nt][3];
        }
        if ((lane & 3) == 0) {
            m_s[warp][r_lo] = m_lo; l_s[warp][r_lo] = l_lo;
            m_s[warp][r_hi] = m_hi; l_s[warp][r_hi] = l_hi;
        }
    }
    __syncthreads();
    const bool single = rg.n_splits - rg.first_split == 1;
    for (int idx = tid; idx < G * HD; idx += kDecThreads) {
        const int g = idx / HD, d = idx - g * HD;
        float M = fmaxf(fmaxf(m_s[0][g], m_s[1][g]), fmaxf(m_s[2][g], m_s[3][g]));
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = m_s[w][g] == -INFINITY ? 0.f : exp2f(m_s[w][g] - M);
            acc += f * obuf[(w * kDecRows + g) * HD + d];
            L += f * l_s[w][g];
        }
        const int head = kvh * G + g;
        if (single) {
            out[static_cast<size_t>(row) * nq * HD + head * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            const size_t p = (static_cast<size_t>(i) * nq + head) * max_splits + split;
            part_o[p * HD + d] = acc;
            if (d == 0) { part_ml[2 * p] = M; part_ml[2 * p + 1] = L; }
        }
    }
}

template <int HD>
int launch_decode(const void* qkv, int row_stride, int row_base, int req_base, int n_decode,
                  const void* kcache, const void* vcache, const int* block_table, int bt_stride,
                  const int* ctx_len, int nq, int nkv, int page_size, float scale, int window,
                  float* part_o, float* part_ml, int max_splits, void* out, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(kDecRows + 2 * kDecChunk) * HD * 2;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(paged_decode_split_kernel<HD>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(max_splits, nkv, n_decode);
    launch_pdl(paged_decode_split_kernel<HD>, dim3(grid), dim3(kDecThreads), smem, stream, 
        static_cast<const __nv_bfloat16*>(qkv), row_stride, row_base, req_base,
        static_cast<const __nv_bfloat16*>(kcache), static_cast<const __nv_bfloat16*>(vcache),
        block_table, bt_stride, ctx_len, nq, nkv, page_size, scale * 1.4426950408889634f, window,
        part_o, part_ml, max_splits, static_cast<__nv_bfloat16*>(out));
    int rc = launch_status();
    if (rc != 0 || max_splits == 1) return rc;
    return launch_decode_merge<HD>(part_o, part_ml, max_splits, kDecChunk, ctx_len, row_base, req_base,
                                   n_decode, nq, window, static_cast<__nv_bfloat16*>(out), stream);
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_decode_chunk() { return kDecChunk; }

// 1 if the split-KV kernel takes this geometry (bfloat16 only), else 0.
SOMI_API int somi_decode_supported(int nq, int nkv, int hd) {
    if (nkv <= 0 || nq % nkv) return 0;
    if (nq / nkv > kDecRows) return 0;
    return hd == 32 || hd == 64 || hd == 128;
}

// Scratch: part_o float32 [n_decode, nq, max_splits, hd], part_ml float32 [n_decode, nq, max_splits, 2].
SOMI_API int somi_paged_attention_decode(
    const void* qkv, int row_stride, int row_base, int req_base, int n_decode, const void* kcache,
    const void* vcache, const int* block_table, int bt_stride, const int* ctx_len, int nq, int nkv,
    int hd, int page_size, float scale, int window, float* part_o, float* part_ml, int max_splits,
    void* out, cudaStream_t stream) {
    if (n_decode <= 0) return 0;
    if (!somi_decode_supported(nq, nkv, hd) || page_size <= 0 || max_splits <= 0 ||
        n_decode > 65535 || nkv > 65535)
        return SOMI_ERR_UNSUPPORTED;
#define SOMI_DEC(HD)                                                                             \
    return launch_decode<HD>(qkv, row_stride, row_base, req_base, n_decode, kcache, vcache,      \
                             block_table, bt_stride, ctx_len, nq, nkv, page_size, scale, window, \
                             part_o, part_ml, max_splits, out, stream)
    if (hd == 32) SOMI_DEC(32);
    if (hd == 64) SOMI_DEC(64);
    SOMI_DEC(128);
#undef SOMI_DEC
}

// ------------------------------------------------------------------------------------------
// The same split-KV decode attention for callers that cannot allocate device memory.
// Declared in attention_decode_static.h; it has no counterpart in the reference.
//
// Some hosts of this library may not call cudaMalloc at the moment they need attention: a
// serving process that gave the whole device to its own pool at start-up, a caller inside a
// latency-critical loop where an allocation would synchronise the device, or one that simply
// has no allocator handle to give us.  For them the per-chunk partial results live in a
// file-scope device array of fixed size instead of caller-provided scratch.  Every GPU that
// loads the library holds these kStaticScratchFloats * 4 bytes (8 MiB) until the process exits.
//
// In host code the array's name is only a host-side stand-in for the device symbol, not a
// device address, so the address is asked for once per device with cudaGetSymbolAddress (with
// that device current) and that pointer is what the kernels get.
namespace somi {

constexpr size_t kStaticScratchFloats = size_t(2) << 20;           // 2 Mi floats = 8 MiB
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) float g_static_decode_scratch[kStaticScratchFloats];
static float* g_static_scratch_ptr[kStaticMaxDevices] = {};        // host: device address per GPU

// Returns the device address of the static scratch on the current device (nullptr on failure);
// the first call on a device asks the runtime for it.
static float* static_scratch_on_current_device(int* status) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) {
        *status = e != cudaSuccess ? static_cast<int>(e) : SOMI_ERR_UNSUPPORTED;
        return nullptr;
    }
    float* p = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_decode_scratch);
        if (e != cudaSuccess || addr == nullptr) {
            *status = e != cudaSuccess ? static_cast<int>(e) : SOMI_ERR_UNSUPPORTED;
            return nullptr;
        }
        p = static_cast<float*>(addr);
        __atomic_store_n(&g_static_scratch_ptr[dev], p, __ATOMIC_RELEASE);
    }
    *status = 0;
    return p;
}

}  // namespace somi

SOMI_API long long somi_paged_attention_decode_static_capacity() {
    return static_cast<long long>(kStaticScratchFloats);
}

SOMI_API const char* somi_paged_attention_decode_static_strerror(int code) {
    switch (code) {
        case 0: return "success";
        case SOMI_ERR_UNSUPPORTED:
            return "sizes not supported by the split-KV decode attention kernel";
        case SOMI_ERR_SCRATCH_TOO_SMALL:
            return "n_decode * num_heads * max_splits * (head_dim + 2) exceeds the static scratch "
                   "of 2 Mi floats; use somi_paged_attention_decode with caller-provided scratch";
        default: return "CUDA runtime error (the value is the cudaError_t)";
    }
}

SOMI_API int somi_paged_attention_decode_static(
    const void* qkv, int row_stride, int row_base, int req_base, int n_decode, const void* kcache,
    const void* vcache, const int* block_table, int bt_stride, const int* ctx_len, int nq, int nkv,
    int hd, int page_size, float scale, int window, int max_splits, void* out,
    cudaStream_t stream) {
    if (n_decode <= 0) return 0;
    if (!somi_decode_supported(nq, nkv, hd) || page_size <= 0 || max_splits <= 0 ||
        n_decode > 65535 || nkv > 65535)
        return SOMI_ERR_UNSUPPORTED;
    // n_decode * nq * max_splits slots of (hd + 2) floats must fit; the test is made with
    // divisions, so that no product of caller-given numbers can wrap around and pass it
    const size_t cap_slots = kStaticScratchFloats / (static_cast<size_t>(hd) + 2);
    if (nq <= 0 || static_cast<size_t>(max_splits) > cap_slots) return SOMI_ERR_SCRATCH_TOO_SMALL;
    const size_t rows_allowed = cap_slots / static_cast<size_t>(max_splits);     // n_decode * nq
    if (static_cast<size_t>(nq) > rows_allowed ||
        static_cast<size_t>(n_decode) > rows_allowed / static_cast<size_t>(nq))
        return SOMI_ERR_SCRATCH_TOO_SMALL;
    const size_t slots = static_cast<size_t>(n_decode) * nq * max_splits;
    // The array's address is looked up for the CURRENT device: `stream` must belong to it (as
    // every pointer argument does); the caller makes that device current before the call.
    int status = 0;
    float* scratch = static_scratch_on_current_device(&status);
    if (scratch == nullptr) return status;
    // Layout inside the array: partial outputs first, then (maximum, sum) pairs.  Nothing here
    // has to start at zero: every slot that the merge kernel reads is written by the split
    // kernel of the same call, and slots of chunks a request does not have are never read.
    float* part_o = scratch;
    float* part_ml = scratch + slots * hd;
    return somi_paged_attention_decode(qkv, row_stride, row_base, req_base, n_decode, kcache,
                                       vcache, block_table, bt_stride, ctx_len, nq, nkv, hd,
                                       page_size, scale, window, part_o, part_ml, max_splits, out,
                                       stream);
}
