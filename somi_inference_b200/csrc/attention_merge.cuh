// Merge of the partial results of split-KV decode attention: for every (request, query head)
// the chunks' outputs, each with its maximum and sum, are added up into one bfloat16 row.
//
// Two kernels.  Few chunks: one thread per output element walks through them (the chain is
// short and the launch is what counts).  Many chunks (long contexts): the warps of the CTA
// take the chunks in turn, so that a warp's loads of different chunks are in flight together,
// and their sums meet in shared memory; with one thread per element a context of 32k tokens
// was a chain of 257 dependent steps per CTA and took longer than the attention itself.
#pragma once

#include "common.cuh"

namespace somi {

constexpr int kMergeWideFrom = 33;     // chunks per request from which the warps share them
constexpr int kMergeWarps = 8;

namespace {      // every file that includes this has kernels of its own (no symbol is shared)

struct MergeRange {
    int first_split, n_splits;
};
// the chunks a request reads: `chunk` keys each, from the window's first key to the newest
__device__ __forceinline__ MergeRange merge_range(int ctx_len, int window, int chunk) {
    MergeRange r;
    const int first_key = window > 0 ? max(0, ctx_len - window + 1) : 0;
    r.first_split = first_key / chunk;
    r.n_splits = (ctx_len + 1 + chunk - 1) / chunk;
    return r;
}

// CHUNK: the keys per partial result, known at compile time here: the range is found with
// shifts (a division by a run-time value at the head of this short kernel cost 1 µs).
template <int HD, int CHUNK>
__global__ void __launch_bounds__(HD)
decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    int max_splits, const int* __restrict__ ctx_len, int row_base,
                    int req_base, int nq, int window, __nv_bfloat16* __restrict__ out) {
    const int i = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const MergeRange rg = merge_range(ctx_len[req_base + i], window, CHUNK);
    if (rg.n_splits - rg.first_split == 1) return;       // written by the split kernel
    const size_t base = (static_cast<size_t>(i) * nq + head) * max_splits;
    float M = -INFINITY;
    for (int s = rg.first_split; s < rg.n_splits; ++s) M = fmaxf(M, part_ml[2 * (base + s)]);
    float acc = 0.f, L = 0.f;
    for (int s = rg.first_split; s < rg.n_splits; ++s) {
        const float f = exp2f(part_ml[2 * (base + s)] - M);
        acc += f * part_o[(base + s) * HD + d];
        L += f * part_ml[2 * (base + s) + 1];
    }
    out[static_cast<size_t>(row_base + i) * nq * HD + head * HD + d] = __float2bfloat16_rn(acc / L);
}

template <int HD>
__global__ void __launch_bounds__(kMergeWarps * 32)
decode_merge_wide_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         int max_splits, int chunk, const int* __restrict__ ctx_len, int row_base,
                         int req_base, int nq, int window, __nv_bfloat16* __restrict__ out) {
    constexpr int V = (HD + 31) / 32;                     // output elements per lane
    __shared__ float red_o[kMergeWarps][HD];
    __shared__ float red_l[kMergeWarps];
    __shared__ float red_m[kMergeWarps];
    const int i = blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();
    pdl_wait();
    const MergeRange rg = merge_range(ctx_len[req_base + i], window, chunk);
    if (rg.n_splits - rg.first_split == 1) return;
    const size_t base = (static_cast<size_t>(i) * nq + head) * max_splits;
    // the maximum over all chunks
    float M = -INFINITY;
    for (int s = rg.first_split + tid; s < rg.n_splits; s += kMergeWarps * 32)
        M = fmaxf(M, part_ml[2 * (base + s)]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) red_m[warp] = M;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < kMergeWarps; ++w) M = fmaxf(M, red_m[w]);
    // each warp adds up every kMergeWarps-th chunk
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;
    float L = 0.f;
#pragma unroll 4
    for (int s = rg.first_split + warp; s < rg.n_splits; s += kMergeWarps) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + 2 * (base + s));
        const float f = exp2f(ml.x - M);
        const float* o = part_o + (base + s) * HD;
#pragma unroll
        for (int v = 0; v < V; ++v)
            if (HD % 32 == 0 || lane + 32 * v < HD) acc[v] += f * o[lane + 32 * v];
        L += f * ml.y;
    }
#pragma unroll
    for (int v = 0; v < V; ++v)
        if (HD % 32 == 0 || lane + 32 * v < HD) red_o[warp][lane + 32 * v] = acc[v];
    if (lane == 0) red_l[warp] = L;
    __syncthreads();
    for (int d = tid; d < HD; d += kMergeWarps * 32) {
        float a = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kMergeWarps; ++w) {
            a += red_o[w][d];
            l += red_l[w];
        }
        out[static_cast<size_t>(row_base + i) * nq * HD + head * HD + d] = __float2bfloat16_rn(a / l);
    }
}

}  // namespace

// Launch the merge for `n_decode` requests (none if every request has a single chunk).
template <int HD>
static int launch_decode_merge(const float* part_o, const float* part_ml, int max_splits, int chunk,
                        const int* ctx_len, int row_base, int req_base, int n_decode, int nq,
                        int window, __nv_bfloat16* out, cudaStream_t stream) {
    dim3 grid(n_decode, nq);
    if (max_splits >= kMergeWideFrom || chunk != 128)
        launch_pdl(decode_merge_wide_kernel<HD>, grid, dim3(kMergeWarps * 32), 0, stream, part_o,
                   part_ml, max_splits, chunk, ctx_len, row_base, req_base, nq, window, out);
    else
        launch_pdl(decode_merge_kernel<HD, 128>, grid, dim3(HD), 0, stream, part_o, part_ml,
                   max_splits, ctx_len, row_base, req_base, nq, window, out);
    return launch_status();
}

}  // namespace somi
