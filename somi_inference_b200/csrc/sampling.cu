// Sampling of one token per logits row, one CTA per row, no scratch memory.
//
// Order of operations as in the reference sampler (somi_inference/core/sampler.py:81-176):
// repetition penalty over the set of history tokens (logit > 0 ? logit / p : logit * p),
// division by the temperature, top-k, top-p on the softmax of what top-k left, and then
// argmax (temperature 0; lowest index wins ties) or a draw from the softmax of what is left.
// The draw is an inverse-CDF walk in index order with a uniform number from a counter-based
// generator keyed by (seed, counter) of the row, so a request's tokens do not depend on what
// else is in the batch.  Thresholds of top-k and top-p are found by radix selection over the
// order-preserving integer image of the floats (four passes of 8 bits); probability mass is
// accumulated in 40-bit fixed point with integer atomics, which makes it order-independent.
// Values exactly equal to the k-th largest are all kept.
#include "common.cuh"

namespace somi {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned int float_key(float f) {
    const unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__host__ __device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned int counter) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (static_cast<unsigned long long>(counter) + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);     // 24 bits: [0, 1)
}

struct RowView {
    const float* logits;
    const unsigned int* bitmap;   // history tokens (shared memory), or nullptr
    float penalty;
    float inv_temperature;        // 1 when temperature is 0
    __device__ __forceinline__ float at(int i) const {
        float l = logits[i];
        if (bitmap && ((bitmap[i >> 5] >> (i & 31)) & 1u)) l = l > 0.f ? l / penalty : l * penalty;
        return l * inv_temperature;
    }
};

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ penalty, const unsigned long long* __restrict__ seed,
              const unsigned int* __restrict__ counter, const int* __restrict__ hist_off,
              const int* __restrict__ hist_tok, int* __restrict__ out) {
    extern __shared__ unsigned int bitmap[];              // (V + 31) / 32 words
    __shared__ unsigned long long hist[256];
    __shared__ float red_f[33];
    __shared__ int red_i[33];
    __shared__ unsigned int sh_prefix;
    __shared__ unsigned long long sh_remaining;
    __shared__ float sh_total;
    __shared__ int sh_found;

    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const float temp = temperature[row];
    const float pen = penalty[row];
    const int h0 = hist_off[row], h1 = hist_off[row + 1];
    const bool use_pen = pen != 1.0f && h1 > h0;
    if (use_pen) {
        for (int i = tid; i < (V + 31) / 32; i += kSampleThreads) bitmap[i] = 0u;
        __syncthreads();
        for (int i = h0 + tid; i < h1; i += kSampleThreads) {
            const int t = hist_tok[i];
            if (t >= 0 && t < V) atomicOr(&bitmap[t >> 5], 1u << (t & 31));
        }
        __syncthreads();
    }
    RowView x{logits + static_cast<size_t>(row) * V, use_pen ? bitmap : nullptr, pen,
              temp > 0.f ? 1.0f / temp : 1.0f};
    // note: the reference divides by the temperature; multiplying by its reciprocal differs
    // by one rounding, which cannot change an ordering and moves probabilities by 1e-7 relative.

    // ---- maximum and its lowest index
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    if (!use_pen && (V & 3) == 0) {
        // four logits per load, several loads in flight: this pass is all a greedy row needs
        const float4* row4 = reinterpret_cast<const float4*>(x.logits);
        const float it = x.inv_temperature;
#pragma unroll 4
        for (int i = tid; i < (V >> 2); i += kSampleThreads) {
            const float4 q = row4[i];
            const float v0 = q.x * it, v1 = q.y * it, v2 = q.z * it, v3 = q.w * it;
            if (v0 > best) { best = v0; best_i = 4 * i; }
            if (v1 > best) { best = v1; best_i = 4 * i + 1; }
            if (v2 > best) { best = v2; best_i = 4 * i + 2; }
            if (v3 > best) { best = v3; best_i = 4 * i + 3; }
        }
    } else {
        for (int i = tid; i < V; i += kSampleThreads) {
            const float v = x.at(i);
            if (v > best) { best = v; best_i = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { red_f[warp] = best; red_i[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = red_f[lane];
        best_i = red_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { red_f[32] = best; red_i[32] = best_i; }
    }
    __syncthreads();
    const float row_max = red_f[32];
    if (temp <= 0.f) {
        if (tid == 0) out[row] = red_i[32] == 0x7fffffff ? 0 : red_i[32];
        return;
    }

    // ---- top-k: key of the k-th largest value
    unsigned int key_floor = 0u;       // keep keys >= key_floor
    const int k = top_k[row];
    if (k > 0 && k < V) {
        unsigned int prefix = 0u, mask = 0u;
        if (tid == 0) sh_remaining = static_cast<unsigned long long>(k);
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) hist[tid] = 0ull;
            __syncthreads();
            for (int i = tid; i < V; i += kSampleThreads) {
                const unsigned int key = float_key(x.at(i));
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1ull);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long rem = sh_remaining;
                int digit = 0;
                for (int b = 255; b >= 0; --b) {
                    if (hist[b] >= rem) { digit = b; break; }
                    rem -= hist[b];
                }
                sh_remaining = rem;
                sh_prefix = prefix | (static_cast<unsigned int>(digit) << shift);
            }
            __syncthreads();
            prefix = sh_prefix;
            mask |= 255u << shift;
        }
        key_floor = prefix;
    }

    // ---- softmax denominator over what top-k left
    const float p_top = top_p[row];
    if (p_top < 1.0f) {
        float z = 0.f;
        for (int i = tid; i < V; i += kSampleThreads) {
            const float v = x.at(i);
            if (float_key(v) >= key_floor) z += expf(v - row_max);
        }
        z = block_sum(z, red_f);
        const float scale = 1099511627776.0f / z;           // 2^40 / Z
        unsigned int prefix = 0u, mask = 0u;
        if (tid == 0) sh_remaining = static_cast<unsigned long long>(static_cast<double>(p_top) * 1099511627776.0);
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) hist[tid] = 0ull;
            __syncthreads();
            for (int i = tid; i < V; i += kSampleThreads) {
                const float v = x.at(i);
                const unsigned int key = float_key(v);
                if (key >= key_floor && (key & mask) == prefix)
                    atomicAdd(&hist[(key >> shift) & 255u],
                              static_cast<unsigned long long>(expf(v - row_max) * scale));
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long rem = sh_remaining;
                int digit = -1, lowest = 0;
                for (int b = 255; b >= 0; --b) {
                    if (hist[b] == 0ull) continue;
                    lowest = b;
                    if (hist[b] > rem) { digit = b; break; }   // inclusive mass passes top_p here
                    rem -= hist[b];
                }
                if (digit < 0) { digit = lowest; rem = 0ull; }  // rounding: everything is kept
                sh_remaining = rem;
                sh_prefix = prefix | (static_cast<unsigned int>(digit) << shift);
            }
            __syncthreads();
            prefix = sh_prefix;
            mask |= 255u << shift;
        }
        if (prefix > key_floor) key_floor = prefix;
    }

    // ---- total mass of what is left, then the inverse-CDF walk in index order
    float z = 0.f;
    for (int i = tid; i < V; i += kSampleThreads) {
        const float v = x.at(i);
        if (float_key(v) >= key_floor) z += expf(v - row_max);
    }
    z = block_sum(z, red_f);
    const float target = uniform_from(seed[row], counter[row]) * z;
    if (tid == 0) { sh_total = 0.f; sh_found = 0x7fffffff; }
    __syncthreads();
    int last_kept = -1;
    for (int base = 0; base < V; base += kSampleThreads) {
        const int i = base + tid;
        float w = 0.f;
        if (i < V) {
            const float v = x.at(i);
            if (float_key(v) >= key_floor) { w = expf(v - row_max); last_kept = i; }
        }
        float incl = w;                       // inclusive scan over the block
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        if (lane == 31) red_f[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            float t = red_f[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float n = __shfl_up_sync(0xffffffffu, t, o);
                if (lane >= o) t += n;
            }
            red_f[lane] = t;
        }
        __syncthreads();
        const float before = sh_total + (warp > 0 ? red_f[warp - 1] : 0.f);
        if (w > 0.f && before + incl > target) atomicMin(&sh_found, i);
        __syncthreads();
        if (sh_found != 0x7fffffff) break;
        if (tid == 0) sh_total += red_f[31];
        __syncthreads();
    }
    if (sh_found != 0x7fffffff) {
        if (tid == 0) out[row] = sh_found;
        return;
    }
    // rounding left the target at or beyond the total: the last kept token
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) last_kept = max(last_kept, __shfl_xor_sync(0xffffffffu, last_kept, o));
    if (lane == 0) red_i[warp] = last_kept;
    __syncthreads();
    if (tid == 0) {
        int m = -1;
        for (int w = 0; w < kSampleThreads / 32; ++w) m = max(m, red_i[w]);
        out[row] = m < 0 ? 0 : m;
    }
}

}  // namespace somi

using namespace somi;

SOMI_API float somi_sample_uniform(unsigned long long seed, unsigned int counter) {
    return uniform_from(seed, counter);
}

SOMI_API int somi_sample(const float* logits, int rows, int V, const float* temperature,
                         const int* top_k, const float* top_p, const float* penalty,
                         const unsigned long long* seed, const unsigned int* counter,
                         const int* hist_off, const int* hist_tok, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = static_cast<size_t>((V + 31) / 32) * sizeof(unsigned int);
    if (smem > 160 * 1024) return SOMI_ERR_UNSUPPORTED;      // vocabularies beyond 1.3 M tokens
    if (smem > 40 * 1024)
        cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(sample_kernel, dim3(rows), dim3(kSampleThreads), smem, stream, logits, V, temperature, top_k, top_p,
                                                         penalty, seed, counter, hist_off,
                                                         hist_tok, out);
    return launch_status();
}
