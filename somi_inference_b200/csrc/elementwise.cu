// Memory-bound kernels of a decoder step: embedding gather, residual sum fused
// with RMS normalisation, rotary encoding fused with the cache write, SiLU(gate)*up.
// All arithmetic is float32; inputs and outputs are float32 or bfloat16.
#include "common.cuh"

namespace somi {

// ---------------------------------------------------------------- embedding
// out[t, :] = float(table[ids[t], :])
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out, int H) {
    const int t = blockIdx.x;
    const T* row = table + static_cast<size_t>(ids[t]) * H;
    float* o = out + static_cast<size_t>(t) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

// ------------------------------------------------------ residual + RMS norm
// r = residual[row] (+ delta[row]); if write_back: residual[row] = r;
// out[b] = r / sqrt(mean(r^2) + eps) * weight, where row = rows ? rows[b] : b.
// The row is kept in shared memory (H floats) between the two passes.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const void* __restrict__ weight, int weight_dtype, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int H,
                                   int write_back) {
    extern __shared__ float row_buf[];
    __shared__ float scratch[33];
    const int b = blockIdx.x;
    const size_t row = rows ? static_cast<size_t>(rows[b]) : static_cast<size_t>(b);
    float* r = residual + row * H;
    const TD* d = delta ? delta + row * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (d) v += to_float(d[i]);
        if (write_back && d) r[i] = v;
        row_buf[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
    TO* o = out + static_cast<size_t>(b) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_float<TO>(row_buf[i] * inv * load_as_float(weight, weight_dtype, i));
}

// ------------------------------------------- rotary encoding + cache write
// qkv: [T, (nq + 2 nkv) * hd].  For every token: rotate the first `rot` dims of
// each query and key head by angle = position * inv_freq[i] (pairs i, i + rot/2),
// write q and k back in place, and, if slot_map is given, write k (rotated) and
// v to cache[page][kv_head][offset][:], slot = page * page_size + offset.
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int nq, int nkv, int hd,
                                  int rot, const int* __restrict__ slot_map,
                                  T* __restrict__ kcache, T* __restrict__ vcache, int page_size) {
    extern __shared__ float cs[];   // cos[rot/2], sin[rot/2]
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const float pos = static_cast<float>(positions[t]);
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    __syncthreads();
    T* row = qkv + static_cast<size_t>(t) * (nq + 2 * nkv) * hd;
    const int slot = slot_map ? slot_map[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    // queries and keys: rotated pairs
    for (int idx = threadIdx.x; idx < (nq + nkv) * half; idx += blockDim.x) {
        const int head = idx / half, i = idx - head * half;
        T* x = row + static_cast<size_t>(head) * hd;
        const float a = to_float(x[i]), b = to_float(x[i + half]);
        const float c = cs[i], s = cs[half + i];
        const T o1 = from_float<T>(a * c - b * s);
        const T o2 = from_float<T>(b * c + a * s);
        x[i] = o1;
        x[i + half] = o2;
        if (slot >= 0 && head >= nq) {
            T* kc = kcache + ((static_cast<size_t>(page) * nkv + (head - nq)) * page_size + off) * hd;
            kc[i] = o1;
            kc[i + half] = o2;
        }
    }
    if (slot < 0) return;
    // key dims beyond the rotated part, and the values
    const int tail = hd - rot;
    for (int idx = threadIdx.x; idx < nkv * tail; idx += blockDim.x) {
        const int head = idx / tail, i = rot + (idx - head * tail);
        kcache[((static_cast<size_t>(page) * nkv + head) * page_size + off) * hd + i] =
            row[static_cast<size_t>(nq + head) * hd + i];
    }
    const T* v = row + static_cast<size_t>(nq + nkv) * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        const int head = idx / hd, i = idx - head * hd;
        vcache[((static_cast<size_t>(page) * nkv + head) * page_size + off) * hd + i] = v[idx];
    }
}

// ------------------------------------------------------------- SiLU * up
// out[t, i] = silu(gu[t, i]) * gu[t, I + i],  silu(z) = z / (1 + exp(-z))
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t n) {
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = idx / I, i = idx - t * I;
        const float g = to_float(gu[t * 2 * I + i]);
        const float u = to_float(gu[t * 2 * I + I + i]);
        out[idx] = from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_embed(const int* ids, const void* table, int dtype, float* out, int T, int H,
                        cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == SOMI_F32)
        embed_kernel<float><<<T, threads, 0, stream>>>(ids, static_cast<const float*>(table), out, H);
    else
        embed_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
            ids, static_cast<const __nv_bfloat16*>(table), out, H);
    return launch_status();
}

SOMI_API int somi_add_rmsnorm(float* residual, const void* delta, int delta_dtype,
                              const void* weight, int weight_dtype, float eps, void* out,
                              int out_dtype, const int* rows, int n_out, int H, int write_back,
                              cudaStream_t stream) {
    if (n_out <= 0) return 0;
    const size_t smem = static_cast<size_t>(H) * sizeof(float);
    if (smem > 200 * 1024) return SOMI_ERR_UNSUPPORTED;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define SOMI_LAUNCH_NORM(TD, TO)                                                                 \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        add_rmsnorm_kernel<TD, TO><<<n_out, threads, smem, stream>>>(                            \
            residual, static_cast<const TD*>(delta), weight, weight_dtype, eps,                  \
            static_cast<TO*>(out), rows, H, write_back);                                         \
    } while (0)
    if (delta_dtype == SOMI_F32 && out_dtype == SOMI_F32) SOMI_LAUNCH_NORM(float, float);
    else if (delta_dtype == SOMI_BF16 && out_dtype == SOMI_BF16) SOMI_LAUNCH_NORM(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == SOMI_F32 && out_dtype == SOMI_BF16) SOMI_LAUNCH_NORM(float, __nv_bfloat16);
    else SOMI_LAUNCH_NORM(__nv_bfloat16, float);
#undef SOMI_LAUNCH_NORM
    return launch_status();
}

SOMI_API int somi_rope_store(void* qkv, int dtype, const int* positions, const float* inv_freq,
                             int T, int nq, int nkv, int hd, int rot, const int* slot_map,
                             void* kcache, void* vcache, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > hd || (rot & 1)) return SOMI_ERR_UNSUPPORTED;
    const size_t smem = static_cast<size_t>(rot > 0 ? rot : 2) * sizeof(float);
    if (dtype == SOMI_F32)
        rope_store_kernel<float><<<T, 256, smem, stream>>>(
            static_cast<float*>(qkv), positions, inv_freq, nq, nkv, hd, rot, slot_map,
            static_cast<float*>(kcache), static_cast<float*>(vcache), page_size);
    else
        rope_store_kernel<__nv_bfloat16><<<T, 256, smem, stream>>>(
            static_cast<__nv_bfloat16*>(qkv), positions, inv_freq, nq, nkv, hd, rot, slot_map,
            static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), page_size);
    return launch_status();
}

SOMI_API int somi_silu_mul(const void* gu, void* out, int dtype, long long T, int I,
                           cudaStream_t stream) {
    const size_t n = static_cast<size_t>(T) * I;
    if (n == 0) return 0;
    const int threads = 256;
    const int blocks = static_cast<int>(n / threads + 1 < 148 * 16 ? n / threads + 1 : 148 * 16);
    if (dtype == SOMI_F32)
        silu_mul_kernel<float><<<blocks, threads, 0, stream>>>(
            static_cast<const float*>(gu), static_cast<float*>(out), I, n);
    else
        silu_mul_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), I, n);
    return launch_status();
}
