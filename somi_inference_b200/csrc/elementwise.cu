// Memory-bound kernels of a decoder step: embedding gather, residual sum fused
// with RMS normalisation, rotary encoding fused with the cache write, SiLU(gate)*up.
// All arithmetic is float32; inputs and outputs are float32 or bfloat16.

#include "common.cuh"

namespace somi {

// Four consecutive elements at once (16 bytes of float32, 8 bytes of bfloat16).
struct F4 { float v[4]; };
__device__ __forceinline__ F4 load4(const float* p) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    return F4{{t.x, t.y, t.z, t.w}};
}
__device__ __forceinline__ F4 load4(const __nv_bfloat16* p) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    return F4{{__low2float(a), __high2float(a), __low2float(b), __high2float(b)}};
}
__device__ __forceinline__ void store4(float* p, const F4& f) {
    *reinterpret_cast<float4*>(p) = make_float4(f.v[0], f.v[1], f.v[2], f.v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const F4& f) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f.v[0], f.v[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(f.v[2], f.v[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}
struct F2 { float x, y; };
__device__ __forceinline__ F2 load2(const float* p) {
    const float2 t = *reinterpret_cast<const float2*>(p);
    return F2{t.x, t.y};
}
__device__ __forceinline__ F2 load2(const __nv_bfloat16* p) {
    const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(p);
    return F2{__low2float(t), __high2float(t)};
}
__device__ __forceinline__ void store2(float* p, float x, float y) {
    *reinterpret_cast<float2*>(p) = make_float2(x, y);
}
__device__ __forceinline__ void store2(__nv_bfloat16* p, float x, float y) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y);
}
__device__ __forceinline__ F4 load4_any(const void* p, int dtype, size_t i) {
    return dtype == SOMI_F32 ? load4(reinterpret_cast<const float*>(p) + i)
                             : load4(reinterpret_cast<const __nv_bfloat16*>(p) + i);
}

// ---------------------------------------------------------------- embedding
// out[t, :] = float(table[ids[t], :])
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = table + static_cast<size_t>(ids[t]) * H;
    float* o = out + static_cast<size_t>(t) * H;
    if ((H & 3) == 0) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) store4(o + i, load4(row + i));
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

// ------------------------------------------------------ residual + RMS norm
// r = residual[row] (+ delta[row]); if write_back: residual[row] = r;
// out[b] = r / sqrt(mean(r^2) + eps) * weight, where row = rows ? rows[b] : b.
// The row is kept in shared memory (H floats) between the two passes.
// `delta` may be `splits` partial sums (float32 only) that lie `split_stride` elements apart; they
// are added in order, so the result does not depend on how the producer was scheduled.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   int splits, long long split_stride,
                                   const void* __restrict__ weight, int weight_dtype, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int H,
                                   int write_back) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    // the norm's weight is written by no kernel [constant]: a thread's first four columns are
    // fetched while the kernel before this one finishes
    F4 w_first = F4{{0.f, 0.f, 0.f, 0.f}};
    if ((H & 3) == 0 && threadIdx.x * 4 < H) w_first = load4_any(weight, weight_dtype, threadIdx.x * 4);
    pdl_wait();
    const int b = blockIdx.x;
    const size_t row = rows ? static_cast<size_t>(rows[b]) : static_cast<size_t>(b);
    float* r = residual + row * H;
    const TD* d = delta ? delta + row * H : nullptr;
    float ss = 0.f;
    TO* o = out + static_cast<size_t>(b) * H;
    if ((H & 3) == 0 && splits == 1 && H <= static_cast<int>(blockDim.x) * 16) {
        // Up to four vectors a thread and one delta: every load of the row is issued before the
        // first result is needed (a loop would wait for each vector's round trip in turn).
        F4 v[4];
        const int step = blockDim.x * 4;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x * 4 + k * step;
            if (i < H) v[k] = load4(r + i);
        }
        if (d) {
            F4 dv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = threadIdx.x * 4 + k * step;
                if (i < H) dv[k] = load4(d + i);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = threadIdx.x * 4 + k * step;
                if (i < H) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[k].v[e] += dv[k].v[e];
                    if (write_back) store4(r + i, v[k]);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x * 4 + k * step;
            if (i < H) {
#pragma unroll
                for (int e = 0; e < 4; ++e) ss += v[k].v[e] * v[k].v[e];
            }
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x * 4 + k * step;
            if (i < H) {
                const F4 w = k == 0 ? w_first : load4_any(weight, weight_dtype, i);
                F4 y;
#pragma unroll
                for (int e = 0; e < 4; ++e) y.v[e] = v[k].v[e] * inv * w.v[e];
                store4(o + i, y);
            }
        }
        return;
    }
    if ((H & 3) == 0) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            F4 v = load4(r + i);
            if (d) {
#pragma unroll 4
                for (int sp = 0; sp < splits; ++sp) {
                    const F4 dv = load4(d + sp * split_stride + i);
#pragma unroll
                    for (int k = 0; k < 4; ++k) v.v[k] += dv.v[k];
                }
                if (write_back) store4(r + i, v);
            }
            store4(row_buf + i, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) ss += v.v[k] * v.v[k];
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            F4 v = load4(row_buf + i);
            const F4 w = i == threadIdx.x * 4 ? w_first : load4_any(weight, weight_dtype, i);
#pragma unroll
            for (int k = 0; k < 4; ++k) v.v[k] = v.v[k] * inv * w.v[k];
            store4(o + i, v);
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (d)
            for (int sp = 0; sp < splits; ++sp) v += to_float(d[sp * split_stride + i]);
        if (write_back && d) r[i] = v;
        row_buf[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
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
    pdl_launch_dependents();
    // positions and slots [descriptor] and frequencies [constant] are written by no kernel of
    // the step: the angles are ready when the projection is
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const float pos = static_cast<float>(ld_step(positions + t));
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    const int slot = slot_map ? ld_step(slot_map + t) : -1;
    pdl_wait();
    __syncthreads();
    T* row = qkv + static_cast<size_t>(t) * (nq + 2 * nkv) * hd;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    // queries and keys: rotated pairs (two neighbouring pairs per thread where sizes allow)
    if ((half & 1) == 0 && (hd & 1) == 0) {
        const int hp = half >> 1;
        for (int idx = threadIdx.x; idx < (nq + nkv) * hp; idx += blockDim.x) {
            const int head = idx / hp, i = (idx - head * hp) << 1;
            T* x = row + static_cast<size_t>(head) * hd;
            const F2 a = load2(x + i), b = load2(x + i + half);
            const float c0 = cs[i], c1 = cs[i + 1], s0 = cs[half + i], s1 = cs[half + i + 1];
            const float o1x = rope_lo(a.x, b.x, c0, s0), o1y = rope_lo(a.y, b.y, c1, s1);
            const float o2x = rope_hi(a.x, b.x, c0, s0), o2y = rope_hi(a.y, b.y, c1, s1);
            store2(x + i, o1x, o1y);
            store2(x + i + half, o2x, o2y);
            if (slot >= 0 && head >= nq) {
                T* kc = kcache + ((static_cast<size_t>(page) * nkv + (head - nq)) * page_size + off) * hd;
                store2(kc + i, o1x, o1y);
                store2(kc + i + half, o2x, o2y);
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < (nq + nkv) * half; idx += blockDim.x) {
            const int head = idx / half, i = idx - head * half;
            T* x = row + static_cast<size_t>(head) * hd;
            const float a = to_float(x[i]), b = to_float(x[i + half]);
            const float c = cs[i], s = cs[half + i];
            const T o1 = from_float<T>(rope_lo(a, b, c, s));
            const T o2 = from_float<T>(rope_hi(a, b, c, s));
            x[i] = o1;
            x[i + half] = o2;
            if (slot >= 0 && head >= nq) {
                T* kc = kcache + ((static_cast<size_t>(page) * nkv + (head - nq)) * page_size + off) * hd;
                kc[i] = o1;
                kc[i + half] = o2;
            }
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
    if ((hd & 3) == 0) {
        const int q4 = hd >> 2;
        for (int idx = threadIdx.x; idx < nkv * q4; idx += blockDim.x) {
            const int head = idx / q4, i = (idx - head * q4) << 2;
            store4(vcache + ((static_cast<size_t>(page) * nkv + head) * page_size + off) * hd + i,
                   load4(v + head * hd + i));
        }
        return;
    }
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        const int head = idx / hd, i = idx - head * hd;
        vcache[((static_cast<size_t>(page) * nkv + head) * page_size + off) * hd + i] = v[idx];
    }
}

// The bfloat16 case for many tokens: four tokens per CTA (one, while that still leaves fewer
// CTAs than four per SM: steps of a few dozen decode tokens), 16-byte accesses.
// A work item is 8 consecutive dims of one head: a rotated pair of 8-dim groups (i, i + rot/2)
// of a query or key head, 8 unrotated key dims, or 8 value dims.  Needs rot/2, hd - rot and hd
// to be multiples of 8 and 16-byte aligned rows.
constexpr int kRopeToks = 4;
__device__ __forceinline__ void unpack8(const uint4& r, float (&f)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        f[2 * k] = __uint_as_float(w[k] << 16);
        f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
        w[k] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__global__ void __launch_bounds__(256)
rope_store_bf16x8_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                         const float* __restrict__ inv_freq, int T, int nq, int nkv, int hd, int rot,
                         const int* __restrict__ slot_map, __nv_bfloat16* __restrict__ kcache,
                         __nv_bfloat16* __restrict__ vcache, int page_size, int toks_per_cta) {
    extern __shared__ float cs[];                 // per token: cos[rot/2], sin[rot/2]
    __shared__ int slot_s[kRopeToks];
    pdl_launch_dependents();
    // before the wait: positions and slots [descriptor], frequencies [constant]
    const int t0 = blockIdx.x * toks_per_cta;
    const int n_tok = min(toks_per_cta, T - t0);
    const int half = rot >> 1;
    for (int idx = threadIdx.x; idx < n_tok * half; idx += blockDim.x) {
        const int tt = idx / half, i = idx - tt * half;
        float sn, c;
        sincosf(static_cast<float>(ld_step(positions + t0 + tt)) * inv_freq[i], &sn, &c);
        cs[tt * rot + i] = c;
        cs[tt * rot + half + i] = sn;
    }
    if (threadIdx.x < n_tok) slot_s[threadIdx.x] = slot_map ? ld_step(slot_map + t0 + threadIdx.x) : -1;
    pdl_wait();
    __syncthreads();
    const int width = (nq + 2 * nkv) * hd;
    const int g_rot = half >> 3, g_tail = (hd - rot) >> 3, g_v = hd >> 3;
    const int n_rot = (nq + nkv) * g_rot;               // rotated pairs of the q and k heads
    const int n_qtail = 0;                              // unrotated query dims stay where they are
    const int n_ktail = nkv * g_tail, n_val = nkv * g_v;
    const int per_tok = n_rot + n_qtail + n_ktail + n_val;
    for (int idx = threadIdx.x; idx < n_tok * per_tok; idx += blockDim.x) {
        const int tt = idx / per_tok;
        int w = idx - tt * per_tok;
        __nv_bfloat16* row = qkv + static_cast<size_t>(t0 + tt) * width;
        const int slot = slot_s[tt];
        const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
        if (w < n_rot) {
            const int head = w / g_rot, i = (w - head * g_rot) << 3;
            __nv_bfloat16* x = row + static_cast<size_t>(head) * hd;
            float a[8], b[8], o1[8], o2[8];
            unpack8(*reinterpret_cast<const uint4*>(x + i), a);
            unpack8(*reinterpret_cast<const uint4*>(x + i + half), b);
            const float* c = cs + tt * rot + i;
            const float* sn = c + half;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                o1[k] = rope_lo(a[k], b[k], c[k], sn[k]);
                o2[k] = rope_hi(a[k], b[k], c[k], sn[k]);
            }
            const uint4 r1 = pack8(o1), r2 = pack8(o2);
            *reinterpret_cast<uint4*>(x + i) = r1;
            *reinterpret_cast<uint4*>(x + i + half) = r2;
            if (slot >= 0 && head >= nq) {
                __nv_bfloat16* kc = kcache + ((static_cast<size_t>(page) * nkv + (head - nq)) * page_size + off) * hd;
                *reinterpret_cast<uint4*>(kc + i) = r1;
                *reinterpret_cast<uint4*>(kc + i + half) = r2;
            }
            continue;
        }
        if (slot < 0) continue;
        w -= n_rot;
        if (w < n_ktail) {
            const int head = w / g_tail, i = rot + ((w - head * g_tail) << 3);
            *reinterpret_cast<uint4*>(kcache + ((static_cast<size_t>(page) * nkv + head) * page_size + off) * hd + i) =
                *reinterpret_cast<const uint4*>(row + static_cast<size_t>(nq + head) * hd + i);
            continue;
        }
        w -= n_ktail;
        const int head = w / g_v, i = (w - head * g_v) << 3;
        *reinterpret_cast<uint4*>(vcache + ((static_cast<size_t>(page) * nkv + head) * page_size + off) * hd + i) =
            *reinterpret_cast<const uint4*>(row + static_cast<size_t>(nq + nkv + head) * hd + i);
    }
}

// The same, reading the projection as `splits` float32 partial sums [splits][T][(nq+2nkv)*hd]
// (what a split-K product leaves) plus a bias: sums them in order, rotates, writes the queries
// to `q_out` rows (bfloat16, same row layout as qkv) and keys/values to the cache only.
__global__ void rope_store_partial_kernel(const float* __restrict__ parts, int splits,
                                          long long split_stride, const void* __restrict__ bias,
                                          int bias_dtype, __nv_bfloat16* __restrict__ q_out,
                                          const int* __restrict__ positions,
                                          const float* __restrict__ inv_freq, int nq, int nkv,
                                          int hd, int rot, const int* __restrict__ slot_map,
                                          __nv_bfloat16* __restrict__ kcache,
                                          __nv_bfloat16* __restrict__ vcache, int page_size,
                                          int heads_per_cta) {
    extern __shared__ float cs[];
    pdl_launch_dependents();
    // before the wait: positions and slots [descriptor], frequencies [constant]
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const int width = (nq + 2 * nkv) * hd;
    const float pos = static_cast<float>(ld_step(positions + t));
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    const int slot = slot_map ? ld_step(slot_map + t) : -1;
    pdl_wait();             // the partial sums (and the bias add) come after it
    __syncthreads();
    const float* prow = parts + static_cast<size_t>(t) * width;
    auto value = [&](int col) {
        float v = bias ? load_as_float(bias, bias_dtype, col) : 0.f;
        for (int sp = 0; sp < splits; ++sp) v += prow[sp * split_stride + col];
        return v;
    };
    auto value4 = [&](int col) {          // four consecutive columns
        F4 v = bias ? load4_any(bias, bias_dtype, col) : F4{{0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
        for (int sp = 0; sp < splits; ++sp) {
            const F4 p = load4(prow + sp * split_stride + col);
#pragma unroll
            for (int k = 0; k < 4; ++k) v.v[k] += p.v[k];
        }
        return v;
    };
    __nv_bfloat16* qrow = q_out + static_cast<size_t>(t) * width;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    // this CTA's share of the nq + 2 nkv heads (queries, keys, values in that order)
    const int h0 = blockIdx.y * heads_per_cta, h1 = min(nq + 2 * nkv, h0 + heads_per_cta);
    const int rot_end = min(h1, slot >= 0 ? nq + nkv : nq);    // keys matter only if they are stored
    const int n_rot = max(0, rot_end - h0);
    if ((half & 3) == 0 && (hd & 3) == 0) {
        const int hq = half >> 2;
        for (int idx = threadIdx.x; idx < n_rot * hq; idx += blockDim.x) {
            const int head = h0 + idx / hq, i = (idx % hq) << 2;
            const F4 a = value4(head * hd + i), b = value4(head * hd + i + half);
            F4 o1, o2;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float c = cs[i + k], s = cs[half + i + k];
                o1.v[k] = rope_lo(a.v[k], b.v[k], c, s);
                o2.v[k] = rope_hi(a.v[k], b.v[k], c, s);
            }
            __nv_bfloat16* dst = head < nq
                ? qrow + head * hd
                : kcache + ((static_cast<size_t>(page) * nkv + (head - nq)) * page_size + off) * hd;
            store4(dst + i, o1);
            store4(dst + i + half, o2);
        }
        const int tail4 = (hd - rot) >> 2;
        for (int idx = threadIdx.x; idx < n_rot * tail4; idx += blockDim.x) {
            const int head = h0 + idx / tail4, i = rot + ((idx % tail4) << 2);
            __nv_bfloat16* dst = head < nq
                ? qrow + head * hd
                : kcache + ((static_cast<size_t>(page) * nkv + (head - nq)) * page_size + off) * hd;
            store4(dst + i, value4(head * hd + i));
        }
        if (slot < 0) return;
        const int v0 = max(h0, nq + nkv), q4 = hd >> 2;
        for (int idx = threadIdx.x; idx < max(0, h1 - v0) * q4; idx += blockDim.x) {
            const int head = v0 + idx / q4 - (nq + nkv), i = (idx % q4) << 2;
            store4(vcache + ((static_cast<size_t>(page) * nkv + head) * page_size + off) * hd + i,
                   value4((nq + nkv + head) * hd + i));
        }
        return;
    }
    for (int idx = threadIdx.x; idx < n_rot * half; idx += blockDim.x) {
        const int head = h0 + idx / half, i = idx % half;
        const float a = value(head * hd + i), b = value(head * hd + i + half);
        const float c = cs[i], s = cs[half + i];
        const __nv_bfloat16 o1 = __float2bfloat16_rn(rope_lo(a, b, c, s));
        const __nv_bfloat16 o2 = __float2bfloat16_rn(rope_hi(a, b, c, s));
        if (head < nq) {
            qrow[head * hd + i] = o1;
            qrow[head * hd + i + half] = o2;
        } else {
            __nv_bfloat16* kc = kcache + ((static_cast<size_t>(page) * nkv + (head - nq)) * page_size + off) * hd;
            kc[i] = o1;
            kc[i + half] = o2;
        }
    }
    const int tail = hd - rot;
    for (int idx = threadIdx.x; idx < n_rot * tail; idx += blockDim.x) {
        const int head = h0 + idx / tail, i = rot + idx % tail;
        const __nv_bfloat16 o = __float2bfloat16_rn(value(head * hd + i));
        if (head < nq) qrow[head * hd + i] = o;
        else kcache[((static_cast<size_t>(page) * nkv + (head - nq)) * page_size + off) * hd + i] = o;
    }
    if (slot < 0) return;
    const int v0 = max(h0, nq + nkv);
    for (int idx = threadIdx.x; idx < max(0, h1 - v0) * hd; idx += blockDim.x) {
        const int head = v0 + idx / hd - (nq + nkv), i = idx % hd;
        vcache[((static_cast<size_t>(page) * nkv + head) * page_size + off) * hd + i] =
            __float2bfloat16_rn(value((nq + nkv + head) * hd + i));
    }
}

// ------------------------------------------------------------- SiLU * up
// out[t, i] = silu(gate) * up,  silu(z) = z / (1 + exp(-z)).
// `interleaved`: gate and up alternate along the row (g0, u0, g1, u1, ...) instead of lying in
// two halves; that is how a product over row-interleaved gate/up weights comes out.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t n,
                                int interleaved) {
    pdl_launch_dependents();
    pdl_wait();
    if ((I & 3) == 0) {
        const size_t n4 = n >> 2;
        const int I4 = I >> 2;
        for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n4;
             idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
            const size_t t = idx / I4, i = (idx - t * I4) << 2;
            F4 g, u;
            if (interleaved) {
                const F4 a = load4(gu + t * 2 * I + 2 * i), b = load4(gu + t * 2 * I + 2 * i + 4);
                g = F4{{a.v[0], a.v[2], b.v[0], b.v[2]}};
                u = F4{{a.v[1], a.v[3], b.v[1], b.v[3]}};
            } else {
                g = load4(gu + t * 2 * I + i);
                u = load4(gu + t * 2 * I + I + i);
            }
            F4 r;
#pragma unroll
            for (int k = 0; k < 4; ++k) r.v[k] = g.v[k] / (1.0f + expf(-g.v[k])) * u.v[k];
            store4(out + t * I + i, r);
        }
        return;
    }
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = idx / I, i = idx - t * I;
        const float g = to_float(gu[t * 2 * I + (interleaved ? 2 * i : i)]);
        const float u = to_float(gu[t * 2 * I + (interleaved ? 2 * i + 1 : I + i)]);
        out[idx] = from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

// The bfloat16 case with I a multiple of 8: a thread reads 32 bytes (8 gate and 8 up values),
// writes 16, one row of the grid per token, no index division; exp and the division are the
// fast float32 forms, whose error is far below a bfloat16 step.
template <int INTERLEAVED>
__global__ void __launch_bounds__(256)
silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= I) return;
    const __nv_bfloat16* row = gu + t * 2 * I;
    uint4 a, b;
    if (INTERLEAVED) {
        a = *reinterpret_cast<const uint4*>(row + 2 * i);
        b = *reinterpret_cast<const uint4*>(row + 2 * i + 8);
    } else {
        a = *reinterpret_cast<const uint4*>(row + i);
        b = *reinterpret_cast<const uint4*>(row + I + i);
    }
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    float g[8], u[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        // a bfloat16 is the upper half of the float32 with the same value
        const float a_lo = __uint_as_float(aw[k] << 16), a_hi = __uint_as_float(aw[k] & 0xffff0000u);
        const float b_lo = __uint_as_float(bw[k] << 16), b_hi = __uint_as_float(bw[k] & 0xffff0000u);
        if (INTERLEAVED) {
            g[k] = a_lo; u[k] = a_hi; g[4 + k] = b_lo; u[4 + k] = b_hi;
        } else {
            g[2 * k] = a_lo; g[2 * k + 1] = a_hi; u[2 * k] = b_lo; u[2 * k + 1] = b_hi;
        }
    }
    uint32_t r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float x = __fdividef(g[2 * k], 1.0f + __expf(-g[2 * k])) * u[2 * k];
        const float y = __fdividef(g[2 * k + 1], 1.0f + __expf(-g[2 * k + 1])) * u[2 * k + 1];
        const __nv_bfloat162 p = __floats2bfloat162_rn(x, y);
        r[k] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + t * I + i) = make_uint4(r[0], r[1], r[2], r[3]);
}

}  // namespace somi

using namespace somi;

// Switches programmatic dependent launch on (default) or off for every kernel of the library.
SOMI_API void somi_set_pdl(int on) { pdl_enabled() = on ? 1 : 0; }

SOMI_API int somi_embed(const int* ids, const void* table, int dtype, float* out, int T, int H,
                        cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == SOMI_F32)
        launch_pdl(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, ids, static_cast<const float*>(table), out, H);
    else
        launch_pdl(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, 
            ids, static_cast<const __nv_bfloat16*>(table), out, H);
    return launch_status();
}

SOMI_API int somi_add_rmsnorm(float* residual, const void* delta, int delta_dtype,
                              int delta_splits, long long delta_split_stride, const void* weight, int weight_dtype, float eps, void* out,
                              int out_dtype, const int* rows, int n_out, int H, int write_back,
                              cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (delta_splits < 1 || (delta_splits > 1 && delta_dtype != SOMI_F32)) return SOMI_ERR_UNSUPPORTED;
    const size_t smem = static_cast<size_t>(H) * sizeof(float);
    if (smem > 200 * 1024) return SOMI_ERR_UNSUPPORTED;
    // Few rows (a decode step): the step waits for this kernel, so a row is read in one pass with a
    // thread per four columns.  (A thread-block cluster per row, with the sum of squares through
    // distributed shared memory, was slower: its two cluster barriers cost more than they saved.)
    // Many rows: fewer threads per row, more rows per SM.
    int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    // (rows that add up split-K partial sums read `splits` times as much: they keep the one-pass
    // form while there is at most a CTA per SM or two, so that every load of a row is in flight
    // at once)
    if ((n_out <= 32 || (delta_splits > 1 && n_out <= 256)) && (H & 3) == 0)
        threads = min(1024, ((H / 4 + 31) / 32) * 32);
#define SOMI_LAUNCH_NORM(TD, TO)                                                                 \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        launch_pdl(add_rmsnorm_kernel<TD, TO>, dim3(n_out), dim3(threads), smem, stream,         \
            residual, static_cast<const TD*>(delta), delta_splits, delta_split_stride, weight,   \
            weight_dtype, eps,                                                                   \
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
    const auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (dtype == SOMI_BF16 && T > 32 && rot > 0 && (rot & 15) == 0 && ((hd - rot) & 7) == 0 &&
        (hd & 7) == 0 && aligned16(qkv) && aligned16(kcache) && aligned16(vcache)) {
        const int toks = T <= 4 * 148 ? 1 : kRopeToks;
        launch_pdl(rope_store_bf16x8_kernel, dim3((T + toks - 1) / toks), dim3(256),
                   smem * toks, stream, static_cast<__nv_bfloat16*>(qkv), positions, inv_freq, T,
                   nq, nkv, hd, rot, slot_map, static_cast<__nv_bfloat16*>(kcache),
                   static_cast<__nv_bfloat16*>(vcache), page_size, toks);
        return launch_status();
    }
    if (dtype == SOMI_F32)
        launch_pdl(rope_store_kernel<float>, dim3(T), dim3(256), smem, stream, 
            static_cast<float*>(qkv), positions, inv_freq, nq, nkv, hd, rot, slot_map,
            static_cast<float*>(kcache), static_cast<float*>(vcache), page_size);
    else
        launch_pdl(rope_store_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, 
            static_cast<__nv_bfloat16*>(qkv), positions, inv_freq, nq, nkv, hd, rot, slot_map,
            static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), page_size);
    return launch_status();
}

SOMI_API int somi_rope_store_partial(const float* parts, int splits, long long split_stride,
                                     const void* bias, int bias_dtype, void* q_out,
                                     const int* positions, const float* inv_freq, int T, int nq,
                                     int nkv, int hd, int rot, const int* slot_map, void* kcache,
                                     void* vcache, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > hd || (rot & 1) || splits < 1) return SOMI_ERR_UNSUPPORTED;
    const size_t smem = static_cast<size_t>(rot > 0 ? rot : 2) * sizeof(float);
    // a token's heads are spread over several CTAs: few tokens would otherwise use few SMs
    const int heads_per_cta = T > 32 ? nq + 2 * nkv : 4;
    const int chunks = (nq + 2 * nkv + heads_per_cta - 1) / heads_per_cta;
    launch_pdl(rope_store_partial_kernel, dim3(T, chunks), dim3(128), smem, stream,
        parts, splits, split_stride, bias, bias_dtype, static_cast<__nv_bfloat16*>(q_out),
        positions, inv_freq, nq, nkv, hd, rot, slot_map, static_cast<__nv_bfloat16*>(kcache),
        static_cast<__nv_bfloat16*>(vcache), page_size, heads_per_cta);
    return launch_status();
}

SOMI_API int somi_silu_mul(const void* gu, void* out, int dtype, long long T, int I,
                           int interleaved, cudaStream_t stream) {
    const size_t n = static_cast<size_t>(T) * I;
    if (n == 0) return 0;
    if (dtype == SOMI_BF16 && (I & 7) == 0 && T <= 65535 &&
        (reinterpret_cast<uintptr_t>(gu) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        const dim3 grid((I / 8 + 255) / 256, static_cast<unsigned>(T));
        if (interleaved)
            launch_pdl(silu_mul_bf16x8_kernel<1>, grid, dim3(256), 0, stream,
                       static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), I);
        else
            launch_pdl(silu_mul_bf16x8_kernel<0>, grid, dim3(256), 0, stream,
                       static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), I);
        return launch_status();
    }
    const int threads = 256;
    const size_t work = (I & 3) == 0 ? n / 4 : n;
    const int blocks = static_cast<int>(work / threads + 1 < 148 * 16 ? work / threads + 1 : 148 * 16);
    if (dtype == SOMI_F32)
        launch_pdl(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, 
            static_cast<const float*>(gu), static_cast<float*>(out), I, n, interleaved);
    else
        launch_pdl(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, 
            static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), I, n, interleaved);
    return launch_status();
}
