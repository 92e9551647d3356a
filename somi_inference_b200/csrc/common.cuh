// Shared helpers for the sm_100a kernels of this library.
//
// Every exported launcher is `extern "C"`, takes raw device pointers, sizes and
// the stream, launches on that stream and returns the cudaError_t of the launch
// as an int (0 = success).  Floating tensors come with a dtype code:
// 0 = float32, 1 = bfloat16.  Sizes that a kernel cannot take are refused with
// SOMI_ERR_UNSUPPORTED before anything is launched; never a wrong result.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SOMI_F32 0
#define SOMI_BF16 1
#define SOMI_ERR_UNSUPPORTED 10001   // outside every cudaError_t value in use
#define SOMI_ERR_SCRATCH_TOO_SMALL 10002

#define SOMI_API extern "C" __attribute__((visibility("default")))

namespace somi {

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float load_as_float(const void* p, int dtype, size_t i) {
    return dtype == SOMI_F32 ? reinterpret_cast<const float*>(p)[i]
                             : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result.  `scratch` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    float r = scratch[32];
    __syncthreads();
    return r;
}

// The rotation of a pair (a at dim i, b at dim i + rot/2) by (cos, sin), with the roundings
// spelled out so that every kernel that rotates gives the same bits.
__device__ __forceinline__ float rope_lo(float a, float b, float c, float s) {
    return __fmaf_rn(a, c, -__fmul_rn(b, s));
}
__device__ __forceinline__ float rope_hi(float a, float b, float c, float s) {
    return __fmaf_rn(b, c, __fmul_rn(a, s));
}

inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

// ---- programmatic dependent launch
// Every kernel of this library is launched with the programmatic-serialization attribute: it
// may be scheduled while its predecessor in the stream is still running, so that its launch
// latency and its set-up (barriers, tensor memory, index arithmetic) overlap the predecessor's
// tail.  A kernel calls `pdl_launch_dependents()` as its first statement, so that its own
// successor may be scheduled, and `pdl_wait()` before it writes global memory at all and before
// any early return.  `pdl_wait()` returns when the predecessor has completed; the predecessor
// completed only after its own wait, so after the wait every earlier kernel is complete.
//
// BEFORE the wait nothing of the kind holds: kernel N may be resident while N-1 is still before
// its own wait and N-2 is running.  So before the wait a kernel may read only memory that NO
// kernel of the same step writes:
//   [constant]   model constants (weights, norm weights, inverse frequencies, tensor maps);
//   [descriptor] the step's descriptor, uploaded by a memcpy that completed before the step's
//                first kernel started (a copy is not launched programmatically);
//   [old-cache]  cache slots of positions below the request's cached length of this step: they
//                were written by earlier steps, and the descriptor copy between two steps is a
//                full barrier in the stream.
// Outputs of ANY kernel of the same step (not only the direct predecessor's) are off limits
// before the wait.  Reads before a wait are tagged with one of the three classes above.
//
// What changes from step to step at fixed addresses ([descriptor], and the tables that lead to
// [old-cache]) is read with `ld_step` before the wait: `ld.global.cg`, served from L2, where the
// copy of the descriptor arrived before the step's first kernel started.  A plain load of a
// `const __restrict__` pointer may go through the SM's read-only cache, whose contents are only
// defined for data that nobody writes during the kernel's lifetime; a kernel that starts before
// its predecessor has ended stretches that lifetime, so these few loads take the path whose
// coherence does not depend on it.  After the wait plain loads are used.  Bulk tensor copies
// (TMA) read through L2 as well.
__device__ __forceinline__ int ld_step(const int* p) { return __ldcg(p); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

inline int& pdl_enabled() {
    static int on = 1;
    return on;
}

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                      cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

}  // namespace somi
