// A kernel that belongs to a part defined in the tests, not to the engine: it is compiled from
// this folder by the engine's builder and launched by the part itself on the current stream.
//     y[t, i] = x[t, i] * sigmoid(g[i] * x[t, i]) + b[i] * x[t, (i + 1) mod H]
// It follows the one rule every kernel of a step has to keep: wait for the kernels before it
// (`pdl_wait`) before the first access to what they wrote.
#include "common.cuh"

namespace toy {

template <typename T>
__global__ void gated_shift_kernel(const T* __restrict__ x, const float* __restrict__ g,
                                   const float* __restrict__ b, T* __restrict__ y, int n_tokens, int H) {
    somi::pdl_launch_dependents();
    somi::pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * H) return;
    const int t = i / H, c = i - t * H;
    const float v = somi::to_float(x[i]);
    const float next = somi::to_float(x[t * H + (c + 1 == H ? 0 : c + 1)]);
    const float gate = 1.0f / (1.0f + expf(-g[c] * v));
    y[i] = somi::from_float<T>(v * gate + b[c] * next);
}

}  // namespace toy

SOMI_API int toy_gated_shift(const void* x, int dtype, const float* g, const float* b, void* y,
                             int n_tokens, int H, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0) return SOMI_ERR_UNSUPPORTED;
    const int n = n_tokens * H;
    const dim3 grid((n + 255) / 256), block(256);
    if (dtype == SOMI_F32)
        somi::launch_pdl(toy::gated_shift_kernel<float>, grid, block, 0, stream,
                         static_cast<const float*>(x), g, b, static_cast<float*>(y), n_tokens, H);
    else if (dtype == SOMI_BF16)
        somi::launch_pdl(toy::gated_shift_kernel<__nv_bfloat16>, grid, block, 0, stream,
                         static_cast<const __nv_bfloat16*>(x), g, b, static_cast<__nv_bfloat16*>(y),
                         n_tokens, H);
    else
        return SOMI_ERR_UNSUPPORTED;
    return somi::launch_status();
}
