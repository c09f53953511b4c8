// Layer norm with weight and bias, and the soft cap of the logits.
//
//   y = (x - mean) / sqrt(var + eps) * w + b,   var = mean((x - mean)^2)      float32 arithmetic, two passes over the row
//   z <- cap * tanh(z / cap)
//
// A warp per output row (eight rows a block); the 32 partial sums meet in a fixed shuffle tree, so a row's result does not depend
// on the rest of the batch.  The output is float32 or bfloat16; with float32 it may be the input itself (every value is read
// and written by the same lane, after the row's two sums are complete).  `rows` (optional) names the input row of each output row.
#include "common.cuh"

namespace vk {

template <typename T>
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const float* x, const float* __restrict__ w, const float* __restrict__ b,
                                                             const int32_t* __restrict__ rows, T* y, int out_rows, int n, float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    dependency_wait();
    let_dependents_start();
    if (r >= out_rows) return;
    const float* in = x + (size_t)(rows ? rows[r] : r) * n;
    T* out = y + (size_t)r * n;
    float sum = 0.0f;
    for (int i = lane; i < n; i += 32) sum += in[i];
    const float mean = warp_sum(sum) / (float)n;
    float ss = 0.0f;
    for (int i = lane; i < n; i += 32) { const float d = in[i] - mean; ss = fmaf(d, d, ss); }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
    for (int i = lane; i < n; i += 32) out[i] = from_f32<T>(fmaf((in[i] - mean) * inv, w[i], b[i]));
}

__global__ void softcap_kernel(float* __restrict__ z, size_t n, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) z[i] = cap * tanhf(z[i] / cap);
}

// act = activation(gate) * up;  gu [tokens, 2*inter]: gate columns, then up columns.  kind as activate_rt numbers them.
template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ gu, T* __restrict__ act, size_t tokens, int inter, int kind) {
    const size_t n = tokens * (size_t)inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter;
        const int c = (int)(i % inter);
        const float g = to_f32<T>(gu[t * 2 * inter + c]);
        const float u = to_f32<T>(gu[t * 2 * inter + inter + c]);
        act[i] = from_f32<T>(activate_rt(kind, g) * u);
    }
}

}  // namespace vk

using namespace vk;

static inline int ln_grid_for(size_t n, int threads) {
    size_t g = (n + threads - 1) / threads;
    return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

// x float32 [*, n]; y [out_rows, n] float32 (dtype 0; may be x itself when rows is null) or bfloat16 (dtype 1).
VK_API int vk_layernorm_rows(const float* x, const float* w, const float* b, const int32_t* rows, void* y, int out_rows, int n, float eps,
                             int dtype, cudaStream_t stream) {
    if (out_rows <= 0) return VK_OK;
    if (n <= 0) return VK_BAD_SHAPE;
    if (dtype == 0 && rows && y == (const void*)x) return VK_BAD_SHAPE;
    const int grid = (out_rows + 7) / 8;
    if (dtype == 0) return launch_dependent(layernorm_rows_kernel<float>, dim3(grid), dim3(256), 0, stream, x, w, b, rows, (float*)y, out_rows, n, eps);
    return launch_dependent(layernorm_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, x, w, b, rows, (__nv_bfloat16*)y, out_rows, n, eps);
}

VK_API int vk_softcap(float* z, size_t n, float cap, cudaStream_t stream) {
    if (n == 0) return VK_OK;
    if (!(cap > 0.0f)) return VK_BAD_SHAPE;
    softcap_kernel<<<ln_grid_for(n, 256), 256, 0, stream>>>(z, n, cap);
    return launch_status();
}

// kind: 0 gelu (erf), 1 gelu (tanh), 2 silu, as the element-wise activation numbers them
VK_API int vk_act_mul(const void* gu, void* act, int tokens, int inter, int kind, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (inter <= 0 || kind < 0 || kind > 2) return VK_BAD_SHAPE;
    const size_t n = (size_t)tokens * inter;
    if (dtype == 0) act_mul_kernel<float><<<ln_grid_for(n, 256), 256, 0, stream>>>((const float*)gu, (float*)act, tokens, inter, kind + 1);
    else act_mul_kernel<__nv_bfloat16><<<ln_grid_for(n, 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)act, tokens, inter, kind + 1);
    return launch_status();
}
