// Layer norm with weight and bias, and the soft cap of the logits.
//
//   y = (x - mean) / sqrt(var + eps) * w + b,   var = mean((x - mean)^2)      float32 arithmetic, two passes over the row
//   z <- cap * tanh(z / cap)
//
// A block per output row; a row's sums meet in a fixed order, so its result does not depend on the rest of the batch.  The output
// is float32 or bfloat16; with float32 it may be the input itself (every value is read and written by the same thread, after the
// row's two sums are complete).  `rows` (optional) names the input row of each output row.
#include "common.cuh"

namespace vk {

constexpr int LN_THREADS = 128;
constexpr int LN_KEEP = 8;          // rows of up to 4 * LN_THREADS * LN_KEEP values stay in registers between the passes

template <typename T> __device__ __forceinline__ void ln_store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void ln_store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void ln_store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// A block per output row.  Rows whose width is a multiple of four (and 16-byte aligned) of up to 4,096 values are read once, all
// of a thread's 16-byte pieces asked for before any is used, and kept in registers for the two sums and the result; other rows are
// read three times.  The sums of a row meet in a fixed order that depends on the width alone.
template <typename T>
__global__ void __launch_bounds__(LN_THREADS) layernorm_rows_kernel(const float* x, const float* __restrict__ w, const float* __restrict__ b,
                                                                    const int32_t* __restrict__ rows, T* y, int out_rows, int n, float eps) {
    __shared__ float scratch[32];
    const int tid = threadIdx.x, r = blockIdx.x;
    dependency_wait();
    let_dependents_start();
    const float* in = x + (size_t)(rows ? rows[r] : r) * n;
    T* out = y + (size_t)r * n;
    const bool vec = (n % 4 == 0) && n <= 4 * LN_THREADS * LN_KEEP && (reinterpret_cast<uintptr_t>(in) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(w) % 16 == 0) && (reinterpret_cast<uintptr_t>(b) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(out) % (4 * sizeof(T)) == 0);
    if (vec) {
        float4 v[LN_KEEP];
#pragma unroll
        for (int j = 0; j < LN_KEEP; j++) {
            const int i = (tid + j * LN_THREADS) * 4;
            v[j] = i < n ? *reinterpret_cast<const float4*>(in + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < LN_KEEP; j++) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        const float mean = block_sum(sum, scratch) / (float)n;
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < LN_KEEP; j++) {
            if ((tid + j * LN_THREADS) * 4 < n) {
                const float d0 = v[j].x - mean, d1 = v[j].y - mean, d2 = v[j].z - mean, d3 = v[j].w - mean;
                ss = fmaf(d0, d0, ss); ss = fmaf(d1, d1, ss); ss = fmaf(d2, d2, ss); ss = fmaf(d3, d3, ss);
            }
        }
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
#pragma unroll
        for (int j = 0; j < LN_KEEP; j++) {
            const int i = (tid + j * LN_THREADS) * 4;
            if (i < n) {
                const float4 ww = *reinterpret_cast<const float4*>(w + i), bb = *reinterpret_cast<const float4*>(b + i);
                ln_store4<T>(out + i, fmaf((v[j].x - mean) * inv, ww.x, bb.x), fmaf((v[j].y - mean) * inv, ww.y, bb.y),
                             fmaf((v[j].z - mean) * inv, ww.z, bb.z), fmaf((v[j].w - mean) * inv, ww.w, bb.w));
            }
        }
        return;
    }
    float sum = 0.0f;
    for (int i = tid; i < n; i += LN_THREADS) sum += in[i];
    const float mean = block_sum(sum, scratch) / (float)n;
    float ss = 0.0f;
    for (int i = tid; i < n; i += LN_THREADS) { const float d = in[i] - mean; ss = fmaf(d, d, ss); }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
    for (int i = tid; i < n; i += LN_THREADS) out[i] = from_f32<T>(fmaf((in[i] - mean) * inv, w[i], b[i]));
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
    if (dtype == 0) return launch_dependent(layernorm_rows_kernel<float>, dim3(out_rows), dim3(LN_THREADS), 0, stream, x, w, b, rows, (float*)y, out_rows, n, eps);
    return launch_dependent(layernorm_rows_kernel<__nv_bfloat16>, dim3(out_rows), dim3(LN_THREADS), 0, stream, x, w, b, rows, (__nv_bfloat16*)y, out_rows, n, eps);
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
