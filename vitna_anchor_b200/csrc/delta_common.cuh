// What the kernels of the delta rule's two forms (one decay a head; a decay per head and key channel) share.
#pragma once
#include "common.cuh"

namespace vk {

constexpr int DR_MAX_TAPS = 16;
constexpr int DR_KPT = 32;         // most values of a column one lane holds
constexpr int DR_DEPENDENT_TOKENS = 64;    // launches of up to this many tokens are programmatic dependents

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

__device__ __forceinline__ void dr_cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

}  // namespace vk
