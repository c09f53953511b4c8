// The gated delta rule: a recurrent mixer with a matrix state per head.
//
// A token's projections arrive as one float32 row
//     proj[t] = [ q (G*dk) | k (G*dk) | v (H*dv) | gate (H*dv) | b (H) | a (H) ]
// (G key heads of size dk shared by H/G value heads of size dv each).  Three kernels follow the product:
//
//  1. prepare: a causal convolution over time on every q, k and v channel (taps weights per channel, the last one
//     the current token's; inputs before a request's first position are zero, inputs before this step's first token
//     come from the request's state), silu; q and k heads scaled to unit length, q also by dk^-1/2;
//     beta = sigmoid(b); decay = exp(-exp(A_log) * softplus(a + dt_bias)).
//  2. recurrence, per request and head, token after token, on the state S [dk][dv]:
//         S <- decay S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//     The columns of S never meet, so a column lives in the registers of R neighbouring lanes (dk/R values each)
//     and the two sums over dk are lane shuffles; a block holds a head's columns (or a part of them) and stages
//     sixteen tokens of q, k, v, decay and beta at a time in shared memory.  The state is kept transposed
//     ([H][dv][dk]) so that a lane's values are contiguous.  The same kernel moves the last taps-1 inputs of the
//     convolution into the request's state once the tokens of the step have been read.
//  3. gate: o / rms(o) over dv, times a weight shared by the heads, times silu(gate), in the compute dtype.
//
// Everything here is float32; only the result of 3 is rounded to the compute dtype for the output projection.
// A request's per-layer state row is [H*dv*dk floats of S^T][(taps-1)*C floats of convolution inputs], C = 2 G dk + H dv.
#include "common.cuh"

namespace vk {

constexpr int DR_MAX_TAPS = 16;
constexpr int DR_CHUNK = 16;       // tokens staged at a time by the recurrence
constexpr int DR_KPT = 32;         // most values of a column one lane holds

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// One block per token.  smem: act [C].
__global__ void __launch_bounds__(256) delta_prepare_kernel(
    const float* __restrict__ proj, const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const int32_t* __restrict__ token_seg, const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
    const float* __restrict__ state, size_t state_stride, size_t conv_off, float* __restrict__ prep, int G, int H, int dk, int dv, int taps) {
    extern __shared__ float act[];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int C = 2 * G * dk + H * dv, N = C + H * dv + 2 * H, P = C + 2 * H;
    const int seg = token_seg[t];
    const int i = t - seg_starts[seg];                       // place of the token in this step's portion of its request
    const int slot = seg_slots[seg];
    const float* old = slot >= 0 ? state + (size_t)slot * state_stride + conv_off : nullptr;   // [taps-1][C]
    for (int c = tid; c < C; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = taps - 1; j >= 0; j--) {               // oldest input first
            const int src = i - j;
            float x;
            if (src >= 0) x = proj[(size_t)(t - j) * N + c];
            else x = old ? old[(size_t)(taps - 1 + src) * C + c] : 0.0f;
            acc = fmaf(conv_w[(size_t)c * taps + (taps - 1 - j)], x, acc);
        }
        act[c] = silu_f(acc);
    }
    __syncthreads();
    float* out = prep + (size_t)t * P;
    const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    for (int hq = warp; hq < 2 * G; hq += nwarps) {          // q heads, then k heads
        const float* v = act + (size_t)hq * dk;
        float ss = 0.0f;
        for (int d = lane; d < dk; d += 32) ss = fmaf(v[d], v[d], ss);
        ss = warp_sum(ss);
        float inv = 1.0f / sqrtf(ss + 1e-6f);
        if (hq < G) inv *= 1.0f / sqrtf((float)dk);
        for (int d = lane; d < dk; d += 32) out[(size_t)hq * dk + d] = v[d] * inv;
    }
    for (int c = 2 * G * dk + tid; c < C; c += blockDim.x) out[c] = act[c];
    for (int h = tid; h < H; h += blockDim.x) {
        const float b = proj[(size_t)t * N + C + H * dv + h], a = proj[(size_t)t * N + C + H * dv + H + h];
        out[C + h] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
        out[C + H + h] = 1.0f / (1.0f + expf(-b));
    }
}

// grid (segments, H, column parts); block = cols * R threads, thread = (column, lane of the column).
__global__ void __launch_bounds__(1024) delta_recurrence_kernel(
    const float* __restrict__ prep, const float* __restrict__ proj, const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
    float* __restrict__ state, size_t state_stride, size_t conv_off, float* __restrict__ o, int G, int H, int dk, int dv, int taps,
    int R, int kpt, int cols) {
    extern __shared__ float sm[];
    const int seg = blockIdx.x, h = blockIdx.y, part = blockIdx.z, tid = threadIdx.x;
    const int slot = seg_slots[seg];
    if (slot < 0) return;                                    // a padding segment of a captured batch
    const int start = seg_starts[seg], n = seg_starts[seg + 1] - start;
    const int C = 2 * G * dk + H * dv, N = C + H * dv + 2 * H, P = C + 2 * H;
    const int g = h / (H / G);
    float* row = state + (size_t)slot * state_stride;

    // staged per chunk: q [CH][dk], k [CH][dk], v [CH][cols], decay [CH], beta [CH]
    float* q_s = sm;
    float* k_s = q_s + DR_CHUNK * dk;
    float* v_s = k_s + DR_CHUNK * dk;
    float* d_s = v_s + DR_CHUNK * cols;
    float* b_s = d_s + DR_CHUNK;

    const int r = tid % R, cl = tid / R;
    const int col = part * cols + cl;
    const bool live = cl < cols && col < dv;
    const int k0 = r * kpt;
    float s[DR_KPT];
    float* srow = row + ((size_t)h * dv + (live ? col : 0)) * dk;
#pragma unroll
    for (int i = 0; i < DR_KPT; i++) s[i] = (live && i < kpt && k0 + i < dk) ? srow[k0 + i] : 0.0f;

    for (int c0 = 0; c0 < n; c0 += DR_CHUNK) {
        const int cn = n - c0 < DR_CHUNK ? n - c0 : DR_CHUNK;
        __syncthreads();
        for (int e = tid; e < cn * dk; e += blockDim.x) {
            const int j = e / dk, d = e % dk;
            const float* p = prep + (size_t)(start + c0 + j) * P;
            q_s[e] = p[(size_t)g * dk + d];
            k_s[e] = p[(size_t)(G + g) * dk + d];
        }
        for (int e = tid; e < cn * cols; e += blockDim.x) {
            const int j = e / cols, c = part * cols + e % cols;
            v_s[e] = c < dv ? prep[(size_t)(start + c0 + j) * P + 2 * G * dk + (size_t)h * dv + c] : 0.0f;
        }
        for (int j = tid; j < cn; j += blockDim.x) {
            d_s[j] = prep[(size_t)(start + c0 + j) * P + C + h];
            b_s[j] = prep[(size_t)(start + c0 + j) * P + C + H + h];
        }
        __syncthreads();
        for (int j = 0; j < cn; j++) {
            const float* kk = k_s + j * dk + k0;
            const float* qq = q_s + j * dk + k0;
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < DR_KPT; i++)
                if (i < kpt && k0 + i < dk) dot = fmaf(s[i], kk[i], dot);
            for (int w = R >> 1; w > 0; w >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, w);
            const float dec = d_s[j];
            const float u = b_s[j] * (v_s[j * cols + (cl < cols ? cl : 0)] - dec * dot);
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < DR_KPT; i++)
                if (i < kpt && k0 + i < dk) {
                    s[i] = fmaf(kk[i], u, dec * s[i]);
                    acc = fmaf(s[i], qq[i], acc);
                }
            for (int w = R >> 1; w > 0; w >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
            if (live && r == 0) o[((size_t)(start + c0 + j) * H + h) * dv + col] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DR_KPT; i++)
            if (i < kpt && k0 + i < dk) srow[k0 + i] = s[i];
    }

    // the convolution's memory: the last taps-1 inputs of the request, this step's tokens included.  The blocks
    // of a segment share the channels.
    if (taps > 1) {
        float* cs = row + conv_off;
        const int nb = gridDim.y * gridDim.z, b = h * gridDim.z + part;
        for (int c = b * blockDim.x + tid; c < C; c += nb * blockDim.x) {
            float keep[DR_MAX_TAPS];
#pragma unroll
            for (int rr = 0; rr < DR_MAX_TAPS; rr++) {
                if (rr < taps - 1) {
                    const int src = n - (taps - 1) + rr;
                    keep[rr] = src >= 0 ? proj[(size_t)(start + src) * N + c] : cs[(size_t)(rr + n) * C + c];
                }
            }
#pragma unroll
            for (int rr = 0; rr < DR_MAX_TAPS; rr++)
                if (rr < taps - 1) cs[(size_t)rr * C + c] = keep[rr];
        }
    }
}

// A warp per (token, head): out = o / rms(o) * w * silu(gate).
template <typename T>
__global__ void __launch_bounds__(256) delta_gate_kernel(const float* __restrict__ o, const float* __restrict__ proj, const float* __restrict__ norm_w,
                                                         float eps, T* __restrict__ out, int tokens, int G, int H, int dk, int dv) {
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= tokens * H) return;
    const int t = unit / H, h = unit % H;
    const int C = 2 * G * dk + H * dv, N = C + H * dv + 2 * H;
    const float* in = o + (size_t)unit * dv;
    const float* gate = proj + (size_t)t * N + C + (size_t)h * dv;
    float ss = 0.0f;
    for (int d = lane; d < dv; d += 32) ss = fmaf(in[d], in[d], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) out[(size_t)unit * dv + d] = from_f32<T>(((in[d] * inv) * norm_w[d]) * silu_f(gate[d]));
}

}  // namespace vk

using namespace vk;

// Floats of one request's state in one layer.
VK_API size_t vk_delta_state_floats(int G, int H, int dk, int dv, int taps) {
    return (size_t)H * dv * dk + (size_t)(taps > 1 ? taps - 1 : 0) * (2 * (size_t)G * dk + (size_t)H * dv);
}

// proj [tokens][C + H*dv + 2H] float32; conv_w [C][taps]; state [slots][state_stride] float32; prep [tokens][C + 2H].
VK_API int vk_delta_prepare(const float* proj, const float* conv_w, const float* a_log, const float* dt_bias, const int32_t* token_seg,
                            const int32_t* seg_starts, const int32_t* seg_slots, const float* state, size_t state_stride, float* prep, int tokens,
                            int G, int H, int dk, int dv, int taps, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1) return VK_BAD_SHAPE;
    if (taps > DR_MAX_TAPS) return VK_TOO_LARGE;
    const size_t C = 2 * (size_t)G * dk + (size_t)H * dv;
    const size_t smem = C * sizeof(float);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    delta_prepare_kernel<<<tokens, 256, smem, stream>>>(proj, conv_w, a_log, dt_bias, token_seg, seg_starts, seg_slots, state, state_stride,
                                                        (size_t)H * dv * dk, prep, G, H, dk, dv, taps);
    return launch_status();
}

VK_API int vk_delta_recurrence(const float* prep, const float* proj, const int32_t* seg_starts, const int32_t* seg_slots, float* state,
                               size_t state_stride, float* o, int segments, int G, int H, int dk, int dv, int taps, cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1) return VK_BAD_SHAPE;
    if (taps > DR_MAX_TAPS || dk > 32 * DR_KPT || H > 65535) return VK_TOO_LARGE;
    int R = 1;
    while ((dk + R - 1) / R > DR_KPT) R *= 2;                // a lane holds at most DR_KPT values of a column
    while (R < 32 && dv * R < 128 && (dk + R - 1) / R > 4) R *= 2;       // small heads: more lanes a column
    const int kpt = (dk + R - 1) / R;
    int cols = dv;
    while (cols * R > 512) cols = (cols + 1) / 2;            // wide heads: several blocks share a head's columns
    const int parts = (dv + cols - 1) / cols;
    const int threads = ((cols * R + 31) / 32) * 32;
    const size_t smem = (size_t)(DR_CHUNK * (2 * dk + cols + 2)) * sizeof(float);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_recurrence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    delta_recurrence_kernel<<<dim3(segments, H, parts), threads, smem, stream>>>(prep, proj, seg_starts, seg_slots, state, state_stride,
                                                                                 (size_t)H * dv * dk, o, G, H, dk, dv, taps, R, kpt, cols);
    return launch_status();
}

VK_API int vk_delta_gate(const float* o, const float* proj, const float* norm_w, float eps, void* out, int tokens, int G, int H, int dk, int dv,
                         int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || dk <= 0 || dv <= 0) return VK_BAD_SHAPE;
    const int grid = (tokens * H + 7) / 8;
    if (dtype == 0) delta_gate_kernel<float><<<grid, 256, 0, stream>>>(o, proj, norm_w, eps, (float*)out, tokens, G, H, dk, dv);
    else delta_gate_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(o, proj, norm_w, eps, (__nv_bfloat16*)out, tokens, G, H, dk, dv);
    return launch_status();
}
