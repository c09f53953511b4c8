// The gated delta rule with a decay per head AND key channel: the state's rows decay at rates of their own.
//
// A token's projections arrive as one float32 row
//     proj[t] = [ q (G*dk) | k (G*dk) | v (H*dv) | b (H) | a1 (ra) | g1 (rg) ]
// (G key heads of size dk shared by H/G value heads of size dv each; a1 and g1 are the narrow halves of two low-rank
// projections).  Three kernels follow the product:
//
//  1. prepare: the causal convolution with silu on q, k and v, unit length for q (also dk^-1/2) and k, as in the form with one
//     decay a head; beta = sigmoid(b); the decay's logarithm  -exp(A_log[h]) * softplus(a2 a1 + dt_bias)  for every head and
//     key channel; the output gate sigmoid(g2 g1) for every head and value channel.  The wide halves a2 and g2 are applied
//     here, in float32, a column of the transposed matrix a thread.
//  2. recurrence, per request and head, token after token, on the state S [dk][dv]:
//         S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//     A column of S lives in the registers of R neighbouring lanes, as in the other form.  Tokens are taken M at a time.
//     With L_t the sum of the group's log decays up to token t (a vector over key channels) and S the state before the group,
//         D_j = S^T (e^{L_j} k_j),  E_j = S^T (e^{L_j} q_j)        (2M sums over dk, independent of one another)
//     and then, for t = 1..M, no further sum over dk:
//         u_t = beta_t (v_t - D_t);   D_j += A[t][j] u_t (j > t);   E_j += B[t][j] u_t (j >= t);   o_t = E_t
//         A[t][j] = sum_d k_t[d] k_j[d] e^{L_j[d] - L_t[d]},   B[t][j] = sum_d k_t[d] q_j[d] e^{L_j[d] - L_t[d]}
//     and S <- diag(e^{L_M}) S + sum_t (e^{L_M - L_t} k_t) u_t^T.  Every exponent is <= 0.  The block works out A, B and the scaled
//     vectors once per chunk for all its columns.  M = 1 is the plain recurrence (single decoded tokens).
//  3. gate: o / rms(o) over dv, times a weight shared by the heads, times the gate of 1, in the compute dtype.
//
// Everything is float32.  A request's state row is the other form's: [H*dv*dk floats of S^T][(taps-1)*C convolution inputs].
#include "delta_common.cuh"

namespace vk {

// prep row: q | k | v | log decay (H*dk) | beta (H) | gate (H*dv)
__host__ __device__ inline int cd_prep_width(int G, int H, int dk, int dv) { return (2 * G * dk + 2 * H * dv + H * dk + H + 3) / 4 * 4; }

// One block per token.  smem: act [C], a1 [ra], g1 [rg].
__global__ void __launch_bounds__(1024) cdelta_prepare_kernel(
    const float* __restrict__ proj, const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const float* __restrict__ a2t, const float* __restrict__ g2t, const int32_t* __restrict__ token_seg, const int32_t* __restrict__ seg_starts,
    const int32_t* __restrict__ seg_slots, const float* __restrict__ state, size_t state_stride, size_t conv_off, float* __restrict__ prep,
    int P, int G, int H, int dk, int dv, int taps, int ra, int rg) {
    extern __shared__ float act[];
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int C = 2 * G * dk + H * dv, N = C + H + ra + rg;
    float* lr = act + C;                                     // a1, then g1
    const int seg = token_seg[t];
    const int i = t - seg_starts[seg];
    const int slot = seg_slots[seg];
    const float* old = slot >= 0 ? state + (size_t)slot * state_stride + conv_off : nullptr;   // [taps-1][C]
    const float* in = proj + (size_t)t * N;
    for (int c = tid; c < C; c += blockDim.x) {
        float x[DR_MAX_TAPS], w[DR_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < DR_MAX_TAPS; j++) {
            if (j < taps) {
                const int src = i - j;
                x[j] = src >= 0 ? proj[(size_t)(t - j) * N + c] : (old ? old[(size_t)(taps - 1 + src) * C + c] : 0.0f);
                w[j] = conv_w[(size_t)c * taps + (taps - 1 - j)];
            }
        }
        float acc = 0.0f;
#pragma unroll
        for (int j = DR_MAX_TAPS - 1; j >= 0; j--)          // oldest input first
            if (j < taps) acc = fmaf(w[j], x[j], acc);
        act[c] = silu_f(acc);
    }
    for (int r = tid; r < ra + rg; r += blockDim.x) lr[r] = in[C + H + r];
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
    const int HK = H * dk, HV = H * dv;
    for (int c = tid; c < HK; c += blockDim.x) {             // the decay's logarithm; the recurrence takes exp of sums of it
        float acc = 0.0f;
        for (int r = 0; r < ra; r++) acc = fmaf(a2t[(size_t)r * HK + c], lr[r], acc);
        out[C + c] = -expf(a_log[c / dk]) * softplus_f(acc + dt_bias[c]);
    }
    for (int h = tid; h < H; h += blockDim.x) out[C + HK + h] = sigmoid_f(in[C + h]);
    for (int c = tid; c < HV; c += blockDim.x) {
        float acc = 0.0f;
        for (int r = 0; r < rg; r++) acc = fmaf(g2t[(size_t)r * HV + c], lr[ra + r], acc);
        out[C + HK + H + c] = sigmoid_f(acc);
    }
}

// grid (segments, H, column parts); block = cols * R threads, thread = (column, lane of the column); a lane holds KPT values of
// its column in pieces of four: piece i of lane r is rows (i*R + r)*4 .. +3 of S (zero beyond dk).
// One staged buffer: q [chunk][dkp], k [chunk][dkp], l [chunk][dkp] (log decays, then their running sums), kt [chunk][dkp]
// (e^{L} k), v [chunk][cols], beta [chunk], products [chunk/M][2][M][M].
template <int KPT, int M>
__global__ void __launch_bounds__(256) cdelta_recurrence_kernel(
    const float* __restrict__ prep, int P, const float* __restrict__ proj, int N, const int32_t* __restrict__ seg_starts,
    const int32_t* __restrict__ seg_slots, float* __restrict__ state, size_t state_stride, size_t conv_off, float* __restrict__ o, int G, int H,
    int dk, int dv, int taps, int R, int cols, int chunk, int vec) {
    extern __shared__ __align__(16) float sm[];
    const int seg = blockIdx.x, h = blockIdx.y, part = blockIdx.z, tid = threadIdx.x;
    dependency_wait();
    let_dependents_start();
    const int slot = seg_slots[seg];
    if (slot < 0) return;                                    // a padding segment of a captured batch
    const int start = seg_starts[seg], n = seg_starts[seg + 1] - start;
    const int C = 2 * G * dk + H * dv;
    const int g = h / (H / G);
    const int dkp = R * KPT;                                 // dk rounded up to what the lanes hold (a power of two)
    const int dk4 = dk / 4, dkp4 = dkp / 4;
    const int sh4 = 31 - __clz(dkp4);
    float* row = state + (size_t)slot * state_stride;

    const int buf_floats = chunk * (4 * dkp + cols + 1 + 2 * M);
    const int r = tid % R, cl = tid / R;
    const int col = part * cols + cl;
    const bool live = cl < cols && col < dv;
    float s[KPT];
    float* srow = row + ((size_t)h * dv + (live ? col : 0)) * dk;
#pragma unroll
    for (int i = 0; i < KPT / 4; i++) {
        const int k0 = (i * R + r) * 4;
        if (vec) {
            const float4 v = (live && k0 < dk) ? *reinterpret_cast<const float4*>(srow + k0) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            s[4 * i] = v.x; s[4 * i + 1] = v.y; s[4 * i + 2] = v.z; s[4 * i + 3] = v.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) s[4 * i + e] = (live && k0 + e < dk) ? srow[k0 + e] : 0.0f;
        }
    }

    auto stage = [&](int c0, int b) {
        float* q_s = sm + b * buf_floats;
        float* k_s = q_s + chunk * dkp;
        float* l_s = k_s + chunk * dkp;
        float* v_s = l_s + 2 * chunk * dkp;
        float* b_s = v_s + chunk * cols;
        const int cn = n - c0 < chunk ? n - c0 : chunk;
        for (int e = tid; e < cn * dkp4; e += blockDim.x) {
            const int j = e >> sh4, d4 = e & (dkp4 - 1);
            const float* p = prep + (size_t)(start + c0 + j) * P;
            if (!vec) {
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const int d = d4 * 4 + x;
                    if (d < dk) {
                        dr_cp_async4(q_s + e * 4 + x, p + (size_t)g * dk + d);
                        dr_cp_async4(k_s + e * 4 + x, p + (size_t)(G + g) * dk + d);
                        dr_cp_async4(l_s + e * 4 + x, p + C + (size_t)h * dk + d);
                    } else {
                        q_s[e * 4 + x] = 0.0f;
                        k_s[e * 4 + x] = 0.0f;
                        l_s[e * 4 + x] = 0.0f;
                    }
                }
            } else if (d4 < dk4) {
                dr_cp_async16(q_s + e * 4, p + (size_t)g * dk + d4 * 4);
                dr_cp_async16(k_s + e * 4, p + (size_t)(G + g) * dk + d4 * 4);
                dr_cp_async16(l_s + e * 4, p + C + (size_t)h * dk + d4 * 4);
            } else {
                *reinterpret_cast<float4*>(q_s + e * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                *reinterpret_cast<float4*>(k_s + e * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                *reinterpret_cast<float4*>(l_s + e * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
        for (int j = 0; j < cn; j++) {
            for (int cc = tid; cc < cols; cc += blockDim.x) {
                const int c = part * cols + cc;
                if (c < dv) dr_cp_async4(v_s + j * cols + cc, prep + (size_t)(start + c0 + j) * P + 2 * G * dk + (size_t)h * dv + c);
                else v_s[j * cols + cc] = 0.0f;
            }
        }
        for (int j = tid; j < cn; j += blockDim.x) dr_cp_async4(b_s + j, prep + (size_t)(start + c0 + j) * P + C + (size_t)H * dk + h);
        const int cnp = (cn + M - 1) / M * M;                // tokens that do nothing fill the last group
        for (int e = cn * dkp + tid; e < cnp * dkp; e += blockDim.x) { q_s[e] = 0.0f; k_s[e] = 0.0f; l_s[e] = 0.0f; }
        for (int e = cn * cols + tid; e < cnp * cols; e += blockDim.x) v_s[e] = 0.0f;
        for (int j = cn + tid; j < cnp; j += blockDim.x) b_s[j] = 0.0f;
    };

    stage(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    int b = 0;
    for (int c0 = 0; c0 < n; c0 += chunk, b ^= 1) {
        const int cn = n - c0 < chunk ? n - c0 : chunk;
        if (c0 + chunk < n) stage(c0 + chunk, b ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        float* q_s = sm + b * buf_floats;
        float* k_s = q_s + chunk * dkp;
        float* l_s = k_s + chunk * dkp;
        float* kt_s = l_s + chunk * dkp;
        const float* v_s = kt_s + chunk * dkp;
        const float* b_s = v_s + chunk * cols;
        float* gram = const_cast<float*>(b_s) + chunk;       // [groups][2][M][M]
        const int cnp = (cn + M - 1) / M * M;
        const int groups = cnp / M;
        // running sums of the log decays inside every group, a (group, channel) a thread
        for (int e = tid; e < groups * dkp; e += blockDim.x) {
            const int grp = e / dkp, d = e - grp * dkp;
            float run = 0.0f;
#pragma unroll
            for (int t = 0; t < M; t++) {
                run += l_s[(grp * M + t) * dkp + d];
                l_s[(grp * M + t) * dkp + d] = run;
            }
        }
        __syncthreads();
        for (int e = tid; e < cnp * 2 * M; e += blockDim.x) {        // entry e = ((group * 2 + which) * M + t) * M + j
            const int jj = e % M, t = (e / M) % M, which = (e / (M * M)) % 2, grp = e / (2 * M * M);
            float acc = 0.0f;
            if (which ? jj >= t : jj > t) {
                const float* x = k_s + (grp * M + t) * dkp;
                const float* y = (which ? q_s : k_s) + (grp * M + jj) * dkp;
                const float* lt = l_s + (grp * M + t) * dkp;
                const float* lj = l_s + (grp * M + jj) * dkp;
                float a0 = 0.0f, a1 = 0.0f;
                for (int ii = 0; ii < dkp; ii += 2) {
                    const int i0 = (ii + 2 * tid) & (dkp - 1);       // neighbouring threads start at other banks
                    a0 = fmaf(x[i0] * y[i0], jj == t ? 1.0f : expf(lj[i0] - lt[i0]), a0);
                    a1 = fmaf(x[i0 + 1] * y[i0 + 1], jj == t ? 1.0f : expf(lj[i0 + 1] - lt[i0 + 1]), a1);
                }
                acc = a0 + a1;
            }
            gram[e] = acc;
        }
        __syncthreads();
        // kt = e^{L_t} k_t,  q <- e^{L_t} q_t,  k <- e^{L_M - L_t} k_t; the last row of a group's l stays: e^{L_M} is taken below
        for (int e = tid; e < cnp * dkp; e += blockDim.x) {
            const int j = e / dkp, d = e - j * dkp;
            const int last = (j / M) * M + M - 1;
            const float lt = l_s[e], lm = l_s[last * dkp + d];
            const float et = expf(lt), kv = k_s[e];
            kt_s[e] = et * kv;
            q_s[e] *= et;
            k_s[e] = expf(lm - lt) * kv;
        }
        __syncthreads();
        const int clc = cl < cols ? cl : 0;
        for (int j0 = 0; j0 < cn; j0 += M) {
            float D[M], E[M];
#pragma unroll
            for (int t = 0; t < M; t++) {
                const float4* kk = reinterpret_cast<const float4*>(kt_s + (j0 + t) * dkp) + r;
                const float4* qq = reinterpret_cast<const float4*>(q_s + (j0 + t) * dkp) + r;
                float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
                for (int i = 0; i < KPT / 4; i++) {
                    const float4 kv = kk[i * R], qv = qq[i * R];
                    a0 = fmaf(s[4 * i], kv.x, a0); a1 = fmaf(s[4 * i + 1], kv.y, a1);
                    a0 = fmaf(s[4 * i + 2], kv.z, a0); a1 = fmaf(s[4 * i + 3], kv.w, a1);
                    b0 = fmaf(s[4 * i], qv.x, b0); b1 = fmaf(s[4 * i + 1], qv.y, b1);
                    b0 = fmaf(s[4 * i + 2], qv.z, b0); b1 = fmaf(s[4 * i + 3], qv.w, b1);
                }
                D[t] = a0 + a1;
                E[t] = b0 + b1;
            }
            for (int w = R >> 1; w > 0; w >>= 1) {
#pragma unroll
                for (int t = 0; t < M; t++) {
                    D[t] += __shfl_xor_sync(0xffffffffu, D[t], w);
                    E[t] += __shfl_xor_sync(0xffffffffu, E[t], w);
                }
            }
            const float* gk = gram + (j0 / M) * 2 * M * M;
            const float* gq = gk + M * M;
            float uw[M];
#pragma unroll
            for (int t = 0; t < M; t++) {
                const float u = b_s[j0 + t] * (v_s[(j0 + t) * cols + clc] - D[t]);
#pragma unroll
                for (int j = t + 1; j < M; j++) D[j] = fmaf(gk[t * M + j], u, D[j]);
#pragma unroll
                for (int j = t; j < M; j++) E[j] = fmaf(gq[t * M + j], u, E[j]);
                if (live && r == 0 && j0 + t < cn) o[((size_t)(start + c0 + j0 + t) * H + h) * dv + col] = E[t];
                uw[t] = u;
            }
            const float4* lm = reinterpret_cast<const float4*>(l_s + (j0 + M - 1) * dkp) + r;
#pragma unroll
            for (int i = 0; i < KPT / 4; i++) {
                const float4 lv = lm[i * R];
                float x0 = expf(lv.x) * s[4 * i], x1 = expf(lv.y) * s[4 * i + 1], x2 = expf(lv.z) * s[4 * i + 2], x3 = expf(lv.w) * s[4 * i + 3];
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const float4 kv = (reinterpret_cast<const float4*>(k_s + (j0 + t) * dkp) + r)[i * R];
                    x0 = fmaf(kv.x, uw[t], x0); x1 = fmaf(kv.y, uw[t], x1); x2 = fmaf(kv.z, uw[t], x2); x3 = fmaf(kv.w, uw[t], x3);
                }
                s[4 * i] = x0; s[4 * i + 1] = x1; s[4 * i + 2] = x2; s[4 * i + 3] = x3;
            }
        }
        __syncthreads();                                     // the buffer may be staged again
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < KPT / 4; i++) {
            const int k0 = (i * R + r) * 4;
            if (vec) {
                if (k0 < dk) *reinterpret_cast<float4*>(srow + k0) = make_float4(s[4 * i], s[4 * i + 1], s[4 * i + 2], s[4 * i + 3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (k0 + e < dk) srow[k0 + e] = s[4 * i + e];
            }
        }
    }

    // the convolution's memory: the last taps-1 inputs of the request, this step's tokens included
    if (taps > 1) {
        float* cs = row + conv_off;
        const int nb = gridDim.y * gridDim.z, bi = h * gridDim.z + part;
        for (int c = bi * blockDim.x + tid; c < C; c += nb * blockDim.x) {
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

// A warp per (token, head): out = o / rms(o) * w * gate, the gate as the prepare kernel left it.
template <typename T>
__global__ void __launch_bounds__(256) cdelta_gate_kernel(const float* __restrict__ o, const float* __restrict__ prep, int P, int gate_off,
                                                          const float* __restrict__ norm_w, float eps, T* __restrict__ out, int tokens, int H, int dv) {
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    dependency_wait();
    let_dependents_start();
    if (unit >= tokens * H) return;
    const int t = unit / H, h = unit % H;
    const float* in = o + (size_t)unit * dv;
    const float* gate = prep + (size_t)t * P + gate_off + (size_t)h * dv;
    float ss = 0.0f;
    for (int d = lane; d < dv; d += 32) ss = fmaf(in[d], in[d], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) out[(size_t)unit * dv + d] = from_f32<T>(((in[d] * inv) * norm_w[d]) * gate[d]);
}

}  // namespace vk

using namespace vk;

VK_API int vk_cdelta_prep_width(int G, int H, int dk, int dv) { return cd_prep_width(G, H, dk, dv); }

// proj [tokens][C + H + ra + rg] float32; conv_w [C][taps]; a2t [ra][H*dk], g2t [rg][H*dv] (the wide halves, transposed);
// dt_bias [H*dk]; a_log [H]; state [slots][state_stride] float32; prep [tokens][vk_cdelta_prep_width].
VK_API int vk_cdelta_prepare(const float* proj, const float* conv_w, const float* a_log, const float* dt_bias, const float* a2t, const float* g2t,
                             const int32_t* token_seg, const int32_t* seg_starts, const int32_t* seg_slots, const float* state, size_t state_stride,
                             float* prep, int tokens, int G, int H, int dk, int dv, int taps, int ra, int rg, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1 || ra < 1 || rg < 1) return VK_BAD_SHAPE;
    const int P = cd_prep_width(G, H, dk, dv);
    if (taps > DR_MAX_TAPS) return VK_TOO_LARGE;
    const size_t C = 2 * (size_t)G * dk + (size_t)H * dv;
    const size_t smem = (C + ra + rg) * sizeof(float);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
    if (smem > 48 * 1024) cudaFuncSetAttribute(cdelta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int wide = (int)((C + 31) / 32 * 32);
    const int threads = tokens <= DR_DEPENDENT_TOKENS ? (wide < 1024 ? wide : 1024) : 256;
    if (tokens <= DR_DEPENDENT_TOKENS)
        return launch_dependent(cdelta_prepare_kernel, dim3(tokens), dim3(threads), smem, stream, proj, conv_w, a_log, dt_bias, a2t, g2t, token_seg,
                                seg_starts, seg_slots, state, state_stride, (size_t)H * dv * dk, prep, P, G, H, dk, dv, taps, ra, rg);
    return launch_plain(cdelta_prepare_kernel, dim3(tokens), dim3(threads), smem, stream, proj, conv_w, a_log, dt_bias, a2t, g2t, token_seg,
                        seg_starts, seg_slots, state, state_stride, (size_t)H * dv * dk, prep, P, G, H, dk, dv, taps, ra, rg);
}

VK_API int vk_cdelta_recurrence(const float* prep, const float* proj, int proj_width, const int32_t* seg_starts, const int32_t* seg_slots,
                                float* state, size_t state_stride, float* o, int segments, int tokens, int G, int H, int dk, int dv, int taps,
                                cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1) return VK_BAD_SHAPE;
    const int vec = dk % 4 == 0 && (H * dv) % 4 == 0 && ((uintptr_t)prep % 16) == 0 && ((uintptr_t)state % 16) == 0 && state_stride % 4 == 0;
    if (taps > DR_MAX_TAPS || dk > 32 * DR_KPT || H > 65535) return VK_TOO_LARGE;
    const int P = cd_prep_width(G, H, dk, dv);
    int R = 1;
    while ((dk + R - 1) / R > DR_KPT) R *= 2;
    while (R < 32 && (dk + R - 1) / R > 8) R *= 2;
    while (R < 32 && dv * R < 128 && (dk + R - 1) / R > 4) R *= 2;
    int kpt = 4;
    while (kpt * R < dk) kpt *= 2;
    int cols = dv;
    while (cols * R > 256) cols = (cols + 1) / 2;
    while ((long long)segments * H * ((dv + cols - 1) / cols) < 148 && cols * R > 64 && cols % 2 == 0) cols /= 2;
    const int parts = (dv + cols - 1) / cols;
    const int threads = ((cols * R + 31) / 32) * 32;
    const int longest = tokens > 0 ? tokens : 1;
    const int M = longest > 1 ? 4 : 1;
    int chunk = 64;
    auto bytes = [&](int c) { return (size_t)2 * c * (4 * R * kpt + cols + 1 + 2 * M) * sizeof(float); };
    while (chunk > 8 && (chunk / 2 >= longest || bytes(chunk) > 64 * 1024)) chunk /= 2;
    const size_t smem = bytes(chunk);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
#define GO(K, MM)                                                                                                                        \
    {                                                                                                                                    \
        auto kern = cdelta_recurrence_kernel<K, MM>;                                                                                     \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                       \
        if (tokens <= DR_DEPENDENT_TOKENS)                                                                                               \
            return launch_dependent(kern, dim3(segments, H, parts), dim3(threads), smem, stream, prep, P, proj, proj_width, seg_starts,  \
                                    seg_slots, state, state_stride, (size_t)H * dv * dk, o, G, H, dk, dv, taps, R, cols, chunk, vec);    \
        return launch_plain(kern, dim3(segments, H, parts), dim3(threads), smem, stream, prep, P, proj, proj_width, seg_starts, seg_slots, \
                            state, state_stride, (size_t)H * dv * dk, o, G, H, dk, dv, taps, R, cols, chunk, vec);                      \
    }
    if (M == 1) {
        if (kpt == 4) GO(4, 1) else if (kpt == 8) GO(8, 1) else if (kpt == 16) GO(16, 1) else GO(32, 1)
    } else {
        if (kpt == 4) GO(4, 4) else if (kpt == 8) GO(8, 4) else if (kpt == 16) GO(16, 4) else GO(32, 4)
    }
#undef GO
    return launch_status();
}

VK_API int vk_cdelta_gate(const float* o, const float* prep, const float* norm_w, float eps, void* out, int tokens, int G, int H, int dk, int dv,
                          int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || dk <= 0 || dv <= 0) return VK_BAD_SHAPE;
    const int grid = (tokens * H + 7) / 8;
    const int P = cd_prep_width(G, H, dk, dv), off = 2 * G * dk + H * dv + H * dk + H;
    if (tokens <= DR_DEPENDENT_TOKENS) {
        if (dtype == 0) return launch_dependent(cdelta_gate_kernel<float>, dim3(grid), dim3(256), 0, stream, o, prep, P, off, norm_w, eps, (float*)out, tokens, H, dv);
        return launch_dependent(cdelta_gate_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, o, prep, P, off, norm_w, eps, (__nv_bfloat16*)out, tokens, H, dv);
    }
    if (dtype == 0) return launch_plain(cdelta_gate_kernel<float>, dim3(grid), dim3(256), 0, stream, o, prep, P, off, norm_w, eps, (float*)out, tokens, H, dv);
    return launch_plain(cdelta_gate_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, o, prep, P, off, norm_w, eps, (__nv_bfloat16*)out, tokens, H, dv);
}
