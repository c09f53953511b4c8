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
//     and S <- diag(e^{L_M}) S + sum_t (e^{L_M - L_t} k_t) u_t^T.  Every exponent is <= 0.  A, B and the scaled vectors are worked out
//     vectors in a kernel of its own for all groups side by side (a warp a token and head), so that the chain from token to token
//     holds no exponential and no sum over dk beyond the 2M above.  M = 1 is the plain recurrence (single decoded tokens).
//  3. gate: o / rms(o) over dv, times a weight shared by the heads, times the gate of 1, in the compute dtype.
//
// Everything is float32.  A request's state row is the other form's: [H*dv*dk floats of S^T][(taps-1)*C convolution inputs].
#include "delta_common.cuh"

namespace vk {

// prep row: q | k | v | log decay (H*dk) | beta (H) | gate (H*dv)
__host__ __device__ inline int cd_prep_width(int G, int H, int dk, int dv) { return (2 * G * dk + 2 * H * dv + H * dk + H + 3) / 4 * 4; }

// A block takes TOK consecutive tokens: per token the convolution, unit lengths and beta, then for all of them at once the wide
// halves of the two low-rank projections, so that a value of a2 or g2 is fetched once for TOK tokens (a prompt's launch; a step
// of few tokens takes TOK = 1 and as many blocks as tokens).  smem: act [C], then a1 | g1 of every token [TOK][ra + rg].
template <int TOK>
__global__ void __launch_bounds__(1024) cdelta_prepare_kernel(
    const float* __restrict__ proj, const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const float* __restrict__ a2t, const float* __restrict__ g2t, const int32_t* __restrict__ token_seg, const int32_t* __restrict__ seg_starts,
    const int32_t* __restrict__ seg_slots, const float* __restrict__ state, size_t state_stride, size_t conv_off, float* __restrict__ prep,
    int P, int tokens, int G, int H, int dk, int dv, int taps, int ra, int rg) {
    extern __shared__ float act[];
    dependency_wait();
    let_dependents_start();
    const int tid = threadIdx.x;
    const int C = 2 * G * dk + H * dv, N = C + H + ra + rg, LR = ra + rg;
    float* lr = act + C;                                     // [TOK][a1 | g1]
    const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    const int tb = blockIdx.x * TOK;
    for (int k = 0; k < TOK; k++) {
        const int t = tb + k;
        if (t >= tokens) break;
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
            for (int j = DR_MAX_TAPS - 1; j >= 0; j--)      // oldest input first
                if (j < taps) acc = fmaf(w[j], x[j], acc);
            act[c] = silu_f(acc);
        }
        for (int r = tid; r < LR; r += blockDim.x) lr[k * LR + r] = in[C + H + r];
        __syncthreads();
        float* out = prep + (size_t)t * P;
        for (int hq = warp; hq < 2 * G; hq += nwarps) {      // q heads, then k heads
            const float* v = act + (size_t)hq * dk;
            float ss = 0.0f;
            for (int d = lane; d < dk; d += 32) ss = fmaf(v[d], v[d], ss);
            ss = warp_sum(ss);
            float inv = 1.0f / sqrtf(ss + 1e-6f);
            if (hq < G) inv *= 1.0f / sqrtf((float)dk);
            for (int d = lane; d < dk; d += 32) out[(size_t)hq * dk + d] = v[d] * inv;
        }
        for (int c = 2 * G * dk + tid; c < C; c += blockDim.x) out[c] = act[c];
        for (int h = tid; h < H; h += blockDim.x) out[C + (size_t)H * dk + h] = sigmoid_f(in[C + h]);
        __syncthreads();                                     // act is written again for the next token
    }
    const int HK = H * dk, HV = H * dv;
    const int nt = tokens - tb < TOK ? tokens - tb : TOK;
    for (int c = tid; c < HK; c += blockDim.x) {             // the decay's logarithm; the recurrence takes exp of sums of it
        float acc[TOK];
#pragma unroll
        for (int k = 0; k < TOK; k++) acc[k] = 0.0f;
        for (int r = 0; r < ra; r++) {
            const float w = a2t[(size_t)r * HK + c];
#pragma unroll
            for (int k = 0; k < TOK; k++) acc[k] = fmaf(w, lr[k * LR + r], acc[k]);
        }
        const float rate = -expf(a_log[c / dk]), bias = dt_bias[c];
#pragma unroll
        for (int k = 0; k < TOK; k++)
            if (k < nt) prep[(size_t)(tb + k) * P + C + c] = rate * softplus_f(acc[k] + bias);
    }
    for (int c = tid; c < HV; c += blockDim.x) {
        float acc[TOK];
#pragma unroll
        for (int k = 0; k < TOK; k++) acc[k] = 0.0f;
        for (int r = 0; r < rg; r++) {
            const float w = g2t[(size_t)r * HV + c];
#pragma unroll
            for (int k = 0; k < TOK; k++) acc[k] = fmaf(w, lr[k * LR + ra + r], acc[k]);
        }
#pragma unroll
        for (int k = 0; k < TOK; k++)
            if (k < nt) prep[(size_t)(tb + k) * P + C + HK + H + c] = sigmoid_f(acc[k]);
    }
}

// What the recurrence needs of a group of M tokens and does not depend on the state, for all groups side by side: a warp per
// (token, head).  A token's group is the M tokens from the last multiple of M before its place in this step's portion of its
// request (the last group of a portion may be shorter).  Row (t, h) of `grp`, GW = 4 * dkr + 8 floats (dkr = dk rounded up to a
// multiple of four; the padding is zero):
//     e^{L_t} k_t | e^{L_t} q_t | e^{L_last - L_t} k_t | e^{L_t} | A[t][0..M-1] | B[t][0..M-1]
// with L_t the sum of the group's log decays up to and including token t, A[t][j] = sum_d k_t k_j e^{L_j - L_t} for j > t and
// B[t][j] = sum_d k_t q_j e^{L_j - L_t} for j >= t (zero elsewhere).
template <int M>
__global__ void __launch_bounds__(256) cdelta_groups_kernel(const float* __restrict__ prep, int P, const int32_t* __restrict__ token_seg,
                                                            const int32_t* __restrict__ seg_starts, float* __restrict__ grp, int tokens, int G,
                                                            int H, int dk, int dv) {
    dependency_wait();
    let_dependents_start();
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= tokens * H) return;
    const int t = unit / H, h = unit - t * H;
    const int g = h / (H / G);
    const int seg = token_seg[t];
    const int first = seg_starts[seg], i = t - first, n = seg_starts[seg + 1] - first;
    const int p = i % M, t0 = t - p;
    const int gl = n - (i - p) < M ? n - (i - p) : M;           // tokens of this group
    const int C = 2 * G * dk + H * dv, dkr = (dk + 3) / 4 * 4, GW = 4 * dkr + 8;      // eight floats for the products whatever M is: rows stay 16-byte aligned
    float* out = grp + (size_t)unit * GW;
    float a[M], b[M];
#pragma unroll
    for (int j = 0; j < M; j++) { a[j] = 0.0f; b[j] = 0.0f; }
    for (int d = lane; d < dkr; d += 32) {
        if (d >= dk) { out[d] = 0.0f; out[dkr + d] = 0.0f; out[2 * dkr + d] = 0.0f; out[3 * dkr + d] = 0.0f; continue; }
        float L[M];
        float run = 0.0f;
#pragma unroll
        for (int j = 0; j < M; j++) {
            if (j < gl) run += prep[(size_t)(t0 + j) * P + C + (size_t)h * dk + d];
            L[j] = run;
        }
        const float lt = L[p], last = L[M - 1];
        const float kt = prep[(size_t)t * P + (size_t)(G + g) * dk + d], qt = prep[(size_t)t * P + (size_t)g * dk + d];
        const float et = expf(lt);
        out[d] = et * kt;
        out[dkr + d] = et * qt;
        out[2 * dkr + d] = expf(last - lt) * kt;
        out[3 * dkr + d] = et;
#pragma unroll
        for (int j = 0; j < M; j++) {
            if (j == p) b[j] = fmaf(kt, qt, b[j]);
            else if (j > p && j < gl) {
                const float w = kt * expf(L[j] - lt);
                a[j] = fmaf(w, prep[(size_t)(t0 + j) * P + (size_t)(G + g) * dk + d], a[j]);
                b[j] = fmaf(w, prep[(size_t)(t0 + j) * P + (size_t)g * dk + d], b[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < M; j++) { a[j] = warp_sum(a[j]); b[j] = warp_sum(b[j]); }
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < M; j++) { out[4 * dkr + j] = a[j]; out[4 * dkr + M + j] = b[j]; }
    }
}

// grid (segments, H, column parts); block = cols * R threads, thread = (column, lane of the column); a lane holds KPT values of
// its column in pieces of four: piece i of lane r is rows (i*R + r)*4 .. +3 of S (zero beyond dk).
// One staged buffer: kt, qt, kf, el [chunk][dkp] each (the four vectors of the groups kernel), v [chunk][cols], beta [chunk],
// products [chunk][2][M].  Tokens are staged `chunk` at a time by cp.async, a chunk ahead of the arithmetic.
template <int KPT, int M>
__global__ void __launch_bounds__(256) cdelta_recurrence_kernel(
    const float* __restrict__ prep, int P, const float* __restrict__ grp, const float* __restrict__ proj, int N,
    const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots, float* __restrict__ state, size_t state_stride,
    size_t conv_off, float* __restrict__ o, int G, int H, int dk, int dv, int taps, int R, int cols, int chunk, int vec) {
    extern __shared__ __align__(16) float sm[];
    const int seg = blockIdx.x, h = blockIdx.y, part = blockIdx.z, tid = threadIdx.x;
    dependency_wait();
    let_dependents_start();
    const int slot = seg_slots[seg];
    if (slot < 0) return;                                    // a padding segment of a captured batch
    const int start = seg_starts[seg], n = seg_starts[seg + 1] - start;
    const int C = 2 * G * dk + H * dv;
    const int dkp = R * KPT;                                 // dk rounded up to what the lanes hold (a power of two)
    const int dkr = (dk + 3) / 4 * 4, dkr4 = dkr / 4, dkp4 = dkp / 4, GW = 4 * dkr + 8;      // eight floats for the products whatever M is: rows stay 16-byte aligned
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
        float* vec_s = sm + b * buf_floats;                  // kt | qt | kf | el, [chunk][dkp] each
        float* v_s = vec_s + 4 * chunk * dkp;
        float* b_s = v_s + chunk * cols;
        float* gram = b_s + chunk;                           // [chunk][2][M]
        const int cn = n - c0 < chunk ? n - c0 : chunk;
        const int cnp = (cn + M - 1) / M * M;                // tokens that do nothing fill the last group
        for (int e = tid; e < cnp * dkp4; e += blockDim.x) {
            const int j = e >> sh4, d4 = e & (dkp4 - 1);
            if (j < cn && d4 < dkr4) {
                const float* src = grp + ((size_t)(start + c0 + j) * H + h) * GW + d4 * 4;
#pragma unroll
                for (int w = 0; w < 4; w++) dr_cp_async16(vec_s + (w * chunk + j) * dkp + d4 * 4, src + w * dkr);
            } else {
#pragma unroll
                for (int w = 0; w < 4; w++) *reinterpret_cast<float4*>(vec_s + (w * chunk + j) * dkp + d4 * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
        for (int e = tid; e < cnp * 2 * M; e += blockDim.x) {
            const int j = e / (2 * M), w = e - j * 2 * M;
            if (j < cn) dr_cp_async4(gram + e, grp + ((size_t)(start + c0 + j) * H + h) * GW + 4 * dkr + w);
            else gram[e] = 0.0f;
        }
        for (int e = tid; e < cnp * cols; e += blockDim.x) {
            const int j = e / cols, cc = e - j * cols;
            const int c = part * cols + cc;
            if (j < cn && c < dv) dr_cp_async4(v_s + e, prep + (size_t)(start + c0 + j) * P + 2 * G * dk + (size_t)h * dv + c);
            else v_s[e] = 0.0f;
        }
        for (int j = tid; j < cnp; j += blockDim.x) {
            if (j < cn) dr_cp_async4(b_s + j, prep + (size_t)(start + c0 + j) * P + C + (size_t)H * dk + h);
            else b_s[j] = 0.0f;
        }
    };

    stage(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    int b = 0;
    for (int c0 = 0; c0 < n; c0 += chunk, b ^= 1) {
        const int cn = n - c0 < chunk ? n - c0 : chunk;
        if (c0 + chunk < n) stage(c0 + chunk, b ^ 1);        // the other buffer was read a chunk ago; the barrier below stands between
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const float* kt_s = sm + b * buf_floats;
        const float* q_s = kt_s + chunk * dkp;
        const float* kf_s = q_s + chunk * dkp;
        const float* el_s = kf_s + chunk * dkp;
        const float* v_s = el_s + chunk * dkp;
        const float* b_s = v_s + chunk * cols;
        const float* gram = b_s + chunk;
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
            float uw[M];
#pragma unroll
            for (int t = 0; t < M; t++) {
                const float* gk = gram + (j0 + t) * 2 * M;
                const float u = b_s[j0 + t] * (v_s[(j0 + t) * cols + clc] - D[t]);
#pragma unroll
                for (int j = t + 1; j < M; j++) D[j] = fmaf(gk[j], u, D[j]);
#pragma unroll
                for (int j = t; j < M; j++) E[j] = fmaf(gk[M + j], u, E[j]);
                if (live && r == 0 && j0 + t < cn) o[((size_t)(start + c0 + j0 + t) * H + h) * dv + col] = E[t];
                uw[t] = u;
            }
            const int lastj = j0 + M - 1 < cn ? j0 + M - 1 : cn - 1;       // the group's last token holds e^{L} of the whole group
            const float4* lm = reinterpret_cast<const float4*>(el_s + lastj * dkp) + r;
#pragma unroll
            for (int i = 0; i < KPT / 4; i++) {
                const float4 lv = lm[i * R];
                float x0 = lv.x * s[4 * i], x1 = lv.y * s[4 * i + 1], x2 = lv.z * s[4 * i + 2], x3 = lv.w * s[4 * i + 3];
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const float4 kv = (reinterpret_cast<const float4*>(kf_s + (j0 + t) * dkp) + r)[i * R];
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

// Single decoded tokens: everything between the projections and the output projection in ONE kernel.  grid (segments, G): a
// block has a key head's q and k and the H/G value heads that read them, so every channel of the convolution belongs to one
// block, which reads its memory, uses it and moves it on.  The block works out its heads' decays (dk values a head) and gates
// from the narrow halves a1 and g1, then takes the state's columns (H/G * dv of them) in passes of blockDim / R columns, R lanes a
// column, KPT <= 16 values a lane in pieces of four.
template <typename T, int KPT>
__global__ void __launch_bounds__(1024) cdelta_decode_kernel(
    const float* __restrict__ proj, const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const float* __restrict__ a2t, const float* __restrict__ g2t, const float* __restrict__ norm_w, float eps,
    const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots, float* __restrict__ state, size_t state_stride,
    size_t conv_off, T* __restrict__ out, int G, int H, int dk, int dv, int taps, int ra, int rg, int R) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float scal[2];
    const int seg = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    dependency_wait();
    let_dependents_start();
    const int slot = seg_slots[seg];
    if (slot < 0) return;                                    // a padding segment of a captured batch
    const int t = seg_starts[seg];
    const int HG = H / G, C = 2 * G * dk + H * dv, N = C + H + ra + rg;
    const int dkp = R * KPT, cols = HG * dv;
    float* row = state + (size_t)slot * state_stride;
    float* cs = row + conv_off;                              // [taps-1][C]
    float* q_s = sm;                                         // [dkp]
    float* k_s = q_s + dkp;                                  // [dkp]
    float* d_s = k_s + dkp;                                  // [HG][dkp] the decays (16-byte aligned like q_s and k_s)
    float* v_s = d_s + HG * dkp;                             // [cols]
    float* o_s = v_s + cols;                                 // [cols]
    float* g_s = o_s + cols;                                 // [cols] the output gate
    float* lr = g_s + cols;                                  // a1 | g1
    const float* in = proj + (size_t)t * N;

    for (int idx = tid; idx < 2 * dkp + cols; idx += blockDim.x) {
        int ch = -1;
        if (idx < dkp) { if (idx < dk) ch = g * dk + idx; }
        else if (idx < 2 * dkp) { if (idx - dkp < dk) ch = (G + g) * dk + (idx - dkp); }
        else ch = 2 * G * dk + g * cols + (idx - 2 * dkp);
        float val = 0.0f;
        if (ch >= 0) {
            float x[DR_MAX_TAPS], w[DR_MAX_TAPS];
#pragma unroll
            for (int j = 0; j < DR_MAX_TAPS; j++)
                if (j < taps) {
                    x[j] = j == 0 ? in[ch] : cs[(size_t)(taps - 1 - j) * C + ch];
                    w[j] = conv_w[(size_t)ch * taps + (taps - 1 - j)];
                }
            float acc = 0.0f;
#pragma unroll
            for (int j = DR_MAX_TAPS - 1; j >= 0; j--)
                if (j < taps) acc = fmaf(w[j], x[j], acc);
            val = silu_f(acc);
#pragma unroll
            for (int rr = 0; rr < DR_MAX_TAPS; rr++)          // row rr becomes the input of taps-2-rr tokens ago
                if (rr < taps - 1) cs[(size_t)rr * C + ch] = x[taps - 2 - rr];
        }
        if (idx < 2 * dkp) sm[idx] = val;                    // q_s, then k_s
        else v_s[idx - 2 * dkp] = val;
    }
    for (int r = tid; r < ra + rg; r += blockDim.x) lr[r] = in[C + H + r];
    __syncthreads();
    if (warp < 2) {                                          // unit length for q (and dk^-1/2) and k
        const float* v = warp == 0 ? q_s : k_s;
        float ss = 0.0f;
        for (int d = lane; d < dk; d += 32) ss = fmaf(v[d], v[d], ss);
        ss = warp_sum(ss);
        float inv = 1.0f / sqrtf(ss + 1e-6f);
        if (warp == 0) inv *= 1.0f / sqrtf((float)dk);
        if (lane == 0) scal[warp] = inv;
    }
    const int HK = H * dk, HV = H * dv;
    for (int e = tid; e < HG * dkp; e += blockDim.x) {       // this block's heads' decays (1 where the lanes hold nothing)
        const int hh = e / dkp, d = e - hh * dkp;
        float dec = 1.0f;
        if (d < dk) {
            const int c = (g * HG + hh) * dk + d;
            float acc = 0.0f;
            for (int r = 0; r < ra; r++) acc = fmaf(a2t[(size_t)r * HK + c], lr[r], acc);
            dec = expf(-expf(a_log[g * HG + hh]) * softplus_f(acc + dt_bias[c]));
        }
        d_s[e] = dec;
    }
    for (int e = tid; e < cols; e += blockDim.x) {
        const int c = g * cols + e;
        float acc = 0.0f;
        for (int r = 0; r < rg; r++) acc = fmaf(g2t[(size_t)r * HV + c], lr[ra + r], acc);
        g_s[e] = sigmoid_f(acc);
    }
    __syncthreads();
    for (int d = tid; d < dk; d += blockDim.x) { q_s[d] *= scal[0]; k_s[d] *= scal[1]; }
    __syncthreads();

    const int r = tid % R, per_pass = blockDim.x / R;
    for (int c0 = 0; c0 < cols; c0 += per_pass) {
        const int ci = c0 + tid / R;
        const bool live = ci < cols;
        const int hh = live ? ci / dv : 0, col = live ? ci % dv : 0, h = g * HG + hh;
        const float beta = sigmoid_f(in[C + h]);
        float* srow = row + ((size_t)h * dv + col) * dk;
        const float* dec = d_s + hh * dkp;
        float s[KPT];
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
        for (int i = 0; i < KPT / 4; i++) {
            const int k0 = (i * R + r) * 4;
            const float4 v = (live && k0 < dk) ? *reinterpret_cast<const float4*>(srow + k0) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float4 kv = *reinterpret_cast<const float4*>(k_s + k0), dv4 = *reinterpret_cast<const float4*>(dec + k0);
            s[4 * i] = dv4.x * v.x; s[4 * i + 1] = dv4.y * v.y; s[4 * i + 2] = dv4.z * v.z; s[4 * i + 3] = dv4.w * v.w;
            a0 = fmaf(s[4 * i], kv.x, fmaf(s[4 * i + 2], kv.z, a0));
            a1 = fmaf(s[4 * i + 1], kv.y, fmaf(s[4 * i + 3], kv.w, a1));
        }
        float dot = a0 + a1;
        for (int w = R >> 1; w > 0; w >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, w);
        const float u = beta * (v_s[live ? ci : 0] - dot);
        a0 = a1 = 0.0f;
#pragma unroll
        for (int i = 0; i < KPT / 4; i++) {
            const int k0 = (i * R + r) * 4;
            const float4 kv = *reinterpret_cast<const float4*>(k_s + k0), qv = *reinterpret_cast<const float4*>(q_s + k0);
            const float x0 = fmaf(kv.x, u, s[4 * i]), x1 = fmaf(kv.y, u, s[4 * i + 1]);
            const float x2 = fmaf(kv.z, u, s[4 * i + 2]), x3 = fmaf(kv.w, u, s[4 * i + 3]);
            a0 = fmaf(x0, qv.x, fmaf(x2, qv.z, a0));
            a1 = fmaf(x1, qv.y, fmaf(x3, qv.w, a1));
            if (live && k0 < dk) *reinterpret_cast<float4*>(srow + k0) = make_float4(x0, x1, x2, x3);
        }
        float acc = a0 + a1;
        for (int w = R >> 1; w > 0; w >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
        if (live && r == 0) o_s[ci] = acc;
    }
    __syncthreads();
    for (int hh = warp; hh < HG; hh += (int)(blockDim.x >> 5)) {                  // o / rms(o) * w * gate, a warp a head
        const int h = g * HG + hh;
        const float* ov = o_s + hh * dv;
        float ss = 0.0f;
        for (int d = lane; d < dv; d += 32) ss = fmaf(ov[d], ov[d], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int d = lane; d < dv; d += 32) out[((size_t)t * H + h) * dv + d] = from_f32<T>(((ov[d] * inv) * norm_w[d]) * g_s[hh * dv + d]);
    }
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
    const bool few = tokens <= DR_DEPENDENT_TOKENS;
    const int tok = few ? 1 : 4;
    const size_t smem = (C + (size_t)tok * (ra + rg)) * sizeof(float);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(cdelta_prepare_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(cdelta_prepare_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    const int wide = (int)((C + 31) / 32 * 32);
    if (few)                                                 // few tokens: a channel a thread, and the launch may begin early
        return launch_dependent(cdelta_prepare_kernel<1>, dim3(tokens), dim3(wide < 1024 ? wide : 1024), smem, stream, proj, conv_w, a_log, dt_bias,
                                a2t, g2t, token_seg, seg_starts, seg_slots, state, state_stride, (size_t)H * dv * dk, prep, P, tokens, G, H, dk, dv,
                                taps, ra, rg);
    return launch_plain(cdelta_prepare_kernel<4>, dim3((tokens + 3) / 4), dim3(256), smem, stream, proj, conv_w, a_log, dt_bias, a2t, g2t, token_seg,
                        seg_starts, seg_slots, state, state_stride, (size_t)H * dv * dk, prep, P, tokens, G, H, dk, dv, taps, ra, rg);
}

// Floats of the scratch between the groups kernel and the recurrence for a step of `tokens` tokens.
VK_API size_t vk_cdelta_group_floats(int tokens, int H, int dk) { return (size_t)tokens * H * (4 * ((dk + 3) / 4 * 4) + 8); }

// Two launches: the groups' vectors and products for all tokens side by side (into grp, vk_cdelta_group_floats), then the
// recurrence, which also writes the state and the convolution's memory.
VK_API int vk_cdelta_recurrence(const float* prep, const float* proj, int proj_width, const int32_t* token_seg, const int32_t* seg_starts,
                                const int32_t* seg_slots, float* state, size_t state_stride, float* grp, float* o, int segments, int tokens,
                                int G, int H, int dk, int dv, int taps, cudaStream_t stream) {
    if (segments <= 0 || tokens <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1) return VK_BAD_SHAPE;
    if (((uintptr_t)grp % 16) || ((uintptr_t)prep % 4)) return VK_BAD_ALIGNMENT;
    const int vec = dk % 4 == 0 && ((uintptr_t)state % 16) == 0 && state_stride % 4 == 0;     // the state's rows in 16-byte pieces
    if (taps > DR_MAX_TAPS || dk > 32 * DR_KPT || H > 65535) return VK_TOO_LARGE;
    const int P = cd_prep_width(G, H, dk, dv);
    const int M = tokens > 1 ? 4 : 1;                        // tokens taken together (see the kernels); no segment is longer than the step
    const bool dependent = tokens <= DR_DEPENDENT_TOKENS;
    {
        const int grid = (tokens * H + 7) / 8;
        int rc;
        if (M == 1) rc = dependent ? launch_dependent(cdelta_groups_kernel<1>, dim3(grid), dim3(256), 0, stream, prep, P, token_seg, seg_starts, grp, tokens, G, H, dk, dv)
                                   : launch_plain(cdelta_groups_kernel<1>, dim3(grid), dim3(256), 0, stream, prep, P, token_seg, seg_starts, grp, tokens, G, H, dk, dv);
        else rc = dependent ? launch_dependent(cdelta_groups_kernel<4>, dim3(grid), dim3(256), 0, stream, prep, P, token_seg, seg_starts, grp, tokens, G, H, dk, dv)
                            : launch_plain(cdelta_groups_kernel<4>, dim3(grid), dim3(256), 0, stream, prep, P, token_seg, seg_starts, grp, tokens, G, H, dk, dv);
        if (rc != 0) return rc;
    }
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
    int chunk = 64;
    auto bytes = [&](int c) { return (size_t)2 * c * (4 * R * kpt + cols + 1 + 2 * M) * sizeof(float); };
    while (chunk > 8 && (chunk / 2 >= tokens || bytes(chunk) > 64 * 1024)) chunk /= 2;
    const size_t smem = bytes(chunk);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
#define GO(K, MM)                                                                                                                        \
    {                                                                                                                                    \
        auto kern = cdelta_recurrence_kernel<K, MM>;                                                                                     \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                       \
        if (dependent)                                                                                                                   \
            return launch_dependent(kern, dim3(segments, H, parts), dim3(threads), smem, stream, prep, P, grp, proj, proj_width, seg_starts, \
                                    seg_slots, state, state_stride, (size_t)H * dv * dk, o, G, H, dk, dv, taps, R, cols, chunk, vec);    \
        return launch_plain(kern, dim3(segments, H, parts), dim3(threads), smem, stream, prep, P, grp, proj, proj_width, seg_starts,     \
                            seg_slots, state, state_stride, (size_t)H * dv * dk, o, G, H, dk, dv, taps, R, cols, chunk, vec);            \
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

static size_t cdelta_decode_smem(int G, int H, int dk, int dv, int ra, int rg) {
    const size_t HG = H / G;
    return (2 * 32 * 16 + 3 * HG * dv + HG * 32 * 16 + ra + rg) * sizeof(float);       // the most the kernel can ask for
}

// Whether the one-kernel form for single decoded tokens takes these sizes (key size a multiple of four up to 512).
VK_API int vk_cdelta_decode_takes(int G, int H, int dk, int dv, int taps, int ra, int rg) {
    return G > 0 && H > 0 && H % G == 0 && dk % 4 == 0 && dk >= 4 && dk <= 32 * 16 && dv > 0 && taps >= 1 && taps <= DR_MAX_TAPS && ra > 0 &&
           rg > 0 && cdelta_decode_smem(G, H, dk, dv, ra, rg) <= 160 * 1024;
}

// Every segment is ONE token.  proj, a2t, g2t as for vk_cdelta_prepare; out [tokens][H*dv] in dtype; the state is read and written.
VK_API int vk_cdelta_decode(const float* proj, const float* conv_w, const float* a_log, const float* dt_bias, const float* a2t, const float* g2t,
                            const float* norm_w, float eps, const int32_t* seg_starts, const int32_t* seg_slots, float* state,
                            size_t state_stride, void* out, int segments, int G, int H, int dk, int dv, int taps, int ra, int rg, int dtype,
                            cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (!vk_cdelta_decode_takes(G, H, dk, dv, taps, ra, rg)) return VK_BAD_SHAPE;
    if (((uintptr_t)state % 16) || state_stride % 4 || G > 65535) return VK_BAD_ALIGNMENT;
    const int HG = H / G, cols = HG * dv;
    int R = 1;
    while ((dk + R - 1) / R > 16) R *= 2;                    // a lane holds at most sixteen values of a column
    while (R < 32 && cols * R * 2 <= 256 && (dk + R - 1) / R > 4) R *= 2;      // few columns: more lanes a column
    int kpt = 4;
    while (kpt * R < dk) kpt *= 2;
    const int want = (cols * R + 31) / 32 * 32;
    const int threads = want < 256 ? 256 : (want > 1024 ? 1024 : want);
    const size_t smem = (size_t)(2 * R * kpt + 3 * cols + HG * R * kpt + ra + rg) * sizeof(float);
#define GO(TT, K)                                                                                                                       \
    {                                                                                                                                   \
        auto kern = cdelta_decode_kernel<TT, K>;                                                                                        \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                      \
        return launch_dependent(kern, dim3(segments, G), dim3(threads), smem, stream, proj, conv_w, a_log, dt_bias, a2t, g2t, norm_w, eps, \
                                seg_starts, seg_slots, state, state_stride, (size_t)H * dv * dk, (TT*)out, G, H, dk, dv, taps, ra, rg, R); \
    }
    if (dtype == 0) {
        if (kpt == 4) GO(float, 4) else if (kpt == 8) GO(float, 8) else GO(float, 16)
    } else {
        if (kpt == 4) GO(__nv_bfloat16, 4) else if (kpt == 8) GO(__nv_bfloat16, 8) else GO(__nv_bfloat16, 16)
    }
#undef GO
}
