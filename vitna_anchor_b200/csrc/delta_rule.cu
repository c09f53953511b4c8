// The gated delta rule: a recurrent mixer with a matrix state per head.
//
// A token's projections arrive as one float32 row
//     proj[t] = [ q (G*dk) | k (G*dk) | v (H*dv) | gate (H*dv) | b (H) | a (H) ]
// (G key heads of size dk shared by H/G value heads of size dv each).  Three kernels follow the product:
//
//  1. prepare: a causal convolution over time on every q, k and v channel (taps weights per channel, the last one
//     the current token's; inputs before a request's first position are zero, inputs before this step's first token
//     come from the request's state), silu; q and k heads scaled to unit length, q also by dk^-1/2;
//     beta = sigmoid(b); decay = exp(-exp(A_log) * softplus(a + dt_bias)) (its logarithm is what is handed on).
//  2. recurrence, per request and head, token after token, on the state S [dk][dv]:
//         S <- decay S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//     The columns of S never meet, so a column lives in the registers of R neighbouring lanes (dk/R values each)
//     and the two sums over dk are lane shuffles; a block holds a head's columns (or a part of them) and stages
//     a chunk of tokens' q, k, v, decay and beta at a time in shared memory, a chunk ahead of the arithmetic.  The state is kept transposed
//     ([H][dv][dk]) so that a lane's values are contiguous.  The same kernel moves the last taps-1 inputs of the
//     convolution into the request's state once the tokens of the step have been read.
//  3. gate: o / rms(o) over dv, times a weight shared by the heads, times silu(gate), in the compute dtype.
//
// Everything here is float32; only the result of 3 is rounded to the compute dtype for the output projection.
// A request's per-layer state row is [H*dv*dk floats of S^T][(taps-1)*C floats of convolution inputs], C = 2 G dk + H dv.
#include "delta_common.cuh"

namespace vk {

// One block per token.  smem: act [C].  A channel's inputs are all asked for before any is used: with few tokens in the step
// the kernel is as long as its chain of trips to memory.
__global__ void __launch_bounds__(1024) delta_prepare_kernel(
    const float* __restrict__ proj, const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const int32_t* __restrict__ token_seg, const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
    const float* __restrict__ state, size_t state_stride, size_t conv_off, float* __restrict__ prep, int P, int G, int H, int dk, int dv,
    int taps) {
    extern __shared__ float act[];
    dependency_wait();
    let_dependents_start();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int C = 2 * G * dk + H * dv, N = C + H * dv + 2 * H;
    const int seg = token_seg[t];
    const int i = t - seg_starts[seg];                       // place of the token in this step's portion of its request
    const int slot = seg_slots[seg];
    const float* old = slot >= 0 ? state + (size_t)slot * state_stride + conv_off : nullptr;   // [taps-1][C]
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
        out[C + h] = -expf(a_log[h]) * softplus_f(a + dt_bias[h]);       // the decay's logarithm; the recurrence takes exp of it
        out[C + H + h] = 1.0f / (1.0f + expf(-b));
    }
}

// grid (segments, H, column parts); block = cols * R threads, thread = (column, lane of the column).  A lane holds KPT values
// of its column in pieces of four: piece i of lane r is rows (i*R + r)*4 .. +3 of S (zero beyond dk), so that the lanes of a
// column read neighbouring 16 bytes of a staged key.  Tokens are staged `chunk` at a time into one of two buffers by
// cp.async (16 bytes a copy: prep's rows are padded to a multiple of four floats), a chunk ahead of the arithmetic.
//
// Inside a chunk the tokens are taken M at a time.  With S the state before token 1 of such a group and, for a column,
//     D_j = (S^T k_j),  E_j = (S^T q_j)                           (2M sums over dk, independent of one another)
// the M steps of the recurrence need no further sum over dk: for t = 1..M
//     D_j, E_j <- g_t D_j, g_t E_j  (j >= t);    u_t = beta_t (v_t - D_t);    D_j += (k_t.k_j) u_t  (j > t);
//     E_j += (k_t.q_j) u_t  (j >= t);            o_t = E_t
// and then S <- (g_1..g_M) S + sum_t (g_{t+1}..g_M) u_t k_t.  The products k_t.k_j and k_t.q_j are the same for every column
// of the head; the block works them out once per chunk.  So the chain from token to token is a handful of scalar
// operations, and the long sums and the lanes' shuffles of M tokens overlap.  A group that reaches past the segment's end is
// filled with tokens that do nothing (beta 0, decay 1, zero vectors).  M = 1 (single decoded tokens) is the plain recurrence.
template <int KPT, int M>
__global__ void __launch_bounds__(256) delta_recurrence_kernel(
    const float* __restrict__ prep, int P, const float* __restrict__ proj, const int32_t* __restrict__ seg_starts,
    const int32_t* __restrict__ seg_slots, float* __restrict__ state, size_t state_stride, size_t conv_off, float* __restrict__ o, int G, int H,
    int dk, int dv, int taps, int R, int cols, int chunk, int vec) {
    extern __shared__ __align__(16) float sm[];
    const int seg = blockIdx.x, h = blockIdx.y, part = blockIdx.z, tid = threadIdx.x;
    dependency_wait();
    let_dependents_start();
    const int slot = seg_slots[seg];
    if (slot < 0) return;                                    // a padding segment of a captured batch
    const int start = seg_starts[seg], n = seg_starts[seg + 1] - start;
    const int C = 2 * G * dk + H * dv, N = C + H * dv + 2 * H;
    const int g = h / (H / G);
    const int dkp = R * KPT;                                 // dk rounded up to what the lanes hold (a power of two)
    const int dk4 = dk / 4, dkp4 = dkp / 4;
    const int sh4 = 31 - __clz(dkp4);
    float* row = state + (size_t)slot * state_stride;

    // one buffer: q [chunk][dkp], k [chunk][dkp], v [chunk][cols], log decay [chunk], beta [chunk], products [chunk/M][2][M][M]
    const int buf_floats = chunk * (2 * dkp + cols + 2 + 2 * M);
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
        } else {                                             // dk is no multiple of four, or a row is not 16-byte aligned
#pragma unroll
            for (int e = 0; e < 4; e++) s[4 * i + e] = (live && k0 + e < dk) ? srow[k0 + e] : 0.0f;
        }
    }

    auto stage = [&](int c0, int b) {
        float* q_s = sm + b * buf_floats;
        float* k_s = q_s + chunk * dkp;
        float* v_s = k_s + chunk * dkp;
        float* d_s = v_s + chunk * cols;
        float* b_s = d_s + chunk;
        const int cn = n - c0 < chunk ? n - c0 : chunk;
        for (int e = tid; e < cn * dkp4; e += blockDim.x) {
            const int j = e >> sh4, d4 = e & (dkp4 - 1);     // dkp4 is a power of two
            const float* p = prep + (size_t)(start + c0 + j) * P;
            if (!vec) {
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const int d = d4 * 4 + x;
                    if (d < dk) {
                        dr_cp_async4(q_s + e * 4 + x, p + (size_t)g * dk + d);
                        dr_cp_async4(k_s + e * 4 + x, p + (size_t)(G + g) * dk + d);
                    } else {
                        q_s[e * 4 + x] = 0.0f;
                        k_s[e * 4 + x] = 0.0f;
                    }
                }
            } else if (d4 < dk4) {
                dr_cp_async16(q_s + e * 4, p + (size_t)g * dk + d4 * 4);
                dr_cp_async16(k_s + e * 4, p + (size_t)(G + g) * dk + d4 * 4);
            } else {
                *reinterpret_cast<float4*>(q_s + e * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                *reinterpret_cast<float4*>(k_s + e * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
        for (int j = 0; j < cn; j++) {
            for (int cc = tid; cc < cols; cc += blockDim.x) {
                const int c = part * cols + cc;
                if (c < dv) dr_cp_async4(v_s + j * cols + cc, prep + (size_t)(start + c0 + j) * P + 2 * G * dk + (size_t)h * dv + c);
                else v_s[j * cols + cc] = 0.0f;
            }
        }
        for (int j = tid; j < cn; j += blockDim.x) {         // the decay arrives as its logarithm
            dr_cp_async4(d_s + j, prep + (size_t)(start + c0 + j) * P + C + h);
            dr_cp_async4(b_s + j, prep + (size_t)(start + c0 + j) * P + C + H + h);
        }
        const int cnp = (cn + M - 1) / M * M;                // tokens that do nothing fill the last group
        for (int e = cn * dkp + tid; e < cnp * dkp; e += blockDim.x) { q_s[e] = 0.0f; k_s[e] = 0.0f; }
        for (int e = cn * cols + tid; e < cnp * cols; e += blockDim.x) v_s[e] = 0.0f;
        for (int j = cn + tid; j < cnp; j += blockDim.x) { d_s[j] = 0.0f; b_s[j] = 0.0f; }
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
        const float* q_s = sm + b * buf_floats;
        const float* k_s = q_s + chunk * dkp;
        const float* v_s = k_s + chunk * dkp;
        float* d_s = sm + b * buf_floats + chunk * (2 * dkp + cols);
        const float* b_s = d_s + chunk;
        float* gram = d_s + 2 * chunk;                       // [groups][2][M][M]: k_t.k_j, then k_t.q_j
        const int cnp = (cn + M - 1) / M * M;
        for (int j = tid; j < cnp; j += blockDim.x) d_s[j] = expf(d_s[j]);
        for (int e = tid; e < cnp * 2 * M; e += blockDim.x) {        // entry e = ((group * 2 + which) * M + t) * M + j
            const int jj = e % M, t = (e / M) % M, which = (e / (M * M)) % 2, grp = e / (2 * M * M);
            float acc = 0.0f;
            if (which ? jj >= t : jj > t) {
                const float4* x = reinterpret_cast<const float4*>(k_s + (grp * M + t) * dkp);
                const float4* y = reinterpret_cast<const float4*>((which ? q_s : k_s) + (grp * M + jj) * dkp);
                float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
                for (int ii = 0; ii < dkp4; ii++) {           // neighbouring threads start at neighbouring pieces: other banks
                    const int i = (ii + tid) & (dkp4 - 1);
                    const float4 xv = x[i], yv = y[i];
                    a0 = fmaf(xv.x, yv.x, a0); a1 = fmaf(xv.y, yv.y, a1); a2 = fmaf(xv.z, yv.z, a2); a3 = fmaf(xv.w, yv.w, a3);
                }
                acc = (a0 + a1) + (a2 + a3);
            }
            gram[e] = acc;
        }
        __syncthreads();
        const int clc = cl < cols ? cl : 0;
        for (int j0 = 0; j0 < cn; j0 += M) {
            float D[M], E[M];
#pragma unroll
            for (int t = 0; t < M; t++) {
                const float4* kk = reinterpret_cast<const float4*>(k_s + (j0 + t) * dkp) + r;
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
            float uw[M], dec[M];
#pragma unroll
            for (int t = 0; t < M; t++) {
                dec[t] = d_s[j0 + t];
#pragma unroll
                for (int j = t; j < M; j++) { D[j] *= dec[t]; E[j] *= dec[t]; }
                const float u = b_s[j0 + t] * (v_s[(j0 + t) * cols + clc] - D[t]);
#pragma unroll
                for (int j = t + 1; j < M; j++) D[j] = fmaf(gk[t * M + j], u, D[j]);
#pragma unroll
                for (int j = t; j < M; j++) E[j] = fmaf(gq[t * M + j], u, E[j]);
                if (live && r == 0 && j0 + t < cn) o[((size_t)(start + c0 + j0 + t) * H + h) * dv + col] = E[t];
                uw[t] = u;
            }
            float all = 1.0f;                                // decays after token t, and of the whole group
#pragma unroll
            for (int t = M - 1; t >= 0; t--) { uw[t] *= all; all *= dec[t]; }
#pragma unroll
            for (int i = 0; i < KPT / 4; i++) {
                float x0 = all * s[4 * i], x1 = all * s[4 * i + 1], x2 = all * s[4 * i + 2], x3 = all * s[4 * i + 3];
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

    // the convolution's memory: the last taps-1 inputs of the request, this step's tokens included.  The blocks
    // of a segment share the channels.
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

// A warp per (token, head): out = o / rms(o) * w * silu(gate).
template <typename T>
__global__ void __launch_bounds__(256) delta_gate_kernel(const float* __restrict__ o, const float* __restrict__ proj, const float* __restrict__ norm_w,
                                                         float eps, T* __restrict__ out, int tokens, int G, int H, int dk, int dv) {
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    dependency_wait();
    let_dependents_start();
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

// Single decoded tokens: everything between the projections and the output projection in ONE kernel.  grid (segments, G): a
// block has a key head's q and k and the H/G value heads that read them, so every channel of the convolution belongs to one
// block, which reads its memory, uses it and moves it on.  The state's columns (H/G * dv of them) are taken in passes of
// blockDim / R columns, R lanes a column, KPT <= 16 values a lane in pieces of four as in the kernel above; the block is as wide
// as the columns need (up to 1,024 threads), since every pass is a trip to memory.
template <typename T, int KPT>
__global__ void __launch_bounds__(1024) delta_decode_kernel(
    const float* __restrict__ proj, const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const float* __restrict__ norm_w, float eps, const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
    float* __restrict__ state, size_t state_stride, size_t conv_off, T* __restrict__ out, int G, int H, int dk, int dv, int taps, int R) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float scal[2];
    const int seg = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    dependency_wait();
    let_dependents_start();
    const int slot = seg_slots[seg];
    if (slot < 0) return;                                    // a padding segment of a captured batch
    const int t = seg_starts[seg];
    const int HG = H / G, C = 2 * G * dk + H * dv, N = C + H * dv + 2 * H;
    const int dkp = R * KPT, cols = HG * dv;
    float* row = state + (size_t)slot * state_stride;
    float* cs = row + conv_off;                              // [taps-1][C]
    float* q_s = sm;                                         // [dkp]
    float* k_s = q_s + dkp;                                  // [dkp]
    float* v_s = k_s + dkp;                                  // [cols]
    float* o_s = v_s + cols;                                 // [cols]
    const float* in = proj + (size_t)t * N;

    // the convolution with silu, and its memory moved on by the thread that read it
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
        sm[idx] = val;                                       // q_s, k_s and v_s lie in this order
    }
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
    __syncthreads();
    for (int d = tid; d < dk; d += blockDim.x) { q_s[d] *= scal[0]; k_s[d] *= scal[1]; }
    __syncthreads();

    const int r = tid % R, per_pass = blockDim.x / R;
    for (int c0 = 0; c0 < cols; c0 += per_pass) {
        const int ci = c0 + tid / R;
        const bool live = ci < cols;
        const int hh = live ? ci / dv : 0, col = live ? ci % dv : 0, h = g * HG + hh;
        const float b = in[C + H * dv + h], a = in[C + H * dv + H + h];
        const float dec = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
        const float beta = 1.0f / (1.0f + expf(-b));
        float* srow = row + ((size_t)h * dv + col) * dk;
        float s[KPT];
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
        for (int i = 0; i < KPT / 4; i++) {
            const int k0 = (i * R + r) * 4;
            const float4 v = (live && k0 < dk) ? *reinterpret_cast<const float4*>(srow + k0) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float4 kv = *reinterpret_cast<const float4*>(k_s + k0);
            s[4 * i] = v.x; s[4 * i + 1] = v.y; s[4 * i + 2] = v.z; s[4 * i + 3] = v.w;
            a0 = fmaf(v.x, kv.x, fmaf(v.z, kv.z, a0));
            a1 = fmaf(v.y, kv.y, fmaf(v.w, kv.w, a1));
        }
        float dot = a0 + a1;
        for (int w = R >> 1; w > 0; w >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, w);
        const float u = beta * (v_s[live ? ci : 0] - dec * dot);
        a0 = a1 = 0.0f;
#pragma unroll
        for (int i = 0; i < KPT / 4; i++) {
            const int k0 = (i * R + r) * 4;
            const float4 kv = *reinterpret_cast<const float4*>(k_s + k0), qv = *reinterpret_cast<const float4*>(q_s + k0);
            const float x0 = fmaf(kv.x, u, dec * s[4 * i]), x1 = fmaf(kv.y, u, dec * s[4 * i + 1]);
            const float x2 = fmaf(kv.z, u, dec * s[4 * i + 2]), x3 = fmaf(kv.w, u, dec * s[4 * i + 3]);
            a0 = fmaf(x0, qv.x, fmaf(x2, qv.z, a0));
            a1 = fmaf(x1, qv.y, fmaf(x3, qv.w, a1));
            if (live && k0 < dk) *reinterpret_cast<float4*>(srow + k0) = make_float4(x0, x1, x2, x3);
        }
        float acc = a0 + a1;
        for (int w = R >> 1; w > 0; w >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
        if (live && r == 0) o_s[ci] = acc;
    }
    __syncthreads();
    for (int hh = warp; hh < HG; hh += (int)(blockDim.x >> 5)) {                  // o / rms(o) * w * silu(gate), a warp a head
        const int h = g * HG + hh;
        const float* ov = o_s + hh * dv;
        float ss = 0.0f;
        for (int d = lane; d < dv; d += 32) ss = fmaf(ov[d], ov[d], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int d = lane; d < dv; d += 32)
            out[((size_t)t * H + h) * dv + d] = from_f32<T>(((ov[d] * inv) * norm_w[d]) * silu_f(in[C + (size_t)h * dv + d]));
    }
}

}  // namespace vk

using namespace vk;

// Floats of one request's state in one layer, rounded up to a multiple of four (rows stay 16-byte aligned).
VK_API size_t vk_delta_state_floats(int G, int H, int dk, int dv, int taps) {
    return ((size_t)H * dv * dk + (size_t)(taps > 1 ? taps - 1 : 0) * (2 * (size_t)G * dk + (size_t)H * dv) + 3) / 4 * 4;
}

// Floats of a row of prep: q | k | v | log decay | beta, padded to a multiple of four.
VK_API int vk_delta_prep_width(int G, int H, int dk, int dv) { return (2 * G * dk + H * dv + 2 * H + 3) / 4 * 4; }

// proj [tokens][C + H*dv + 2H] float32; conv_w [C][taps]; state [slots][state_stride] float32; prep [tokens][vk_delta_prep_width].
VK_API int vk_delta_prepare(const float* proj, const float* conv_w, const float* a_log, const float* dt_bias, const int32_t* token_seg,
                            const int32_t* seg_starts, const int32_t* seg_slots, const float* state, size_t state_stride, float* prep, int tokens,
                            int G, int H, int dk, int dv, int taps, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1) return VK_BAD_SHAPE;
    const int P = vk_delta_prep_width(G, H, dk, dv);
    if (taps > DR_MAX_TAPS) return VK_TOO_LARGE;
    const size_t C = 2 * (size_t)G * dk + (size_t)H * dv;
    const size_t smem = C * sizeof(float);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // few tokens (decoding): the launch may begin under the end of the kernel before it; a prompt's launches stay ordinary, since
    // blocks that wait for a long kernel before them would hold the places its own later blocks need
    const int wide = (int)((C + 31) / 32 * 32);
    const int threads = tokens <= DR_DEPENDENT_TOKENS ? (wide < 1024 ? wide : 1024) : 256;     // few tokens: a channel a thread
    if (tokens <= DR_DEPENDENT_TOKENS)
        return launch_dependent(delta_prepare_kernel, dim3(tokens), dim3(threads), smem, stream, proj, conv_w, a_log, dt_bias, token_seg, seg_starts,
                                seg_slots, state, state_stride, (size_t)H * dv * dk, prep, P, G, H, dk, dv, taps);
    return launch_plain(delta_prepare_kernel, dim3(tokens), dim3(256), smem, stream, proj, conv_w, a_log, dt_bias, token_seg, seg_starts,
                        seg_slots, state, state_stride, (size_t)H * dv * dk, prep, P, G, H, dk, dv, taps);
}

VK_API int vk_delta_recurrence(const float* prep, const float* proj, const int32_t* seg_starts, const int32_t* seg_slots, float* state,
                               size_t state_stride, float* o, int segments, int tokens, int G, int H, int dk, int dv, int taps,
                               cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1) return VK_BAD_SHAPE;
    const int vec = dk % 4 == 0 && ((uintptr_t)prep % 16) == 0 && ((uintptr_t)state % 16) == 0 && state_stride % 4 == 0;     // 16-byte copies
    if (taps > DR_MAX_TAPS || dk > 32 * DR_KPT || H > 65535) return VK_TOO_LARGE;
    const int P = vk_delta_prep_width(G, H, dk, dv);
    // lanes a column: as few as keep a lane's values within DR_KPT, more for small heads (shorter sums between two tokens)
    int R = 1;
    while ((dk + R - 1) / R > DR_KPT) R *= 2;
    while (R < 32 && (dk + R - 1) / R > 8) R *= 2;           // eight values a lane measured best (2,048 tokens: 0.73 ms against 0.81 at 4 or 16)
    while (R < 32 && dv * R < 128 && (dk + R - 1) / R > 4) R *= 2;
    int kpt = 4;
    while (kpt * R < dk) kpt *= 2;
    int cols = dv;
    while (cols * R > 256) cols = (cols + 1) / 2;            // wide heads: several blocks share a head's columns
    // few segments (a prompt): the chain from token to token is what takes the time, and it is shortest when a multiprocessor's
    // schedulers have one warp each to serve (measured: blocks of 64 threads 0.62 ms, of 256 threads 0.92 ms for 2,048 tokens of
    // nine heads of 64 x 64); narrower blocks also put a head's columns on more multiprocessors
    while ((long long)segments * H * ((dv + cols - 1) / cols) < 148 && cols * R > 64 && cols % 2 == 0) cols /= 2;
    const int parts = (dv + cols - 1) / cols;
    const int threads = ((cols * R + 31) / 32) * 32;
    const int longest = tokens > 0 ? tokens : 1;             // no segment is longer than the step
    const int M = longest > 1 ? 4 : 1;                       // tokens taken together (see the kernel)
    int chunk = 64;
    while (chunk > 8 && (chunk / 2 >= longest || (size_t)2 * chunk * (2 * R * kpt + cols + 2 + 2 * M) * sizeof(float) > 64 * 1024)) chunk /= 2;
    const size_t smem = (size_t)2 * chunk * (2 * R * kpt + cols + 2 + 2 * M) * sizeof(float);
    if (smem > 200 * 1024) return VK_TOO_LARGE;
#define GO(K, MM)                                                                                                                      \
    {                                                                                                                                  \
        auto kern = delta_recurrence_kernel<K, MM>;                                                                                    \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                     \
        if (tokens <= DR_DEPENDENT_TOKENS)                                                                                             \
            return launch_dependent(kern, dim3(segments, H, parts), dim3(threads), smem, stream, prep, P, proj, seg_starts, seg_slots, \
                                    state, state_stride, (size_t)H * dv * dk, o, G, H, dk, dv, taps, R, cols, chunk, vec);            \
        return launch_plain(kern, dim3(segments, H, parts), dim3(threads), smem, stream, prep, P, proj, seg_starts, seg_slots, state,  \
                            state_stride, (size_t)H * dv * dk, o, G, H, dk, dv, taps, R, cols, chunk, vec);                           \
    }
    if (M == 1) {
        if (kpt == 4) GO(4, 1) else if (kpt == 8) GO(8, 1) else if (kpt == 16) GO(16, 1) else GO(32, 1)
    } else {
        if (kpt == 4) GO(4, 4) else if (kpt == 8) GO(8, 4) else if (kpt == 16) GO(16, 4) else GO(32, 4)
    }
#undef GO
    return launch_status();
}

VK_API int vk_delta_gate(const float* o, const float* proj, const float* norm_w, float eps, void* out, int tokens, int G, int H, int dk, int dv,
                         int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VK_OK;
    if (G <= 0 || H <= 0 || dk <= 0 || dv <= 0) return VK_BAD_SHAPE;
    const int grid = (tokens * H + 7) / 8;
    if (tokens <= DR_DEPENDENT_TOKENS) {
        if (dtype == 0) return launch_dependent(delta_gate_kernel<float>, dim3(grid), dim3(256), 0, stream, o, proj, norm_w, eps, (float*)out, tokens, G, H, dk, dv);
        return launch_dependent(delta_gate_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, o, proj, norm_w, eps, (__nv_bfloat16*)out, tokens, G, H, dk, dv);
    }
    if (dtype == 0) return launch_plain(delta_gate_kernel<float>, dim3(grid), dim3(256), 0, stream, o, proj, norm_w, eps, (float*)out, tokens, G, H, dk, dv);
    return launch_plain(delta_gate_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, o, proj, norm_w, eps, (__nv_bfloat16*)out, tokens, G, H, dk, dv);
}

// Whether the one-kernel form for single decoded tokens takes these sizes.
VK_API int vk_delta_decode_takes(int G, int H, int dk, int dv, int taps) {
    return G > 0 && H > 0 && H % G == 0 && dk % 4 == 0 && dk >= 4 && dk <= 32 * 16 && dv > 0 && taps >= 1 && taps <= DR_MAX_TAPS &&
           (size_t)(2 * 32 * 16 + 2 * (H / G) * dv) * sizeof(float) <= 160 * 1024;
}

// Every segment is ONE token.  proj as above; out [tokens][H*dv] in dtype; the state is read and written.
VK_API int vk_delta_decode(const float* proj, const float* conv_w, const float* a_log, const float* dt_bias, const float* norm_w, float eps,
                           const int32_t* seg_starts, const int32_t* seg_slots, float* state, size_t state_stride, void* out, int segments, int G,
                           int H, int dk, int dv, int taps, int dtype, cudaStream_t stream) {
    if (segments <= 0) return VK_OK;
    if (!vk_delta_decode_takes(G, H, dk, dv, taps)) return VK_BAD_SHAPE;
    if (((uintptr_t)state % 16) || state_stride % 4 || G > 65535) return VK_BAD_ALIGNMENT;
    const int cols = (H / G) * dv;
    int R = 1;
    while ((dk + R - 1) / R > 16) R *= 2;                    // a lane holds at most sixteen values of a column
    while (R < 32 && cols * R * 2 <= 256 && (dk + R - 1) / R > 4) R *= 2;      // few columns: more lanes a column
    int kpt = 4;
    while (kpt * R < dk) kpt *= 2;
    const int want = (cols * R + 31) / 32 * 32;
    const int threads = want < 256 ? 256 : (want > 1024 ? 1024 : want);
    const size_t smem = (size_t)(2 * R * kpt + 2 * cols) * sizeof(float);
#define GO(TT, K)                                                                                                                       \
    {                                                                                                                                   \
        auto kern = delta_decode_kernel<TT, K>;                                                                                         \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                      \
        return launch_dependent(kern, dim3(segments, G), dim3(threads), smem, stream, proj, conv_w, a_log, dt_bias, norm_w, eps, seg_starts, \
                                seg_slots, state, state_stride, (size_t)H * dv * dk, (TT*)out, G, H, dk, dv, taps, R);                  \
    }
    if (dtype == 0) {
        if (kpt == 4) GO(float, 4) else if (kpt == 8) GO(float, 8) else GO(float, 16)
    } else {
        if (kpt == 4) GO(__nv_bfloat16, 4) else if (kpt == 8) GO(__nv_bfloat16, 8) else GO(__nv_bfloat16, 16)
    }
#undef GO
}
