// The gated delta rule over a prompt's portion in chunks: what can be worked out without the state is worked out for all
// chunks at once, and only a short pass per chunk runs in order.
//
// For a chunk of C tokens with the state S before it, L_t = ln(g_1 .. g_t) (the decays up to t, inside the chunk):
//     A[t][i] = beta_t e^(L_t - L_i) (k_t . k_i)   (i < t)          the updates u_t solve  (I + A) U = diag(beta) V - diag(beta e^L) K S
//     so with  U' = (I + A)^-1 diag(beta) V   and   W = (I + A)^-1 diag(beta e^L) K :     U = U' - W S
//     P[t][i] = e^(L_t - L_i) (q_t . k_i)          (i <= t)         O = diag(e^L) Q S + P U
//     S <- e^(L_C) S + (diag(e^(L_C - L)) K)^T U
// Kernel 1 (a block per chunk and head, all chunks of the step side by side): L, A, P, the triangular solve for U' and W by
// forward substitution, and the scaled copies of Q and K; everything goes to a scratch.  Kernel 2 (a block per request, head
// and slice of the state's columns) walks the request's chunks in order with the state slice in shared memory: three small
// products a chunk.  All float32 on CUDA cores: the decays, beta, the unit vectors and the state are 32-bit quantities of this
// mixer, and the sums are of float32 values.  The results equal the token-by-token recurrence up to the order of sums.
// A chunk that reaches past its segment's end is filled with tokens that do nothing.  Inputs are the rows `delta_prepare`
// writes (q | k | v | log decay | beta).
//
// The form with a decay per head AND key channel (template flag CH; inputs are the rows `cdelta_prepare` writes, q | k | v | log
// decay [H][dk] | beta [H] | ..): L_t is a vector over the key channels, and the decays no longer leave the sums over dk:
//     A[t][i] = beta_t sum_d k_t[d] k_i[d] e^(L_t[d] - L_i[d]),     P[t][i] = sum_d q_t[d] k_i[d] e^(L_t[d] - L_i[d])
// (an exponential per pair and channel; for 4 x 4 pieces below the diagonal it is split as e^(L_t - r) e^(r - L_i) with r = L of the
// piece's last column token, both factors at most 1, which makes eight exponentials a channel for a piece instead of sixteen; a piece's
// channels are shared out over two to eight threads),
// W and Qg carry e^(L_t[d]), KgT carries e^(L_C[d] - L_i[d]), and the state's rows decay by the vector e^(L_C[d]), which follows
// U' in the scratch.  Everything else, the triangular solve and the scan included, is the same code.
#include "common.cuh"

namespace vk {

constexpr int DC_THREADS = 256;
constexpr int DC_MAX_TAPS = 16;
constexpr int DC_MAX_DK = 128;

__device__ __forceinline__ void dc_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Which segment and which of its chunks the step's chunk number `b` is; false when the step has fewer chunks.
template <int C>
__device__ __forceinline__ bool find_chunk(const int32_t* seg_starts, int segments, int b, int& seg, int& c0) {
    int acc = 0;
    for (int s = 0; s < segments; s++) {
        const int n = seg_starts[s + 1] - seg_starts[s];
        const int nc = (n + C - 1) / C;
        if (b < acc + nc) { seg = s; c0 = (b - acc) * C; return true; }
        acc += nc;
    }
    return false;
}

// Floats of scratch for one (chunk, head):  W [C][dk] | Qg [C][dk] | KgT [dk][C] | P [C][C] | U' [C][dv] | e^(L_C) and padding [4]
// (with a decay per channel: e^(L_C[d]) for every d, padded to a multiple of four)
__host__ __device__ __forceinline__ size_t dc_stride(int C, int dk, int dv, bool ch = false) {
    return (size_t)C * (3 * dk + C + dv) + (ch ? (dk + 3) / 4 * 4 : 4);
}

// grid (chunks of the step, H); 256 threads = a 16 x 16 arrangement for the products.
template <int C, bool CH>
__global__ void __launch_bounds__(DC_THREADS) delta_chunk_prepare_kernel(const float* __restrict__ prep, int P, const int32_t* __restrict__ seg_starts,
                                                                         const int32_t* __restrict__ seg_slots, int segments,
                                                                         float* __restrict__ scratch, int G, int H, int dk, int dv) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float L[C], beta[C];
    __shared__ int where[2];
    const int tid = threadIdx.x, h = blockIdx.y;
    if (tid == 0) {
        int seg = -1, c0 = 0;
        if (!find_chunk<C>(seg_starts, segments, blockIdx.x, seg, c0) || seg_slots[seg] < 0) seg = -1;
        where[0] = seg;
        where[1] = c0;
    }
    __syncthreads();
    const int seg = where[0], c0 = where[1];
    if (seg < 0) return;
    const int start = seg_starts[seg], n = seg_starts[seg + 1] - start;
    const int cn = n - c0 < C ? n - c0 : C;
    const int Cq = 2 * G * dk + H * dv, g = h / (H / G);
    const int ldk = dk + 1, ldc = C + 1, nr = dv + dk;
    float* k_s = sm;                       // [C][dk+1]
    float* q_s = k_s + C * ldk;            // [C][dk+1]
    float* A_s = q_s + C * ldk;            // [C][C+1]
    float* P_s = A_s + C * ldc;            // [C][C+1]
    float* x_s = P_s + C * ldc;            // [C][dv + dk]: the right sides, then the solutions
    float* Lv = x_s + C * nr;              // CH: [C][dk+1], the decays' logarithms of every channel, then their running sums

    if (tid < C) {
        const bool on = tid < cn;
        if (!CH) L[tid] = on ? prep[(size_t)(start + c0 + tid) * P + Cq + h] : 0.0f;
        beta[tid] = on ? prep[(size_t)(start + c0 + tid) * P + Cq + (CH ? H * dk : H) + h] : 0.0f;
    }
    if (CH) {
        for (int e = tid; e < C * dk; e += DC_THREADS) {
            const int t = e / dk, d = e - t * dk;
            Lv[t * ldk + d] = t < cn ? prep[(size_t)(start + c0 + t) * P + Cq + (size_t)h * dk + d] : 0.0f;
        }
    }
    for (int e = tid; e < C * dk; e += DC_THREADS) {
        const int t = e / dk, d = e - t * dk;
        const float* row = prep + (size_t)(start + c0 + t) * P;
        k_s[t * ldk + d] = t < cn ? row[(size_t)(G + g) * dk + d] : 0.0f;
        q_s[t * ldk + d] = t < cn ? row[(size_t)g * dk + d] : 0.0f;
    }
    __syncthreads();
    if (CH) {                               // the decays' logarithms summed up to each token, a channel a thread
        for (int d = tid; d < dk; d += DC_THREADS) {
            float acc = 0.0f;
            for (int t = 0; t < C; t++) { acc += Lv[t * ldk + d]; Lv[t * ldk + d] = acc; }
        }
    } else if (tid == 0) {
        float acc = 0.0f;
        for (int t = 0; t < C; t++) { acc += L[t]; L[t] = acc; }
    }
    __syncthreads();
    for (int e = tid; e < C * nr; e += DC_THREADS) {
        const int t = e / nr, c = e - t * nr;
        float v = 0.0f;
        if (t < cn) v = c < dv ? beta[t] * prep[(size_t)(start + c0 + t) * P + 2 * G * dk + (size_t)h * dv + c]
                               : beta[t] * expf(CH ? Lv[t * ldk + (c - dv)] : L[t]) * k_s[t * ldk + (c - dv)];
        x_s[e] = v;
    }
    if (CH) {
        // k k^T and q k^T with the pairs' decays, in 4 x 4 pieces.  The exponentials make a piece expensive, so the channels of a
        // piece are shared out: the threads that would have a piece above the diagonal take half of the channels of the piece
        // mirrored below it, and with C = 32 (a quarter as many pieces as threads) every piece's channels are cut in four again.
        // The parts of a piece are added in a fixed order, one barrier a part.
        constexpr int NB = C / 4, NPC = NB * NB, S = DC_THREADS / NPC;
        for (int e = tid; e < C * ldc; e += DC_THREADS) { A_s[e] = 0.0f; P_s[e] = 0.0f; }
        const int piece = tid % NPC, dsplit = tid / NPC;
        int ty = piece / NB, tx = piece % NB;
        const bool mirror = tx > ty;
        if (mirror) { const int z = ty; ty = tx; tx = z; }
        const bool diag = tx == ty;
        const int parts = diag ? S : 2 * S, part = diag ? dsplit : dsplit * 2 + (mirror ? 1 : 0);
        float kk[4][4], qk[4][4];
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int b = 0; b < 4; b++) kk[a][b] = qk[a][b] = 0.0f;
        for (int d = part * dk / parts; d < (part + 1) * dk / parts; d++) {
            float kt[4], qt[4], ki[4], lt[4], li[4];
#pragma unroll
            for (int a = 0; a < 4; a++) {
                kt[a] = k_s[(ty * 4 + a) * ldk + d];
                qt[a] = q_s[(ty * 4 + a) * ldk + d];
                ki[a] = k_s[(tx * 4 + a) * ldk + d];
                lt[a] = Lv[(ty * 4 + a) * ldk + d];
                li[a] = Lv[(tx * 4 + a) * ldk + d];
            }
            if (diag) {                     // the exponent of every pair by itself: six below the diagonal, none on or above it
#pragma unroll
                for (int a = 0; a < 4; a++)
#pragma unroll
                    for (int b = 0; b <= a; b++) {
                        const float w = b < a ? expf(lt[a] - lt[b]) * ki[b] : ki[b];
                        kk[a][b] = fmaf(kt[a], w, kk[a][b]);
                        qk[a][b] = fmaf(qt[a], w, qk[a][b]);
                    }
            } else {                        // every row token comes after every column token: e^(L_t - r) e^(r - L_i), r = L of the last
                const float ref = li[3];    // column token, both factors at most 1
#pragma unroll
                for (int a = 0; a < 4; a++) {
                    const float et = expf(lt[a] - ref);
                    kt[a] *= et;
                    qt[a] *= et;
                    ki[a] *= expf(ref - li[a]);
                }
#pragma unroll
                for (int a = 0; a < 4; a++)
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        kk[a][b] = fmaf(kt[a], ki[b], kk[a][b]);
                        qk[a][b] = fmaf(qt[a], ki[b], qk[a][b]);
                    }
            }
        }
        for (int ph = 0; ph < 2 * S; ph++) {
            __syncthreads();
            if (part == ph) {
#pragma unroll
                for (int a = 0; a < 4; a++)
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        const int t = ty * 4 + a, i = tx * 4 + b;
                        if (i < t) A_s[t * ldc + i] += beta[t] * kk[a][b];
                        if (i <= t) P_s[t * ldc + i] += qk[a][b];
                    }
            }
        }
    } else
    // k k^T and q k^T in 4 x 4 pieces: thread (ty, tx) has rows ty*4.., columns tx*4.. (C = 64: one piece a thread; C = 32: a quarter idle)
    {
        const int ty = tid / 16, tx = tid % 16;
        if (ty * 4 < C && tx * 4 < C) {
            float kk[4][4], qk[4][4];
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int b = 0; b < 4; b++) kk[a][b] = qk[a][b] = 0.0f;
            if (tx <= ty) {                 // pieces above the diagonal are never read
                for (int d = 0; d < dk; d++) {
                    float kt[4], qt[4], ki[4];
#pragma unroll
                    for (int a = 0; a < 4; a++) {
                        kt[a] = k_s[(ty * 4 + a) * ldk + d];
                        qt[a] = q_s[(ty * 4 + a) * ldk + d];
                        ki[a] = k_s[(tx * 4 + a) * ldk + d];
                    }
#pragma unroll
                    for (int a = 0; a < 4; a++)
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            kk[a][b] = fmaf(kt[a], ki[b], kk[a][b]);
                            qk[a][b] = fmaf(qt[a], ki[b], qk[a][b]);
                        }
                }
            }
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const int t = ty * 4 + a, i = tx * 4 + b;
                    const float ratio = i <= t ? expf(L[t] - L[i]) : 0.0f;
                    A_s[t * ldc + i] = i < t ? beta[t] * ratio * kk[a][b] : 0.0f;
                    P_s[t * ldc + i] = ratio * qk[a][b];
                }
        }
    }
    __syncthreads();
    // (I + A) X = right sides, a column a thread, rows in order
    for (int c = tid; c < nr; c += DC_THREADS) {
        for (int t = 1; t < C; t++) {
            float a0 = x_s[t * nr + c], a1 = 0.0f;
            int i = 0;
            for (; i + 1 < t; i += 2) {
                a0 = fmaf(-A_s[t * ldc + i], x_s[i * nr + c], a0);
                a1 = fmaf(-A_s[t * ldc + i + 1], x_s[(i + 1) * nr + c], a1);
            }
            if (i < t) a0 = fmaf(-A_s[t * ldc + i], x_s[i * nr + c], a0);
            x_s[t * nr + c] = a0 + a1;
        }
    }
    __syncthreads();
    float* out = scratch + ((size_t)blockIdx.x * H + h) * dc_stride(C, dk, dv, CH);
    float* W_g = out;
    float* Q_g = W_g + C * dk;
    float* K_g = Q_g + C * dk;             // transposed: [dk][C]
    float* P_g = K_g + C * dk;
    float* U_g = P_g + C * C;
    const float LC = CH ? 0.0f : L[C - 1];
    for (int e = tid; e < C * dk; e += DC_THREADS) {
        const int t = e / dk, d = e - t * dk;
        W_g[e] = x_s[t * nr + dv + d];
        Q_g[e] = expf(CH ? Lv[t * ldk + d] : L[t]) * q_s[t * ldk + d];
    }
    for (int e = tid; e < dk * C; e += DC_THREADS) {
        const int d = e / C, i = e - d * C;
        K_g[e] = expf(CH ? Lv[(C - 1) * ldk + d] - Lv[i * ldk + d] : LC - L[i]) * k_s[i * ldk + d];
    }
    for (int e = tid; e < C * C; e += DC_THREADS) P_g[e] = P_s[(e / C) * ldc + e % C];
    for (int e = tid; e < C * dv; e += DC_THREADS) U_g[e] = x_s[(e / dv) * nr + e % dv];
    if (CH) {
        for (int d = tid; d < dk; d += DC_THREADS) U_g[C * dv + d] = expf(Lv[(C - 1) * ldk + d]);
    } else if (tid == 0) U_g[C * dv] = expf(LC);
}

// grid (segments, H, column slices); 256 threads; COLS columns of the state a block.  A chunk's operands arrive by cp.async in one of
// two buffers, a chunk ahead.
template <int C, int COLS, bool CH>
__global__ void __launch_bounds__(256) delta_chunk_scan_kernel(const float* __restrict__ scratch, const float* __restrict__ proj, int N,
                                                               const int32_t* __restrict__ seg_starts, const int32_t* __restrict__ seg_slots,
                                                               float* __restrict__ state, size_t state_stride, size_t conv_off,
                                                               float* __restrict__ o, int G, int H, int dk, int dv, int taps) {
    extern __shared__ __align__(16) float sm[];
    constexpr int T = 256, RG = T / COLS;                   // row groups: a thread has column tid % COLS and rows tid / COLS + RG * j
    const int seg = blockIdx.x, h = blockIdx.y, part = blockIdx.z, tid = threadIdx.x;
    const int slot = seg_slots[seg];
    if (slot < 0) return;
    const int start = seg_starts[seg], n = seg_starts[seg + 1] - start;
    int base = 0;                                            // the step's chunk number of this segment's first chunk
    for (int s = 0; s < seg; s++) base += (seg_starts[s + 1] - seg_starts[s] + C - 1) / C;
    const int Cq = 2 * G * dk + H * dv;                     // N: floats of a row of proj
    const size_t stride = dc_stride(C, dk, dv, CH);
    const int c = tid % COLS, r0 = tid / COLS, col = part * COLS + c;
    const bool live = col < dv;
    float* row = state + (size_t)slot * state_stride;

    const int opnd = C * (3 * dk + C);      // floats of a chunk's W, Qg, KgT and P, which lie in this order
    const int lds = dk + 4, ldu = C + 4;    // the state's and the updates' slices are kept transposed: a column's values lie together,
    float* S_s = sm;                        // [COLS][dk + 4]        so that every load below is 16 bytes
    float* U_s = S_s + COLS * lds;          // [COLS][C + 4]
    float* bufs = U_s + COLS * ldu;         // two buffers of `opnd` floats
    for (int e = tid; e < dk * COLS; e += T) {
        const int cc = e / dk, d = e - cc * dk, gc = part * COLS + cc;
        S_s[cc * lds + d] = gc < dv ? row[((size_t)h * dv + gc) * dk + d] : 0.0f;
    }
    for (int e = tid; e < opnd / 4; e += T) dc_cp_async16(bufs + e * 4, scratch + ((size_t)base * H + h) * stride + e * 4);
    asm volatile("cp.async.commit_group;" ::: "memory");
    int turn = 0;
    for (int c0 = 0, b = base; c0 < n; c0 += C, b++, turn ^= 1) {
        const float* in = scratch + ((size_t)b * H + h) * stride;
        const int cn = n - c0 < C ? n - c0 : C;
        __syncthreads();                                     // the other buffer is free, the state slice is written
        if (c0 + C < n) {
            const float* nxt = in + (size_t)H * stride;
            for (int e = tid; e < opnd / 4; e += T) dc_cp_async16(bufs + (turn ^ 1) * opnd + e * 4, nxt + e * 4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        const float* W_s = bufs + turn * opnd;  // [C][dk]
        const float* Q_s = W_s + C * dk;        // [C][dk]
        const float* K_s = Q_s + C * dk;        // [dk][C]
        const float* P_s = K_s + C * dk;        // [C][C]
        const float* U_g = in + (size_t)opnd;
        float up[C / RG];                                    // U' of this thread's places
#pragma unroll
        for (int j = 0; j < C / RG; j++) up[j] = live ? U_g[(size_t)(r0 + RG * j) * dv + col] : 0.0f;
        const float gC = CH ? 0.0f : U_g[(size_t)C * dv];
        float gv[DC_MAX_DK / RG];                            // CH: the chunk's decay of each of this thread's rows of the state
        if (CH) {
#pragma unroll
            for (int j = 0; j < DC_MAX_DK / RG; j++) gv[j] = r0 + RG * j < dk ? U_g[(size_t)C * dv + r0 + RG * j] : 0.0f;
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        // W S and Qg S together: the state's values are loaded once for both
        float ws[C / RG], qs[C / RG];
#pragma unroll
        for (int j = 0; j < C / RG; j++) ws[j] = qs[j] = 0.0f;
        const float* sc = S_s + c * lds;
        for (int d = 0; d < dk; d += 4) {
            const float4 sv = *reinterpret_cast<const float4*>(sc + d);
#pragma unroll
            for (int j = 0; j < C / RG; j++) {
                const float4 w = *reinterpret_cast<const float4*>(W_s + (r0 + RG * j) * dk + d);
                const float4 q = *reinterpret_cast<const float4*>(Q_s + (r0 + RG * j) * dk + d);
                ws[j] = fmaf(w.x, sv.x, fmaf(w.y, sv.y, fmaf(w.z, sv.z, fmaf(w.w, sv.w, ws[j]))));
                qs[j] = fmaf(q.x, sv.x, fmaf(q.y, sv.y, fmaf(q.z, sv.z, fmaf(q.w, sv.w, qs[j]))));
            }
        }
        float* uc = U_s + c * ldu;
#pragma unroll
        for (int j = 0; j < C / RG; j++) uc[r0 + RG * j] = up[j] - ws[j];          // U = U' - W S
        __syncthreads();
        // O = Qg S + P U
        for (int i = 0; i < C; i += 4) {
            const float4 uv = *reinterpret_cast<const float4*>(uc + i);
#pragma unroll
            for (int j = 0; j < C / RG; j++) {
                const float4 w = *reinterpret_cast<const float4*>(P_s + (r0 + RG * j) * C + i);
                qs[j] = fmaf(w.x, uv.x, fmaf(w.y, uv.y, fmaf(w.z, uv.z, fmaf(w.w, uv.w, qs[j]))));
            }
        }
#pragma unroll
        for (int j = 0; j < C / RG; j++) {
            const int t = r0 + RG * j;
            if (live && t < cn) o[((size_t)(start + c0 + t) * H + h) * dv + col] = qs[j];
        }
        // S <- e^(L_C) S + KgT U: a thread has rows r0 + RG * j of its column; the new values wait in registers until every
        // thread has read the old state
        float s_new[DC_MAX_DK / RG];
#pragma unroll
        for (int j = 0; j < DC_MAX_DK / RG; j++) s_new[j] = 0.0f;
        for (int i = 0; i < C; i += 4) {
            const float4 uv = *reinterpret_cast<const float4*>(uc + i);
#pragma unroll
            for (int j = 0; j < DC_MAX_DK / RG; j++) {
                const int d = r0 + RG * j;
                if (d < dk) {
                    const float4 w = *reinterpret_cast<const float4*>(K_s + d * C + i);
                    s_new[j] = fmaf(w.x, uv.x, fmaf(w.y, uv.y, fmaf(w.z, uv.z, fmaf(w.w, uv.w, s_new[j]))));
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < DC_MAX_DK / RG; j++) {
            const int d = r0 + RG * j;
            if (d < dk) S_s[c * lds + d] = fmaf(CH ? gv[j] : gC, S_s[c * lds + d], s_new[j]);
        }
    }
    __syncthreads();
    for (int e = tid; e < dk * COLS; e += T) {
        const int cc = e / dk, d = e - cc * dk, gc = part * COLS + cc;
        if (gc < dv) row[((size_t)h * dv + gc) * dk + d] = S_s[cc * lds + d];
    }
    // the convolution's memory: the last taps-1 inputs of the request, this step's tokens included
    if (taps > 1) {
        float* cs = row + conv_off;
        const int nb = gridDim.y * gridDim.z, bi = h * gridDim.z + part;
        for (int ch = bi * T + tid; ch < Cq; ch += nb * T) {
            float keep[DC_MAX_TAPS];
#pragma unroll
            for (int rr = 0; rr < DC_MAX_TAPS; rr++)
                if (rr < taps - 1) {
                    const int src = n - (taps - 1) + rr;
                    keep[rr] = src >= 0 ? proj[(size_t)(start + src) * N + ch] : cs[(size_t)(rr + n) * Cq + ch];
                }
#pragma unroll
            for (int rr = 0; rr < DC_MAX_TAPS; rr++)
                if (rr < taps - 1) cs[(size_t)rr * Cq + ch] = keep[rr];
        }
    }
}

}  // namespace vk

using namespace vk;

static int dc_chunk(int dk) { return dk <= 64 ? 64 : 32; }

// Whether the chunked kernels take these sizes (else the token-by-token kernel does the work).
VK_API int vk_delta_chunked_takes(int G, int H, int dk, int dv, int taps) {
    const int C = dc_chunk(dk);
    return G > 0 && H > 0 && H % G == 0 && dk % 4 == 0 && dk >= 8 && dk <= 128 && dv > 0 && dv % 4 == 0 && dv <= 256 && taps >= 1 &&
           taps <= DC_MAX_TAPS;
}

// Bytes of scratch for a step of `tokens` tokens in `segments` segments.
VK_API size_t vk_delta_chunked_scratch_bytes(int tokens, int segments, int H, int dk, int dv) {
    const int C = dc_chunk(dk);
    return ((size_t)tokens / C + segments + 1) * H * dc_stride(C, dk, dv) * sizeof(float);
}

template <bool CH>
static int delta_chunked_launch(const float* prep, int prep_width, const float* proj, int proj_width, const int32_t* seg_starts,
                                const int32_t* seg_slots, float* state, size_t state_stride, float* o, float* scratch, int segments, int tokens,
                                int G, int H, int dk, int dv, int taps, cudaStream_t stream) {
    if (segments <= 0 || tokens <= 0) return VK_OK;
    if (!vk_delta_chunked_takes(G, H, dk, dv, taps)) return VK_BAD_SHAPE;
    if (((uintptr_t)scratch % 16) || H > 65535) return VK_BAD_ALIGNMENT;
    const int C = dc_chunk(dk);
    const int chunks = tokens / C + segments;
    const size_t smem1 = (size_t)(2 * C * (dk + 1) + 2 * C * (C + 1) + C * (dv + dk) + (CH ? C * (dk + 1) : 0)) * sizeof(float);
    constexpr int COLS = 16;
    const size_t smem2 = (size_t)(COLS * (dk + 4) + COLS * (C + 4) + 2 * C * (3 * dk + C)) * sizeof(float);
    const int parts = (dv + COLS - 1) / COLS;
    if (smem1 > 200 * 1024 || smem2 > 200 * 1024) return VK_TOO_LARGE;
#define GO(CC)                                                                                                                             \
    {                                                                                                                                      \
        auto k1 = delta_chunk_prepare_kernel<CC, CH>;                                                                                      \
        auto k2 = delta_chunk_scan_kernel<CC, COLS, CH>;                                                                                   \
        cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);                                                 \
        cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);                                                 \
        int rc = launch_plain(k1, dim3(chunks, H), dim3(DC_THREADS), smem1, stream, prep, prep_width, seg_starts, seg_slots, segments,    \
                              scratch, G, H, dk, dv);                                                                                      \
        if (rc != 0) return rc;                                                                                                            \
        return launch_plain(k2, dim3(segments, H, parts), dim3(256), smem2, stream, (const float*)scratch, proj, proj_width, seg_starts,  \
                            seg_slots, state, state_stride, (size_t)H * dv * dk, o, G, H, dk, dv, taps);                                   \
    }
    if (C == 64) GO(64) else GO(32)
#undef GO
}

// prep [tokens][prep width] as delta_prepare leaves it; proj as for the token-by-token kernel; o [tokens][H*dv] float32.
VK_API int vk_delta_chunked(const float* prep, int prep_width, const float* proj, const int32_t* seg_starts, const int32_t* seg_slots, float* state,
                            size_t state_stride, float* o, float* scratch, int segments, int tokens, int G, int H, int dk, int dv, int taps,
                            cudaStream_t stream) {
    return delta_chunked_launch<false>(prep, prep_width, proj, 2 * G * dk + 2 * H * dv + 2 * H, seg_starts, seg_slots, state, state_stride, o,
                                       scratch, segments, tokens, G, H, dk, dv, taps, stream);
}

// The form with a decay per head and key channel: prep as cdelta_prepare leaves it, proj rows of proj_width floats (the
// convolution's inputs first).  The sizes are those vk_delta_chunked_takes.
VK_API size_t vk_cdelta_chunked_scratch_bytes(int tokens, int segments, int H, int dk, int dv) {
    const int C = dc_chunk(dk);
    return ((size_t)tokens / C + segments + 1) * H * dc_stride(C, dk, dv, true) * sizeof(float);
}

VK_API int vk_cdelta_chunked(const float* prep, int prep_width, const float* proj, int proj_width, const int32_t* seg_starts,
                             const int32_t* seg_slots, float* state, size_t state_stride, float* o, float* scratch, int segments, int tokens,
                             int G, int H, int dk, int dv, int taps, cudaStream_t stream) {
    return delta_chunked_launch<true>(prep, prep_width, proj, proj_width, seg_starts, seg_slots, state, state_stride, o, scratch, segments,
                                      tokens, G, H, dk, dv, taps, stream);
}
