// Linear attention whose decay is computed from the input, one number per key channel and token, over a
// float32 state that is carried from step to step:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        S is [dk][dv] per request slot and head, a_t in (0, 1]^dk
//   o_t = S_t^T q_t
//
// Two mixers feed it (prep kernel, `mode`):
//   0  "gla"     q = zq * qscale, k = zk, v = zv, log a = logsigmoid(za + bias) / tau
//   1  "hgrn2"   q = silu(zq), v = zv, f = low + (1 - low) sigmoid(zf + bias), a = f, k = 1 - f
// The prep kernel writes q, k, v and g = log a as float32 (everything that enters the recurrence is 32-bit);
// g is clamped at -80 so that sums of it stay finite (exp(-80) is zero beside anything it is added to).
//
// Routes (the same numbers up to float32 rounding):
//   scan     one CTA per (segment, head) walks the tokens one by one: decoded tokens and short portions
//   chunked  long portions in chunks of C tokens, with b_i = g_1 + ... + g_i inside a chunk (b_n = B):
//            (1) every chunk: U = sum_j (k_j exp(B - b_j)) v_j^T and B, in parallel;
//            (2) per (segment, head): the state before every chunk, S <- diag(exp(B)) S + U, the last into the slot;
//            (3) every chunk: o_i = S^T (q_i exp(b_i)) + sum_(j<=i) [sum_e q_i[e] k_j[e] exp(b_i[e] - b_j[e])] v_j.
//            Every exponent is a sum of g's, hence <= 0: nothing overflows however strong the decay.
//
// tok_seg[t] (ascending) names the segment of token t, seg_slot[s] its state slot.  A segment whose first
// token sits at position 0 starts from a zero state whatever the slot holds.
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {

constexpr float G_FLOOR = -80.f;

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float log_sigmoidf_(float z) {      // log(1 / (1 + e^-z)) without overflow
    return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

struct Parts {            // a float32 product, possibly split-K parts
    const float* p;
    int nsplit;
    size_t stride;
    int ld;
};
__device__ __forceinline__ float load(const Parts& a, size_t t, int col) {
    const size_t idx = t * a.ld + col;
    float v = a.p[idx];
    for (int s = 1; s < a.nsplit; ++s) v += a.p[idx + (size_t)s * a.stride];
    return v;
}

// ---- prep ---------------------------------------------------------------------------------------------
// grid (T, slices of the columns), any block: columns of head-major [H * dk] / [H * dv] rows.  mode 0: the decay's
// logits are a low-rank product, z = A2 (columns a0 .. a0 + rank of the main product) + bias, taken here in float32.
template <typename WT>
__global__ void prep_kernel(Parts main, int q0, int k0, int v0, int a0, const WT* __restrict__ a2, int rank,
                            const float* __restrict__ bias, const float* __restrict__ low, float qscale,
                            float inv_tau, int mode, float* __restrict__ q, float* __restrict__ k,
                            float* __restrict__ v, float* __restrict__ g, int QW, int VW) {
    extern __shared__ float lr[];       // [rank]
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    if (mode == 0) {
        for (int r = threadIdx.x; r < rank; r += blockDim.x) lr[r] = load(main, t, a0 + r);
        __syncthreads();
    }
    const int span = (max(QW, VW) + gridDim.y - 1) / gridDim.y, c0 = blockIdx.y * span, c1 = c0 + span;
    for (int i = c0 + threadIdx.x; i < min(QW, c1); i += blockDim.x) {
        const float zq = load(main, t, q0 + i);
        if (mode == 0) {
            float za = 0.f;
            const WT* row = a2 + (size_t)i * rank;
            for (int r = 0; r < rank; ++r) za = fmaf(lr[r], to_float(row[r]), za);
            za += bias[i];
            q[t * QW + i] = zq * qscale;
            k[t * QW + i] = load(main, t, k0 + i);
            g[t * QW + i] = fmaxf(log_sigmoidf_(za) * inv_tau, G_FLOOR);
        } else {
            const float s = sigmoidf_(load(main, t, a0 + i) + bias[i]);
            const float lo = low[i];
            const float f = lo + (1.f - lo) * s;
            q[t * QW + i] = zq * sigmoidf_(zq);
            k[t * QW + i] = 1.f - f;
            g[t * QW + i] = fmaxf(logf(f), G_FLOOR);
        }
    }
    for (int i = c0 + threadIdx.x; i < min(VW, c1); i += blockDim.x) v[t * VW + i] = load(main, t, v0 + i);
}

// ---- behind the recurrence: one norm per head, an optional multiplier ------------------------------------------
// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w[:] * silu(gate[t, h dv + :]); one warp per (t, h)
template <typename OT>
__global__ void head_norm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, Parts gate,
                                 int gate0, OT* __restrict__ out, size_t pairs, int H, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t th = (size_t)blockIdx.x * warps + warp;
    if (th >= pairs) return;
    const size_t t = th / H;
    const int h = (int)(th - t * H);
    const float* row = o + th * dv;
    float ss = 0.f;
    for (int e = lane; e < dv; e += 32) ss += row[e] * row[e];
    ss = warp_sum(ss);
    const float rinv = 1.f / sqrtf(ss / (float)dv + eps);
    for (int e = lane; e < dv; e += 32) {
        float y = row[e] * rinv * w[e];
        if (gate.p) {
            const float z = load(gate, t, gate0 + h * dv + e);
            y *= z * sigmoidf_(z);
        }
        out[th * dv + e] = from_float<OT>(y);
    }
}

struct Rec {
    const float* q;           // [T][H * dk]
    const float* k;
    const float* g;
    const float* v;           // [T][H * dv]
    float* state;             // [slots][H][dk][dv]
    float* out;               // [T][H * dv]
    const int* tok_seg;
    const int* seg_slot;
    const int* positions;
    int T, H, dk, dv, writable;
};

__device__ __forceinline__ void segment_range(const int* tok_seg, int T, int seg, int& begin, int& end) {
    int lo = 0, hi = T;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tok_seg[mid] < seg) lo = mid + 1; else hi = mid; }
    begin = lo;
    hi = T;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tok_seg[mid] <= seg) lo = mid + 1; else hi = mid; }
    end = lo;
}

// ---- token by token ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
scan_kernel(const Rec a, int max_tokens) {
    extern __shared__ __align__(16) float sm[];
    const int dk = a.dk, dv = a.dv;
    float* St = sm;                     // [dk][dv]
    float* qs = St + dk * dv;           // [dk]
    float* ks = qs + dk;
    float* as = ks + dk;
    float* vs = as + dk;                // [dv]
    const int R = max(1, (int)blockDim.x / dv);
    float* po = vs + dv;                // [R][dv]
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.x, h = blockIdx.y;
    int t0, t1;
    segment_range(a.tok_seg, a.T, seg, t0, t1);
    if (t1 <= t0 || (max_tokens > 0 && t1 - t0 > max_tokens)) return;
    float* slot = a.state + ((size_t)a.seg_slot[seg] * a.H + h) * dk * dv;
    const bool fresh = a.positions[t0] == 0;
    const bool by4 = (dk * dv) % 4 == 0 && ((uintptr_t)a.state & 15) == 0;      // a slot then starts on 16 bytes
    if (by4) {
        for (int i = 4 * threadIdx.x; i < dk * dv; i += 4 * blockDim.x)
            *reinterpret_cast<float4*>(St + i) = fresh ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(slot + i);
    } else {
        for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) St[i] = fresh ? 0.f : slot[i];
    }
    const int QW = a.H * dk, VW = a.H * dv;
    for (int t = t0; t < t1; ++t) {
        for (int i = threadIdx.x; i < dk; i += blockDim.x) {
            const size_t idx = (size_t)t * QW + h * dk + i;
            qs[i] = a.q[idx];
            ks[i] = a.k[idx];
            as[i] = expf(a.g[idx]);
        }
        for (int j = threadIdx.x; j < dv; j += blockDim.x) vs[j] = a.v[(size_t)t * VW + h * dv + j];
        __syncthreads();
        for (int u = threadIdx.x; u < R * dv; u += blockDim.x) {
            const int r = u / dv, j = u - r * dv;
            const float vj = vs[j];
            float part = 0.f;
            for (int i = r; i < dk; i += R) {
                const float s = fmaf(as[i], St[i * dv + j], ks[i] * vj);
                St[i * dv + j] = s;
                part = fmaf(s, qs[i], part);
            }
            po[u] = part;
        }
        __syncthreads();
        for (int j = threadIdx.x; j < dv; j += blockDim.x) {
            float o = 0.f;
            for (int r = 0; r < R; ++r) o += po[r * dv + j];
            a.out[(size_t)t * VW + h * dv + j] = o;
        }
    }
    __syncthreads();
    if (a.writable) {
        if (by4) {
            for (int i = 4 * threadIdx.x; i < dk * dv; i += 4 * blockDim.x)
                *reinterpret_cast<float4*>(slot + i) = *reinterpret_cast<const float4*>(St + i);
        } else {
            for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) slot[i] = St[i];
        }
    }
}

// ---- tiles of the chunked route -------------------------------------------------------------------------------
// A chunk's rows sit in shared memory with their channels rounded up to fours (zeros beyond the head's own), so that
// every product below runs on float4 loads and register tiles; rows beyond the chunk's tokens are zero as well.
constexpr int SB = 16;                 // tokens per block of the scores inside a chunk
__device__ __forceinline__ int round4(int n) { return (n + 3) & ~3; }
inline size_t round4h(int n) { return (size_t)((n + 3) & ~3); }
// floats behind the output kernel's q, v and scores: b and k of the chunk, later rows of S (never fewer than four)
__host__ __device__ inline int stage_floats(int dkp, int dvp, int C) { return max(2 * C * (dkp + 4), 4 * dvp); }
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// 16 bytes from global to shared memory without a register in between; zeros instead where `real` is false
__device__ __forceinline__ void copy16(float* dst, const float* src, bool real) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = real ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copies_done() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// dst[j][0 .. dpad) = src[t0 + j][col0 .. col0 + d) for j < n, zero elsewhere; C rows, ld apart, a warp per row.
// `vec`: d is a multiple of 4 and every row starts on 16 bytes, so that the rows go as asynchronous copies
// (the caller waits with copies_done() before its barrier).
__device__ __forceinline__ void load_rows(float* dst, int ld, const float* __restrict__ src, size_t W, int t0, int n,
                                          int col0, int d, int dpad, int C, int vec) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int j = warp; j < C; j += warps) {
        const float* row = src + (size_t)(t0 + min(j, n - 1)) * W + col0;
        if (vec) {
            for (int i = 4 * lane; i < d; i += 128) copy16(dst + j * ld + i, row + i, j < n);
        } else {
            for (int i = lane; i < dpad; i += 32) dst[j * ld + i] = (j < n && i < d) ? row[i] : 0.f;
        }
    }
}

// in place: b[j][i] <- b[0][i] + ... + b[j][i], one channel per thread (rows beyond the tokens hold zeros, so they
// end up with the last token's sum)
__device__ __forceinline__ void running_sum_rows(float* b, int ld, int dpad, int C) {
    for (int i = threadIdx.x; i < dpad; i += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < C; ++j) {
            acc += b[j * ld + i];
            b[j * ld + i] = acc;
        }
    }
}

__device__ __forceinline__ void fma4(float (&acc)[4], float s, const float4& v) {
    acc[0] = fmaf(s, v.x, acc[0]);
    acc[1] = fmaf(s, v.y, acc[1]);
    acc[2] = fmaf(s, v.z, acc[2]);
    acc[3] = fmaf(s, v.w, acc[3]);
}

// ---- chunked (1): every chunk's own contribution U [dk][dv] and its total log decay B [dk] -------------------
// chunks: {segment, first token, tokens (<= C), index of the chunk in its segment}; U holds dk * dv + dk floats a
// chunk and head.  A thread owns up to 8 x 8 of U: key channels {4 ti .. +3, 64 + 4 ti .. +3} by value channels
// {4 te .. +3, 64 + 4 te .. +3}, so that a warp's loads of a row are contiguous.
__global__ void __launch_bounds__(256)
chunk_state_kernel(const Rec a, const int* __restrict__ chunks, float* __restrict__ U, int C, int vec) {
    extern __shared__ __align__(16) float sm[];
    const int dk = a.dk, dv = a.dv, dkp = round4(dk), dvp = round4(dv), LK = dkp + 4;
    float* b = sm;                      // [C][LK]   running log decay
    float* ks = b + C * LK;             // [C][LK]   k_j exp(B - b_j)
    float* vs = ks + C * LK;            // [C][dvp]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y;
    const int t0 = chunks[4 * c + 1], n = chunks[4 * c + 2];
    const size_t QW = (size_t)a.H * dk, VW = (size_t)a.H * dv;
    load_rows(b, LK, a.g, QW, t0, n, h * dk, dk, dkp, C, vec);
    load_rows(ks, LK, a.k, QW, t0, n, h * dk, dk, dkp, C, vec);
    load_rows(vs, dvp, a.v, VW, t0, n, h * dv, dv, dvp, C, vec);
    copies_done();
    __syncthreads();
    running_sum_rows(b, LK, dkp, C);
    __syncthreads();
    const float* B = b + (n - 1) * LK;
    for (int j = threadIdx.x >> 5; j < n; j += blockDim.x >> 5)
        for (int i = threadIdx.x & 31; i < dkp; i += 32) ks[j * LK + i] *= expf(B[i] - b[j * LK + i]);
    __syncthreads();
    float* u = U + ((size_t)c * a.H + h) * (dk * dv + dk);
    const int ti = threadIdx.x >> 4, te = threadIdx.x & 15, gk = dkp >> 2, ge = dvp >> 2;
    for (int ia = ti; ia < gk; ia += 32)
        for (int eb = te; eb < ge; eb += 32) {
            const int i0 = 4 * ia, i1 = 4 * (ia + 16), e0 = 4 * eb, e1 = 4 * (eb + 16);
            const bool hi = ia + 16 < gk, he = eb + 16 < ge;
            float acc[8][2][4];
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[r][0][x] = acc[r][1][x] = 0.f;
            const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < n; ++j) {
                const float4 k0 = ld4(ks + j * LK + i0), k1 = hi ? ld4(ks + j * LK + i1) : zero;
                const float4 v0 = ld4(vs + j * dvp + e0), v1 = he ? ld4(vs + j * dvp + e1) : zero;
                const float kk[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    fma4(acc[r][0], kk[r], v0);
                    fma4(acc[r][1], kk[r], v1);
                }
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int i = (r < 4 ? i0 : i1) + (r & 3);
                if (i >= dk || (r >= 4 && !hi)) continue;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int e = half ? e1 : e0;
                    if (half && !he) continue;
                    float* dst = u + (size_t)i * dv + e;
                    if (vec) {
                        *reinterpret_cast<float4*>(dst) = make_float4(acc[r][half][0], acc[r][half][1], acc[r][half][2], acc[r][half][3]);
                    } else {
#pragma unroll
                        for (int x = 0; x < 4; ++x)
                            if (e + x < dv) dst[x] = acc[r][half][x];
                    }
                }
            }
        }
    for (int i = threadIdx.x; i < dk; i += blockDim.x) u[dk * dv + i] = B[i];
}

// ---- chunked (2): states at the chunks' starts -----------------------------------------------------------
// seg_chunks: {segment, first chunk, chunks, first token}.  U[c] is replaced by the state BEFORE chunk c.
__global__ void __launch_bounds__(256)
chunk_prefix_kernel(const Rec a, const int* __restrict__ seg_chunks, float* __restrict__ U) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y;
    const int seg = seg_chunks[4 * s], c0 = seg_chunks[4 * s + 1], nc = seg_chunks[4 * s + 2], t0 = seg_chunks[4 * s + 3];
    const int dk = a.dk, dv = a.dv;
    const int idx = blockIdx.z * blockDim.x + threadIdx.x;
    if (idx >= dk * dv) return;
    const int row = idx / dv;
    float* slot = a.state + ((size_t)a.seg_slot[seg] * a.H + h) * dk * dv;
    const size_t stride = (size_t)a.H * (dk * dv + dk);
    float* u = U + ((size_t)c0 * a.H + h) * (dk * dv + dk);
    float S = a.positions[t0] == 0 ? 0.f : slot[idx];
    for (int c = 0; c < nc; c += 4) {
        float own[4], dec[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            own[i] = c + i < nc ? u[(size_t)(c + i) * stride + idx] : 0.f;
            dec[i] = c + i < nc ? u[(size_t)(c + i) * stride + dk * dv + row] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (c + i < nc) {
                u[(size_t)(c + i) * stride + idx] = S;
                S = fmaf(expf(dec[i]), S, own[i]);
            }
    }
    if (a.writable) slot[idx] = S;
}

// ---- chunked (3): outputs ------------------------------------------------------------------------------
// o_i = S^T (q_i exp(b_i)) + sum_(j<=i) A[i][j] v_j with A[i][j] = sum_e q_i[e] k_j[e] exp(b_i[e] - b_j[e]).
// The chunk is cut into blocks of SB tokens.  Inside a block every pair takes its own exponentials.  Between blocks
// the exponent is split at r = b of the last token before i's block: (q_i exp(b_i - r)) . (k_j exp(r - b_j)), both
// factors' exponents being sums of g's (<= 0), so the pair's score is one plain dot product and the rows are scaled in
// place, block after block.  Then [q exp(b) | A] meets [S ; v] in register tiles of 4 tokens (one of every block)
// by 8 value channels, S staged through the shared memory that b and k no longer need.
__global__ void __launch_bounds__(256)
chunk_out_kernel(const Rec a, const int* __restrict__ chunks, const float* __restrict__ U, int C, int vec) {
    extern __shared__ __align__(16) float sm[];
    const int dk = a.dk, dv = a.dv, dkp = round4(dk), dvp = round4(dv), LK = dkp + 4, LA = C + 4, nb = C / SB;
    float* qs = sm;                     // [C][LK]
    float* vs = qs + C * LK;            // [C][dvp]
    float* A = vs + C * dvp;            // [C][LA]
    float* b = A + C * LA;              // [C][LK]   running log decay; from here on, later, rows of S (stage_floats)
    float* ks = b + C * LK;             // [C][LK]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int t0 = chunks[4 * c + 1], n = chunks[4 * c + 2];
    const size_t QW = (size_t)a.H * dk, VW = (size_t)a.H * dv;
    const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    load_rows(b, LK, a.g, QW, t0, n, h * dk, dk, dkp, C, vec);
    load_rows(qs, LK, a.q, QW, t0, n, h * dk, dk, dkp, C, vec);
    load_rows(ks, LK, a.k, QW, t0, n, h * dk, dk, dkp, C, vec);
    load_rows(vs, dvp, a.v, VW, t0, n, h * dv, dv, dvp, C, vec);
    for (int idx = tid; idx < C * LA; idx += blockDim.x) A[idx] = 0.f;
    copies_done();
    __syncthreads();
    running_sum_rows(b, LK, dkp, C);
    __syncthreads();
    // pairs of one block: eight lanes share a pair's channels
    {
        const int grp = tid >> 3, l8 = tid & 7, per = SB * (SB + 1) / 2, total = nb * per, g4 = dkp >> 2;
        for (int p0 = 0; p0 < total; p0 += 32) {
            const int p = p0 + grp;
            float s = 0.f;
            int i = 0, j = 0;
            if (p < total) {
                const int I = p / per, rem = p - I * per;
                int r = 0;
                while ((r + 1) * (r + 2) / 2 <= rem) ++r;
                i = I * SB + r;
                j = I * SB + rem - r * (r + 1) / 2;
                for (int e4 = l8; e4 < g4; e4 += 8) {
                    const float4 q4 = ld4(qs + i * LK + 4 * e4), k4 = ld4(ks + j * LK + 4 * e4);
                    const float4 bi = ld4(b + i * LK + 4 * e4), bj = ld4(b + j * LK + 4 * e4);
                    s = fmaf(q4.x * k4.x, expf(bi.x - bj.x), s);
                    s = fmaf(q4.y * k4.y, expf(bi.y - bj.y), s);
                    s = fmaf(q4.z * k4.z, expf(bi.z - bj.z), s);
                    s = fmaf(q4.w * k4.w, expf(bi.w - bj.w), s);
                }
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (p < total && l8 == 0) A[i * LA + j] = s;
        }
    }
    __syncthreads();
    // pairs of different blocks
    for (int I = 1; I < nb; ++I) {
        const float* r1 = b + (I * SB - 1) * LK;                 // b of the last token before block I
        const float* r0 = I > 1 ? b + ((I - 1) * SB - 1) * LK : nullptr;
        for (int j = warp; j < (I + 1) * SB; j += warps)
            for (int e = lane; e < dkp; e += 32) {
                if (j >= I * SB) qs[j * LK + e] *= expf(b[j * LK + e] - r1[e]);
                else if (j >= (I - 1) * SB) ks[j * LK + e] *= expf(r1[e] - b[j * LK + e]);
                else ks[j * LK + e] *= expf(r1[e] - r0[e]);
            }
        __syncthreads();
        const int ai = I * SB + (tid & 15), jq = tid >> 4;
        if (jq < 4 * I) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const float* qrow = qs + ai * LK;
            const float* krow = ks + 4 * jq * LK;
            for (int e = 0; e < dkp; e += 4) {
                const float4 q4 = ld4(qrow + e);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float4 k4 = ld4(krow + x * LK + e);
                    acc[x] = fmaf(q4.x, k4.x, fmaf(q4.y, k4.y, fmaf(q4.z, k4.z, fmaf(q4.w, k4.w, acc[x]))));
                }
            }
            *reinterpret_cast<float4*>(A + ai * LA + 4 * jq) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        __syncthreads();
    }
    // q_i exp(b_i): what meets the state before the chunk (rows of later blocks already carry exp(b_i - r))
    for (int j = warp; j < C; j += warps) {
        const float* bb = j < SB ? b + j * LK : b + (j / SB * SB - 1) * LK;
        for (int e = lane; e < dkp; e += 32) qs[j * LK + e] *= expf(bb[e]);
    }
    const float* S = U + ((size_t)c * a.H + h) * (dk * dv + dk);
    float* Sst = b;                                              // [rows][dvp]
    const int slab = min(dkp, (stage_floats(dkp, dvp, C) / dvp) & ~3);      // at least four rows of S
    const int ti = tid >> 4, te = tid & 15, ge = dvp >> 2;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int et = 0; et < ge; et += 32) {
        const int eb = et + te, e0 = 4 * eb, e1 = 4 * (eb + 16);
        const bool act = eb < ge, he = eb + 16 < ge;
        float acc[4][2][4];
#pragma unroll
        for (int m = 0; m < 4; ++m)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[m][0][x] = acc[m][1][x] = 0.f;
        for (int s0 = 0; s0 < dkp; s0 += slab) {
            const int rows = min(slab, dkp - s0);
            __syncthreads();
            if (vec) {              // whole rows, one after the other
                for (int idx = 4 * tid; idx < rows * dv; idx += 4 * blockDim.x) copy16(Sst + idx, S + (size_t)s0 * dv + idx, true);
                copies_done();
            } else {
                for (int r = warp; r < rows; r += warps)
                    for (int e = lane; e < dvp; e += 32)
                        Sst[r * dvp + e] = (s0 + r < dk && e < dv) ? S[(size_t)(s0 + r) * dv + e] : 0.f;
            }
            __syncthreads();
            if (act)
                for (int r = 0; r < rows; r += 4) {
                    float qq[4][4];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const float4 q4 = m < nb ? ld4(qs + (m * SB + ti) * LK + s0 + r) : zero;
                        qq[m][0] = q4.x; qq[m][1] = q4.y; qq[m][2] = q4.z; qq[m][3] = q4.w;
                    }
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float4 s4 = ld4(Sst + (r + x) * dvp + e0), s5 = he ? ld4(Sst + (r + x) * dvp + e1) : zero;
#pragma unroll
                        for (int m = 0; m < 4; ++m) {
                            fma4(acc[m][0], qq[m][x], s4);
                            fma4(acc[m][1], qq[m][x], s5);
                        }
                    }
                }
        }
        if (act) {
            for (int J = 0; J < nb; ++J)
                for (int jj = 0; jj < SB; jj += 4) {
                    float aa[4][4];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const float4 a4 = (m >= J && m < nb) ? ld4(A + (m * SB + ti) * LA + J * SB + jj) : zero;
                        aa[m][0] = a4.x; aa[m][1] = a4.y; aa[m][2] = a4.z; aa[m][3] = a4.w;
                    }
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const int j = J * SB + jj + x;
                        const float4 v4 = ld4(vs + j * dvp + e0), v5 = he ? ld4(vs + j * dvp + e1) : zero;
#pragma unroll
                        for (int m = 0; m < 4; ++m)
                            if (m >= J) {
                                fma4(acc[m][0], aa[m][x], v4);
                                fma4(acc[m][1], aa[m][x], v5);
                            }
                    }
                }
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int i = m * SB + ti;
                if (m >= nb || i >= n) continue;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (half && !he) continue;
                    float* dst = a.out + (size_t)(t0 + i) * VW + h * dv + (half ? e1 : e0);
                    if (vec) {
                        *reinterpret_cast<float4*>(dst) = make_float4(acc[m][half][0], acc[m][half][1], acc[m][half][2], acc[m][half][3]);
                    } else {
#pragma unroll
                        for (int x = 0; x < 4; ++x)
                            if ((half ? e1 : e0) + x < dv) dst[x] = acc[m][half][x];
                    }
                }
            }
        }
    }
}

size_t scan_smem(int dk, int dv, int threads) {
    const int R = threads / dv > 0 ? threads / dv : 1;
    return sizeof(float) * ((size_t)dk * dv + 3 * dk + dv + (size_t)R * dv);
}
size_t out_smem(int dk, int dv, int C) {
    const size_t LK = round4h(dk) + 4;
    return sizeof(float) * (C * LK + (size_t)C * round4h(dv) + (size_t)C * (C + 4) +
                            (size_t)stage_floats((int)round4h(dk), (int)round4h(dv), C));
}
size_t state_smem(int dk, int dv, int C) {
    const size_t LK = round4h(dk) + 4;
    return sizeof(float) * (2 * C * LK + (size_t)C * round4h(dv));
}

constexpr size_t SMEM_MAX = 200 * 1024;

}  // namespace

MHB_EXPORT int mhb_gated_linear_prep(const float* main_p, int main_nsplit, long long main_stride, int main_ld, int q0,
                                     int k0, int v0, int a0, const void* a2, int a2_dtype, int rank, const float* bias,
                                     const float* low, float qscale, float inv_tau, int mode, float* q, float* k,
                                     float* v, float* g, int T, int QW, int VW, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (mode != 0 && mode != 1) return fail("gated_linear_prep: unknown mode %d", mode);
    if (mode == 0 && (rank < 1 || rank > 8192)) return fail("gated_linear_prep: a low-rank decay of rank %d", rank);
    Parts main{main_p, main_nsplit, (size_t)main_stride, main_ld};
    const size_t smem = mode == 0 ? sizeof(float) * rank : 0;
    MHB_DISPATCH_DTYPE(a2_dtype, WT, {
        // few tokens: a CTA per 256 columns, so that a decoded token's row is spread over many SMs
        const int cols = QW > VW ? QW : VW, slices = T >= 64 ? 1 : (cols + 255) / 256;
        cudaError_t e = launch_kernel(prep_kernel<WT>, dim3(T, slices), dim3(256), smem, stream, main, q0, k0, v0, a0,
                                      (const WT*)a2, rank, bias, low, qscale, inv_tau, mode, q, k, v, g, QW, VW);
        if (e != cudaSuccess) return fail("gated_linear_prep: %s", cudaGetErrorString(e));
    });
    return check_launch("gated_linear_prep");
}

MHB_EXPORT int mhb_gated_linear_head_norm(const float* o, const float* w, float eps, const float* gate, int gate_nsplit,
                                          long long gate_stride, int gate_ld, int gate0, void* out, int out_dtype, int T,
                                          int H, int dv, cudaStream_t stream) {
    if (T <= 0) return 0;
    Parts gp{gate, gate_nsplit, (size_t)gate_stride, gate_ld};
    const size_t pairs = (size_t)T * H;
    const int warps = 8;
    MHB_DISPATCH_DTYPE(out_dtype, OT, {
        cudaError_t e = launch_kernel(head_norm_kernel<OT>, dim3((unsigned)((pairs + warps - 1) / warps)), dim3(32 * warps),
                                      0, stream, o, w, eps, gp, gate0, (OT*)out, pairs, H, dv);
        if (e != cudaSuccess) return fail("gated_linear_head_norm: %s", cudaGetErrorString(e));
    });
    return check_launch("gated_linear_head_norm");
}

static Rec make_rec(const float* q, const float* k, const float* g, const float* v, float* state, float* out,
                    const int* tok_seg, const int* seg_slot, const int* positions, int T, int H, int dk, int dv,
                    int writable) {
    Rec a;
    a.q = q; a.k = k; a.g = g; a.v = v; a.state = state; a.out = out;
    a.tok_seg = tok_seg; a.seg_slot = seg_slot; a.positions = positions;
    a.T = T; a.H = H; a.dk = dk; a.dv = dv; a.writable = writable;
    return a;
}

MHB_EXPORT int mhb_gated_linear_scan(const float* q, const float* k, const float* g, const float* v, float* state,
                                     float* out, const int* tok_seg, const int* seg_slot, const int* positions, int T,
                                     int S, int H, int dk, int dv, int writable, int max_tokens, cudaStream_t stream) {
    if (T <= 0 || S <= 0) return 0;
    const int threads = 256;
    const size_t smem = scan_smem(dk, dv, threads);
    if (smem > SMEM_MAX) return fail("gated_linear_scan: a state of %d x %d does not fit an SM's shared memory", dk, dv);
    static size_t raised = 0;
    if (smem > 48 * 1024 && smem > raised) {
        if (cudaFuncSetAttribute(scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX) != cudaSuccess)
            return fail("gated_linear_scan: cannot raise the shared-memory limit");
        raised = SMEM_MAX;
    }
    Rec a = make_rec(q, k, g, v, state, out, tok_seg, seg_slot, positions, T, H, dk, dv, writable);
    cudaError_t e = launch_kernel(scan_kernel, dim3(S, H), dim3(threads), smem, stream, a, max_tokens);
    if (e != cudaSuccess) return fail("gated_linear_scan: %s", cudaGetErrorString(e));
    return check_launch("gated_linear_scan");
}

// Shared memory of the chunked route for chunks of C tokens (the caller picks the largest C that fits).
MHB_EXPORT long long mhb_gated_linear_chunk_smem(int dk, int dv, int C) {
    const size_t a = out_smem(dk, dv, C), b = state_smem(dk, dv, C);
    return (long long)(a > b ? a : b);
}

MHB_EXPORT int mhb_gated_linear_chunked(const float* q, const float* k, const float* g, const float* v, float* state,
                                        float* out, const int* tok_seg, const int* seg_slot, const int* positions, int T,
                                        int H, int dk, int dv, int writable, const int* chunks, int num_chunks,
                                        const int* seg_chunks, int num_segs, float* scratch, int C, cudaStream_t stream) {
    if (num_chunks <= 0 || num_segs <= 0) return 0;
    const size_t so = out_smem(dk, dv, C), ss = state_smem(dk, dv, C);
    if (C < SB || C > 4 * SB || C % SB) return fail("gated_linear_chunked: chunks of %d tokens (16, 32, 48 or 64)", C);
    if (so > SMEM_MAX || ss > SMEM_MAX)
        return fail("gated_linear_chunked: chunks of %d tokens of %d x %d do not fit", C, dk, dv);
    // whole float4 stores where every row of the outputs starts on 16 bytes
    const int vec = dk % 4 == 0 && dv % 4 == 0 &&
                    ((uintptr_t)scratch | (uintptr_t)out | (uintptr_t)q | (uintptr_t)k | (uintptr_t)g | (uintptr_t)v) % 16 == 0;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX) != cudaSuccess ||
            cudaFuncSetAttribute(chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX) != cudaSuccess)
            return fail("gated_linear_chunked: cannot raise the shared-memory limit");
        raised = true;
    }
    Rec a = make_rec(q, k, g, v, state, out, tok_seg, seg_slot, positions, T, H, dk, dv, writable);
    cudaError_t e = launch_kernel(chunk_state_kernel, dim3(num_chunks, H), dim3(256), ss, stream, a, chunks, scratch, C, vec);
    if (e != cudaSuccess) return fail("gated_linear_chunked (1): %s", cudaGetErrorString(e));
    e = launch_kernel(chunk_prefix_kernel, dim3(num_segs, H, (dk * dv + 255) / 256), dim3(256), 0, stream, a, seg_chunks,
                      scratch);
    if (e != cudaSuccess) return fail("gated_linear_chunked (2): %s", cudaGetErrorString(e));
    e = launch_kernel(chunk_out_kernel, dim3(num_chunks, H), dim3(256), so, stream, a, chunks, (const float*)scratch, C, vec);
    if (e != cudaSuccess) return fail("gated_linear_chunked (3): %s", cudaGetErrorString(e));
    return check_launch("gated_linear_chunked");
}
