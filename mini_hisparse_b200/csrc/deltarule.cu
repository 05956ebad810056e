// The gated delta rule: a linear recurrence over a float32 state per head whose write is an error correction.
//
//   S <- g_t S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t        S [dk][dv] per head
//
// with q, k, v from short causal convolutions over time (one filter per channel, then silu), q and k made unit
// vectors per head, beta a sigmoid and g = exp(-exp(A_log) softplus(a + dt_bias)) one number per head and token.
// Every column of S evolves on its own (column j sees v_t[j] only), so the recurrence is cut along the value
// columns: a group of 4 lanes owns one column, each lane a run of dk / 4 rows in registers (the token's k and q
// come as float4 from shared memory, where cp.async put them while the 16 tokens before were walked; the sums run
// in four chains), and the two dot products of a token are finished by two shuffles each.  Decoded tokens and prompt portions take the same
// kernel; a segment that starts at position 0 starts from zero, whatever its slot held.
//
//   delta_prep        per token: the convolutions of the q, k, v columns of the input projection (float32, possibly
//                     split-K parts) over this step's rows and, before the segment's first row, the slot's last
//                     taps - 1 inputs; silu; unit q (times dk^-1/2) and k; beta; g.  All float32.
//   delta_conv_keep   per segment, after delta_prep: the last taps - 1 inputs of the segment go to its slot.
//   delta_scan        the recurrence: one CTA of two warps per (segment, head, 16 value columns).
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int MAX_TAPS = 16;
constexpr int LPC = 4;          // lanes per state column
constexpr int COLS = 16;        // state columns per CTA

struct Parts {
    const float* p;
    int nsplit;
    size_t stride;
    int ld;
    __device__ __forceinline__ float at(size_t row, int col) const {
        const size_t idx = row * ld + col;
        float v = p[idx];
        for (int s = 1; s < nsplit; ++s) v += p[idx + (size_t)s * stride];
        return v;
    }
};

__device__ __forceinline__ int segment_begin(const int* tok_seg, int T, int seg) {
    int lo = 0, hi = T;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tok_seg[mid] < seg) lo = mid + 1; else hi = mid; }
    return lo;
}
__device__ __forceinline__ int segment_end(const int* tok_seg, int T, int seg) {
    int lo = 0, hi = T;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tok_seg[mid] <= seg) lo = mid + 1; else hi = mid; }
    return lo;
}

__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct PrepArgs {
    Parts proj;                 // [T][ld]: columns c0 .. hold [q | k | v], b0 .. beta's logits, a0 .. the decay's
    int c0, b0, a0;
    const float* taps;          // [C][ntaps], the last tap is the current token's
    const float* A_log;         // [H]
    const float* dt_bias;       // [H]
    const float* keep;          // [slots][keep_stride]: a slot's last ntaps - 1 inputs [ntaps - 1][C]
    size_t keep_stride;
    const int* tok_seg;
    const int* seg_slot;
    const int* positions;
    float* q;                   // [T][G dk]
    float* k;                   // [T][G dk]
    float* v;                   // [T][H dv]
    float* beta;                // [T][H]
    float* decay;               // [T][H]
    int T, H, G, dk, dv, ntaps;
    float qscale, unit_eps;
};

__global__ void __launch_bounds__(256)
prep_kernel(const PrepArgs a) {
    extern __shared__ float sh[];           // [2 G dk]: q and k after silu
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int seg = a.tok_seg[t];
    const int t0 = segment_begin(a.tok_seg, a.T, seg);
    const int pos = a.positions[t], start = a.positions[t0];
    const int QK = a.G * a.dk, VW = a.H * a.dv, C = 2 * QK + VW, K = a.ntaps;
    const float* kept = a.keep + (size_t)a.seg_slot[seg] * a.keep_stride;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float y = 0.f;
        for (int i = 0; i < K; ++i) {
            const int p = pos - (K - 1) + i;
            if (p < 0) continue;
            const float z = p >= start ? a.proj.at((size_t)(t - (pos - p)), a.c0 + c)
                                       : kept[(size_t)(p - (start - (K - 1))) * C + c];
            y = fmaf(a.taps[(size_t)c * K + i], z, y);
        }
        y = silu(y);
        if (c < 2 * QK) sh[c] = y;
        else a.v[(size_t)t * VW + (c - 2 * QK)] = y;
    }
    for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
        a.beta[(size_t)t * a.H + h] = 1.f / (1.f + expf(-a.proj.at(t, a.b0 + h)));
        a.decay[(size_t)t * a.H + h] = expf(-expf(a.A_log[h]) * softplus(a.proj.at(t, a.a0 + h) + a.dt_bias[h]));
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int head = warp; head < 2 * a.G; head += nwarps) {       // q heads, then k heads
        const float* row = sh + head * a.dk;
        float ss = 0.f;
        for (int e = lane; e < a.dk; e += 32) ss += row[e] * row[e];
        const float r = (head < a.G ? a.qscale : 1.f) / sqrtf(warp_sum(ss) + a.unit_eps);
        float* dst = head < a.G ? a.q + (size_t)t * QK + head * a.dk : a.k + (size_t)t * QK + (head - a.G) * a.dk;
        for (int e = lane; e < a.dk; e += 32) dst[e] = row[e] * r;
    }
}

// one CTA per segment; a thread owns a channel's column of the kept rows, so reading the old rows and writing the
// new ones needs no barrier
__global__ void __launch_bounds__(256)
conv_keep_kernel(Parts proj, int c0, float* keep, size_t keep_stride, const int* tok_seg, const int* seg_slot,
                 const int* positions, int T, int C, int ntaps) {
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.x;
    const int t0 = segment_begin(tok_seg, T, seg), t1 = segment_end(tok_seg, T, seg);
    if (t1 <= t0) return;
    const int n = t1 - t0, R = ntaps - 1;
    const int start = positions[t0];
    float* kept = keep + (size_t)seg_slot[seg] * keep_stride;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float rows[MAX_TAPS];
        for (int r = 0; r < R; ++r) {              // new row r holds the input at position start + n - R + r
            const int back = R - r;                // that many positions before the segment's end
            float z = 0.f;
            if (back <= n) z = proj.at((size_t)(t1 - back), c0 + c);
            else if (start + n - back >= 0) z = kept[(size_t)(r + n) * C + c];      // old row r + n, still inside
            rows[r] = z;
        }
        for (int r = 0; r < R; ++r) kept[(size_t)r * C + c] = rows[r];
    }
}

struct ScanArgs {
    const float* q;        // [T][G dk]
    const float* k;
    const float* v;        // [T][H dv]
    const float* beta;     // [T][H]
    const float* decay;    // [T][H]
    float* state;          // [slots][state_stride]: [H][dk][dv]
    size_t state_stride;
    float* out;            // [T][H dv]
    const int* tok_seg;
    const int* seg_slot;
    const int* positions;
    int T, H, G, dk, dv, writable;
};

__device__ __forceinline__ void copy_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// RPL: rows of a column per lane (dk <= LPC * RPL; lane `sub` of a column owns the rows sub * RPL ...).  CH: tokens whose
// inputs are staged at once; the next CH tokens' inputs arrive by cp.async while these are walked.
// CPT: columns per thread (two recurrences whose chains fill each other's waits; see the launch for why it is 1).
template <int RPL, int CH, int CPT>
__global__ void __launch_bounds__(LPC * COLS / CPT)
scan_kernel(const ScanArgs a) {
    constexpr int RUN = RPL + 4;             // a lane's run of rows, padded so that the four lanes' float4 loads meet no bank twice
    __shared__ __align__(16) float qs[2][CH][LPC * RUN];
    __shared__ __align__(16) float ks[2][CH][LPC * RUN];
    __shared__ float vs[2][CH][COLS];
    __shared__ float bs[2][CH], gs[2][CH];
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
    const int t0 = segment_begin(a.tok_seg, a.T, seg), t1 = segment_end(a.tok_seg, a.T, seg);
    if (t1 <= t0) return;
    const int dk = a.dk, dv = a.dv;
    const int hk = h / (a.H / a.G);
    const int sub = threadIdx.x % LPC, cl = threadIdx.x / LPC;
    int cols_here[CPT];                                        // a thread's columns inside the CTA's 16
#pragma unroll
    for (int c = 0; c < CPT; ++c) cols_here[c] = cl + c * (COLS / CPT);
    bool live[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) live[c] = col0 + cols_here[c] < dv;
    const int QK = a.G * dk, VW = a.H * dv;
    // what no copy ever writes (rows beyond dk, columns beyond dv) stays zero
    for (int i = threadIdx.x; i < 2 * CH * LPC * RUN; i += blockDim.x) { (&qs[0][0][0])[i] = 0.f; (&ks[0][0][0])[i] = 0.f; }
    for (int i = threadIdx.x; i < 2 * CH * COLS; i += blockDim.x) (&vs[0][0][0])[i] = 0.f;
    __syncthreads();
    const bool by4 = dk % 4 == 0 && ((uintptr_t)a.q & 15) == 0 && ((uintptr_t)a.k & 15) == 0;     // rows then start on 16 bytes
    auto stage_in = [&](int st, int c0) {
        const int n = min(CH, t1 - c0);
        if (by4) {
            const int per = dk / 4;
            for (int idx = threadIdx.x; idx < n * per; idx += blockDim.x) {
                const int tt = idx / per, i = (idx - tt * per) * 4;
                const size_t src = (size_t)(c0 + tt) * QK + hk * dk + i;
                const int at = (i / RPL) * RUN + i % RPL;
                copy_async16(&qs[st][tt][at], a.q + src);
                copy_async16(&ks[st][tt][at], a.k + src);
            }
        } else {
            for (int idx = threadIdx.x; idx < n * dk; idx += blockDim.x) {
                const int tt = idx / dk, i = idx - tt * dk;
                const size_t src = (size_t)(c0 + tt) * QK + hk * dk + i;
                const int at = (i / RPL) * RUN + i % RPL;
                copy_async4(&qs[st][tt][at], a.q + src);
                copy_async4(&ks[st][tt][at], a.k + src);
            }
        }
        const int cols = min(COLS, dv - col0);
        for (int idx = threadIdx.x; idx < n * cols; idx += blockDim.x) {
            const int tt = idx / cols, c = idx - tt * cols;
            copy_async4(&vs[st][tt][c], a.v + (size_t)(c0 + tt) * VW + h * dv + col0 + c);
        }
        if (threadIdx.x < n) {
            copy_async4(&bs[st][threadIdx.x], a.beta + (size_t)(c0 + threadIdx.x) * a.H + h);
            copy_async4(&gs[st][threadIdx.x], a.decay + (size_t)(c0 + threadIdx.x) * a.H + h);
        }
    };
    stage_in(0, t0);
    copy_async_commit();
    float* slot = a.state + (size_t)a.seg_slot[seg] * a.state_stride + (size_t)h * dk * dv;
    const bool fresh = a.positions[t0] == 0;
    float S[CPT][RPL];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int i = sub * RPL + r;
            S[c][r] = (!fresh && live[c] && i < dk) ? slot[(size_t)i * dv + col0 + cols_here[c]] : 0.f;
        }
    int st = 0;
    for (int c0 = t0; c0 < t1; c0 += CH, st ^= 1) {
        const int n = min(CH, t1 - c0);
        if (c0 + CH < t1) stage_in(st ^ 1, c0 + CH);
        copy_async_commit();
        copy_async_wait<1>();          // everything but the copies just issued has landed
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float g = gs[st][tt];
            float kr[RPL];
            const float4* k4 = reinterpret_cast<const float4*>(&ks[st][tt][sub * RUN]);
#pragma unroll
            for (int r = 0; r < RPL / 4; ++r) {
                const float4 x = k4[r];
                kr[4 * r] = x.x; kr[4 * r + 1] = x.y; kr[4 * r + 2] = x.z; kr[4 * r + 3] = x.w;
            }
            float d[CPT][4];           // four chains a column, so that no product waits for the one before
#pragma unroll
            for (int c = 0; c < CPT; ++c) d[c][0] = d[c][1] = d[c][2] = d[c][3] = 0.f;
#pragma unroll
            for (int r = 0; r < RPL; r += 4)
#pragma unroll
                for (int c = 0; c < CPT; ++c)
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        S[c][r + x] *= g;
                        d[c][x] = fmaf(S[c][r + x], kr[r + x], d[c][x]);
                    }
            float u[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float dot = (d[c][0] + d[c][1]) + (d[c][2] + d[c][3]);
#pragma unroll
                for (int o = 1; o < LPC; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                u[c] = bs[st][tt] * (vs[st][tt][cols_here[c]] - dot);
                d[c][0] = d[c][1] = d[c][2] = d[c][3] = 0.f;
            }
            const float4* q4 = reinterpret_cast<const float4*>(&qs[st][tt][sub * RUN]);
#pragma unroll
            for (int r = 0; r < RPL / 4; ++r) {
                const float4 x4 = q4[r];
                const float qv[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
                for (int c = 0; c < CPT; ++c)
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        S[c][4 * r + x] = fmaf(kr[4 * r + x], u[c], S[c][4 * r + x]);
                        d[c][x] = fmaf(S[c][4 * r + x], qv[x], d[c][x]);
                    }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float o = (d[c][0] + d[c][1]) + (d[c][2] + d[c][3]);
#pragma unroll
                for (int x = 1; x < LPC; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
                if (sub == 0 && live[c]) a.out[(size_t)(c0 + tt) * VW + h * dv + col0 + cols_here[c]] = o;
            }
        }
        __syncthreads();               // this stage is free for the copies of the chunk after the next
    }
    copy_async_wait<0>();
    if (a.writable) {
#pragma unroll
        for (int c = 0; c < CPT; ++c)
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                const int i = sub * RPL + r;
                if (live[c] && i < dk) slot[(size_t)i * dv + col0 + cols_here[c]] = S[c][r];
            }
    }
}
}  // namespace

MHB_EXPORT int mhb_delta_prep(const float* proj, int nsplit, long long split_stride, int ld, int c0, int b0, int a0,
                              const float* taps, const float* A_log, const float* dt_bias, const float* keep,
                              long long keep_stride, const int* tok_seg, const int* seg_slot, const int* positions,
                              float* q, float* k, float* v, float* beta, float* decay, int T, int H, int G, int dk,
                              int dv, int ntaps, float qscale, float unit_eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (ntaps < 1 || ntaps > MAX_TAPS) return fail("delta_prep: %d taps (1 to %d)", ntaps, MAX_TAPS);
    if (G < 1 || H % G) return fail("delta_prep: %d heads over %d q/k heads", H, G);
    PrepArgs a;
    a.proj = Parts{proj, nsplit, (size_t)split_stride, ld};
    a.c0 = c0; a.b0 = b0; a.a0 = a0; a.taps = taps; a.A_log = A_log; a.dt_bias = dt_bias; a.keep = keep;
    a.keep_stride = (size_t)keep_stride; a.tok_seg = tok_seg; a.seg_slot = seg_slot; a.positions = positions;
    a.q = q; a.k = k; a.v = v; a.beta = beta; a.decay = decay; a.T = T; a.H = H; a.G = G; a.dk = dk; a.dv = dv;
    a.ntaps = ntaps; a.qscale = qscale; a.unit_eps = unit_eps;
    const size_t smem = sizeof(float) * 2 * (size_t)G * dk;
    if (smem > 48 * 1024) return fail("delta_prep: q and k of %d x %d do not fit the kernel's shared memory", G, dk);
    cudaError_t e = launch_kernel(prep_kernel, dim3(T), dim3(256), smem, stream, a);
    if (e != cudaSuccess) return fail("delta_prep: %s", cudaGetErrorString(e));
    return check_launch("delta_prep");
}

MHB_EXPORT int mhb_delta_conv_keep(const float* proj, int nsplit, long long split_stride, int ld, int c0, float* keep,
                                   long long keep_stride, const int* tok_seg, const int* seg_slot, const int* positions,
                                   int T, int S, int C, int ntaps, cudaStream_t stream) {
    if (T <= 0 || S <= 0 || ntaps <= 1) return 0;
    if (ntaps > MAX_TAPS) return fail("delta_conv_keep: %d taps (up to %d)", ntaps, MAX_TAPS);
    cudaError_t e = launch_kernel(conv_keep_kernel, dim3(S), dim3(256), 0, stream,
                                  Parts{proj, nsplit, (size_t)split_stride, ld}, c0, keep, (size_t)keep_stride, tok_seg,
                                  seg_slot, positions, T, C, ntaps);
    if (e != cudaSuccess) return fail("delta_conv_keep: %s", cudaGetErrorString(e));
    return check_launch("delta_conv_keep");
}

MHB_EXPORT int mhb_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* decay,
                              float* state, long long state_stride, float* out, const int* tok_seg, const int* seg_slot,
                              const int* positions, int T, int S, int H, int G, int dk, int dv, int writable,
                              cudaStream_t stream) {
    if (T <= 0 || S <= 0) return 0;
    if (G < 1 || H % G) return fail("delta_scan: %d heads over %d q/k heads", H, G);
    if (dk > 256) return fail("delta_scan: keys %d wide (up to 256)", dk);
    ScanArgs a;
    a.q = q; a.k = k; a.v = v; a.beta = beta; a.decay = decay; a.state = state; a.state_stride = (size_t)state_stride;
    a.out = out; a.tok_seg = tok_seg; a.seg_slot = seg_slot; a.positions = positions; a.T = T; a.H = H; a.G = G;
    a.dk = dk; a.dv = dv; a.writable = writable;
    dim3 grid(S, H, (dv + COLS - 1) / COLS);
    cudaError_t e;
    // One column a thread: with two (CPT = 2) a warp's chains do fill each other's waits (1.3 times the work a cycle),
    // but a prompt of one request then has half as many warps, and they are what fills the GPU: 16 heads x 128 columns
    // took 850 us with two columns a thread and 560 us with one.
    if (dk <= 16) e = launch_kernel(scan_kernel<4, 16, 1>, grid, dim3(LPC * COLS), 0, stream, a);
    else if (dk <= 32) e = launch_kernel(scan_kernel<8, 16, 1>, grid, dim3(LPC * COLS), 0, stream, a);
    else if (dk <= 64) e = launch_kernel(scan_kernel<16, 16, 1>, grid, dim3(LPC * COLS), 0, stream, a);
    else if (dk <= 128) e = launch_kernel(scan_kernel<32, 16, 1>, grid, dim3(LPC * COLS), 0, stream, a);
    else e = launch_kernel(scan_kernel<64, 8, 1>, grid, dim3(LPC * COLS), 0, stream, a);
    if (e != cudaSuccess) return fail("delta_scan: %s", cudaGetErrorString(e));
    return check_launch("delta_scan");
}
