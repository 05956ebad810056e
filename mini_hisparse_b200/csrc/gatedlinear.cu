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
// grid (T), any block: columns of head-major [H * dk] / [H * dv] rows.  mode 0: the decay's logits are a low-rank
// product, z = A2 (columns a0 .. a0 + rank of the main product) + bias, taken here in float32.
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
    for (int i = threadIdx.x; i < QW; i += blockDim.x) {
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
    for (int i = threadIdx.x; i < VW; i += blockDim.x) v[t * VW + i] = load(main, t, v0 + i);
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
    extern __shared__ float sm[];
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
    for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) St[i] = fresh ? 0.f : slot[i];
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
    if (a.writable)
        for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) slot[i] = St[i];
}

// inclusive running sum of g over the chunk's tokens, one key channel per thread: b[j][i], rows dk + 1 apart
__device__ __forceinline__ void running_log_decay(const Rec& a, int t0, int n, int h, float* b) {
    const int dk = a.dk, QW = a.H * dk;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < n; ++j) {
            acc += a.g[(size_t)(t0 + j) * QW + h * dk + i];
            b[j * (dk + 1) + i] = acc;
        }
    }
}

// ---- chunked (1): every chunk's own contribution U [dk][dv] and its total log decay B [dk] -------------------
// chunks: {segment, first token, tokens (<= C), index of the chunk in its segment}; U holds dk * dv + dk floats a
// chunk and head
__global__ void __launch_bounds__(256)
chunk_state_kernel(const Rec a, const int* __restrict__ chunks, float* __restrict__ U, int C) {
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv;
    float* b = sm;                      // [C][dk + 1]
    float* ks = b + C * (dk + 1);       // [C][dk + 1]  k_j exp(B - b_j)
    float* vs = ks + C * (dk + 1);      // [C][dv]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y;
    const int t0 = chunks[4 * c + 1], n = chunks[4 * c + 2];
    const int QW = a.H * dk, VW = a.H * dv;
    running_log_decay(a, t0, n, h, b);
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * dk; idx += blockDim.x) {
        const int j = idx / dk, i = idx - j * dk;
        ks[j * (dk + 1) + i] = a.k[(size_t)(t0 + j) * QW + h * dk + i] * expf(b[(n - 1) * (dk + 1) + i] - b[j * (dk + 1) + i]);
    }
    for (int idx = threadIdx.x; idx < n * dv; idx += blockDim.x) {
        const int j = idx / dv, e = idx - j * dv;
        vs[idx] = a.v[(size_t)(t0 + j) * VW + h * dv + e];
    }
    __syncthreads();
    float* u = U + ((size_t)c * a.H + h) * (dk * dv + dk);
    for (int idx = threadIdx.x; idx < dk * dv; idx += blockDim.x) {
        const int i = idx / dv, e = idx - i * dv;
        float s = 0.f;
        for (int j = 0; j < n; ++j) s = fmaf(ks[j * (dk + 1) + i], vs[j * dv + e], s);
        u[idx] = s;
    }
    for (int i = threadIdx.x; i < dk; i += blockDim.x) u[dk * dv + i] = b[(n - 1) * (dk + 1) + i];
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
__global__ void __launch_bounds__(256)
chunk_out_kernel(const Rec a, const int* __restrict__ chunks, const float* __restrict__ U, int C) {
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv;
    float* b = sm;                      // [C][dk + 1]
    float* qs = b + C * (dk + 1);       // [C][dk + 1]
    float* ks = qs + C * (dk + 1);      // [C][dk + 1]
    float* vs = ks + C * (dk + 1);      // [C][dv]
    float* A = vs + C * dv;             // [C][C + 1]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y;
    const int t0 = chunks[4 * c + 1], n = chunks[4 * c + 2];
    const int QW = a.H * dk, VW = a.H * dv;
    running_log_decay(a, t0, n, h, b);
    for (int idx = threadIdx.x; idx < n * dk; idx += blockDim.x) {
        const int j = idx / dk, i = idx - j * dk;
        const size_t src = (size_t)(t0 + j) * QW + h * dk + i;
        qs[j * (dk + 1) + i] = a.q[src];
        ks[j * (dk + 1) + i] = a.k[src];
    }
    for (int idx = threadIdx.x; idx < n * dv; idx += blockDim.x) {
        const int j = idx / dv, e = idx - j * dv;
        vs[idx] = a.v[(size_t)(t0 + j) * VW + h * dv + e];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * n; idx += blockDim.x) {
        const int i = idx / n, j = idx - i * n;
        float s = 0.f;
        if (j <= i) {
            const float* qi = qs + i * (dk + 1);
            const float* kj = ks + j * (dk + 1);
            const float* bi = b + i * (dk + 1);
            const float* bj = b + j * (dk + 1);
            for (int e = 0; e < dk; ++e) s = fmaf(qi[e] * kj[e], expf(bi[e] - bj[e]), s);
        }
        A[i * (C + 1) + j] = s;
    }
    __syncthreads();
    // q_i exp(b_i) in place: what meets the state before the chunk
    for (int idx = threadIdx.x; idx < n * dk; idx += blockDim.x) {
        const int j = idx / dk, i = idx - j * dk;
        qs[j * (dk + 1) + i] *= expf(b[j * (dk + 1) + i]);
    }
    __syncthreads();
    const float* S = U + ((size_t)c * a.H + h) * (dk * dv + dk);
    for (int idx = threadIdx.x; idx < n * dv; idx += blockDim.x) {
        const int i = idx / dv, e = idx - i * dv;
        const float* qi = qs + i * (dk + 1);
        float o = 0.f;
        for (int r = 0; r < dk; ++r) o = fmaf(S[r * dv + e], qi[r], o);
        const float* Ai = A + i * (C + 1);
        for (int j = 0; j <= i; ++j) o = fmaf(Ai[j], vs[j * dv + e], o);
        a.out[(size_t)(t0 + i) * VW + h * dv + e] = o;
    }
}

size_t scan_smem(int dk, int dv, int threads) {
    const int R = threads / dv > 0 ? threads / dv : 1;
    return sizeof(float) * ((size_t)dk * dv + 3 * dk + dv + (size_t)R * dv);
}
size_t out_smem(int dk, int dv, int C) { return sizeof(float) * ((size_t)3 * C * (dk + 1) + (size_t)C * dv + (size_t)C * (C + 1)); }
size_t state_smem(int dk, int dv, int C) { return sizeof(float) * ((size_t)2 * C * (dk + 1) + (size_t)C * dv); }

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
        cudaError_t e = launch_kernel(prep_kernel<WT>, dim3(T), dim3(256), smem, stream, main, q0, k0, v0, a0,
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
    if (so > SMEM_MAX || ss > SMEM_MAX) return fail("gated_linear_chunked: chunks of %d tokens of %d x %d do not fit", C, dk, dv);
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX) != cudaSuccess ||
            cudaFuncSetAttribute(chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX) != cudaSuccess)
            return fail("gated_linear_chunked: cannot raise the shared-memory limit");
        raised = true;
    }
    Rec a = make_rec(q, k, g, v, state, out, tok_seg, seg_slot, positions, T, H, dk, dv, writable);
    cudaError_t e = launch_kernel(chunk_state_kernel, dim3(num_chunks, H), dim3(256), ss, stream, a, chunks, scratch, C);
    if (e != cudaSuccess) return fail("gated_linear_chunked (1): %s", cudaGetErrorString(e));
    e = launch_kernel(chunk_prefix_kernel, dim3(num_segs, H, (dk * dv + 255) / 256), dim3(256), 0, stream, a, seg_chunks,
                      scratch);
    if (e != cudaSuccess) return fail("gated_linear_chunked (2): %s", cudaGetErrorString(e));
    e = launch_kernel(chunk_out_kernel, dim3(num_chunks, H), dim3(256), so, stream, a, chunks, (const float*)scratch, C);
    if (e != cudaSuccess) return fail("gated_linear_chunked (3): %s", cudaGetErrorString(e));
    return check_launch("gated_linear_chunked");
}
