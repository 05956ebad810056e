// Memory-bound kernels of blocks that normalise AFTER the residual sum, and of mixers that
// normalise or gate their own vectors:
//
//   norm_mix        x <- keep * x + rms(alpha * x + delta) * w, and a copy of x in the compute dtype
//                   (post-norm: keep = 0; a normalised branch added to the stream: alpha = 0, keep = 1)
//   act_rows        relu(z)^2 (and other activations by code, or a plain conversion) of a product that may
//                   come in split-K parts
//   table_gate      gelu_tanh(z[t, j]) * table[token[t], column0 + j]
//   gated_rmsnorm   rms(o) * w * sigmoid(g)
//   qknorm_rope_append   RMS norm over the WHOLE q projection and over the whole k projection (all
//                   heads at once), rotation of the first rdim elements of every head, q to a
//                   matrix, k and v into the pages of the cache
//
// Everything is computed in float32; inputs from a split-K product arrive as `nsplit` float32
// partial matrices `split_stride` elements apart and are summed in index order.
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {

__device__ __forceinline__ float load_parts(const float* p, size_t idx, int nsplit, size_t split_stride) {
    float v = p[idx];
    for (int s = 1; s < nsplit; ++s) v += p[idx + (size_t)s * split_stride];
    return v;
}
template <typename T>
__device__ __forceinline__ float load_parts_t(const T* p, size_t idx, int nsplit, size_t split_stride) {
    float v = to_float(p[idx]);
    for (int s = 1; s < nsplit; ++s) v += to_float(p[idx + (size_t)s * split_stride]);
    return v;
}

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float gelu_tanhf(float z) {
    const float c = 0.7978845608028654f;      // sqrt(2 / pi)
    return 0.5f * z * (1.f + tanhf(c * (z + 0.044715f * z * z * z)));
}

template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *(const float4*)p; }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 u = *(const uint2*)p;
    const __nv_bfloat162 a = *(const __nv_bfloat162*)&u.x, b = *(const __nv_bfloat162*)&u.y;
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *(float4*)p = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *(const uint32_t*)&a;
    u.y = *(const uint32_t*)&b;
    *(uint2*)p = u;
}
template <typename T>
__device__ __forceinline__ float4 load4_parts(const T* p, size_t idx, int nsplit, size_t split_stride) {
    float4 v = load4<T>(p + idx);
    for (int s = 1; s < nsplit; ++s) {
        const float4 w = load4<T>(p + idx + (size_t)s * split_stride);
        v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    return v;
}

// ---- x <- keep x + rms(alpha x + delta) w ---------------------------------------------------------
template <typename DT, typename OT>
__global__ void norm_mix_kernel(float* __restrict__ x, const DT* __restrict__ delta, int nsplit,
                                size_t split_stride, const float* __restrict__ weight, float eps,
                                float alpha, float keep, OT* __restrict__ copy, int H) {
    extern __shared__ float row[];           // alpha x + delta of this row
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    float* xr = x + r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = alpha != 0.f ? alpha * xr[i] : 0.f;
        if (delta) s += load_parts_t(delta, r * H + i, nsplit, split_stride);
        row[i] = s;
        ss += s * s;
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(total / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float n = row[i] * rstd * weight[i];
        if (keep != 0.f) n += keep * xr[i];
        xr[i] = n;
        if (copy) copy[r * H + i] = from_float<OT>(n);
    }
}

// The same with four elements per thread and step (H % 4 == 0, every row 16-byte aligned).
template <typename DT, typename OT>
__global__ void norm_mix_vec_kernel(float* __restrict__ x, const DT* __restrict__ delta, int nsplit,
                                    size_t split_stride, const float* __restrict__ weight, float eps,
                                    float alpha, float keep, OT* __restrict__ copy, int H) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    float* xr = x + r * H;
    float ss = 0.f;
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        if (alpha != 0.f) {
            const float4 v = *(const float4*)(xr + i);
            s = make_float4(alpha * v.x, alpha * v.y, alpha * v.z, alpha * v.w);
        }
        if (delta) {
            const float4 d = load4_parts(delta, r * H + i, nsplit, split_stride);
            s.x += d.x; s.y += d.y; s.z += d.z; s.w += d.w;
        }
        *(float4*)(row + i) = s;
        ss += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(total / (float)H + eps);
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
        const float4 s = *(const float4*)(row + i), w = *(const float4*)(weight + i);
        float4 n = make_float4(s.x * rstd * w.x, s.y * rstd * w.y, s.z * rstd * w.z, s.w * rstd * w.w);
        if (keep != 0.f) {
            const float4 v = *(const float4*)(xr + i);
            n.x += keep * v.x; n.y += keep * v.y; n.z += keep * v.z; n.w += keep * v.w;
        }
        *(float4*)(xr + i) = n;
        if (copy) store4<OT>(copy + r * H + i, n);
    }
}

// ---- activations of a product ----------------------------------------------------------------------
enum { ACT_RELU2 = 0, ACT_SILU = 1, ACT_GELU_TANH = 2, ACT_COPY = 3 };

template <typename IT, typename OT>
__global__ void act_rows_kernel(const IT* __restrict__ z, int nsplit, size_t split_stride, OT* __restrict__ out,
                                size_t n, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = load_parts_t(z, i, nsplit, split_stride);
    float a;
    if (act == ACT_RELU2) { a = fmaxf(v, 0.f); a *= a; }
    else if (act == ACT_SILU) a = v * sigmoidf(v);
    else if (act == ACT_GELU_TANH) a = gelu_tanhf(v);
    else a = v;
    out[i] = from_float<OT>(a);
}

__device__ __forceinline__ float act_of(float v, int act) {
    if (act == ACT_RELU2) { const float a = fmaxf(v, 0.f); return a * a; }
    if (act == ACT_SILU) return v * sigmoidf(v);
    if (act == ACT_GELU_TANH) return gelu_tanhf(v);
    return v;
}

// four elements per thread (n % 4 == 0, 16-byte aligned, parts a multiple of four elements apart)
template <typename IT, typename OT>
__global__ void act_rows_vec_kernel(const IT* __restrict__ z, int nsplit, size_t split_stride, OT* __restrict__ out,
                                    size_t n, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = 4 * ((size_t)blockIdx.x * blockDim.x + threadIdx.x);
    if (i >= n) return;
    const float4 v = load4_parts(z, i, nsplit, split_stride);
    store4<OT>(out + i, make_float4(act_of(v.x, act), act_of(v.y, act), act_of(v.z, act), act_of(v.w, act)));
}

// ---- gelu_tanh(z) * table[token, column0 + j] -------------------------------------------------------
template <typename IT, typename WT, typename OT>
__global__ void table_gate_kernel(const IT* __restrict__ z, int nsplit, size_t split_stride,
                                  const WT* __restrict__ table, int table_width, int column0, int vocab,
                                  const int* __restrict__ tokens, OT* __restrict__ out, int T, int D,
                                  int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)T * D) return;
    const int t = (int)(i / D), j = (int)(i - (size_t)t * D);
    const int tok = tokens[t];
    float e = 0.f;
    if (tok >= 0 && tok < vocab) e = to_float(table[(size_t)tok * table_width + column0 + j]);
    else if (status) atomicOr(status, 1);
    out[i] = from_float<OT>(gelu_tanhf(load_parts_t(z, i, nsplit, split_stride)) * e);
}

// ---- rms(o) * w * sigmoid(g) -------------------------------------------------------------------------
template <typename OT>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_nsplit,
                                     size_t gate_split_stride, int gate_ld, const float* __restrict__ weight,
                                     float eps, OT* __restrict__ out, int N) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    const float* orow = o + r * N;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) { const float v = orow[i]; ss += v * v; }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(total / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        float n = orow[i] * rstd * weight[i];
        if (gate) n *= sigmoidf(load_parts(gate, r * gate_ld + i, gate_nsplit, gate_split_stride));
        out[r * N + i] = from_float<OT>(n);
    }
}

// ---- q/k norm over the whole projection, rotation, append ------------------------------------------
// A row of the product holds [q: nq * dk | k: nkv * dk | v: nkv * dv | anything else]; a layer that
// reads another layer's cache has [q | anything else] and has_kv = 0.  One page of the cache holds
// [keys: nkv][P][dk] followed by [values: nkv][P][dv].
template <typename QT, typename CT>
__global__ void qknorm_rope_append_kernel(const float* __restrict__ qkv, int nsplit, size_t split_stride, int ld,
                                          const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                          float eps, const int* __restrict__ positions,
                                          const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                          int table_width, const float* __restrict__ inv_freq, int rdim,
                                          QT* __restrict__ q_out, CT* __restrict__ cache, int nq, int nkv, int dk,
                                          int dv, int P, int num_pages, int has_kv, int* __restrict__ status,
                                          int per_head, float v_eps, size_t page_extra) {
    extern __shared__ float sh[];            // q row, k row, cos, sin (and the v row, if it is normalised)
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int qw = nq * dk, kw = has_kv ? nkv * dk : 0, vw = has_kv ? nkv * dv : 0;
    const int rhalf = rdim >> 1;
    float* qs = sh;
    float* ks = qs + qw;
    float* cs = ks + kw;
    float* sn = cs + rhalf;
    const size_t base = (size_t)t * ld;
    float ssq = 0.f, ssk = 0.f;
    for (int i = threadIdx.x; i < qw + kw; i += blockDim.x) {
        const float v = load_parts(qkv, base + i, nsplit, split_stride);
        sh[i] = v;
        if (i < qw) ssq += v * v; else ssk += v * v;
    }
    for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c;
        sn[i] = s;
    }
    float* vs = sn + rhalf;                  // [vw], only with v_eps > 0
    if (v_eps > 0.f)
        for (int i = threadIdx.x; i < vw; i += blockDim.x) vs[i] = load_parts(qkv, base + qw + kw + i, nsplit, split_stride);
    if (per_head) {
        // one norm per head over its dk elements, the weight [dk] shared by the heads: a warp per head
        __syncthreads();
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
        for (int head = warp; head < (qw + kw) / dk; head += nwarps) {
            float* row = sh + head * dk;
            const float* w = head < nq ? q_weight : k_weight;
            float ss = 0.f;
            for (int e = lane; e < dk; e += 32) ss += row[e] * row[e];
            const float r = 1.f / sqrtf(warp_sum(ss) / (float)dk + eps);
            for (int e = lane; e < dk; e += 32) row[e] = row[e] * r * w[e];
        }
    } else {
        const float tq = block_sum(ssq, scratch);
        const float tk = block_sum(ssk, scratch);
        const float rq = 1.f / sqrtf(tq / (float)qw + eps);
        const float rk = kw ? 1.f / sqrtf(tk / (float)kw + eps) : 0.f;
        for (int i = threadIdx.x; i < qw + kw; i += blockDim.x)
            sh[i] = i < qw ? sh[i] * rq * q_weight[i] : sh[i] * rk * k_weight[i - qw];
    }
    __syncthreads();
    if (v_eps > 0.f) {
        // every head's value divided by its own root mean square (no weight): a warp per head
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
        for (int head = warp; head < (has_kv ? nkv : 0); head += nwarps) {
            float* row = vs + head * dv;
            float ss = 0.f;
            for (int e = lane; e < dv; e += 32) ss += row[e] * row[e];
            const float r = 1.f / sqrtf(warp_sum(ss) / (float)dv + v_eps);
            for (int e = lane; e < dv; e += 32) row[e] *= r;
        }
        __syncthreads();
    }
    CT* page_k = nullptr;
    CT* page_v = nullptr;
    const int within = pos % P;
    if (has_kv) {
        const int page = block_table[(size_t)tok_seg[t] * table_width + pos / P];
        if (page < 0 || page >= num_pages) {          // never write outside the pool
            if (threadIdx.x == 0 && status) atomicOr(status, 2);
        } else {
            page_k = cache + (size_t)page * ((size_t)nkv * P * (dk + dv) + page_extra);
            page_v = page_k + (size_t)nkv * P * dk;
        }
    }
    // one thread per unit: rdim/2 rotated pairs and dk - rdim plain elements per head
    const int units = rhalf + (dk - rdim);
    const int heads = nq + (has_kv ? nkv : 0);
    for (int idx = threadIdx.x; idx < heads * units; idx += blockDim.x) {
        const int head = idx / units, u = idx - head * units;
        const float* src = sh + head * dk;       // k heads follow the q heads in shared memory
        QT* qdst = head < nq ? q_out + (size_t)t * qw + head * dk : nullptr;
        CT* kdst = (head >= nq && page_k) ? page_k + ((size_t)(head - nq) * P + within) * dk : nullptr;
        if (u < rhalf) {
            const float a = src[u], b = src[u + rhalf];
            const float oa = a * cs[u] - b * sn[u];
            const float ob = b * cs[u] + a * sn[u];
            if (qdst) { qdst[u] = from_float<QT>(oa); qdst[u + rhalf] = from_float<QT>(ob); }
            else if (kdst) { kdst[u] = from_float<CT>(oa); kdst[u + rhalf] = from_float<CT>(ob); }
        } else {
            const int e = rdim + (u - rhalf);
            if (qdst) qdst[e] = from_float<QT>(src[e]);
            else if (kdst) kdst[e] = from_float<CT>(src[e]);
        }
    }
    if (page_v) {
        for (int i = threadIdx.x; i < vw; i += blockDim.x) {
            const int g = i / dv, e = i - g * dv;
            page_v[((size_t)g * P + within) * dv + e] =
                from_float<CT>(v_eps > 0.f ? vs[i] : load_parts(qkv, base + qw + kw + i, nsplit, split_stride));
        }
    }
}

int row_threads(int H) {
    int t = (H + 31) / 32 * 32;
    if (t > 512) t = 512;
    if (t < 64) t = 64;
    return t;
}

template <typename Kern>
int allow_smem(Kern kern, size_t smem, const char* what) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("%s: shared memory %zu: %s", what, smem, cudaGetErrorString(e));
    }
    return 0;
}
}  // namespace

MHB_EXPORT int mhb_norm_mix(float* x, const void* delta, int delta_dtype, int nsplit, long long split_stride,
                            const float* weight, float eps, float alpha, float keep, void* copy, int copy_dtype,
                            int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (nsplit > 1 && delta_dtype != MHB_F32) return fail("norm_mix: split partials must be float32");
    const size_t smem = sizeof(float) * (size_t)H;
    const bool vec = H % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)delta & 15) && !((uintptr_t)weight & 15) &&
                     !((uintptr_t)copy & 15) && split_stride % 4 == 0;
    if (vec) {
        int threads = (H / 4 + 31) / 32 * 32;
        if (threads > 512) threads = 512;
        if (threads < 64) threads = 64;
        MHB_DISPATCH_DTYPE(delta_dtype, DT, MHB_DISPATCH_DTYPE(copy_dtype, OT, {
            auto kern = norm_mix_vec_kernel<DT, OT>;
            if (allow_smem(kern, smem, "norm_mix")) return -1;
            launch_kernel(kern, dim3(R), dim3(threads), smem, stream, x, (const DT*)delta, nsplit,
                          (size_t)split_stride, weight, eps, alpha, keep, (OT*)copy, H);
        }));
        return check_launch("norm_mix");
    }
    MHB_DISPATCH_DTYPE(delta_dtype, DT, MHB_DISPATCH_DTYPE(copy_dtype, OT, {
        auto kern = norm_mix_kernel<DT, OT>;
        if (allow_smem(kern, smem, "norm_mix")) return -1;
        launch_kernel(kern, dim3(R), dim3(row_threads(H)), smem, stream, x, (const DT*)delta, nsplit,
                      (size_t)split_stride, weight, eps, alpha, keep, (OT*)copy, H);
    }));
    return check_launch("norm_mix");
}

MHB_EXPORT int mhb_act_rows(const void* z, int in_dtype, int nsplit, long long split_stride, void* out,
                            int out_dtype, long long n, int act, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (act < 0 || act > ACT_COPY) return fail("act_rows: unknown activation %d", act);
    if (nsplit > 1 && in_dtype != MHB_F32) return fail("act_rows: split partials must be float32");
    const int threads = 256;
    if (n % 4 == 0 && !((uintptr_t)z & 15) && !((uintptr_t)out & 15) && split_stride % 4 == 0) {
        const unsigned vblocks = (unsigned)((n / 4 + threads - 1) / threads);
        MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(out_dtype, OT,
            launch_kernel((act_rows_vec_kernel<IT, OT>), dim3(vblocks), dim3(threads), 0, stream, (const IT*)z, nsplit,
                          (size_t)split_stride, (OT*)out, (size_t)n, act)));
        return check_launch("act_rows");
    }
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(out_dtype, OT,
        launch_kernel((act_rows_kernel<IT, OT>), dim3(blocks), dim3(threads), 0, stream, (const IT*)z, nsplit,
                      (size_t)split_stride, (OT*)out, (size_t)n, act)));
    return check_launch("act_rows");
}

MHB_EXPORT int mhb_table_gate(const void* z, int in_dtype, int nsplit, long long split_stride, const void* table,
                              int table_dtype, int table_width, int column0, int vocab, const int* tokens,
                              void* out, int out_dtype, int T, int D, int* status, cudaStream_t stream) {
    if (T <= 0 || D <= 0) return 0;
    if (column0 < 0 || column0 + D > table_width) return fail("table_gate: columns %d..%d outside a table %d wide", column0, column0 + D, table_width);
    if (nsplit > 1 && in_dtype != MHB_F32) return fail("table_gate: split partials must be float32");
    const int threads = 256;
    const unsigned blocks = (unsigned)(((size_t)T * D + threads - 1) / threads);
    MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(table_dtype, WT, MHB_DISPATCH_DTYPE(out_dtype, OT,
        launch_kernel((table_gate_kernel<IT, WT, OT>), dim3(blocks), dim3(threads), 0, stream, (const IT*)z, nsplit,
                      (size_t)split_stride, (const WT*)table, table_width, column0, vocab, tokens, (OT*)out, T, D,
                      status))));
    return check_launch("table_gate");
}

MHB_EXPORT int mhb_gated_rmsnorm(const float* o, const float* gate, int gate_nsplit, long long gate_split_stride,
                                 int gate_ld, const float* weight, float eps, void* out, int out_dtype, int R, int N,
                                 cudaStream_t stream) {
    if (R <= 0) return 0;
    MHB_DISPATCH_DTYPE(out_dtype, OT,
        launch_kernel(gated_rmsnorm_kernel<OT>, dim3(R), dim3(row_threads(N)), 0, stream, o, gate, gate_nsplit,
                      (size_t)gate_split_stride, gate_ld, weight, eps, (OT*)out, N));
    return check_launch("gated_rmsnorm");
}

// per_head: the two norms run over each head alone, with weights [dk] that the heads share, instead of over the whole
// projections.  v_eps > 0: every head's value is divided by its root mean square (with that eps) before it is stored.
// page_extra: elements of a page behind its keys and values (left alone here).
MHB_EXPORT int mhb_qknorm_rope_append_opts(const float* qkv, int nsplit, long long split_stride, int ld,
                                      const float* q_weight, const float* k_weight, float eps, const int* positions,
                                      const int* tok_seg, const int* block_table, int table_width,
                                      const float* inv_freq, int rdim, void* q_out, void* cache, int dtype, int T,
                                      int nq, int nkv, int dk, int dv, int P, int num_pages, int has_kv, int* status,
                                      int per_head, float v_eps, long long page_extra, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rdim < 0 || rdim > dk || (rdim & 1)) return fail("qknorm_rope_append: %d rotated elements of a head of %d", rdim, dk);
    const int qw = nq * dk, kw = has_kv ? nkv * dk : 0;
    const size_t smem = sizeof(float) * ((size_t)qw + kw + rdim + (v_eps > 0.f && has_kv ? (size_t)nkv * dv : 0));
    MHB_DISPATCH_DTYPE(dtype, CT, {
        auto kern = qknorm_rope_append_kernel<CT, CT>;
        if (allow_smem(kern, smem, "qknorm_rope_append")) return -1;
        launch_kernel(kern, dim3(T), dim3(row_threads(qw + kw)), smem, stream, qkv, nsplit, (size_t)split_stride, ld,
                      q_weight, k_weight, eps, positions, tok_seg, block_table, table_width, inv_freq, rdim,
                      (CT*)q_out, (CT*)cache, nq, nkv, dk, dv, P, num_pages, has_kv, status, per_head, v_eps,
                      (size_t)page_extra);
    });
    return check_launch("qknorm_rope_append");
}

MHB_EXPORT int mhb_qknorm_rope_append(const float* qkv, int nsplit, long long split_stride, int ld,
                                      const float* q_weight, const float* k_weight, float eps, const int* positions,
                                      const int* tok_seg, const int* block_table, int table_width,
                                      const float* inv_freq, int rdim, void* q_out, void* cache, int dtype, int T,
                                      int nq, int nkv, int dk, int dv, int P, int num_pages, int has_kv, int* status,
                                      cudaStream_t stream) {
    return mhb_qknorm_rope_append_opts(qkv, nsplit, split_stride, ld, q_weight, k_weight, eps, positions, tok_seg,
                                       block_table, table_width, inv_freq, rdim, q_out, cache, dtype, T, nq, nkv, dk, dv,
                                       P, num_pages, has_kv, status, 0, 0.f, 0, stream);
}
