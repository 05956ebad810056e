// Parts of blocks whose two sublayers read ONE normalised input, and of the two mixers that come with
// them: attention with several score maps per head over shared values, and attention over a latent
// cache (one row per position that is key and value at once).  Everything here is float32 math on
// the CUDA cores; inputs are float32 products (possibly split-K parts that are summed in order),
// outputs are in the compute dtype unless a sum is still to be taken in 32 bits.
//
//   add_layernorm      x <- x + d1 + d2;  out = (x - mean) / sqrt(var + eps) * w      (no bias)
//   stream_pack        dst[:, col0 : col0 + W] = x + d1 + d2 (compute dtype), optionally x <- 0
//   glu_act            out = act(gate) * up for a stacked [gate | up] product
//   rope_append_maps   rotate the maps of q and k, q out, keys and values into their page
//   latent_prep        unit-RMS latent with weight, shared rotated key part -> page; q's two parts out
//   head_linear        out[t, h, :] = W[h] x[t, h, :]: one small matrix per head
//   maps_combine       o = a1 - lambda a2, o / rms(o) * post, times sigmoid(gate_h)
#include "common.cuh"
#include "mma_helpers.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {

template <typename T>
__device__ __forceinline__ float load_parts(const T* p, size_t idx, int nsplit, size_t split_stride) {
    float v = to_float(p[idx]);
#pragma unroll 4              // the parts' loads in flight together; they are still added in order
    for (int s = 1; s < nsplit; ++s) v += to_float(p[idx + (size_t)s * split_stride]);
    return v;
}

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float gelu_tanhf(float z) {
    const float c = 0.7978845608028654f;      // sqrt(2 / pi)
    return 0.5f * z * (1.f + tanhf(c * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float siluf(float z) { return z / (1.f + expf(-z)); }

// ---- layer norm with up to two products added to the stream first ---------------------------------
// For output row r (source row s = rows ? rows[r] : r): v = x[s] + d1[s] + d2[s]; without `rows` the sum
// is written back (the residual is updated in place).  mean and variance (the mean of the squared
// deviations, taken in a second pass over the row) in float32.
template <typename DT, typename OT, bool VEC>
__global__ void add_layernorm_kernel(float* __restrict__ x, const DT* __restrict__ d1, int n1, size_t s1,
                                     const DT* __restrict__ d2, int n2, size_t s2,
                                     const float* __restrict__ weight, float eps, const int* __restrict__ rows,
                                     OT* __restrict__ out, int H) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * H;
    const bool write_back = (d1 != nullptr || d2 != nullptr) && rows == nullptr;
    float sum = 0.f;
    if (VEC) {          // four elements per thread and load (rows and parts 16-byte aligned, float32 products)
        const float* f1 = (const float*)d1;
        const float* f2 = (const float*)d2;
        for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
            float4 v = *(const float4*)(xr + i);
            if (f1)
#pragma unroll 4
            for (int p = 0; p < n1; ++p) {
                const float4 a = *(const float4*)(f1 + (size_t)p * s1 + (size_t)s * H + i);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            if (f2)
#pragma unroll 4
            for (int p = 0; p < n2; ++p) {
                const float4 a = *(const float4*)(f2 + (size_t)p * s2 + (size_t)s * H + i);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            if (write_back) *(float4*)(xr + i) = v;
            *(float4*)(row + i) = v;
            sum += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = xr[i];
            if (d1) v += load_parts(d1, (size_t)s * H + i, n1, s1);
            if (d2) v += load_parts(d2, (size_t)s * H + i, n2, s2);
            if (write_back) xr[i] = v;
            row[i] = v;
            sum += v;
        }
    }
    const float mean = block_sum(sum, scratch) / (float)H;
    float sq = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float c = row[i] - mean;
        sq += c * c;
    }
    const float var = block_sum(sq, scratch) / (float)H;
    const float rstd = 1.f / sqrtf(var + eps);
    OT* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<OT>((row[i] - mean) * rstd * weight[i]);
}

// ---- the stream's rows into a run of columns of a wider matrix ------------------------------------
template <typename DT, typename OT>
__global__ void stream_pack_kernel(float* __restrict__ x, const DT* __restrict__ d1, int n1, size_t s1,
                                   const DT* __restrict__ d2, int n2, size_t s2, OT* __restrict__ dst,
                                   int dst_ld, int col0, int W, int zero, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / W;
    const int i = (int)(idx - t * W);
    float v = x[idx];
    if (d1) v += load_parts(d1, idx, n1, s1);
    if (d2) v += load_parts(d2, idx, n2, s2);
    dst[t * dst_ld + col0 + i] = from_float<OT>(v);
    if (zero) x[idx] = 0.f;
}

// ---- act(gate) * up ------------------------------------------------------------------------------------
// gu[t] holds 2 I values in blocks: `block` gate values, then the `block` up values of the same indices.
template <typename IT, typename OT>
__global__ void glu_act_kernel(const IT* __restrict__ gu, int nsplit, size_t split_stride, OT* __restrict__ out,
                               int I, int block, int act, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const int gcol = (i / block) * 2 * block + i % block;
    const float g = load_parts(gu, t * 2 * I + gcol, nsplit, split_stride);
    const float u = load_parts(gu, t * 2 * I + gcol + block, nsplit, split_stride);
    const float a = act == 0 ? siluf(g) : gelu_tanhf(g);
    out[idx] = from_float<OT>(a * u);
}

// ---- rotation of q and k maps, append --------------------------------------------------------------
// A row of the product holds [q: nq * d | k: nkv * kparts * d | v: nkv * dv | anything else], nq counting
// every map of every head.  The first rdim elements of every map are rotated (interleaved pairs
// (2i, 2i+1) or half-split pairs (i, i + rdim/2)), angle = float(position) * inv_freq[i].  One page holds
// [keys: nkv][P][kparts * d] followed by [values: nkv][P][dv].
template <typename QT, typename CT>
__global__ void rope_append_maps_kernel(const float* __restrict__ proj, int nsplit, size_t split_stride, int ld,
                                        const int* __restrict__ positions, const int* __restrict__ tok_seg,
                                        const int* __restrict__ block_table, int table_width,
                                        const float* __restrict__ inv_freq, int rdim, int interleaved,
                                        QT* __restrict__ q_out, CT* __restrict__ cache, int nq, int nkv, int kparts,
                                        int d, int dv, int P, int num_pages, int q_pad, int* __restrict__ status) {
    extern __shared__ float sh[];            // cos, sin
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int rhalf = rdim >> 1;
    float* cs = sh;
    float* sn = sh + rhalf;
    for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c;
        sn[i] = s;
    }
    __syncthreads();
    const int qw = nq * d, kmaps = nkv * kparts, kw = kmaps * d, vw = nkv * dv;
    const size_t base = (size_t)t * ld;
    const int within = pos % P;
    CT* page_k = nullptr;
    CT* page_v = nullptr;
    const int page = block_table[(size_t)tok_seg[t] * table_width + pos / P];
    if (page < 0 || page >= num_pages) {          // never write outside the pool
        if (threadIdx.x == 0 && status) atomicOr(status, 2);
    } else {
        page_k = cache + (size_t)page * nkv * P * (kparts * d + dv);
        page_v = page_k + (size_t)nkv * P * kparts * d;
    }
    const int units = rhalf + (d - rdim);     // rotated pairs and plain elements per map
    for (int idx = threadIdx.x; idx < (nq + kmaps) * units; idx += blockDim.x) {
        const int head = idx / units, u = idx - head * units;
        const size_t src = base + (size_t)head * d;      // the k maps follow the q maps in the row
        // q_pad: a q map is a row kparts * d wide that holds the map at its own columns (zeros elsewhere, below)
        QT* qdst = head >= nq ? nullptr
                   : q_pad ? q_out + ((size_t)t * nq + head) * (kparts * d) + (head % kparts) * d
                           : q_out + (size_t)t * qw + head * d;
        CT* kdst = nullptr;
        if (head >= nq && page_k) {
            const int km = head - nq, g = km / kparts, m = km - g * kparts;
            kdst = page_k + ((size_t)g * P + within) * (kparts * d) + m * d;
        }
        if (!qdst && !kdst) continue;
        if (u < rhalf) {
            const int ia = interleaved ? 2 * u : u, ib = interleaved ? 2 * u + 1 : u + rhalf;
            const float a = load_parts(proj, src + ia, nsplit, split_stride);
            const float b = load_parts(proj, src + ib, nsplit, split_stride);
            const float oa = a * cs[u] - b * sn[u];
            const float ob = b * cs[u] + a * sn[u];
            if (qdst) { qdst[ia] = from_float<QT>(oa); qdst[ib] = from_float<QT>(ob); }
            else { kdst[ia] = from_float<CT>(oa); kdst[ib] = from_float<CT>(ob); }
        } else {
            const int e = rdim + (u - rhalf);
            const float a = load_parts(proj, src + e, nsplit, split_stride);
            if (qdst) qdst[e] = from_float<QT>(a);
            else kdst[e] = from_float<CT>(a);
        }
    }
    if (q_pad) {
        const int other = (kparts - 1) * d;           // the columns of a padded row that belong to other maps
        for (int idx = threadIdx.x; idx < nq * other; idx += blockDim.x) {
            const int head = idx / other, e = idx - head * other;
            const int col = e < (head % kparts) * d ? e : e + d;
            q_out[((size_t)t * nq + head) * (kparts * d) + col] = from_float<QT>(0.f);
        }
    }
    if (page_v) {
        for (int i = threadIdx.x; i < vw; i += blockDim.x) {
            const int g = i / dv, e = i - g * dv;
            page_v[((size_t)g * P + within) * dv + e] =
                from_float<CT>(load_parts(proj, base + qw + kw + i, nsplit, split_stride));
        }
    }
}

// ---- the latent cache row and q's two parts ---------------------------------------------------------
// A row of the product holds [q: heads * (d + dr) | latent: rank | shared key part: dr | anything else].
// The latent is divided by its root mean square (eps inside the root) and multiplied by `weight`; the
// shared key part and the last dr elements of every q head are rotated over their whole width.  The
// cache row of the position is [latent | rotated key part]; a page holds [P][rank + dr].
// q_plain [T, heads, d] receives the unrotated parts, q_full [T, heads, rank + dr] the rotated parts in
// its last dr columns (its first `rank` columns are for the product of q_plain with the key expansion).
template <typename QT, typename CT>
__global__ void latent_prep_kernel(const float* __restrict__ proj, int nsplit, size_t split_stride, int ld,
                                   const float* __restrict__ weight, float eps, const int* __restrict__ positions,
                                   const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                   int table_width, const float* __restrict__ inv_freq, int interleaved,
                                   QT* __restrict__ q_plain, QT* __restrict__ q_full, CT* __restrict__ cache,
                                   int heads, int d, int dr, int rank, int P, int num_pages, int write_kv,
                                   int* __restrict__ status) {
    extern __shared__ float sh[];            // cos, sin
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int rhalf = dr >> 1;
    float* cs = sh;
    float* sn = sh + rhalf;
    for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c;
        sn[i] = s;
    }
    const size_t base = (size_t)t * ld;
    const int qw = heads * (d + dr);
    const int width = rank + dr;
    // q: plain parts and rotated parts
    __syncthreads();
    for (int idx = threadIdx.x; idx < heads * d; idx += blockDim.x) {
        const int h = idx / d, e = idx - h * d;
        q_plain[(size_t)t * heads * d + idx] =
            from_float<QT>(load_parts(proj, base + (size_t)h * (d + dr) + e, nsplit, split_stride));
    }
    for (int idx = threadIdx.x; idx < heads * rhalf; idx += blockDim.x) {
        const int h = idx / rhalf, u = idx - h * rhalf;
        const int ia = interleaved ? 2 * u : u, ib = interleaved ? 2 * u + 1 : u + rhalf;
        const size_t src = base + (size_t)h * (d + dr) + d;
        const float a = load_parts(proj, src + ia, nsplit, split_stride);
        const float b = load_parts(proj, src + ib, nsplit, split_stride);
        QT* dst = q_full + ((size_t)t * heads + h) * width + rank;
        dst[ia] = from_float<QT>(a * cs[u] - b * sn[u]);
        dst[ib] = from_float<QT>(b * cs[u] + a * sn[u]);
    }
    if (!write_kv) return;
    // the latent's mean square
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = load_parts(proj, base + qw + i, nsplit, split_stride);
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float rinv = 1.f / sqrtf(total / (float)rank + eps);
    const int page = block_table[(size_t)tok_seg[t] * table_width + pos / P];
    if (page < 0 || page >= num_pages) {          // never write outside the pool
        if (threadIdx.x == 0 && status) atomicOr(status, 2);
        return;
    }
    CT* rowp = cache + ((size_t)page * P + pos % P) * width;
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        rowp[i] = from_float<CT>(load_parts(proj, base + qw + i, nsplit, split_stride) * rinv * weight[i]);
    for (int u = threadIdx.x; u < rhalf; u += blockDim.x) {
        const int ia = interleaved ? 2 * u : u, ib = interleaved ? 2 * u + 1 : u + rhalf;
        const float a = load_parts(proj, base + qw + rank + ia, nsplit, split_stride);
        const float b = load_parts(proj, base + qw + rank + ib, nsplit, split_stride);
        rowp[rank + ia] = from_float<CT>(a * cs[u] - b * sn[u]);
        rowp[rank + ib] = from_float<CT>(b * cs[u] + a * sn[u]);
    }
}

// ---- one small matrix per head -------------------------------------------------------------------------
// out[t, h, n] = sum_k x[t, h, k] * w[h, n, k] (float32 accumulation); x and out are addressed by a row
// stride and a head stride, so both may be runs of columns of wider rows.
constexpr int HL_T = 32, HL_N = 64, HL_K = 32;
template <typename XT, typename WT, typename OT>
__global__ void __launch_bounds__(128)
head_linear_kernel(const XT* __restrict__ x, size_t xs_t, size_t xs_h, const WT* __restrict__ w,
                   OT* __restrict__ out, size_t os_t, size_t os_h, int T, int N, int K) {
    __shared__ float xs[HL_T][HL_K + 1];
    __shared__ float ws[HL_N][HL_K + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * HL_T, n0 = blockIdx.y * HL_N, h = blockIdx.z;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const WT* wh = w + (size_t)h * N * K;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += HL_K) {
        for (int idx = threadIdx.x; idx < HL_T * HL_K; idx += 128) {
            const int r = idx / HL_K, c = idx - r * HL_K;
            const int t = t0 + r, k = k0 + c;
            xs[r][c] = (t < T && k < K) ? to_float(x[(size_t)t * xs_t + (size_t)h * xs_h + k]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < HL_N * HL_K; idx += 128) {
            const int r = idx / HL_K, c = idx - r * HL_K;
            const int n = n0 + r, k = k0 + c;
            ws[r][c] = (n < N && k < K) ? to_float(wh[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < HL_K; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[ty + 8 * i][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ws[tx + 16 * j][kk];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty + 8 * i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n < N) out[(size_t)t * os_t + (size_t)h * os_h + n] = from_float<OT>(acc[i][j]);
        }
    }
}

// The same on the tensor cores (bfloat16 in, float32 accumulation): one CTA per 64 tokens x 64 outputs of a
// head; both tiles are staged whole by cp.async (K padded to a multiple of 32 with zeros), each warp owns 16
// tokens and walks K with mma.sync m16n8k16.  x's strides and K must be multiples of 8 elements.
constexpr int HM_T = 64, HM_N = 64;
template <typename OT>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, size_t xs_t, size_t xs_h, const __nv_bfloat16* __restrict__ w,
                       OT* __restrict__ out, size_t os_t, size_t os_h, int T, int N, int K, int KP) {
    extern __shared__ __align__(16) uint8_t hm_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int LD = KP + 8;                      // padded row, in elements: keeps ldmatrix free of bank conflicts
    const uint32_t xs = (uint32_t)__cvta_generic_to_shared(hm_smem);
    const uint32_t ws = xs + HM_T * LD * 2;
    const int t0 = blockIdx.x * HM_T, n0 = blockIdx.y * HM_N, h = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* wh = w + (size_t)h * N * K;
    const int cpr = KP / 8;                     // 16-byte chunks per row
    for (int c = tid; c < HM_T * cpr; c += 128) {
        const int r = c / cpr, ch = c - r * cpr;
        const bool live = t0 + r < T && ch * 8 < K;
        const __nv_bfloat16* src = live ? x + (size_t)(t0 + r) * xs_t + (size_t)h * xs_h + ch * 8 : x;
        cp_async16(xs + (r * LD + ch * 8) * 2, src, live ? 16 : 0);
    }
    for (int c = tid; c < HM_N * cpr; c += 128) {
        const int r = c / cpr, ch = c - r * cpr;
        const bool live = n0 + r < N && ch * 8 < K;
        const __nv_bfloat16* src = live ? wh + (size_t)(n0 + r) * K + ch * 8 : wh;
        cp_async16(ws + (r * LD + ch * 8) * 2, src, live ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    float acc[HM_N / 8][4];
#pragma unroll
    for (int j = 0; j < HM_N / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const int wrow = warp * 16;
    for (int k = 0; k < KP; k += 32) {
        uint32_t a0[4], a1[4];
        const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1), c = k + 8 * (lane >> 4);
        ldmatrix_x4(xs + (r * LD + c) * 2, a0[0], a0[1], a0[2], a0[3]);
        ldmatrix_x4(xs + (r * LD + c + 16) * 2, a1[0], a1[1], a1[2], a1[3]);
#pragma unroll
        for (int j = 0; j < HM_N / 8; ++j) {
            uint32_t b0, b1, b2, b3;          // 8 outputs x 32 elements of K
            ldmatrix_x4(ws + ((j * 8 + (lane & 7)) * LD + k + 8 * (lane >> 3)) * 2, b0, b1, b2, b3);
            mma_bf16(acc[j], a0, b0, b1);
            mma_bf16(acc[j], a1, b2, b3);
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int t = t0 + wrow + (lane >> 2) + 8 * half;
        if (t >= T) continue;
        OT* o = out + (size_t)t * os_t + (size_t)h * os_h;
        // two neighbours in one store where the pair is whole and its address even
        const bool pairs = sizeof(OT) == 2 && ((os_t | os_h) & 1) == 0 && ((uintptr_t)out & 3) == 0;
#pragma unroll
        for (int j = 0; j < HM_N / 8; ++j) {
            const int n = n0 + j * 8 + (lane & 3) * 2;
            if (pairs && n + 1 < N) {
                *(uint32_t*)(o + n) = pack_bf16(acc[j][2 * half], acc[j][2 * half + 1]);
                continue;
            }
            if (n < N) o[n] = from_float<OT>(acc[j][2 * half]);
            if (n + 1 < N) o[n + 1] = from_float<OT>(acc[j][2 * half + 1]);
        }
    }
}

// ---- the maps of a head into one output ------------------------------------------------------------------
// a [T, heads, 2, dv] float32 (map 1, map 2 of every head); o = a1 - lambda * a2; o <- o / sqrt(mean(o^2) + eps)
// * post; times sigmoid(gate[t][h]) if there is a gate (one column per head of a float32 product).
template <typename OT>
__global__ void maps_combine_kernel(const float* __restrict__ a, float lambda, float eps, float post,
                                    const float* __restrict__ gate, int gate_nsplit, size_t gate_split_stride,
                                    int gate_ld, OT* __restrict__ out, size_t pairs, int heads, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t th = (size_t)blockIdx.x * warps + warp;      // (token, head)
    if (th >= pairs) return;
    const size_t t = th / heads;
    const int h = (int)(th - t * heads);
    const float* a1 = a + th * 2 * dv;
    const float* a2 = a1 + dv;
    float ss = 0.f;
    for (int e = lane; e < dv; e += 32) {
        const float o = a1[e] - lambda * a2[e];
        ss += o * o;
    }
    ss = warp_sum(ss);
    float mul = post / sqrtf(ss / (float)dv + eps);
    if (gate) {
        const size_t idx = t * gate_ld + h;
        float z = gate[idx];
        for (int s = 1; s < gate_nsplit; ++s) z += gate[idx + (size_t)s * gate_split_stride];
        mul *= sigmoidf(z);
    }
    OT* o = out + th * dv;
    for (int e = lane; e < dv; e += 32) o[e] = from_float<OT>((a1[e] - lambda * a2[e]) * mul);
}

int row_threads(int H) {
    int t = (H + 31) / 32 * 32;
    if (t > 512) t = 512;
    if (t < 64) t = 64;
    return t;
}
}  // namespace

MHB_EXPORT int mhb_add_layernorm(float* x, const void* d1, int n1, long long s1, const void* d2, int n2,
                                 long long s2, int delta_dtype, const float* weight, float eps, const int* rows,
                                 void* out, int out_dtype, int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    if ((n1 > 1 || n2 > 1) && delta_dtype != MHB_F32) return fail("add_layernorm: split partials must be float32");
    const size_t smem = sizeof(float) * (size_t)H;
    const bool vec = delta_dtype == MHB_F32 && H % 4 == 0 && s1 % 4 == 0 && s2 % 4 == 0 && ((uintptr_t)x & 15) == 0 &&
                     ((uintptr_t)d1 & 15) == 0 && ((uintptr_t)d2 & 15) == 0;
    const int threads = vec ? row_threads(H / 4) : row_threads(H);
    if (vec) {
        MHB_DISPATCH_DTYPE(out_dtype, OT, {
            auto kern = add_layernorm_kernel<float, OT, true>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return fail("add_layernorm: a row of %d: %s", H, cudaGetErrorString(e));
            }
            launch_kernel(kern, dim3(R), dim3(threads), smem, stream, x, (const float*)d1, n1, (size_t)s1,
                          (const float*)d2, n2, (size_t)s2, weight, eps, rows, (OT*)out, H);
        });
        return check_launch("add_layernorm");
    }
    MHB_DISPATCH_DTYPE(delta_dtype, DT, MHB_DISPATCH_DTYPE(out_dtype, OT, {
        auto kern = add_layernorm_kernel<DT, OT, false>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail("add_layernorm: a row of %d: %s", H, cudaGetErrorString(e));
        }
        launch_kernel(kern, dim3(R), dim3(threads), smem, stream, x, (const DT*)d1, n1, (size_t)s1,
                      (const DT*)d2, n2, (size_t)s2, weight, eps, rows, (OT*)out, H);
    }));
    return check_launch("add_layernorm");
}

MHB_EXPORT int mhb_stream_pack(float* x, const void* d1, int n1, long long s1, const void* d2, int n2, long long s2,
                               int delta_dtype, void* dst, int dst_dtype, int dst_ld, int col0, int T, int W, int zero,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if ((n1 > 1 || n2 > 1) && delta_dtype != MHB_F32) return fail("stream_pack: split partials must be float32");
    if (col0 < 0 || col0 + W > dst_ld) return fail("stream_pack: columns %d..%d of %d", col0, col0 + W, dst_ld);
    const size_t total = (size_t)T * W;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    MHB_DISPATCH_DTYPE(delta_dtype, DT, MHB_DISPATCH_DTYPE(dst_dtype, OT,
        launch_kernel(stream_pack_kernel<DT, OT>, dim3(blocks), dim3(256), 0, stream, x, (const DT*)d1, n1, (size_t)s1,
                      (const DT*)d2, n2, (size_t)s2, (OT*)dst, dst_ld, col0, W, zero, total)));
    return check_launch("stream_pack");
}

MHB_EXPORT int mhb_glu_act(const void* gu, int in_dtype, int nsplit, long long split_stride, void* out, int out_dtype,
                           int T, int I, int block, int act, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (block <= 0 || I % block) return fail("glu_act: block %d does not divide %d", block, I);
    if (nsplit > 1 && in_dtype != MHB_F32) return fail("glu_act: split partials must be float32");
    if (act != 0 && act != 1) return fail("glu_act: unknown activation %d", act);
    const size_t total = (size_t)T * I;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(out_dtype, OT,
        launch_kernel(glu_act_kernel<IT, OT>, dim3(blocks), dim3(256), 0, stream, (const IT*)gu, nsplit,
                      (size_t)split_stride, (OT*)out, I, block, act, total)));
    return check_launch("glu_act");
}

MHB_EXPORT int mhb_rope_append_maps(const float* proj, int nsplit, long long split_stride, int ld,
                                    const int* positions, const int* tok_seg, const int* block_table, int table_width,
                                    const float* inv_freq, int rdim, int interleaved, void* q_out, void* cache,
                                    int dtype, int T, int nq, int nkv, int kparts, int d, int dv, int P, int num_pages,
                                    int q_pad, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rdim % 2 || rdim < 0 || rdim > d) return fail("rope_append_maps: %d rotated elements of %d", rdim, d);
    if (nq * d + nkv * kparts * d + nkv * dv > ld)
        return fail("rope_append_maps: a row of %d holds no q, k and v of these sizes", ld);
    const size_t smem = sizeof(float) * (size_t)(rdim > 0 ? rdim : 2);
    const int threads = row_threads((nq + nkv * kparts) * (d - rdim / 2));
    MHB_DISPATCH_DTYPE(dtype, CT,
        launch_kernel(rope_append_maps_kernel<CT, CT>, dim3(T), dim3(threads), smem, stream, proj, nsplit,
                      (size_t)split_stride, ld, positions, tok_seg, block_table, table_width, inv_freq, rdim,
                      interleaved, (CT*)q_out, (CT*)cache, nq, nkv, kparts, d, dv, P, num_pages, q_pad, status));
    return check_launch("rope_append_maps");
}

MHB_EXPORT int mhb_latent_prep(const float* proj, int nsplit, long long split_stride, int ld, const float* weight,
                               float eps, const int* positions, const int* tok_seg, const int* block_table,
                               int table_width, const float* inv_freq, int interleaved, void* q_plain, void* q_full,
                               void* cache, int dtype, int T, int heads, int d, int dr, int rank, int P, int num_pages,
                               int write_kv, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dr % 2 || dr < 0) return fail("latent_prep: a rotated part of %d elements", dr);
    if (heads * (d + dr) + (write_kv ? rank + dr : 0) > ld) return fail("latent_prep: a row of %d holds no q and latent of these sizes", ld);
    const size_t smem = sizeof(float) * (size_t)(dr > 0 ? dr : 2);
    const int threads = row_threads(heads * d > rank ? heads * d : rank);
    MHB_DISPATCH_DTYPE(dtype, CT,
        launch_kernel(latent_prep_kernel<CT, CT>, dim3(T), dim3(threads), smem, stream, proj, nsplit,
                      (size_t)split_stride, ld, weight, eps, positions, tok_seg, block_table, table_width, inv_freq,
                      interleaved, (CT*)q_plain, (CT*)q_full, (CT*)cache, heads, d, dr, rank, P, num_pages, write_kv,
                      status));
    return check_launch("latent_prep");
}

MHB_EXPORT int mhb_head_linear(const void* x, int x_dtype, long long xs_t, long long xs_h, const void* w, int w_dtype,
                               void* out, int out_dtype, long long os_t, long long os_h, int T, int heads, int N, int K,
                               cudaStream_t stream) {
    if (T <= 0 || heads <= 0 || N <= 0) return 0;
    if (heads > 65535) return fail("head_linear: too many heads");
    const int KP = (K + 31) / 32 * 32;
    const size_t smem = (size_t)(HM_T + HM_N) * (KP + 8) * 2;
    if (x_dtype == MHB_BF16 && w_dtype == MHB_BF16 && K % 8 == 0 && xs_t % 8 == 0 && xs_h % 8 == 0 &&
        ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && smem <= 200 * 1024) {
        dim3 grid((T + HM_T - 1) / HM_T, (N + HM_N - 1) / HM_N, heads);
        MHB_DISPATCH_DTYPE(out_dtype, OT, {
            auto kern = head_linear_mma_kernel<OT>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return fail("head_linear: shared memory %zu: %s", smem, cudaGetErrorString(e));
            }
            launch_kernel(kern, grid, dim3(128), smem, stream, (const __nv_bfloat16*)x, (size_t)xs_t, (size_t)xs_h,
                          (const __nv_bfloat16*)w, (OT*)out, (size_t)os_t, (size_t)os_h, T, N, K, KP);
        });
        return check_launch("head_linear");
    }
    dim3 grid((T + HL_T - 1) / HL_T, (N + HL_N - 1) / HL_N, heads);
    MHB_DISPATCH_DTYPE(x_dtype, XT, MHB_DISPATCH_DTYPE(w_dtype, WT, MHB_DISPATCH_DTYPE(out_dtype, OT,
        launch_kernel(head_linear_kernel<XT, WT, OT>, grid, dim3(128), 0, stream, (const XT*)x, (size_t)xs_t,
                      (size_t)xs_h, (const WT*)w, (OT*)out, (size_t)os_t, (size_t)os_h, T, N, K))));
    return check_launch("head_linear");
}

MHB_EXPORT int mhb_maps_combine(const float* a, float lambda, float eps, float post, const float* gate,
                                int gate_nsplit, long long gate_split_stride, int gate_ld, void* out, int out_dtype,
                                int T, int heads, int dv, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int warps = 4;
    const size_t pairs = (size_t)T * heads;
    dim3 grid((unsigned)((pairs + warps - 1) / warps));
    MHB_DISPATCH_DTYPE(out_dtype, OT,
        launch_kernel(maps_combine_kernel<OT>, grid, dim3(warps * 32), 0, stream, a, lambda, eps, post, gate,
                      gate_nsplit, (size_t)gate_split_stride, gate_ld, (OT*)out, pairs, heads, dv));
    return check_launch("maps_combine");
}
