// A routed feed-forward (mixture of experts) without a word from the host between its kernels:
//
//   moe_route     per token: softmax over the router's outputs, choice scores (softmax + correction), the best
//                 `keep` of `groups` equal groups of neighbours, the `top` best choice scores inside them, and
//                 the chosen outputs' softmax values divided by their sum (+ 1e-20)
//   moe_plan      the chosen (token, expert) pairs grouped by expert: a row per pair, tiles of TILE_ROWS rows of
//                 one expert each (outputs at or beyond `experts` are identity experts and get no row)
//   moe_linear    out[r] = W[expert of r] x[source of r], tile by tile; `glu`: W holds [gate ; up] and the result is
//                 silu(gate x) * (up x).  bfloat16 on mma.sync m16n8k16, float32 (and odd widths) on FFMA tiles;
//                 float32 accumulation in both
//   moe_combine   out[t] = sum_k weight[t, k] * (row of pair (t, k), or the input itself for an identity expert)
//                          + sigmoid(shared gate logit[t]) * shared expert's output[t]
//
// Which row a pair gets inside its expert depends on the order of atomic additions; every row is computed by
// itself and a token's pairs are summed in the order of their choice, so the result does not.
#include "common.cuh"
#include "mma_helpers.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {

constexpr int TILE_ROWS = 64;

__device__ __forceinline__ float load_parts(const float* p, size_t idx, int nsplit, size_t stride) {
    float v = p[idx];
    for (int s = 1; s < nsplit; ++s) v += p[idx + (size_t)s * stride];
    return v;
}

// ---- router ---------------------------------------------------------------------------------------------
// one warp per token; shared memory: per warp n softmax values, n choice scores, `groups` group scores
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, int nsplit, size_t stride, int ld, const float* __restrict__ correction,
             int* __restrict__ chosen, float* __restrict__ weights, int T, int n, int top, int groups, int keep,
             const float* __restrict__ bias) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* s = sm + (size_t)warp * (2 * n + groups);
    float* c = s + n;
    float* gs = c + n;
    float mx = -INFINITY;
    for (int i = lane; i < n; i += 32) {
        const float z = load_parts(logits, (size_t)t * ld + i, nsplit, stride) + (bias ? bias[i] : 0.f);
        s[i] = z;
        mx = fmaxf(mx, z);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) {
        const float e = expf(s[i] - mx);
        s[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    for (int i = lane; i < n; i += 32) {
        s[i] = s[i] / sum;
        c[i] = s[i] + (correction ? correction[i] : 0.f);
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = n / groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int i = 0; i < per; ++i) best = fmaxf(best, c[g * per + i]);
            gs[g] = best;
        }
        __syncwarp();
        // the `keep` best groups, ties to the lower index; a taken group's score becomes NaN-free +inf mark
        for (int r = 0; r < keep; ++r) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gs[g];
                if (v != INFINITY && (v > best || (v == best && g < arg) || arg == 0x7fffffff)) { best = v; arg = g; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
            }
            if (lane == 0 && arg != 0x7fffffff) gs[arg] = INFINITY;
            __syncwarp();
        }
        for (int i = lane; i < n; i += 32)
            if (gs[i / per] != INFINITY) c[i] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    float mine = 0.f;             // lane k keeps the k-th pick
    int mine_at = 0;
    for (int r = 0; r < top; ++r) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int i = lane; i < n; i += 32) {
            const float v = c[i];
            if (v != -INFINITY && (arg == 0x7fffffff || v > best)) { best = v; arg = i; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;          // fewer candidates than picks: cannot happen with a valid configuration
        const float p = s[arg];
        total += p;
        if (lane == (r & 31)) { mine = p; mine_at = arg; }
        if (lane == 0) c[arg] = -INFINITY;
        __syncwarp();
        if ((r & 31) == 31 || r == top - 1) {      // flush up to 32 picks
            const int base = r & ~31;
            if (base + lane <= r) {
                chosen[(size_t)t * top + base + lane] = mine_at;
                weights[(size_t)t * top + base + lane] = mine;     // divided below
            }
        }
    }
    __syncwarp();
    const float inv = 1.f / (total + 1e-20f);
    for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] *= inv;
}

// ---- grouping by expert -----------------------------------------------------------------------------------
// plan (int32): [0] tiles; [1 .. 1 + 3 max_tiles) {expert, first row, one past the last row} per tile;
// then row_token [pairs] and pair_row [pairs] (-1: an identity expert)
__global__ void __launch_bounds__(1024)
plan_kernel(const int* __restrict__ chosen, int pairs, int top, int experts, int max_tiles, int* __restrict__ plan) {
    extern __shared__ int ism[];
    int* count = ism;                   // [experts]
    int* first = count + experts;       // [experts]
    int* cursor = first + experts;      // [experts]
    pdl_launch_dependents();
    pdl_wait();
    int* tiles = plan + 1;
    int* row_token = tiles + 3 * max_tiles;
    int* pair_row = row_token + pairs;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, nt = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = row;
            for (int r = 0; r < count[e] && nt < max_tiles; r += TILE_ROWS) {
                tiles[3 * nt] = e;
                tiles[3 * nt + 1] = row + r;
                tiles[3 * nt + 2] = row + min(count[e], r + TILE_ROWS);
                ++nt;
            }
            row += count[e];
        }
        plan[0] = nt;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < experts) {
            const int r = first[e] + atomicAdd(&cursor[e], 1);
            row_token[r] = i / top;
            pair_row[i] = r;
        } else {
            pair_row[i] = -1;
        }
    }
}

__device__ __forceinline__ float siluf_(float z) { return z / (1.f + expf(-z)); }

// ---- grouped product, CUDA cores ---------------------------------------------------------------------------
// tile: 32 rows x 64 outputs, K in blocks of 32; 128 threads, 4 x 4 outputs each.  glu: outputs n and F + n of W.
constexpr int GL_T = 32, GL_N = 64, GL_K = 32;
template <typename XT, typename OT, bool GLU>
__global__ void __launch_bounds__(128)
linear_kernel(const XT* __restrict__ x, size_t x_ld, const int* __restrict__ plan, int max_tiles, int pairs, int gather,
              const XT* __restrict__ w, OT* __restrict__ out, int N, int K) {
    __shared__ float xs[GL_T][GL_K + 1];
    __shared__ float ws[GLU ? 2 : 1][GL_N][GL_K + 1];
    __shared__ int src[GL_T];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x / (TILE_ROWS / GL_T), sub = blockIdx.x % (TILE_ROWS / GL_T);
    if (tile >= plan[0]) return;
    const int* ti = plan + 1 + 3 * tile;
    const int e = ti[0], r0 = ti[1] + sub * GL_T, r1 = ti[2];
    if (r0 >= r1) return;
    const int* row_token = plan + 1 + 3 * max_tiles;
    const int n0 = blockIdx.y * GL_N;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const size_t wrows = GLU ? 2 * (size_t)N : (size_t)N;
    const XT* we = w + (size_t)e * wrows * K;
    if (threadIdx.x < GL_T) {
        const int r = r0 + threadIdx.x;
        src[threadIdx.x] = r < r1 ? (gather ? row_token[r] : r) : -1;
    }
    __syncthreads();
    float acc[4][4] = {}, acc2[GLU ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += GL_K) {
        for (int idx = threadIdx.x; idx < GL_T * GL_K; idx += 128) {
            const int r = idx / GL_K, c = idx - r * GL_K;
            const int s = src[r], k = k0 + c;
            xs[r][c] = (s >= 0 && k < K) ? to_float(x[(size_t)s * x_ld + k]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < GL_N * GL_K; idx += 128) {
            const int r = idx / GL_K, c = idx - r * GL_K;
            const int n = n0 + r, k = k0 + c;
            const bool live = n < N && k < K;
            ws[0][r][c] = live ? to_float(we[(size_t)n * K + k]) : 0.f;
            if (GLU) ws[GLU ? 1 : 0][r][c] = live ? to_float(we[((size_t)N + n) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < GL_K; ++kk) {
            float xv[4], wv[4], uv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[ty + 8 * i][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                wv[j] = ws[0][tx + 16 * j][kk];
                if (GLU) uv[j] = ws[GLU ? 1 : 0][tx + 16 * j][kk];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
                    if (GLU) acc2[GLU ? i : 0][j] = fmaf(xv[i], uv[j], acc2[GLU ? i : 0][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty + 8 * i;
        if (r >= r1) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            const float v = GLU ? siluf_(acc[i][j]) * acc2[GLU ? i : 0][j] : acc[i][j];
            out[(size_t)r * N + n] = from_float<OT>(v);
        }
    }
}

// ---- grouped product, tensor cores (bfloat16) ---------------------------------------------------------------
// tile: 64 rows x 64 outputs (glu: of gate and of up), K in blocks of 64 that cp.async brings in GM_STAGES - 1 blocks
// ahead of the one the tensor cores work on; 4 warps of 16 rows.  K and x's row stride are multiples of 8 elements.
// Few rows (decoded tokens) wait on the weights: four stages keep more bytes in flight.  Many rows are bound by the
// tensor cores and by how many CTAs an SM holds: two stages.
constexpr int GM_N = 64, GM_K = 64, GM_LD = GM_K + 8, GM_FEW_ROWS = 512;
constexpr size_t gm_smem(bool glu, int stages) { return (size_t)stages * (TILE_ROWS + (glu ? 2 : 1) * GM_N) * GM_LD * 2; }
template <typename OT, bool GLU, int GM_STAGES>
__global__ void __launch_bounds__(128)
linear_mma_kernel(const __nv_bfloat16* __restrict__ x, size_t x_ld, const int* __restrict__ plan, int max_tiles,
                  int pairs, int gather, const __nv_bfloat16* __restrict__ w, OT* __restrict__ out, int N, int K) {
    extern __shared__ __align__(16) unsigned char gm_stages[];       // [GM_STAGES] x {x tile, w tile}
    __shared__ int src[TILE_ROWS];
    constexpr uint32_t XS_BYTES = TILE_ROWS * GM_LD * 2, STAGE_BYTES = XS_BYTES + (GLU ? 2 : 1) * GM_N * GM_LD * 2;
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int* ti = plan + 1 + 3 * tile;
    const int e = ti[0], r0 = ti[1], r1 = ti[2];
    const int* row_token = plan + 1 + 3 * max_tiles;
    const int n0 = blockIdx.y * GM_N;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t wrows = GLU ? 2 * (size_t)N : (size_t)N;
    const __nv_bfloat16* we = w + (size_t)e * wrows * K;
    if (tid < TILE_ROWS) {
        const int r = r0 + tid;
        src[tid] = r < r1 ? (gather ? row_token[r] : r) : -1;
    }
    __syncthreads();
    const uint32_t stages = (uint32_t)__cvta_generic_to_shared(gm_stages);
    float acc[GM_N / 8][4], acc2[GLU ? GM_N / 8 : 1][4];
#pragma unroll
    for (int j = 0; j < GM_N / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
    for (int j = 0; j < (GLU ? GM_N / 8 : 1); ++j) acc2[j][0] = acc2[j][1] = acc2[j][2] = acc2[j][3] = 0.f;
    const int wrow = warp * 16;
    constexpr int CPR = GM_K / 8;
    auto bring = [&](int kb) {                  // block kb of K into its stage
        const int k0 = kb * GM_K;
        const uint32_t xs = stages + (kb % GM_STAGES) * STAGE_BYTES, ws = xs + XS_BYTES;
        for (int c = tid; c < TILE_ROWS * CPR; c += 128) {
            const int r = c / CPR, ch = c - r * CPR;
            const bool live = src[r] >= 0 && k0 + ch * 8 < K;
            const __nv_bfloat16* p = live ? x + (size_t)src[r] * x_ld + k0 + ch * 8 : x;
            cp_async16(xs + (r * GM_LD + ch * 8) * 2, p, live ? 16 : 0);
        }
        for (int c = tid; c < (GLU ? 2 : 1) * GM_N * CPR; c += 128) {
            const int r = c / CPR, ch = c - r * CPR;
            const int half = r / GM_N, n = n0 + (r - half * GM_N);
            const bool live = n < N && k0 + ch * 8 < K;
            const __nv_bfloat16* p = live ? we + ((size_t)half * N + n) * K + k0 + ch * 8 : we;
            cp_async16(ws + (r * GM_LD + ch * 8) * 2, p, live ? 16 : 0);
        }
    };
    const int nk = (K + GM_K - 1) / GM_K;
    for (int kb = 0; kb < GM_STAGES - 1; ++kb) {
        if (kb < nk) bring(kb);
        cp_async_commit();
    }
    for (int kb = 0; kb < nk; ++kb) {
        cp_async_wait<GM_STAGES - 2>();         // block kb has landed (for this thread)
        __syncthreads();                        // for every thread; and everyone is done with block kb - 1,
        if (kb + GM_STAGES - 1 < nk) bring(kb + GM_STAGES - 1);      // whose stage the next block takes
        cp_async_commit();
        const uint32_t xs = stages + (kb % GM_STAGES) * STAGE_BYTES, ws = xs + XS_BYTES;
#pragma unroll
        for (int k = 0; k < GM_K; k += 32) {
            uint32_t a0[4], a1[4];
            const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1), c = k + 8 * (lane >> 4);
            ldmatrix_x4(xs + (r * GM_LD + c) * 2, a0[0], a0[1], a0[2], a0[3]);
            ldmatrix_x4(xs + (r * GM_LD + c + 16) * 2, a1[0], a1[1], a1[2], a1[3]);
#pragma unroll
            for (int j = 0; j < GM_N / 8; ++j) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(ws + ((j * 8 + (lane & 7)) * GM_LD + k + 8 * (lane >> 3)) * 2, b0, b1, b2, b3);
                mma_bf16(acc[j], a0, b0, b1);
                mma_bf16(acc[j], a1, b2, b3);
                if (GLU) {
                    ldmatrix_x4(ws + ((GM_N + j * 8 + (lane & 7)) * GM_LD + k + 8 * (lane >> 3)) * 2, b0, b1, b2, b3);
                    mma_bf16(acc2[GLU ? j : 0], a0, b0, b1);
                    mma_bf16(acc2[GLU ? j : 0], a1, b2, b3);
                }
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = r0 + wrow + (lane >> 2) + 8 * half;
        if (r >= r1) continue;
        OT* o = out + (size_t)r * N;
#pragma unroll
        for (int j = 0; j < GM_N / 8; ++j) {
            const int n = n0 + j * 8 + (lane & 3) * 2;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (n + u >= N) continue;
                const float a = acc[j][2 * half + u];
                o[n + u] = from_float<OT>(GLU ? siluf_(a) * acc2[GLU ? j : 0][2 * half + u] : a);
            }
        }
    }
}

// ---- the weighted sum -------------------------------------------------------------------------------------
template <typename HT>
__global__ void __launch_bounds__(256)
combine_kernel(const float* __restrict__ y, const int* __restrict__ plan, int max_tiles, int pairs,
               const int* __restrict__ chosen, const float* __restrict__ weights, int top, int experts,
               const HT* __restrict__ h, size_t h_ld, const float* __restrict__ shared, int sn, size_t ss,
               const float* __restrict__ sg, int gn, size_t gs, int g_ld, float* __restrict__ out, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int* pair_row = plan + 1 + 3 * max_tiles + pairs;
    float gate = 0.f;
    if (shared) gate = 1.f / (1.f + expf(-load_parts(sg, t * g_ld, gn, gs)));
    for (int j = threadIdx.x; j < W; j += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const size_t i = t * top + k;
            const int r = pair_row[i];
            const float v = r >= 0 ? y[(size_t)r * W + j] : to_float(h[t * h_ld + j]);
            acc = fmaf(weights[i], v, acc);
        }
        if (shared) acc = fmaf(gate, load_parts(shared, t * W + j, sn, ss), acc);
        out[t * W + j] = acc;
    }
}

}  // namespace

MHB_EXPORT int mhb_moe_tile_rows() { return TILE_ROWS; }

// bias (or null): added to the logits before the softmax; correction may be null too (no correction).  With both
// null groups the choice is by the logits themselves and the weights are the softmax over the chosen logits.
MHB_EXPORT int mhb_moe_route_biased(const float* logits, int nsplit, long long stride, int ld, const float* bias,
                                    const float* correction, int* chosen, float* weights, int T, int n, int top,
                                    int groups, int keep, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (top < 1 || top > n) return fail("moe_route: %d picks among %d outputs", top, n);
    if (groups < 1 || n % groups || keep < 1 || keep > groups)
        return fail("moe_route: %d outputs in %d groups of which %d are kept", n, groups, keep);
    if ((long long)(n / groups) * keep < top) return fail("moe_route: the kept groups hold fewer than %d outputs", top);
    const int warps = 4;
    const size_t smem = sizeof(float) * warps * (2 * (size_t)n + groups);
    if (smem > 48 * 1024) return fail("moe_route: %d router outputs are more than the kernel holds", n);
    cudaError_t e = launch_kernel(route_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), smem, stream, logits,
                                  nsplit, (size_t)stride, ld, correction, chosen, weights, T, n, top, groups, keep, bias);
    if (e != cudaSuccess) return fail("moe_route: %s", cudaGetErrorString(e));
    return check_launch("moe_route");
}

MHB_EXPORT int mhb_moe_route(const float* logits, int nsplit, long long stride, int ld, const float* correction,
                             int* chosen, float* weights, int T, int n, int top, int groups, int keep,
                             cudaStream_t stream) {
    return mhb_moe_route_biased(logits, nsplit, stride, ld, nullptr, correction, chosen, weights, T, n, top, groups,
                                keep, stream);
}

MHB_EXPORT int mhb_moe_plan(const int* chosen, int pairs, int top, int experts, int max_tiles, int* plan,
                            cudaStream_t stream) {
    if (pairs <= 0) return 0;
    const size_t smem = sizeof(int) * 3 * (size_t)experts;
    if (smem > 48 * 1024) return fail("moe_plan: %d experts are more than the kernel holds", experts);
    cudaError_t e = launch_kernel(plan_kernel, dim3(1), dim3(1024), smem, stream, chosen, pairs, top, experts, max_tiles,
                                  plan);
    if (e != cudaSuccess) return fail("moe_plan: %s", cudaGetErrorString(e));
    return check_launch("moe_plan");
}

MHB_EXPORT int mhb_moe_linear(const void* x, int x_dtype, long long x_ld, const int* plan, int max_tiles, int pairs,
                              int gather, const void* w, void* out, int out_dtype, int N, int K, int glu,
                              cudaStream_t stream) {
    if (pairs <= 0 || max_tiles <= 0) return 0;
    const bool mma = x_dtype == MHB_BF16 && K % 8 == 0 && x_ld % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
    cudaError_t e;
    if (mma) {
        dim3 grid(max_tiles, (N + GM_N - 1) / GM_N);
        const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
        const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
        const bool few = pairs <= GM_FEW_ROWS;
        if (glu && out_dtype != MHB_BF16) return fail("moe_linear: the gated product writes the compute dtype");
#define MHB_MOE_MMA(OT, GLU, ST)                                                                                      \
    do {                                                                                                              \
        static bool raised = false;                                                                                   \
        if (!raised) {                                                                                                \
            if (cudaFuncSetAttribute(linear_mma_kernel<OT, GLU, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                     (int)gm_smem(GLU, ST)) != cudaSuccess)                                           \
                return fail("moe_linear: cannot raise the shared-memory limit");                                      \
            raised = true;                                                                                            \
        }                                                                                                             \
        e = launch_kernel(linear_mma_kernel<OT, GLU, ST>, grid, dim3(128), gm_smem(GLU, ST), stream, xb, (size_t)x_ld, \
                          plan, max_tiles, pairs, gather, wb, (OT*)out, N, K);                                        \
    } while (0)
        if (glu) {
            if (few) MHB_MOE_MMA(__nv_bfloat16, true, 4); else MHB_MOE_MMA(__nv_bfloat16, true, 2);
        } else if (out_dtype == MHB_F32) {
            if (few) MHB_MOE_MMA(float, false, 4); else MHB_MOE_MMA(float, false, 2);
        } else {
            if (few) MHB_MOE_MMA(__nv_bfloat16, false, 4); else MHB_MOE_MMA(__nv_bfloat16, false, 2);
        }
#undef MHB_MOE_MMA
    } else {
        dim3 grid(max_tiles * (TILE_ROWS / GL_T), (N + GL_N - 1) / GL_N);
        if (x_dtype == MHB_F32) {
            if (out_dtype != MHB_F32) return fail("moe_linear: a float32 product writes float32");
            e = glu ? launch_kernel(linear_kernel<float, float, true>, grid, dim3(128), 0, stream, (const float*)x,
                                    (size_t)x_ld, plan, max_tiles, pairs, gather, (const float*)w, (float*)out, N, K)
                    : launch_kernel(linear_kernel<float, float, false>, grid, dim3(128), 0, stream, (const float*)x,
                                    (size_t)x_ld, plan, max_tiles, pairs, gather, (const float*)w, (float*)out, N, K);
        } else {
            const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
            const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
            if (glu && out_dtype == MHB_BF16)
                e = launch_kernel(linear_kernel<__nv_bfloat16, __nv_bfloat16, true>, grid, dim3(128), 0, stream, xb,
                                  (size_t)x_ld, plan, max_tiles, pairs, gather, wb, (__nv_bfloat16*)out, N, K);
            else if (!glu && out_dtype == MHB_F32)
                e = launch_kernel(linear_kernel<__nv_bfloat16, float, false>, grid, dim3(128), 0, stream, xb, (size_t)x_ld,
                                  plan, max_tiles, pairs, gather, wb, (float*)out, N, K);
            else
                return fail("moe_linear: the gated product writes the compute dtype, the plain one float32");
        }
    }
    if (e != cudaSuccess) return fail("moe_linear: %s", cudaGetErrorString(e));
    return check_launch("moe_linear");
}

MHB_EXPORT int mhb_moe_combine(const float* y, const int* plan, int max_tiles, int pairs, const int* chosen,
                               const float* weights, int top, int experts, const void* h, int h_dtype, long long h_ld,
                               const float* shared, int sn, long long ss, const float* sg, int gn, long long gs, int g_ld,
                               float* out, int T, int W, cudaStream_t stream) {
    if (T <= 0) return 0;
    MHB_DISPATCH_DTYPE(h_dtype, HT, {
        cudaError_t e = launch_kernel(combine_kernel<HT>, dim3(T), dim3(256), 0, stream, y, plan, max_tiles, pairs, chosen,
                                      weights, top, experts, (const HT*)h, (size_t)h_ld, shared, sn, (size_t)ss, sg, gn,
                                      (size_t)gs, g_ld, out, W);
        if (e != cudaSuccess) return fail("moe_combine: %s", cudaGetErrorString(e));
    });
    return check_launch("moe_combine");
}
