// Small kernels around attention whose mask or weights are not the plain causal ones.
//
//   pool_means   block means of cached keys and values.  A page of the pool holds the keys [nkv][P][d] and values
//                [nkv][P][dv] of its P positions and, behind them, pooled keys [nkv][slots][d] and pooled values
//                [nkv][slots][dv], slots = ceil(P / pool).  Block b covers the positions b pool .. b pool + pool - 1;
//                its means are taken over the rows AS THE CACHE HOLDS THEM (after whatever norm and rotation they
//                got, in the cache's dtype), summed in float32, and stored in the page of the block's last
//                position at slot b - floor(page_index P / pool).  One CTA per (token, KV head): the token that
//                completes a block writes it (it runs behind the kernel that appended this step's rows); the
//                others return at once.
//   talk_mix     o[t][h][:] = sum_g talk[h][g] a[t][g][kv(h)][:]: the heads' softmax weights mixed AFTER the
//                softmax, written as a mix of outputs: a[t][g][c] is head g's weights applied to the values of KV
//                head c, and head h keeps the values of its own KV head.  The three strides of `a` (token, head,
//                KV head) are arguments: one kernel writes rows [nkv][dv] wide, another one plane per KV head.
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
template <typename CT>
__global__ void __launch_bounds__(128)
pool_means_kernel(CT* __restrict__ cache, const int* __restrict__ positions, const int* __restrict__ tok_seg,
                  const int* __restrict__ block_table, int table_width, int nkv, int d, int dv, int P, int pool,
                  int num_pages, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, kvh = blockIdx.y;
    const int pos = positions[t];
    if ((pos + 1) % pool) return;
    const int b = pos / pool;                                  // the block that this token completes
    const int slots = (P + pool - 1) / pool;
    const size_t kv_elems = (size_t)nkv * P * (d + dv);
    const size_t page_elems = kv_elems + (size_t)nkv * slots * (d + dv);
    const int* table = block_table + (size_t)tok_seg[t] * table_width;
    const int last_page = pos / P;
    const int dst_page = table[last_page];
    if (dst_page < 0 || dst_page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, 2);
        return;
    }
    const int slot = b - (int)(((long long)last_page * P) / pool);
    const float inv = 1.f / (float)pool;
    for (int e = threadIdx.x; e < d + dv; e += blockDim.x) {
        const bool is_k = e < d;
        float sum = 0.f;
        for (int p = pos - pool + 1; p <= pos; ++p) {
            const int page = table[p / P];
            if (page < 0 || page >= num_pages) continue;       // reported by the append of that row
            const size_t base = (size_t)page * page_elems;
            const int within = p % P;
            sum += to_float(is_k ? cache[base + ((size_t)kvh * P + within) * d + e]
                                 : cache[base + (size_t)nkv * P * d + ((size_t)kvh * P + within) * dv + (e - d)]);
        }
        const size_t base = (size_t)dst_page * page_elems + kv_elems;
        if (is_k) cache[base + ((size_t)kvh * slots + slot) * d + e] = from_float<CT>(sum * inv);
        else cache[base + (size_t)nkv * slots * d + ((size_t)kvh * slots + slot) * dv + (e - d)] = from_float<CT>(sum * inv);
    }
}

template <typename OT>
__global__ void __launch_bounds__(256)
talk_mix_kernel(const float* __restrict__ a, const float* __restrict__ talk, OT* __restrict__ out, int nq, int nkv, int dv,
                size_t tok_stride, size_t head_stride, size_t kv_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int groups = nq / nkv;
    for (int idx = threadIdx.x; idx < nq * dv; idx += blockDim.x) {
        const int h = idx / dv, e = idx - h * dv;
        const float* src = a + (size_t)t * tok_stride + (size_t)(h / groups) * kv_stride + e;
        float o = 0.f;
        for (int g = 0; g < nq; ++g) o = fmaf(talk[h * nq + g], src[(size_t)g * head_stride], o);
        out[(size_t)t * nq * dv + idx] = from_float<OT>(o);
    }
}
}  // namespace

MHB_EXPORT int mhb_pool_means(void* cache, int dtype, const int* positions, const int* tok_seg, const int* block_table,
                              int table_width, int T, int nkv, int d, int dv, int P, int pool, int num_pages, int* status,
                              cudaStream_t stream) {
    if (T <= 0) return 0;
    if (pool < 1 || P < 1) return fail("pool_means: blocks of %d positions over pages of %d", pool, P);
    MHB_DISPATCH_DTYPE(dtype, CT,
        launch_kernel(pool_means_kernel<CT>, dim3(T, nkv), dim3(128), 0, stream, (CT*)cache, positions, tok_seg,
                      block_table, table_width, nkv, d, dv, P, pool, num_pages, status));
    return check_launch("pool_means");
}

MHB_EXPORT int mhb_talk_mix(const float* a, const float* talk, void* out, int dtype, int T, int nq, int nkv, int dv,
                            long long tok_stride, long long head_stride, long long kv_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (nkv < 1 || nq % nkv) return fail("talk_mix: %d heads over %d KV heads", nq, nkv);
    MHB_DISPATCH_DTYPE(dtype, OT,
        launch_kernel(talk_mix_kernel<OT>, dim3(T), dim3(256), 0, stream, a, talk, (OT*)out, nq, nkv, dv,
                      (size_t)tok_stride, (size_t)head_stride, (size_t)kv_stride));
    return check_launch("talk_mix");
}
