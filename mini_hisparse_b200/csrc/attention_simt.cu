// Causal grouped-query attention over the paged KV cache, for prefill portions and decode
// tokens alike, with float32 scores, softmax and accumulation on the CUDA cores.
//
// Math (mini_hisparse/model.py:173-179 for prompts, mini_hisparse/attention.py:26-35 for a
// decoded token): query head h reads KV head h / groups; s_t = (K[t] . q) * scale for every
// cached key t <= the query's position (the token's own key was appended before);
// w = softmax(s); o = sum_t w_t V[t].  An optional window keeps keys t > position - window.
//
// Work is described by items (8 ints each) that the host writes:
//   {segment, first token (index in the batch), tokens, first head in the group, heads,
//    kv_begin, kv_end, split}
// One CTA handles one item for one KV head: rows = tokens x heads (<= 16) against keys
// [kv_begin, kv_end).  split < 0: the normalised output is written to `out`.  split >= 0:
// the CTA writes an un-normalised partial (max, sum, accumulator) and combine merges the
// splits with the rule of reference/attention.py:11-20.
//
// Options that other mixers bring, all off by default:
//   dv != d    values of another width than keys; a page then holds [keys: nkv][P][d] followed by
//              [values: nkv][P][dv] (for dv == d that IS the layout [2][nkv][P][d])
//   sink       one learned number per query head that joins the softmax's denominator as exp(sink_h)
//              that stands for no position: the running (max, sum) starts at (sink_h, 1) instead of
//              (-inf, 0), in the unsplit item or in split 0 only, so a token's parts hold it a single time
//   gate       the output row is multiplied by sigmoid(gate[t][h * dv + e]); the gate comes as the
//              columns of a float32 product (split-K parts summed in order); with gate_per_head the
//              gate is one number per head, gate[t][h]
//   kparts     every KV head's key row holds `kparts` keys of width d side by side, each a score map of
//              its own over the SAME values: query head q belongs to map q % kparts of KV head
//              (q / kparts) / groups, and gridDim.y = nkv * kparts (one CTA per item, KV head and map)
//   softcap    s <- softcap * tanh(s / softcap) on the scaled score, before the mask and the softmax
//   shared_kv  the values ARE the first dv elements of the key rows (a latent cache: one row per
//              position serves as key and as value), so a page holds [nkv][P][kparts * d] and nothing else
//   prefix     with a window, keys that the window has passed can still be seen in one of two forms, walked
//              before the item's own key range by the unsplit item or by split 0 only:
//              pre_kind 1  the first pre_n positions of the sequence stay visible (their own keys and values)
//              pre_kind 2  every block of pre_n positions that ends at or before position - window is seen as
//                          ONE key and value (the block's means, kept in the page's tail: after the keys and
//                          values of its P positions a page holds [nkv][slots][d] pooled keys and
//                          [nkv][slots][dv] pooled values, slots = ceil(P / pre_n); block b lies in the page
//                          of its last position, at slot b - floor(page * P / pre_n))
//   vheads     nkv instead of 1: a query head's weights are applied to the values of EVERY KV head, and the
//              output row is [nkv][dv] wide (for a mixer that mixes the heads' weights afterwards)
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int R_TILE = 16;   // query rows per CTA
constexpr int KT = 32;       // keys per tile: one per lane
constexpr int WARPS = 4;
constexpr int ROWS_PER_WARP = R_TILE / WARPS;
constexpr int ITEM_INTS = 8;

struct AttnArgs {
    const void* q;             // [T, nq, d]
    const void* cache;         // [pages, 2, nkv, P, d] of one layer
    void* out;                 // [T, nq, d]
    float* part_acc;           // [rows, nq, d]
    float* part_ml;            // [rows, nq, 2]
    const int* items;
    const int* positions;      // [T]
    const int* block_table;    // [S, width]
    const int* tok_part_row;   // [T] first partial row of a token
    int num_items, width, nq, nkv, d, P, num_pages, window;
    float scale;
    int dv;                    // value width (== d unless the mixer says otherwise)
    const float* sink;         // [nq] or null
    const float* gate;         // [gate_nsplit][T][gate_ld] or null
    int gate_nsplit, gate_ld;
    size_t gate_split_stride;
    int kparts;                // score maps per KV head (1 unless the mixer says otherwise)
    float softcap;             // 0: none
    int shared_kv;             // values are the head of the key rows
    int gate_per_head;         // the gate has one column per head
    int out_f32;               // `out` is float32 whatever the dtype of q and the cache (a sum is still to come)
    int pre_kind, pre_n;       // keys seen beyond the window: 0 none, 1 the first pre_n positions, 2 means of blocks of pre_n
    int pool_slots;            // pooled rows per page and KV head (pre_kind 2)
    int vheads;                // 1, or nkv: values of every KV head
    int vhead;                 // >= 0 (with vheads 1): the values of this KV head, whatever the query head's own
    size_t page_extra;         // elements of a page behind its keys and values
};

__device__ __forceinline__ float gate_of(const AttnArgs& a, int t, int col) {
    if (!a.gate) return 1.f;
    const size_t idx = (size_t)t * a.gate_ld + col;
    float g = a.gate[idx];
    for (int s = 1; s < a.gate_nsplit; ++s) g += a.gate[idx + (size_t)s * a.gate_split_stride];
    return 1.f / (1.f + expf(-g));
}

template <typename CT, int DPL>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const AttnArgs a) {
    extern __shared__ float smem[];
    const int d = a.d, dv = a.dv * a.vheads;      // dv: the width of an output row
    float* q_s = smem;                       // [R_TILE][d]
    float* k_s = q_s + R_TILE * d;           // [KT][d + 1]
    float* v_s = k_s + KT * (d + 1);         // [KT][dv]
    __shared__ int row_pos[R_TILE];

    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= a.num_items) return;
    const int* it = a.items + (size_t)blockIdx.x * ITEM_INTS;
    const int seg = it[0], tok0 = it[1], ntok = it[2], head0 = it[3], nheads = it[4];
    const int kv_begin = it[5], kv_end = it[6], split = it[7];
    const int kparts = a.kparts;
    const int kvh = blockIdx.y / kparts, map = blockIdx.y - kvh * kparts;
    const int groups = a.nq / (a.nkv * kparts);
    const int nrows = ntok * nheads;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int k_ld = kparts * d;                                   // a key row of one KV head
    const int dv1 = a.dv;                                          // one KV head's values
    const int v_ld = a.shared_kv ? k_ld : dv1;
    const size_t v_plane = a.shared_kv ? 0 : (size_t)a.nkv * a.P * k_ld;
    const size_t kv_elems = (size_t)a.nkv * a.P * k_ld + (a.shared_kv ? 0 : (size_t)a.nkv * a.P * dv1);
    const size_t page_elems = kv_elems + a.page_extra;
    const CT* q = (const CT*)a.q;
    const CT* cache = (const CT*)a.cache;

    // stage the queries (float32) and the rows' positions
    for (int idx = threadIdx.x; idx < R_TILE * d; idx += blockDim.x) {
        const int r = idx / d, e = idx - r * d;
        float v = 0.f;
        if (r < nrows) {
            const int t = tok0 + r / nheads, h = (kvh * groups + head0 + r % nheads) * kparts + map;
            v = to_float(q[((size_t)t * a.nq + h) * d + e]);
        }
        q_s[idx] = v;
    }
    if (threadIdx.x < R_TILE) {
        const int r = threadIdx.x;
        row_pos[r] = r < nrows ? a.positions[tok0 + r / nheads] : -1;
    }
    __syncthreads();

    float m[ROWS_PER_WARP], l[ROWS_PER_WARP], acc[ROWS_PER_WARP][DPL];
#pragma unroll
    for (int rs = 0; rs < ROWS_PER_WARP; ++rs) {
        m[rs] = -INFINITY;
        l[rs] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[rs][i] = 0.f;
        const int r = rs * WARPS + warp;
        if (a.sink && split <= 0 && r < nrows) {      // a single time per token: here or in split 0
            m[rs] = a.sink[(kvh * groups + head0 + r % nheads) * kparts + map];
            l[rs] = 1.f;
        }
    }

    const int* table = a.block_table + (size_t)seg * a.width;
    // keys beyond the window (see "prefix" at the top): positions below `beyond` have left the window of the
    // item's last row, which is the one that sees the most of them
    int pre_end = 0;
    if (a.pre_kind && a.window > 0 && split <= 0 && nrows > 0) {
        const int beyond = a.positions[tok0 + ntok - 1] - a.window + 1;
        if (beyond > 0) pre_end = a.pre_kind == 1 ? min(a.pre_n, beyond) : beyond / a.pre_n;
    }
    for (int phase = pre_end > 0 ? 0 : 1; phase < 2; ++phase) {
    const int begin = phase ? kv_begin : 0, end = phase ? kv_end : pre_end;
    const bool pooled = !phase && a.pre_kind == 2;
    for (int t0 = begin; t0 < end; t0 += KT) {
        // load KT keys and values: warp w takes keys w*8 .. w*8+7, lanes run along d
        for (int j = warp * (KT / WARPS); j < (warp + 1) * (KT / WARPS); ++j) {
            const int kp = t0 + j;
            int page = -1, slot = 0;
            if (kp < end) {
                const int pg = pooled ? (kp * a.pre_n + a.pre_n - 1) / a.P : kp / a.P;
                slot = pooled ? kp - (int)(((long long)pg * a.P) / a.pre_n) : kp - pg * a.P;
                page = table[pg];
                if (page >= a.num_pages) page = -1;
            }
            if (page >= 0) {
                const size_t pbase = (size_t)page * page_elems;
                if (pooled) {
                    const size_t off = pbase + kv_elems + ((size_t)kvh * a.pool_slots + slot) * d;
                    for (int e = lane; e < d; e += 32) k_s[j * (d + 1) + e] = to_float(cache[off + e]);
                    for (int c = 0; c < a.vheads; ++c) {
                        const int vh = a.vheads > 1 ? c : (a.vhead >= 0 ? a.vhead : kvh);
                        const size_t voff = pbase + kv_elems + (size_t)a.nkv * a.pool_slots * d +
                                            ((size_t)vh * a.pool_slots + slot) * dv1;
                        for (int e = lane; e < dv1; e += 32) v_s[j * dv + c * dv1 + e] = to_float(cache[voff + e]);
                    }
                } else {
                    const size_t off = pbase + ((size_t)kvh * a.P + slot) * k_ld + map * d;
                    for (int e = lane; e < d; e += 32) k_s[j * (d + 1) + e] = to_float(cache[off + e]);
                    for (int c = 0; c < a.vheads; ++c) {
                        const int vh = a.vheads > 1 ? c : (a.vhead >= 0 ? a.vhead : kvh);
                        const size_t voff = pbase + v_plane + ((size_t)vh * a.P + slot) * v_ld;
                        for (int e = lane; e < dv1; e += 32) v_s[j * dv + c * dv1 + e] = to_float(cache[voff + e]);
                    }
                }
            } else {
                for (int e = lane; e < d; e += 32) k_s[j * (d + 1) + e] = 0.f;
                for (int e = lane; e < dv; e += 32) v_s[j * dv + e] = 0.f;
            }
        }
        __syncthreads();
        const int kp = t0 + lane;  // this lane's key
#pragma unroll
        for (int rs = 0; rs < ROWS_PER_WARP; ++rs) {
            const int r = rs * WARPS + warp;
            if (r >= nrows) continue;  // uniform within the warp
            const int qp = row_pos[r];
            const float* qr = q_s + r * d;
            const float* kr = k_s + lane * (d + 1);
            float s = 0.f;
            for (int e = 0; e < d; ++e) s = fmaf(qr[e], kr[e], s);
            s *= a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            bool valid;
            if (phase) valid = kp < end && kp <= qp && (a.window <= 0 || kp > qp - a.window);
            else if (pooled) valid = kp < end && qp - a.window + 1 > 0 && kp < (qp - a.window + 1) / a.pre_n;
            else valid = kp < end && kp <= qp - a.window;
            if (!valid) s = -INFINITY;
            const float m_new = fmaxf(m[rs], warp_max(s));
            float p = 0.f, alpha = 1.f;
            if (m_new > -INFINITY) {
                p = valid ? expf(s - m_new) : 0.f;
                alpha = m[rs] > -INFINITY ? expf(m[rs] - m_new) : 0.f;
            }
            l[rs] = l[rs] * alpha + warp_sum(p);
            m[rs] = m_new;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[rs][i] *= alpha;
            for (int j = 0; j < KT; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int e = lane + 32 * i;
                    if (e < dv) acc[rs][i] = fmaf(pj, v_s[j * dv + e], acc[rs][i]);
                }
            }
        }
        __syncthreads();
    }
    }

#pragma unroll
    for (int rs = 0; rs < ROWS_PER_WARP; ++rs) {
        const int r = rs * WARPS + warp;
        if (r >= nrows) continue;
        const int t = tok0 + r / nheads, h = (kvh * groups + head0 + r % nheads) * kparts + map;
        if (split < 0) {
            const float inv = l[rs] > 0.f ? 1.f / l[rs] : 0.f;
            const size_t o0 = ((size_t)t * a.nq + h) * dv;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int e = lane + 32 * i;
                if (e >= dv) continue;
                const float val = acc[rs][i] * inv * gate_of(a, t, a.gate_per_head ? h : h * dv + e);
                if (a.out_f32) ((float*)a.out)[o0 + e] = val;
                else ((CT*)a.out)[o0 + e] = from_float<CT>(val);
            }
        } else {
            const size_t prow = (size_t)a.tok_part_row[t] + split;
            float* pa = a.part_acc + (prow * a.nq + h) * dv;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int e = lane + 32 * i;
                if (e < dv) pa[e] = acc[rs][i];
            }
            if (lane == 0) {
                a.part_ml[(prow * a.nq + h) * 2 + 0] = m[rs];
                a.part_ml[(prow * a.nq + h) * 2 + 1] = l[rs];
            }
        }
    }
}

// Merge the splits of a token (reference/attention.py:11-20):
//   M = max m_s;  w_s = exp(m_s - M) (0 where m_s = -inf);  o = sum w_s acc_s / sum w_s l_s
template <typename OT>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc,
                                         const float* __restrict__ part_ml,
                                         const int* __restrict__ tok_part_row,
                                         const int* __restrict__ tok_nsplit, OT* __restrict__ out,
                                         int nq, int d, int every, const float* __restrict__ gate,
                                         int gate_nsplit, size_t gate_split_stride, int gate_ld,
                                         int gate_per_head) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    // every > 0: each token has exactly that many parts, in the rows t * every ...
    const int ns = every > 0 ? every : tok_nsplit[t];
    if (ns <= 0) return;  // written directly by the attention kernel
    const size_t row0 = every > 0 ? (size_t)t * every : tok_part_row[t];
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[((row0 + s) * nq + h) * 2]);
    float L = 0.f;
    for (int s = 0; s < ns; ++s) {
        const float ms = part_ml[((row0 + s) * nq + h) * 2];
        const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
        L += w * part_ml[((row0 + s) * nq + h) * 2 + 1];
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < ns; ++s) {
            const float ms = part_ml[((row0 + s) * nq + h) * 2];
            const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
            o += w * part_acc[((row0 + s) * nq + h) * d + e];
        }
        float g = 1.f;
        if (gate) {
            const size_t idx = (size_t)t * gate_ld + (gate_per_head ? h : h * d + e);
            float z = gate[idx];
            for (int s = 1; s < gate_nsplit; ++s) z += gate[idx + (size_t)s * gate_split_stride];
            g = 1.f / (1.f + expf(-z));
        }
        out[((size_t)t * nq + h) * d + e] = from_float<OT>(o * inv * g);
    }
}

template <typename CT>
int launch_attention(const AttnArgs& a, int max_items, cudaStream_t stream) {
    const int dvt = a.dv * a.vheads;
    int dpl = (dvt + 31) / 32;
    if (dpl > 8) dpl = dpl <= 12 ? 12 : 16;      // wide values: accumulators for 384 or 512 elements per row
    const size_t smem = sizeof(float) * ((size_t)R_TILE * a.d + (size_t)KT * (a.d + 1) + (size_t)KT * dvt);
    dim3 grid(max_items, a.nkv * a.kparts);
#define MHB_ATTN_CASE(N)                                                                        \
    case N: {                                                                                   \
        auto kern = attention_simt_kernel<CT, N>;                                               \
        if (smem > 48 * 1024) {                                                                 \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                    \
            if (e != cudaSuccess) return fail("attention: shared memory %zu: %s", smem,        \
                                              cudaGetErrorString(e));                           \
        }                                                                                       \
        launch_kernel(kern, grid, dim3(WARPS * 32), smem, stream, a);                           \
        break;                                                                                  \
    }
    switch (dpl) {
        MHB_ATTN_CASE(1) MHB_ATTN_CASE(2) MHB_ATTN_CASE(3) MHB_ATTN_CASE(4)
        MHB_ATTN_CASE(5) MHB_ATTN_CASE(6) MHB_ATTN_CASE(7) MHB_ATTN_CASE(8)
        MHB_ATTN_CASE(12) MHB_ATTN_CASE(16)
        default: return fail("attention: a value width of %d is larger than 512", dvt);
    }
#undef MHB_ATTN_CASE
    return check_launch("attention_simt");
}
}  // namespace

MHB_EXPORT int mhb_attention_simt(const void* q, const void* cache, void* out, int dtype,
                                  float* part_acc, float* part_ml, const int* items, int num_items,
                                  int max_items, const int* positions, const int* block_table,
                                  int width, const int* tok_part_row, int nq, int nkv, int d, int P,
                                  int num_pages, int window, float scale, cudaStream_t stream) {
    if (max_items <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attention: %d query heads over %d KV heads", nq, nkv);
    if (nkv > 65535) return fail("attention: too many KV heads");
    AttnArgs a;
    a.q = q; a.cache = cache; a.out = out; a.part_acc = part_acc; a.part_ml = part_ml;
    a.items = items; a.positions = positions; a.block_table = block_table;
    a.tok_part_row = tok_part_row; a.num_items = num_items; a.width = width; a.nq = nq;
    a.nkv = nkv; a.d = d; a.P = P; a.num_pages = num_pages; a.window = window; a.scale = scale;
    a.dv = d; a.sink = nullptr; a.gate = nullptr; a.gate_nsplit = 1; a.gate_ld = 0; a.gate_split_stride = 0;
    a.kparts = 1; a.softcap = 0.f; a.shared_kv = 0; a.gate_per_head = 0; a.out_f32 = 0;
    a.pre_kind = 0; a.pre_n = 0; a.pool_slots = 0; a.vheads = 1; a.page_extra = 0; a.vhead = -1;
    MHB_DISPATCH_DTYPE(dtype, CT, return launch_attention<CT>(a, max_items, stream));
    return 0;
}

// The same with the options: values dv wide, a sink per query head, a gate on the output.
namespace {
int attention_simt_options(const void* q, const void* cache, void* out, int dtype,
                                      float* part_acc, float* part_ml, const int* items, int num_items,
                                      int max_items, const int* positions, const int* block_table,
                                      int width, const int* tok_part_row, int nq, int nkv, int d, int dv, int P,
                                      int num_pages, int window, float scale, const float* sink,
                                      const float* gate, int gate_nsplit, long long gate_split_stride, int gate_ld,
                                      int kparts, float softcap, int shared_kv, int gate_per_head, int out_f32,
                                      int pre_kind, int pre_n, int all_values, cudaStream_t stream) {
    if (max_items <= 0) return 0;
    if (pre_kind < 0 || pre_kind > 2 || (pre_kind && pre_n < 1)) return fail("attention: keys beyond the window of kind %d over %d positions", pre_kind, pre_n);
    if ((pre_kind || all_values) && (kparts != 1 || shared_kv)) return fail("attention: keys beyond the window and values of every KV head go with plain key and value rows only");
    if (kparts < 1 || nq % (nkv > 0 ? nkv * kparts : 1)) return fail("attention: %d query heads over %d KV heads with %d score maps each", nq, nkv, kparts);
    if ((long long)nkv * kparts > 65535) return fail("attention: too many KV heads");
    if (shared_kv && dv > kparts * d) return fail("attention: values %d wide cannot be the head of key rows %d wide", dv, kparts * d);
    if (nkv <= 0 || nq % nkv) return fail("attention: %d query heads over %d KV heads", nq, nkv);
    if (nkv > 65535) return fail("attention: too many KV heads");
    if (d > 1024) return fail("attention: a key width of %d is larger than 1024", d);
    AttnArgs a;
    a.q = q; a.cache = cache; a.out = out; a.part_acc = part_acc; a.part_ml = part_ml;
    a.items = items; a.positions = positions; a.block_table = block_table;
    a.tok_part_row = tok_part_row; a.num_items = num_items; a.width = width; a.nq = nq;
    a.nkv = nkv; a.d = d; a.P = P; a.num_pages = num_pages; a.window = window; a.scale = scale;
    a.dv = dv; a.sink = sink; a.gate = gate; a.gate_nsplit = gate_nsplit; a.gate_ld = gate_ld;
    a.gate_split_stride = (size_t)gate_split_stride;
    a.kparts = kparts; a.softcap = softcap; a.shared_kv = shared_kv; a.gate_per_head = gate_per_head;
    a.out_f32 = out_f32;
    a.pre_kind = pre_kind; a.pre_n = pre_n; a.vheads = all_values == 1 ? nkv : 1;
    a.vhead = all_values >= 2 ? all_values - 2 : -1;          // 2 + c: the values of KV head c alone
    if (a.vhead >= nkv) return fail("attention: values of KV head %d of %d", a.vhead, nkv);
    a.pool_slots = pre_kind == 2 ? (P + pre_n - 1) / pre_n : 0;
    a.page_extra = (size_t)nkv * a.pool_slots * (d + dv);
    MHB_DISPATCH_DTYPE(dtype, CT, return launch_attention<CT>(a, max_items, stream));
    return 0;
}
}  // namespace

MHB_EXPORT int mhb_attention_simt_ext(const void* q, const void* cache, void* out, int dtype,
                                      float* part_acc, float* part_ml, const int* items, int num_items,
                                      int max_items, const int* positions, const int* block_table,
                                      int width, const int* tok_part_row, int nq, int nkv, int d, int dv, int P,
                                      int num_pages, int window, float scale, const float* sink,
                                      const float* gate, int gate_nsplit, long long gate_split_stride, int gate_ld,
                                      int kparts, float softcap, int shared_kv, int gate_per_head, int out_f32,
                                      cudaStream_t stream) {
    return attention_simt_options(q, cache, out, dtype, part_acc, part_ml, items, num_items, max_items, positions,
                                  block_table, width, tok_part_row, nq, nkv, d, dv, P, num_pages, window, scale, sink,
                                  gate, gate_nsplit, gate_split_stride, gate_ld, kparts, softcap, shared_kv,
                                  gate_per_head, out_f32, 0, 0, 0, stream);
}

// The same with keys that stay visible beyond the window (pre_kind, pre_n) and with the values of every KV head
// under each query head's weights (all_values 1; 2 + c: the values of KV head c alone, for rows too wide to hold all):
// see "prefix" and "vheads" at the top.
MHB_EXPORT int mhb_attention_simt_masked(const void* q, const void* cache, void* out, int dtype,
                                         float* part_acc, float* part_ml, const int* items, int num_items,
                                         int max_items, const int* positions, const int* block_table,
                                         int width, const int* tok_part_row, int nq, int nkv, int d, int dv, int P,
                                         int num_pages, int window, float scale, const float* sink,
                                         const float* gate, int gate_nsplit, long long gate_split_stride, int gate_ld,
                                         int out_f32, int pre_kind, int pre_n, int all_values, cudaStream_t stream) {
    return attention_simt_options(q, cache, out, dtype, part_acc, part_ml, items, num_items, max_items, positions,
                                  block_table, width, tok_part_row, nq, nkv, d, dv, P, num_pages, window, scale, sink,
                                  gate, gate_nsplit, gate_split_stride, gate_ld, 1, 0.f, 0, 0, out_f32, pre_kind,
                                  pre_n, all_values, stream);
}

// every > 0: token t has `every` parts in the rows t * every ... of the partial buffers (tok_part_row and
// tok_nsplit are not read); else token t has tok_nsplit[t] parts from row tok_part_row[t].
MHB_EXPORT int mhb_attention_combine(const float* part_acc, const float* part_ml,
                                     const int* tok_part_row, const int* tok_nsplit, void* out,
                                     int dtype, int T, int nq, int d, int every, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (every <= 0 && (!tok_part_row || !tok_nsplit)) return fail("attention_combine: no list of parts");
    dim3 grid(T, nq);
    const int threads = d >= 128 ? 128 : 32 * ((d + 31) / 32);
    MHB_DISPATCH_DTYPE(dtype, OT,
        launch_kernel(attention_combine_kernel<OT>, grid, dim3(threads), 0, stream, part_acc, part_ml,
                      tok_part_row, tok_nsplit, (OT*)out, nq, d, every, (const float*)nullptr, 1, (size_t)0, 0, 0));
    return check_launch("attention_combine");
}

// The merge with a gate on the output (see the options at the top); d is the VALUE width here.
MHB_EXPORT int mhb_attention_combine_gated(const float* part_acc, const float* part_ml, const int* tok_part_row,
                                           const int* tok_nsplit, void* out, int dtype, int T, int nq, int d,
                                           int every, const float* gate, int gate_nsplit,
                                           long long gate_split_stride, int gate_ld, int gate_per_head,
                                           cudaStream_t stream) {
    if (T <= 0) return 0;
    if (every <= 0 && (!tok_part_row || !tok_nsplit)) return fail("attention_combine: no list of parts");
    dim3 grid(T, nq);
    const int threads = d >= 128 ? 128 : 32 * ((d + 31) / 32);
    MHB_DISPATCH_DTYPE(dtype, OT,
        launch_kernel(attention_combine_kernel<OT>, grid, dim3(threads), 0, stream, part_acc, part_ml,
                      tok_part_row, tok_nsplit, (OT*)out, nq, d, every, gate, gate_nsplit,
                      (size_t)gate_split_stride, gate_ld, gate_per_head));
    return check_launch("attention_combine");
}
