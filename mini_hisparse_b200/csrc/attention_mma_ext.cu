// The tensor-core attention of attention_mma_kernel.cuh with the options that other mixers bring: keys
// and values of different widths (any multiples of 8 up to 128; the tiles are padded to the next
// multiple of 32), a sink per query head in the softmax's denominator, a gate on the output (per element
// or per head), softmax weights that keep 16 bits in the value product, several score maps per KV head
// over shared values, capped scores, values that are the head of the key rows (a latent cache), and
// float32 outputs.  Work items, tile heights and the merge of
// key splits are those of attention_mma.cu.
#include "attention_mma_kernel.cuh"

using namespace mhb;
using namespace mhb_amma;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
template <int D, int ROWS>
int dispatch_dv(int dvp, const AttnArgs& a, int launch_items, cudaStream_t stream) {
    switch (dvp) {
        case 32: return launch<D, 32, ROWS, true>(a, launch_items, stream);
        case 64: return launch<D, 64, ROWS, true>(a, launch_items, stream);
        case 96: return launch<D, 96, ROWS, true>(a, launch_items, stream);
        case 128: return launch<D, 128, ROWS, true>(a, launch_items, stream);
    }
    return fail("attention_mma_ext: values %d wide", dvp);
}
template <int ROWS>
int dispatch_d(int dp, int dvp, const AttnArgs& a, int launch_items, cudaStream_t stream) {
    switch (dp) {
        case 32: return dispatch_dv<32, ROWS>(dvp, a, launch_items, stream);
        case 64: return dispatch_dv<64, ROWS>(dvp, a, launch_items, stream);
        case 96: return dispatch_dv<96, ROWS>(dvp, a, launch_items, stream);
        case 128: return dispatch_dv<128, ROWS>(dvp, a, launch_items, stream);
    }
    return fail("attention_mma_ext: keys %d wide", dp);
}
}  // namespace

MHB_EXPORT int mhb_attention_mma_ext_supports(int d, int dv) {
    return d >= 8 && d <= 128 && d % 8 == 0 && dv >= 8 && dv <= 128 && dv % 8 == 0;
}

namespace {
int attention_mma_options(const void* q, const void* cache, void* out, float* part_acc,
                                     float* part_ml, const int* items, int num_items, int launch_items,
                                     int rows, const int* positions, const int* block_table, int width,
                                     const int* tok_part_row, const int* tok_nsplit, int* counters, int nq,
                                     int nkv, int d, int dv, int P, int num_pages, int window, float scale,
                                     const float* sink, const float* gate, int gate_nsplit,
                                     long long gate_split_stride, int gate_ld, int kparts, float softcap,
                                     int shared_kv, int gate_per_head, int out_f32, int pre_kind, int pre_n,
                                     int value_head, long long out_plane, long long part_plane_rows,
                                     long long counters_plane, cudaStream_t stream) {
    if (launch_items <= 0) return 0;
    if (pre_kind < 0 || pre_kind > 2 || (pre_kind && pre_n < 1)) return fail("attention: keys beyond the window of kind %d over %d positions", pre_kind, pre_n);
    if ((pre_kind || value_head >= 0) && (kparts != 1 || shared_kv)) return fail("attention: keys beyond the window and another head's values go with plain key and value rows only");
    if (value_head >= nkv || value_head < -2) return fail("attention: values of KV head %d of %d", value_head, nkv);
    if (nkv <= 0 || kparts < 1 || nq % (nkv * kparts))
        return fail("attention: %d query heads over %d KV heads with %d score maps each", nq, nkv, kparts);
    if ((long long)nkv * kparts > 65535) return fail("attention: too many KV heads");
    if (shared_kv && dv > kparts * d) return fail("attention: values %d wide cannot be the head of key rows %d wide", dv, kparts * d);
    if (!mhb_attention_mma_ext_supports(d, dv)) return fail("attention_mma_ext: widths %d and %d (multiples of 8 up to 128)", d, dv);
    if (!(scale > 0.f) && sink) return fail("attention_mma_ext: a sink needs a positive scale");
    AttnArgs a;
    fill_args(a, q, cache, out, part_acc, part_ml, items, num_items, positions, block_table, width, tok_part_row,
              tok_nsplit, counters, nq, nkv, P, num_pages, window, scale);
    a.d = d; a.dv = dv; a.sink = sink; a.gate = gate; a.gate_nsplit = gate_nsplit; a.gate_ld = gate_ld;
    a.gate_split_stride = (size_t)gate_split_stride;
    a.kparts = kparts; a.softcap = softcap; a.shared_kv = shared_kv; a.gate_per_head = gate_per_head; a.out_f32 = out_f32;
    a.pre_kind = pre_kind; a.pre_n = pre_n; a.vhead = value_head < 0 ? -1 : value_head;
    if (value_head == -2) {          // every KV head's values, a plane of outputs each
        if (nkv > 65535) return fail("attention: too many KV heads for a plane each");
        a.vplanes = nkv; a.out_plane = (size_t)out_plane; a.part_plane_rows = (size_t)part_plane_rows;
        a.counters_plane = (size_t)counters_plane;
    }
    a.pool_slots = pre_kind == 2 ? (P + pre_n - 1) / pre_n : 0;
    a.page_extra = (size_t)nkv * a.pool_slots * (d + dv);
    const int dp = (d + 31) / 32 * 32, dvp = (dv + 31) / 32 * 32;
    if (rows == 64) return dispatch_d<64>(dp, dvp, a, launch_items, stream);
    if (rows == 16) return dispatch_d<16>(dp, dvp, a, launch_items, stream);
    return fail("attention_mma_ext: tile height %d", rows);
}
}  // namespace

MHB_EXPORT int mhb_attention_mma_ext(const void* q, const void* cache, void* out, float* part_acc,
                                     float* part_ml, const int* items, int num_items, int launch_items,
                                     int rows, const int* positions, const int* block_table, int width,
                                     const int* tok_part_row, const int* tok_nsplit, int* counters, int nq,
                                     int nkv, int d, int dv, int P, int num_pages, int window, float scale,
                                     const float* sink, const float* gate, int gate_nsplit,
                                     long long gate_split_stride, int gate_ld, int kparts, float softcap,
                                     int shared_kv, int gate_per_head, int out_f32, cudaStream_t stream) {
    return attention_mma_options(q, cache, out, part_acc, part_ml, items, num_items, launch_items, rows, positions,
                                 block_table, width, tok_part_row, tok_nsplit, counters, nq, nkv, d, dv, P, num_pages,
                                 window, scale, sink, gate, gate_nsplit, gate_split_stride, gate_ld, kparts, softcap,
                                 shared_kv, gate_per_head, out_f32, 0, 0, -1, 0, 0, 0, stream);
}

// The same with keys that stay visible beyond the window (pre_kind 1: the first pre_n positions; 2: the means of
// blocks of pre_n positions, from the pages' tails) and, with value_head >= 0, every query head's weights applied
// to the values of that one KV head; value_head -2: to the values of every KV head in turn (gridDim.z = nkv), plane z of
// `out` (out_plane elements apart), of the partial buffers (part_plane_rows rows apart) and of the counters
// (counters_plane apart) belonging to KV head z.
MHB_EXPORT int mhb_attention_mma_masked(const void* q, const void* cache, void* out, float* part_acc,
                                        float* part_ml, const int* items, int num_items, int launch_items,
                                        int rows, const int* positions, const int* block_table, int width,
                                        const int* tok_part_row, const int* tok_nsplit, int* counters, int nq,
                                        int nkv, int d, int dv, int P, int num_pages, int window, float scale,
                                        const float* gate, int gate_nsplit, long long gate_split_stride, int gate_ld,
                                        int out_f32, int pre_kind, int pre_n, int value_head, long long out_plane,
                                        long long part_plane_rows, long long counters_plane, cudaStream_t stream) {
    return attention_mma_options(q, cache, out, part_acc, part_ml, items, num_items, launch_items, rows, positions,
                                 block_table, width, tok_part_row, tok_nsplit, counters, nq, nkv, d, dv, P, num_pages,
                                 window, scale, nullptr, gate, gate_nsplit, gate_split_stride, gate_ld, 1, 0.f, 0, 0,
                                 out_f32, pre_kind, pre_n, value_head, out_plane, part_plane_rows, counters_plane, stream);
}
