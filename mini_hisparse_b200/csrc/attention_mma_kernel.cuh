// Causal grouped-query attention over the paged KV cache on the tensor cores (bfloat16 inputs,
// float32 scores, softmax and accumulation), for prefill portions and decode tokens alike.
//
// Math as in attention_simt.cu (mini_hisparse/model.py:173-179, mini_hisparse/attention.py:26-35):
// s_t = (K[t] . q) * scale over the cached keys t <= the query's position (and inside the window,
// if there is one), w = softmax(s), o = sum_t w_t V[t]; query head h reads KV head h / groups.
// The work items are the same 8 ints {segment, first token, tokens, first head of the group,
// heads, kv_begin, kv_end, split}; split >= 0 writes an un-normalised partial.  With a counter
// array the CTA that finishes a token's last split merges all its splits (in split order, so the
// result does not depend on which CTA comes last); without one, attention_combine does it.
//
// One CTA (4 warps) serves one item and one KV head.  The query heads of a KV group are stacked
// into the row dimension of the tile, so a page of keys is read once for the whole group.
//   ROWS = 64 (long portions): each warp owns 16 query rows and walks all keys.
//   ROWS = 16 (decode tokens, tiny portions): the four warps share the 16 rows and each takes
//     16 of the 64 keys of a tile; their partial results are merged at the end.
// Keys and values arrive in tiles of 64 by cp.async (16-byte chunks gathered through the block
// table, two or three stages deep); rows are padded by 16 bytes, which keeps ldmatrix conflict-free for
// every head size that is a multiple of 16.  Products are mma.sync m16n8k16: the score tile
// feeds the value product straight from registers.
#pragma once
#include "common.cuh"
#include "mma_helpers.cuh"

namespace mhb_amma {
using namespace mhb;
constexpr int KT = 64;          // keys per tile
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int ITEM_INTS = 8;
constexpr int MAX_MERGE_SPLITS = 64;   // most key splits of a token that the fused merge takes

struct AttnArgs {
    const __nv_bfloat16* q;     // [T, nq, d]
    const __nv_bfloat16* cache; // [pages, 2, nkv, P, d] of one layer
    __nv_bfloat16* out;         // [T, nq, d]
    float* part_acc;            // [rows, nq, d]
    float* part_ml;             // [rows, nq, 2]
    const int* items;
    const int* positions;
    const int* block_table;
    const int* tok_part_row;
    const int* tok_nsplit;      // splits of each token (used by the fused merge)
    int* counters;              // one per (first token, KV head, head chunk): zero between launches
    int num_items, width, nq, nkv, P, num_pages, window;
    int page_shift;             // log2(P) if P is a power of two, else -1
    float scale;
    // the options (EXT instances only)
    int d, dv;                  // true widths of keys and values (multiples of 8, at most the padded D and DV)
    const float* sink;          // [nq] or null
    const float* gate;          // [gate_nsplit][T][gate_ld] or null
    int gate_nsplit, gate_ld;
    size_t gate_split_stride;
    int kparts;                 // score maps per KV head: its key row holds kparts keys side by side, all over the same values
    float softcap;              // s <- softcap * tanh(s / softcap) on the scaled score (0: none)
    int shared_kv;              // the values are the first dv elements of the key rows; a page holds those rows only
    int gate_per_head;          // the gate has one column per head instead of one per output element
    int out_f32;                // `out` is float32 (a sum of the outputs is still to be taken in 32 bits)
    // keys that stay visible beyond the window, as in attention_simt.cu: pre_kind 1 = the first pre_n positions,
    // 2 = the means of every block of pre_n positions that the window has passed wholly (from the pages' tails,
    // pool_slots rows per KV head); they are walked as tiles of their own before the item's key range
    int pre_kind, pre_n, pool_slots;
    size_t page_extra;          // elements of a page behind its keys and values
    int vhead;                  // >= 0: the values are those of this KV head, whatever the query head's own (-1: its own)
    // vplanes > 0: gridDim.z = vplanes, and the CTAs of plane z take the values of KV head z and write a plane of their
    // own of the output, of the partial buffers and of the merge counters
    int vplanes;
    size_t out_plane, part_plane_rows, counters_plane;
};

__device__ __forceinline__ void store_out(const AttnArgs& a, size_t idx, float v) {
    if (a.out_f32) ((float*)a.out)[idx] = v;
    else a.out[idx] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float gate_of(const AttnArgs& a, int t, int col) {
    if (!a.gate) return 1.f;
    const size_t idx = (size_t)t * a.gate_ld + col;
    float g = a.gate[idx];
    for (int s = 1; s < a.gate_nsplit; ++s) g += a.gate[idx + (size_t)s * a.gate_split_stride];
    return 1.f / (1.f + expf(-g));
}

template <int D, int DV, int ROWS>
struct Layout {
    static constexpr int LD = D + 8;                        // padded key row, in elements
    static constexpr int LDV = DV + 8;                      // padded value row
    static constexpr int Q_BYTES = ROWS * LD * 2;
    static constexpr int K_BYTES = KT * LD * 2;             // keys of one stage
    static constexpr int V_BYTES = KT * LDV * 2;            // values of one stage
    static constexpr int MERGE_BYTES = ROWS == 16 ? WARPS * 16 * (DV + 2) * 4 : 0;
    // decode tiles are bound by memory latency: three stages keep two tiles in flight per CTA
    static constexpr int STAGES = ROWS == 16 ? 3 : 2;
    static constexpr int LOOP_BYTES = Q_BYTES + STAGES * (K_BYTES + V_BYTES);
    static constexpr int TOTAL = LOOP_BYTES > MERGE_BYTES ? LOOP_BYTES : MERGE_BYTES;
};

// D and DV are the widths of keys and values as the tiles hold them.  EXT = false: they are the true
// widths and equal (a page is [2][nkv][P][D]).  EXT = true (the options of a mixer that brings them):
// the true widths a.d <= D and a.dv <= DV may be smaller (multiples of 8; the tiles' tails are zero),
// a page holds [nkv][P][d] keys followed by [nkv][P][dv] values, a sink per query head joins the
// softmax's denominator (the running (max, sum) of ONE thread per row starts at (sink, 1), in the
// unsplit item or in split 0 only), the output is multiplied by sigmoid(gate), and the softmax's
// weights enter the value product as the sum of two bfloat16 numbers (the weight and what rounding
// it lost), which keeps 16 bits of them instead of 8.  Further, with a.kparts > 1 every KV head has that many
// score maps (gridDim.y = nkv * kparts; query head q belongs to map q % kparts; the maps' keys lie side by side
// in the key row and share the values), a.softcap caps the scores, a.shared_kv takes the values from the head
// of the key rows (a latent cache), a.gate_per_head reads one gate per head, a.out_f32 writes float32.
template <int D, int DV, int ROWS, bool EXT>
__global__ void __launch_bounds__(THREADS)
attention_mma_kernel(const AttnArgs a_in) {
    AttnArgs a = a_in;
    if constexpr (EXT) {
        if (a.vplanes > 0) {
            const size_t z = blockIdx.z;
            a.vhead = (int)z;
            a.out = a.out_f32 ? (__nv_bfloat16*)((float*)a.out + z * a.out_plane) : a.out + z * a.out_plane;
            a.part_acc += z * a.part_plane_rows * a.nq * a.dv;
            a.part_ml += z * a.part_plane_rows * a.nq * 2;
            if (a.counters) a.counters += z * a.counters_plane;
        }
    }
    using L = Layout<D, DV, ROWS>;
    constexpr int LD = L::LD, LDV = L::LDV;
    constexpr int KSTEPS = D / 16;        // k-steps of Q K^T
    constexpr int DTILES = DV / 8;        // n-tiles of the output
    const int d_true = EXT ? a.d : D, dv_true = EXT ? a.dv : DV;
    constexpr bool SPLIT_KEYS = ROWS == 16;
    constexpr int NT = SPLIT_KEYS ? 2 : 8;   // score n-tiles (8 keys each) per warp per tile
    constexpr bool Q_IN_REGS = D <= 128;
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ int row_pos[ROWS];

    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= a.num_items) return;
    const int* it = a.items + (size_t)blockIdx.x * ITEM_INTS;
    const int seg = it[0], tok0 = it[1], ntok = it[2], head0 = it[3], nheads = it[4];
    const int kv_begin = it[5], kv_end = it[6], split = it[7];
    const int kparts = EXT ? a.kparts : 1;
    const int kvh = blockIdx.y / kparts, map = blockIdx.y - kvh * kparts;
    const int groups = a.nq / (a.nkv * kparts);
    const int nrows = ntok * nheads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // query head (as q, out and the partial buffers count them) of row r of this tile
    auto head_of = [&](int r) { return (kvh * groups + head0 + r % nheads) * kparts + map; };
    const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t kv_s = q_s + L::Q_BYTES;       // [stage][K|V][KT][LD]
    const int* table = a.block_table + (size_t)seg * a.width;
    const bool shared_kv = EXT && a.shared_kv;
    const int k_ld = kparts * d_true;                    // a key row of one KV head: its maps side by side
    const int v_ld = shared_kv ? k_ld : dv_true;
    const size_t plane = shared_kv ? 0 : (size_t)a.nkv * a.P * k_ld;  // elements between the keys and the values of a page
    const size_t kv_elems = (size_t)a.nkv * a.P * k_ld + (shared_kv ? 0 : (size_t)a.nkv * a.P * dv_true);
    const size_t page_elems = kv_elems + (EXT ? a.page_extra : 0);
    const int vh = (EXT && a.vhead >= 0) ? a.vhead : kvh;          // whose values
    int pre_end = 0;                                               // keys (or block means) beyond the window
    if constexpr (EXT) {
        if (a.pre_kind && a.window > 0 && split <= 0 && nrows > 0) {
            const int beyond = a.positions[tok0 + ntok - 1] - a.window + 1;    // the last row sees the most of them
            if (beyond > 0) pre_end = a.pre_kind == 1 ? min(a.pre_n, beyond) : beyond / a.pre_n;
        }
    }
    const int pre_tiles = (pre_end + KT - 1) / KT;

    // ---- stage the queries --------------------------------------------------------------------
    for (int c = tid; c < ROWS * (D / 8); c += THREADS) {
        const int r = c / (D / 8), ch = c % (D / 8);
        const bool live = r < nrows;
        const int t = tok0 + (live ? r / nheads : 0), h = head_of(live ? r : 0);
        const __nv_bfloat16* src = a.q + ((size_t)t * a.nq + h) * d_true + (ch * 8 < d_true ? ch * 8 : 0);
        cp_async16(q_s + (r * LD + ch * 8) * 2, src, live && ch * 8 < d_true ? 16 : 0);
    }
    if (tid < ROWS) row_pos[tid] = tid < nrows ? a.positions[tok0 + tid / nheads] : -1;

    // Consecutive threads copy consecutive 16-byte chunks of a key row, so a warp's request covers
    // whole rows (full 32-byte sectors).  A thread meets KT * (D/8) / THREADS rows per tile.
    auto load_tile = [&](int stage, int tile) {
        const bool pre = tile < pre_tiles;
        const int t0 = pre ? tile * KT : kv_begin + (tile - pre_tiles) * KT;
        const int end = pre ? pre_end : kv_end;
        const bool pooled = EXT && pre && a.pre_kind == 2;
        constexpr int CPR = D / 8 + DV / 8;                // chunks per position: its key, then its value
        constexpr int ITERS = KT * CPR / THREADS;
        const uint32_t kbase = kv_s + stage * (L::K_BYTES + L::V_BYTES);
        const uint32_t vbase = kbase + L::K_BYTES;
        // 16-row tiles serve a few key tiles per CTA: their time is the fetch of the kernel's instructions (ncu:
        // 70 us whatever the work, stalled on "no instruction"), so their copies stay a loop instead of 16 bodies
#pragma unroll (ROWS == 16 ? 2 : ITERS)
        for (int i = 0; i < ITERS; ++i) {
            const int c = i * THREADS + tid;
            const int j = c / CPR, ch = c % CPR;
            const int kp = t0 + j;
            int page = -1;
            int within = a.page_shift >= 0 ? (kp & (a.P - 1)) : (kp % a.P);
            if (kp < end) {
                if (pooled) {          // block kp lies in the page of its last position
                    const int pg = (kp * a.pre_n + a.pre_n - 1) / a.P;
                    within = kp - (int)(((long long)pg * a.P) / a.pre_n);
                    page = table[pg];
                } else {
                    page = table[a.page_shift >= 0 ? (kp >> a.page_shift) : (kp / a.P)];
                }
                if (page >= a.num_pages) page = -1;
            }
            const __nv_bfloat16* src = a.cache;
            int bytes = page >= 0 ? 16 : 0;
            if (ch < D / 8) {
                if (ch * 8 >= d_true) bytes = 0;           // the tile's tail beyond the true width stays zero
                if (bytes) {
                    if (pooled) src += (size_t)page * page_elems + kv_elems + ((size_t)kvh * a.pool_slots + within) * d_true + ch * 8;
                    else src += (size_t)page * page_elems + ((size_t)kvh * a.P + within) * k_ld + map * d_true + ch * 8;
                }
                cp_async16(kbase + (j * LD + ch * 8) * 2, src, bytes);
            } else {
                const int cv = ch - D / 8;
                if (cv * 8 >= dv_true) bytes = 0;
                if (bytes) {
                    if (pooled) src += (size_t)page * page_elems + kv_elems + (size_t)a.nkv * a.pool_slots * d_true +
                                       ((size_t)vh * a.pool_slots + within) * dv_true + cv * 8;
                    else src += (size_t)page * page_elems + plane + ((size_t)vh * a.P + within) * v_ld + cv * 8;
                }
                cp_async16(vbase + (j * LDV + cv * 8) * 2, src, bytes);
            }
        }
    };

    constexpr int STAGES = L::STAGES;
    const int ntiles = pre_tiles + (kv_end - kv_begin + KT - 1) / KT;
#pragma unroll 1
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st < ntiles) load_tile(st, st);
        cp_async_commit();
    }

    // ---- per-thread state: rows r0 = lane/4 and r0 + 8 of this warp's 16 rows ------------------
    const int wrow = SPLIT_KEYS ? 0 : warp * 16;
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
    const float scale_log2 = a.scale * 1.4426950408889634f;
    if constexpr (EXT) {
        // the sink is a score that is not scaled: in the units of the raw products it is sink / scale.  It
        // is added a single time per row: in one warp (where four warps share the rows) and one thread of the quad.
        if (a.sink && split <= 0 && (!SPLIT_KEYS || warp == 0)) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = wrow + (lane >> 2) + 8 * h;
                if (row < nrows) {
                    m_run[h] = a.sink[head_of(row)] / a.scale;
                    l_run[h] = (lane & 3) == 0 ? 1.f : 0.f;
                }
            }
        }
    }

    for (int itile = 0; itile < ntiles; ++itile) {
        const int stage = itile % STAGES;
        if (itile + STAGES - 1 < ntiles)
            load_tile((itile + STAGES - 1) % STAGES, itile + STAGES - 1);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        if (itile == 0 && Q_IN_REGS) {
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
                const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1), c = k * 16 + 8 * (lane >> 4);
                ldmatrix_x4(q_s + (r * LD + c) * 2, qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
            }
        }
        const uint32_t k_s = kv_s + stage * (L::K_BYTES + L::V_BYTES);
        const uint32_t v_s = k_s + L::K_BYTES;
        const bool pre = itile < pre_tiles;
        const int t0 = pre ? itile * KT : kv_begin + (itile - pre_tiles) * KT;
        const int key0 = SPLIT_KEYS ? warp * 16 : 0;      // first key of this warp inside the tile

        // ---- S = Q K^T -------------------------------------------------------------------------
        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KSTEPS; k += 2) {
            uint32_t qa[2][4];
            if (Q_IN_REGS) {
#pragma unroll
                for (int x = 0; x < 4; ++x) { qa[0][x] = qf[k][x]; qa[1][x] = qf[k + 1 < KSTEPS ? k + 1 : k][x]; }
            } else {
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    if (k + kk < KSTEPS) {
                        const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1), c = (k + kk) * 16 + 8 * (lane >> 4);
                        ldmatrix_x4(q_s + (r * LD + c) * 2, qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                // K rows = keys key0 + 8j .. +7; columns = two k-steps (32 elements) when available
                uint32_t b0, b1, b2, b3;
                const int r = key0 + j * 8 + (lane & 7);
                int c = k * 16 + 8 * (lane >> 3);
                if (KSTEPS % 2 == 1 && k + 1 >= KSTEPS) c = k * 16 + 8 * ((lane >> 3) & 1);   // last odd step: stay inside the row
                ldmatrix_x4(k_s + (r * LD + c) * 2, b0, b1, b2, b3);
                mma_bf16(s[j], qa[0], b0, b1);
                if (k + 1 < KSTEPS) mma_bf16(s[j], qa[1], b2, b3);
            }
        }

        if constexpr (EXT) {
            if (a.softcap > 0.f) {      // the cap works on the scaled score; the tile stays in the raw products' units
                const float to_cap = a.scale / a.softcap, from_cap = a.softcap / a.scale;
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int x = 0; x < 4; ++x) s[j][x] = from_cap * tanhf(s[j][x] * to_cap);
            }
        }
        // ---- mask, online softmax -----------------------------------------------------------------
        float mx[2] = {-INFINITY, -INFINITY};
        int pre_lim[2] = {0, 0};          // in a tile of keys beyond the window: how many of them each of the two rows sees
        if constexpr (EXT) {
            if (pre) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int beyond = row_pos[wrow + (lane >> 2) + 8 * h] - a.window + 1;
                    pre_lim[h] = beyond <= 0 ? 0 : (a.pre_kind == 1 ? min(a.pre_n, beyond) : beyond / a.pre_n);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int row = wrow + (lane >> 2) + 8 * (x >> 1);
                const int kp = t0 + key0 + j * 8 + (lane & 3) * 2 + (x & 1);
                const int qp = row_pos[row];
                bool valid = kp < kv_end && kp <= qp && (a.window <= 0 || kp > qp - a.window);
                if (EXT && pre) valid = kp < pre_lim[x >> 1];
                s[j][x] = valid ? s[j][x] : -INFINITY;
                mx[x >> 1] = fmaxf(mx[x >> 1], s[j][x]);
            }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;
            alpha[h] = exp2f((m_run[h] - m_use[h]) * scale_log2);     // exp2(-inf) = 0 on the first tile
            m_run[h] = m_new;
            l_run[h] *= alpha[h];
        }
        uint32_t pf[NT / 2][4];
        uint32_t pl[EXT ? NT / 2 : 1][4];      // what rounding the weights to bfloat16 lost
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            float p[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                p[x] = exp2f((s[j][x] - m_use[x >> 1]) * scale_log2);
                l_run[x >> 1] += p[x];
            }
            pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
            if constexpr (EXT) {
                float r[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) r[x] = p[x] - __bfloat162float(__float2bfloat16_rn(p[x]));
                pl[j >> 1][(j & 1) * 2 + 0] = pack_bf16(r[0], r[1]);
                pl[j >> 1][(j & 1) * 2 + 1] = pack_bf16(r[2], r[3]);
            }
        }
#pragma unroll
        for (int i = 0; i < DTILES; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }

        // ---- O += P V ---------------------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
            for (int i = 0; i < DTILES; i += 2) {
                uint32_t b0, b1, b2, b3;
                const int r = key0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = i * 8 + 8 * (lane >> 4);
                ldmatrix_x4_trans(v_s + (r * LDV + c) * 2, b0, b1, b2, b3);
                mma_bf16(o[i], pf[kk], b0, b1);
                mma_bf16(o[i + 1], pf[kk], b2, b3);
                if constexpr (EXT) {
                    mma_bf16(o[i], pl[kk], b0, b1);
                    mma_bf16(o[i + 1], pl[kk], b2, b3);
                }
            }
        }
        __syncthreads();      // everyone is done with this stage before it is loaded again
    }
    cp_async_wait<0>();

    // ---- finish: sums across the quad, merge of the warps (16-row mode), output -----------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    if (ntiles == 0) __syncthreads();
    if (SPLIT_KEYS) {
        // scratch (aliases the tiles, which nobody reads any more): [warp][row][D + 2] floats
        float* mg = (float*)smem;
        constexpr int MS = DV + 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            float* dst = mg + (warp * 16 + row) * MS;
#pragma unroll
            for (int i = 0; i < DTILES; ++i) {
                dst[i * 8 + (lane & 3) * 2 + 0] = o[i][2 * h + 0];
                dst[i * 8 + (lane & 3) * 2 + 1] = o[i][2 * h + 1];
            }
            if ((lane & 3) == 0) { dst[DV] = m_run[h]; dst[DV + 1] = l_run[h]; }
        }
        __syncthreads();
        for (int idx = tid; idx < nrows * dv_true; idx += THREADS) {
            const int row = idx / dv_true, e = idx - row * dv_true;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) M = fmaxf(M, mg[(w * 16 + row) * MS + DV]);
            float acc = 0.f, lsum = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float mw = mg[(w * 16 + row) * MS + DV];
                const float wgt = mw == -INFINITY ? 0.f : exp2f((mw - M) * scale_log2);
                acc += wgt * mg[(w * 16 + row) * MS + e];
                lsum += wgt * mg[(w * 16 + row) * MS + DV + 1];
            }
            const int t = tok0 + row / nheads, hq = head_of(row);
            if (split < 0) {
                float res = lsum > 0.f ? acc / lsum : 0.f;
                if constexpr (EXT) {
                    res *= gate_of(a, t, a.gate_per_head ? hq : hq * dv_true + e);
                    store_out(a, ((size_t)t * a.nq + hq) * dv_true + e, res);
                } else {
                    a.out[((size_t)t * a.nq + hq) * dv_true + e] = __float2bfloat16_rn(res);
                }
            } else {
                const size_t prow = (size_t)a.tok_part_row[t] + split;
                a.part_acc[(prow * a.nq + hq) * dv_true + e] = acc;
                if (e == 0) {
                    a.part_ml[(prow * a.nq + hq) * 2 + 0] = M == -INFINITY ? -INFINITY : M * a.scale;
                    a.part_ml[(prow * a.nq + hq) * 2 + 1] = lsum;
                }
            }
        }
        if (split >= 0 && a.counters != nullptr) {
            // the last CTA of this tile's splits merges them (reference/attention.py:11-20)
            __shared__ int is_last;
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const int chunks = (groups + 15) / 16;
                int* counter = a.counters + ((size_t)tok0 * gridDim.y + blockIdx.y) * chunks + head0 / 16;
                const int ns = a.tok_nsplit[tok0];
                const int prev = atomicAdd(counter, 1);
                is_last = prev == ns - 1;
                if (is_last) *counter = 0;
            }
            __syncthreads();
            if (is_last) {
                __threadfence();
                // weights of every (row, split) once, then one load per split and output element
                __shared__ float wgt_s[16][MAX_MERGE_SPLITS];
                __shared__ float inv_s[16];
                const int ns = min(a.tok_nsplit[tok0], MAX_MERGE_SPLITS);
                if (tid < nrows) {
                    const int t = tok0 + tid / nheads, hq = head_of(tid);
                    const size_t row0 = a.tok_part_row[t];
                    float M = -INFINITY;
                    for (int sp = 0; sp < ns; ++sp) M = fmaxf(M, __ldcg(a.part_ml + ((row0 + sp) * a.nq + hq) * 2));
                    float lsum = 0.f;
                    for (int sp = 0; sp < ns; ++sp) {
                        const float ms = __ldcg(a.part_ml + ((row0 + sp) * a.nq + hq) * 2);
                        const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
                        wgt_s[tid][sp] = w;
                        lsum += w * __ldcg(a.part_ml + ((row0 + sp) * a.nq + hq) * 2 + 1);
                    }
                    inv_s[tid] = lsum > 0.f ? 1.f / lsum : 0.f;
                }
                __syncthreads();
                for (int idx = tid; idx < nrows * dv_true; idx += THREADS) {
                    const int row = idx / dv_true, e = idx - row * dv_true;
                    const int t = tok0 + row / nheads, hq = head_of(row);
                    const float* src = a.part_acc + ((size_t)a.tok_part_row[t] * a.nq + hq) * dv_true + e;
                    const size_t step = (size_t)a.nq * dv_true;
                    float acc = 0.f;
#pragma unroll 4
                    for (int sp = 0; sp < ns; ++sp) acc += wgt_s[row][sp] * __ldcg(src + sp * step);
                    acc *= inv_s[row];
                    if constexpr (EXT) {
                        acc *= gate_of(a, t, a.gate_per_head ? hq : hq * dv_true + e);
                        store_out(a, ((size_t)t * a.nq + hq) * dv_true + e, acc);
                    } else {
                        a.out[((size_t)t * a.nq + hq) * dv_true + e] = __float2bfloat16_rn(acc);
                    }
                }
            }
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = wrow + (lane >> 2) + 8 * h;
            if (row >= nrows) continue;
            const int t = tok0 + row / nheads, hq = head_of(row);
            if (split < 0) {
                const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
                const size_t o0 = ((size_t)t * a.nq + hq) * dv_true + (lane & 3) * 2;
                __nv_bfloat16* dst = a.out + o0;
                float gh = 1.f;
                if constexpr (EXT) { if (a.gate_per_head) gh = gate_of(a, t, hq); }
#pragma unroll
                for (int i = 0; i < DTILES; ++i) {
                    if (EXT && i * 8 >= dv_true) break;
                    float g0 = gh, g1 = gh;
                    if constexpr (EXT) {
                        if (!a.gate_per_head) {
                            g0 = gate_of(a, t, hq * dv_true + i * 8 + (lane & 3) * 2);
                            g1 = gate_of(a, t, hq * dv_true + i * 8 + (lane & 3) * 2 + 1);
                        }
                        if (a.out_f32) {
                            *(float2*)((float*)a.out + o0 + i * 8) = make_float2(o[i][2 * h] * inv * g0, o[i][2 * h + 1] * inv * g1);
                            continue;
                        }
                    }
                    *(uint32_t*)(dst + i * 8) = pack_bf16(o[i][2 * h] * inv * g0, o[i][2 * h + 1] * inv * g1);
                }
            } else {
                const size_t prow = (size_t)a.tok_part_row[t] + split;
                float* dst = a.part_acc + (prow * a.nq + hq) * dv_true + (lane & 3) * 2;
#pragma unroll
                for (int i = 0; i < DTILES; ++i) {
                    if (EXT && i * 8 >= dv_true) break;
                    dst[i * 8] = o[i][2 * h];
                    dst[i * 8 + 1] = o[i][2 * h + 1];
                }
                if ((lane & 3) == 0) {
                    a.part_ml[(prow * a.nq + hq) * 2 + 0] = m_run[h] == -INFINITY ? -INFINITY : m_run[h] * a.scale;
                    a.part_ml[(prow * a.nq + hq) * 2 + 1] = l_run[h];
                }
            }
        }
    }
}


template <int D, int DV, int ROWS, bool EXT>
int launch(const AttnArgs& a, int launch_items, cudaStream_t stream) {
    auto kern = attention_mma_kernel<D, DV, ROWS, EXT>;
    constexpr int smem = Layout<D, DV, ROWS>::TOTAL;
    static bool configured = false;
    // static shared memory (row positions, the merge's weights) comes on top: opt in well below 48 KB
    if (!configured && smem > 40 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("attention_mma: shared memory %d: %s", smem, cudaGetErrorString(e));
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    dim3 grid(launch_items, a.nkv * (EXT ? a.kparts : 1), EXT && a.vplanes > 0 ? a.vplanes : 1);
    launch_kernel(kern, grid, dim3(THREADS), smem, stream, a);
    return check_launch("attention_mma");
}

inline void fill_args(AttnArgs& a, const void* q, const void* cache, void* out, float* part_acc, float* part_ml,
                      const int* items, int num_items, const int* positions, const int* block_table, int width,
                      const int* tok_part_row, const int* tok_nsplit, int* counters, int nq, int nkv, int P,
                      int num_pages, int window, float scale) {
    a.q = (const __nv_bfloat16*)q; a.cache = (const __nv_bfloat16*)cache; a.out = (__nv_bfloat16*)out;
    a.part_acc = part_acc; a.part_ml = part_ml; a.items = items; a.positions = positions;
    a.block_table = block_table; a.tok_part_row = tok_part_row; a.tok_nsplit = tok_nsplit;
    a.counters = counters; a.num_items = num_items; a.width = width;
    a.nq = nq; a.nkv = nkv; a.P = P; a.num_pages = num_pages; a.window = window; a.scale = scale;
    a.page_shift = -1;
    if (P > 0 && (P & (P - 1)) == 0) { a.page_shift = 0; while ((1 << a.page_shift) < P) ++a.page_shift; }
    a.d = a.dv = 0; a.sink = nullptr; a.gate = nullptr; a.gate_nsplit = 1; a.gate_ld = 0; a.gate_split_stride = 0;
    a.kparts = 1; a.softcap = 0.f; a.shared_kv = 0; a.gate_per_head = 0; a.out_f32 = 0;
    a.pre_kind = 0; a.pre_n = 0; a.pool_slots = 0; a.page_extra = 0; a.vhead = -1;
    a.vplanes = 0; a.out_plane = a.part_plane_rows = a.counters_plane = 0;
}
}  // namespace mhb_amma
