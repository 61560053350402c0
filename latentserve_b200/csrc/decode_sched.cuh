// Work partitioning for split-KV paged decode attention.
//
// A decode batch is a ragged set of sequences. Instead of a (sequence, split)
// grid, whose programs idle whenever lengths differ, the pages of the whole
// batch are laid end to end on one axis ("units": pages for the dense kernels,
// selected-list entries for the sparse one) and cut into equal chunks, one per
// CTA column. A chunk may span several sequences; each (chunk, sequence) piece
// is a "segment" and yields one partial softmax state. The grid is fixed by
// the launch (graph-capturable); the chunk size follows the sequence lengths
// that are on the device at run time.
//
// Partial slot of segment (chunk c, sequence b) = c + b. Walking the unit axis
// left to right, each new segment increments c or b (or both), so the slot is
// unique, and a sequence's slots are contiguous: [c_lo + b, c_hi + b].
#pragma once

#include "ls_common.cuh"

#define LS_MAX_BATCH 1024          // prefix sums of the batch live in shared memory
#define LS_MODE_DENSE 0
#define LS_MODE_SPARSE 1

namespace ls {

struct DecodeParams {
    const __half* q;
    const void* k_pool;
    const void* v_pool;
    const int* block_tables;
    const int* seq_lens;
    float* part_acc;               // [slots, H, RP, 128]
    float* part_m;                 // [slots, H, RP]   (log2 domain)
    float* part_l;                 // [slots, H, RP]
    int* seg_range;                // [B, 2] first slot, count; [2B] = error flag;
                                   // [2B+2 ..) one arrival counter per (sequence, head)
    __half* out;                   // [B, H, R, 128] final output, or null: partials only
    long long so_b, so_h, so_m;
    // INT8 pools
    const float* k_scale;
    const float* v_scale;
    const float* k_zero;
    const float* v_zero;
    const __half* k_res;
    const int* res_rows;
    // fp16 pools: the step's new K / V rows [B, H, 128], appended by this launch (or null)
    const __half* k_new;
    const __half* v_new;
    long long sn_b, sn_h, svn_b, svn_h;
    // sparse page lists
    const int* sel;
    float ratio;
    int recent;
    int num_sel;
    long long sl_b, sl_h;
    int batch, heads, n_rep;
    int max_pages;                 // block-table row stride (entries)
    int num_blocks;                // pool blocks, for the device-side id check
    int num_res_rows;              // residual rows, likewise
    int num_chunks;
    int min_chunk;
    long long sq_b, sq_h, sq_m;    // q strides (elements)
    long long sk_b, sk_p, sk_h;    // pool strides: block, token, head (elements)
    long long ks_b, ks_h;          // k_scale strides: block, head
    long long vs_b, vs_p, vs_h;    // v_scale strides: block, token, head
    long long sr_r, sr_p, sr_h;    // residual strides: row, token, head
    int early;                     // LS_EARLY_PAGES: old pages may be read before the dependency wait
    int kv_merged;                 // INT8 TMA loader: a page's K and V tiles come by ONE copy (map `kv`)
    int k_off;                     // byte offset of the K tile inside a stage (0, or 2048 when the merged
                                   // copy delivers V first); the V tile sits at 2048 - k_off
    float scale_log2;              // softmax scale * log2(e)
};

// Units a sequence contributes to the work axis.
template <int MODE>
__device__ __forceinline__ int seq_units(const DecodeParams& p, int b) {
    const int L = max(p.seq_lens[b], 0);
    const int np = min((L + LS_PAGE - 1) / LS_PAGE, p.max_pages);
    if (MODE == LS_MODE_SPARSE) {
        // Entries of the (score-sorted) selection this sequence attends: its
        // own budget for its current length, as the reference's sparse kernel
        // computes it in-kernel (kernels/cuda/paged_sparse_fp16.cu:242-247).
        int n = p.num_sel;
        if (p.ratio > 0.f) {
            const int want = p.ratio >= 1.f
                                 ? np
                                 : max(p.recent + 1, (int)ceilf(p.ratio * (float)np));
            n = min(min(want, np), p.num_sel);
        }
        return n;
    }
    return np;
}

// Exclusive prefix sums of units over the batch into cum[0..B]; returns total.
// Called by every thread of the CTA; `scratch` holds one int per warp.
template <int MODE, int THREADS>
__device__ __forceinline__ int build_prefix(const DecodeParams& p, int* cum, int* scratch) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ipt = (p.batch + THREADS - 1) / THREADS;
    const int base = tid * ipt;
    int s = 0;
    for (int i = 0; i < ipt; ++i) {
        const int idx = base + i;
        if (idx < p.batch) s += seq_units<MODE>(p, idx);
    }
    int inc = s;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(LS_FULL_MASK, inc, off);
        if (lane >= off) inc += o;
    }
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    int run = inc - s;
    for (int w = 0; w < warp; ++w) run += scratch[w];
    for (int i = 0; i < ipt; ++i) {
        const int idx = base + i;
        if (idx < p.batch) {
            cum[idx] = run;
            run += seq_units<MODE>(p, idx);
        }
    }
    if (tid == THREADS - 1) cum[p.batch] = run;
    __syncthreads();
    return cum[p.batch];
}

__device__ __forceinline__ int chunk_size(const DecodeParams& p, int total) {
    const int even = (total + p.num_chunks - 1) / p.num_chunks;
    return max(max(even, p.min_chunk), 1);
}

// First sequence whose unit range contains global unit g (g < total).
__device__ __forceinline__ int find_seq(const int* cum, int batch, int g) {
    int lo = 0, hi = batch - 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (cum[mid + 1] > g) hi = mid; else lo = mid + 1;
    }
    return lo;
}

// Slots of every sequence, for the merge kernel. One CTA writes this.
template <int THREADS>
__device__ __forceinline__ void write_seg_ranges(const DecodeParams& p, const int* cum, int chunk) {
    for (int b = threadIdx.x; b < p.batch; b += THREADS) {
        const int lo = cum[b], hi = cum[b + 1];
        int first = 0, count = 0;
        if (hi > lo) {
            const int c_lo = lo / chunk, c_hi = (hi - 1) / chunk;
            first = c_lo + b;
            count = c_hi - c_lo + 1;
        }
        p.seg_range[2 * b] = first;
        p.seg_range[2 * b + 1] = count;
    }
}

// One warp's walk over its pages of a chunk: units lo+w, lo+w+W, ... of every
// segment, segment after segment. The load side and the compute side each
// hold a cursor and advance it independently, so prefetch runs across segment
// boundaries.
struct Cursor {
    int b;        // sequence
    int u;        // unit within the sequence
    int hi;       // end of this segment, in units of the sequence
    int g1;       // end of the chunk on the global axis
    bool done;
};

template <int W>
__device__ __forceinline__ void cursor_normalize(Cursor& c, const int* cum, int batch, int warp) {
    // Bounded: every iteration moves to a later sequence.
    while (!c.done && c.u >= c.hi) {
        if (cum[c.b + 1] >= c.g1) {
            c.done = true;
        } else {
            ++c.b;
            while (c.b < batch - 1 && cum[c.b + 1] == cum[c.b]) ++c.b;
            c.hi = min(c.g1, cum[c.b + 1]) - cum[c.b];
            c.u = warp;
        }
    }
}

template <int W>
__device__ __forceinline__ Cursor cursor_begin(const int* cum, int batch, int b0, int g0, int g1,
                                               int warp) {
    Cursor c;
    c.b = b0;
    c.g1 = g1;
    c.hi = min(g1, cum[b0 + 1]) - cum[b0];
    c.u = g0 - cum[b0] + warp;
    c.done = false;
    cursor_normalize<W>(c, cum, batch, warp);
    return c;
}

template <int W>
__device__ __forceinline__ void cursor_next(Cursor& c, const int* cum, int batch, int warp) {
    c.u += W;
    cursor_normalize<W>(c, cum, batch, warp);
}

}  // namespace ls
