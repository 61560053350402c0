// Page scoring and deterministic top-k for page-sparse decode.
//
//   ls_page_index        Quest upper bound per page from the page's per-channel
//                        K min / max, maximised over the query rows of the GQA
//                        group (reference: kernels/cuda/paged_sparse_fp16.cu:78-130)
//   ls_page_index_heads  the same bound per query row, not maximised, for the
//                        reference's summed-mass scoring (:141-190)
//   ls_topk_pages        indices of the k best pages per (sequence, KV head),
//                        score descending, ties to the lower page index
//                        (reference: torch.topk(sorted=True), kernels/cuda/paged_sparse.py:164-168,
//                        whose tie order is unspecified; this one is fixed)
//
// The score arithmetic keeps the reference's fp32 evaluation order exactly --
// lane l sums channels 4l..4l+3 left to right starting from 0, then pairwise
// sums over lanes at distance 16, 8, 4, 2, 1 -- so that scores, and with them
// the selected indices, are reproducible bit for bit on a CPU. The reference
// does that with an all-lanes butterfly per value (5 shuffles each); here 32
// values (4 pages x 8 padded query rows) are reduced together, each step
// keeping half of the values per lane, which forms exactly the same pairwise
// sums with 31 shuffles for all 32.
#include "ls_common.cuh"

namespace ls {

constexpr int kIndexWarps = 4;
constexpr int kGroup = 4;                    // pages reduced together
constexpr int kItemGroups = 2;               // groups per pipelined item
constexpr int kItemPages = kGroup * kItemGroups;
constexpr int kMaxItems = 3;                 // items a warp stages at once (its span / 8)
constexpr int kItemBytes = kItemPages * 512; // a page's minimum and maximum rows, 256 bytes each
static_assert(kMaxItems == 3, "page_index_kernel writes out its three waits");
#ifndef LS_INDEX_CTAS
#define LS_INDEX_CTAS 4
#endif
constexpr int kIndexCtasPerSm = LS_INDEX_CTAS;   // resident CTAs of the index kernel (registers, 48 KB each)

__device__ __forceinline__ void unpack4h(uint2 raw, float (&f)[4]) {
    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
    const float2 a = __half22float2(h2[0]), b = __half22float2(h2[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// One halving step of the joint reduction: N values per lane in, N/2 out.
// Lanes with bit OFF clear keep values [0, N/2), the others [N/2, N); each
// kept value becomes own + partner's, the same two operands the all-lanes
// butterfly adds at this distance.
template <int N, int OFF>
__device__ __forceinline__ void halve(const float (&in)[N], float (&out)[N / 2], int lane) {
    const bool upper = (lane & OFF) != 0;
#pragma unroll
    for (int k = 0; k < N / 2; ++k) {
        const float keep = upper ? in[k + N / 2] : in[k];
        const float send = upper ? in[k] : in[k + N / 2];
        out[k] = __fadd_rn(keep, __shfl_xor_sync(LS_FULL_MASK, send, OFF));
    }
}

// Bounds of 8 (padded) query rows x 4 pages. On return lane l holds the
// complete bound of page (l >> 3) of the group, query row (l & 7).
// max(q * lo, q * hi) with lo <= hi (a page's channel minimum and maximum) is
// q * hi for q > 0 and q * lo for q < 0. With q+ = max(q, 0) and q- = min(q, 0)
// that product is fma(q+, hi, q- * lo), bit for bit: one of the two factors is
// zero, so one term is a zero and the other is rounded exactly once. No compare,
// no select -- and rows r, r + 1 go through the two halves of packed fp32
// instructions, so a term costs 1.5 instructions instead of 4. The per-lane sums
// run over channels in order, as the reference's do.
__device__ __forceinline__ float bounds_4x8(const f32x2 (&qp)[4][4], const f32x2 (&qn)[4][4], int n_rep,
                                            const uint2 (&lo_raw)[kGroup],
                                            const uint2 (&hi_raw)[kGroup], int lane) {
    float x[32];
#pragma unroll
    for (int pg = 0; pg < kGroup; ++pg) {
        float lo[4], hi[4];
        unpack4h(lo_raw[pg], lo);
        unpack4h(hi_raw[pg], hi);
        f32x2 lo2[4], hi2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            lo2[j] = pack2(lo[j], lo[j]);
            hi2[j] = pack2(hi[j], hi[j]);
        }
#pragma unroll
        for (int rp = 0; rp < 4; ++rp) {
            f32x2 t = pack2(0.f, 0.f);
            if (2 * rp < n_rep) {
#pragma unroll
                for (int j = 0; j < 4; ++j) t = add2(t, fma2(qp[rp][j], hi2[j], mul2(qn[rp][j], lo2[j])));
            }
            unpack2(t, x[pg * 8 + 2 * rp], x[pg * 8 + 2 * rp + 1]);
        }
    }
    float a[16], b[8], c[4], d[2], e[1];
    halve<32, 16>(x, a, lane);
    halve<16, 8>(a, b, lane);
    halve<8, 4>(b, c, lane);
    halve<4, 2>(c, d, lane);
    halve<2, 1>(d, e, lane);
    return e[0];
}

// Monotone map from fp32 to uint32: a > b as floats <=> key(a) > key(b).
// -0 is folded onto +0 first so the two compare equal, as they do as floats.
__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t u = __float_as_uint(x + 0.f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kTopkMaxRow = 8192;              // longest row (a 128K context)

typedef unsigned long long u64;

// One compare-exchange of a bitonic network: keep the larger of (mine, other)
// if `want_max`, else the smaller.
__device__ __forceinline__ u64 bitonic_keep(u64 mine, u64 other, bool want_max) {
    return ((other > mine) == want_max) ? other : mine;
}

// Deterministic top-k by a full sort of the row: one CTA per (sequence, head)
// sorts 64-bit keys (order_key(score) << 32 | ~page) to descending order with a
// bitonic network, so equal scores come out with the lower page first, and
// writes the first k pages. Each thread holds E consecutive keys in registers:
// exchanges at distance < E stay inside the thread, distances E..16E are warp
// shuffles, and only distances >= 32E go through shared memory with a barrier.
// Fewer keys per thread means more warps to hide the network's latency.
template <int kTopkPerThread>
__global__ void __launch_bounds__(1024)
topk_pages_kernel(const float* __restrict__ scores, int* __restrict__ sel, int n, int n_pow2, int k,
                  int heads, long long ss_b, long long ss_h, long long sl_b, long long sl_h) {
    extern __shared__ __align__(8) u64 keys[];
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // lets the attention kernel's prologue overlap the sort
    const int bh = blockIdx.x, b = bh / heads, h = bh % heads;
    const float* row = scores + b * ss_b + h * ss_h;
    const int base = threadIdx.x * kTopkPerThread;
    u64 v[kTopkPerThread];
#pragma unroll
    for (int e = 0; e < kTopkPerThread; ++e) {
        const int i = base + e;
        v[e] = 0ull;                               // padding sorts after every real entry
        if (i < n) v[e] = ((u64)order_key(row[i]) << 32) | (0xffffffffu - (uint32_t)i);
    }
    for (int size = 2; size <= n_pow2; size <<= 1) {
        int stride = size >> 1;
        // For strides >= E every key of this thread sits on the same side of the
        // exchange and in the same sorting direction: one decision per round.
        for (; stride >= 32 * kTopkPerThread; stride >>= 1) {          // other warps: shared memory
            const bool want_max = ((base & stride) == 0) == ((base & size) == 0);
#pragma unroll
            for (int e = 0; e < kTopkPerThread; ++e) keys[base + e] = v[e];
            __syncthreads();
#pragma unroll
            for (int e = 0; e < kTopkPerThread; ++e)
                v[e] = bitonic_keep(v[e], keys[(base + e) ^ stride], want_max);
            __syncthreads();
        }
        for (; stride >= kTopkPerThread; stride >>= 1) {               // same warp: shuffles
            const bool want_max = ((base & stride) == 0) == ((base & size) == 0);
            const int lane_mask = stride / kTopkPerThread;
#pragma unroll
            for (int e = 0; e < kTopkPerThread; ++e)
                v[e] = bitonic_keep(v[e], __shfl_xor_sync(LS_FULL_MASK, v[e], lane_mask), want_max);
        }
#pragma unroll
        for (int st = kTopkPerThread / 2; st > 0; st >>= 1) {          // same thread: registers
            if (st <= stride) {
#pragma unroll
                for (int e = 0; e < kTopkPerThread; ++e) {
                    if ((e & st) == 0) {
                        const bool descending = ((base + e) & size) == 0;
                        const u64 a = v[e], c = v[e | st];
                        const bool swap = (c > a) == descending;
                        v[e] = swap ? c : a;
                        v[e | st] = swap ? a : c;
                    }
                }
            }
        }
    }
    int* dst = sel + b * sl_b + h * sl_h;
#pragma unroll
    for (int e = 0; e < kTopkPerThread; ++e)
        if (base + e < k) dst[base + e] = (int)(0xffffffffu - (uint32_t)(v[e] & 0xffffffffull));
}

// ---------------------------------------------------------------------------
// Selection without the sort, for the fused index -> select -> attend path: the
// attention kernel needs the SET of pages a sequence is owed (its own budget n
// from its own length), not their order by score. One CTA per (sequence, head):
// a 4-pass radix search over the 32-bit order keys finds the n-th largest key T,
// then every key above T is kept, and of the keys equal to T the ones with the
// lowest page numbers (the same tie rule as the sort), by two block scans. Output:
// the kept pages in ascending page order, then -1 up to k. The kept set equals
// the first n entries of the sorted selection, bit for bit.
constexpr int kSelectThreads = 512;

// Shared scratch of select_row.
constexpr int kDigitBits = 11;                 // radix digit: 2048 bins
constexpr int kBins = 1 << kDigitBits;
struct SelectScratch {
    int hist[kBins];
    int warp_tot[32][2];
    unsigned lo, hi;                           // smallest / largest finite key of the row
    int n_inf, n_fin;                          // keys that are +inf / finite
    unsigned prefix;
    int remaining;
};

// How many pages a sequence attends: the rule of the attention kernel
// (kernels/cuda/paged_sparse_fp16.cu:242-247 in the reference).
__device__ __forceinline__ int pages_owed(int len, float ratio, int recent, int k, int n) {
    const int L = max(len, 0);
    const int np = (L + LS_PAGE - 1) / LS_PAGE;
    int want = np;
    if (ratio > 0.f && ratio < 1.f) want = max(recent + 1, (int)ceilf(ratio * (float)np));
    return min(min(want, np), min(k, n));
}

// One row of scores -> the n_keep best pages in ascending page order, then -1 up to k.
// Called by all THREADS threads of a CTA; thread i holds keys [i * E, (i + 1) * E).
//
// The n_keep-th largest key T is found by a radix search from the top, 11 bits a
// pass, that starts below the bits every key of the row has in common (scores of one
// row lie within a few binades, so the upper 8-10 bits of their order keys agree: two
// passes instead of the four a byte-wise search over all 32 bits takes). Then every
// key above T is kept, and of the keys equal to T the ones with the lowest page
// numbers, by two block scans.
template <int THREADS, int E>
__device__ __forceinline__ void select_row(const float* __restrict__ row, int* __restrict__ out, int n,
                                           int k, int n_keep, SelectScratch& sc) {
    static_assert(kBins % THREADS == 0, "every thread scans the same number of bins");
    constexpr int BPT = kBins / THREADS;                    // bins per thread
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned key[E];
    if ((n & 3) == 0 && ((reinterpret_cast<uintptr_t>(row) & 15) == 0)) {
#pragma unroll
        for (int e = 0; e < E; e += 4) {
            const int i = tid * E + e;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < n) v = __ldcg(reinterpret_cast<const float4*>(row + i));
            key[e] = (i < n) ? order_key(v.x) : 0u;          // padding: below every real key
            key[e + 1] = (i < n) ? order_key(v.y) : 0u;
            key[e + 2] = (i < n) ? order_key(v.z) : 0u;
            key[e + 3] = (i < n) ? order_key(v.w) : 0u;
        }
    } else {
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int i = tid * E + e;
            key[e] = (i < n) ? order_key(__ldcg(row + i)) : 0u;
        }
    }
    if (n_keep <= 0) {
        for (int i = tid; i < k; i += THREADS) out[i] = -1;
        return;
    }

    // Forced pages score +inf and pages past the end -inf: both are set aside (the former
    // are always kept, the latter never needed), so that what is searched is the range of
    // the finite scores. The bits above the highest bit in which the smallest and the
    // largest of those differ are common to all of them and need no pass.
    constexpr unsigned kPosInf = 0xff800000u, kNegInf = 0x007fffffu;      // order keys of +inf, -inf
    unsigned lo = 0xffffffffu, hi = 0u;
    int n_inf = 0, n_fin = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        if (tid * E + e < n) {
            if (key[e] == kPosInf) {
                ++n_inf;
            } else if (key[e] != kNegInf) {
                ++n_fin;
                lo = min(lo, key[e]);
                hi = max(hi, key[e]);
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        lo = min(lo, __shfl_xor_sync(LS_FULL_MASK, lo, off));
        hi = max(hi, __shfl_xor_sync(LS_FULL_MASK, hi, off));
        n_inf += __shfl_xor_sync(LS_FULL_MASK, n_inf, off);
        n_fin += __shfl_xor_sync(LS_FULL_MASK, n_fin, off);
    }
    if (tid == 0) {
        sc.lo = 0xffffffffu;
        sc.hi = 0u;
        sc.n_inf = 0;
        sc.n_fin = 0;
    }
    for (int i = tid; i < kBins; i += THREADS) sc.hist[i] = 0;
    __syncthreads();
    if (lane == 0) {
        atomicMin(&sc.lo, lo);
        atomicMax(&sc.hi, hi);
        atomicAdd(&sc.n_inf, n_inf);
        atomicAdd(&sc.n_fin, n_fin);
    }
    __syncthreads();
    lo = sc.lo;
    hi = sc.hi;
    n_inf = sc.n_inf;
    n_fin = sc.n_fin;
    int top = 0, remaining = n_keep;
    unsigned mask = 0xffffffffu, prefix;
    if (n_keep <= n_inf) {
        prefix = kPosInf;                                   // the forced pages alone fill the budget
    } else if (n_keep > n_inf + n_fin) {
        prefix = kNegInf;                                   // more owed than scored: never on a sound table
        remaining = n_keep - n_inf - n_fin;
    } else {
        remaining = n_keep - n_inf;
        top = 32 - __clz(lo ^ hi);                          // undecided low bits (0: all finite keys equal)
        mask = top >= 32 ? 0u : ~((1u << top) - 1u);        // decided (common) high bits
        prefix = hi & mask;
    }
#pragma unroll 1
    while (top > 0) {
        const int w = min(kDigitBits, top), shift = top - w;
        const unsigned dmask = (1u << w) - 1u;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            if ((key[e] & mask) == prefix && key[e] != kPosInf && key[e] != kNegInf && tid * E + e < n)
                atomicAdd(&sc.hist[(key[e] >> shift) & dmask], 1);
        }
        __syncthreads();
        // Thread i owns bins kBins-1 - BPT i .. (descending); inclusive scan over threads.
        int local[BPT], sum = 0;
#pragma unroll
        for (int j = 0; j < BPT; ++j) {
            const int bin = kBins - 1 - (BPT * tid + j);
            local[j] = sc.hist[bin];
            sc.hist[bin] = 0;                               // ready for the next pass
            sum += local[j];
        }
        int incl = sum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(LS_FULL_MASK, incl, off);
            if (lane >= off) incl += v;
        }
        if (lane == 31) sc.warp_tot[warp][0] = incl;
        __syncthreads();
        int before = incl - sum;                            // keys in bins above this thread's
        for (int wq = 0; wq < warp; ++wq) before += sc.warp_tot[wq][0];
        if (before < remaining && remaining <= before + sum) {
#pragma unroll
            for (int j = 0; j < BPT; ++j) {
                if (before + local[j] >= remaining) {
                    sc.prefix = prefix | ((unsigned)(kBins - 1 - (BPT * tid + j)) << shift);
                    sc.remaining = remaining - before;
                    break;
                }
                before += local[j];
            }
        }
        __syncthreads();
        // sc.prefix / sc.remaining / warp_tot are rewritten only after the next pass's first barrier.
        prefix = sc.prefix;
        remaining = sc.remaining;
        mask |= dmask << shift;
        top = shift;
    }
    const unsigned T = prefix;                              // the n_keep-th largest key
    const int take_eq = remaining;                          // keys equal to T to keep, lowest pages first

    // Block scans over (keys equal to T, keys above T), in page order.
    int eq_local = 0, gt_local = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const bool real = tid * E + e < n;
        eq_local += real && key[e] == T;
        gt_local += real && key[e] > T;
    }
    int eq_incl = eq_local, gt_incl = gt_local;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(LS_FULL_MASK, eq_incl, off);
        const int c = __shfl_up_sync(LS_FULL_MASK, gt_incl, off);
        if (lane >= off) {
            eq_incl += a;
            gt_incl += c;
        }
    }
    __syncthreads();                                        // warp_tot of the last pass has been read
    if (lane == 31) {
        sc.warp_tot[warp][0] = eq_incl;
        sc.warp_tot[warp][1] = gt_incl;
    }
    __syncthreads();
    int eq_before = eq_incl - eq_local, gt_before = gt_incl - gt_local;
    for (int w = 0; w < warp; ++w) {
        eq_before += sc.warp_tot[w][0];
        gt_before += sc.warp_tot[w][1];
    }
    // Position of a kept key = kept keys before it = (above T before it) + min(equal before it, take_eq).
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const int i = tid * E + e;
        if (i >= n) break;
        const bool gt = key[e] > T, eq = key[e] == T;
        if (gt || (eq && eq_before < take_eq)) out[gt_before + min(eq_before, take_eq)] = i;
        gt_before += gt;
        eq_before += eq;
    }
    for (int i = n_keep + tid; i < k; i += THREADS) out[i] = -1;
}

// grid (ceil(max_pages / (4 * span)), H, B), block 128: a warp scores `span`
// consecutive pages (8, 16 or 24) of one (sequence, KV head) in items of eight.
// All of the warp's bounds are requested at once with 8-byte cp.async copies into
// the warp's own shared memory, one commit group per item, and each item is
// reduced as soon as its group has landed: one DRAM round trip per warp, and the
// bounds wait in shared memory instead of 64 registers, which is what lets four
// CTAs share an SM. Every lane reads back exactly the bytes it copied, so the
// wait on its own groups is the only synchronisation. The host sizes `span` so
// that the whole grid is resident at once where the problem allows it.
//
// Launched programmatically with `early` set, the block ids and the bounds are
// requested BEFORE the kernel synchronises on its predecessor: the pages whose bounds
// it reads are never a sequence's last page (page 0 and the `recent` last pages are
// not scored at all), and only a last page's bounds change between decode steps. The
// queries, which the predecessor usually wrote, are read after the wait.
//
// PER_HEAD = 0: scores [B,H,P]; PER_HEAD = 1: heads [B,H,R,P].
template <int PER_HEAD>
__global__ void __launch_bounds__(kIndexWarps * 32, kIndexCtasPerSm)
page_index_kernel(const __half* __restrict__ q, const __half* __restrict__ kmin,
                  const __half* __restrict__ kmax, const int* __restrict__ block_tables,
                  const int* __restrict__ seq_lens, float* __restrict__ out, int n_rep,
                  int max_pages, int span, int table_stride, int num_blocks, int recent, int early,
                  long long sq_b, long long sq_h, long long sq_m, long long sb_b, long long sb_h,
                  long long ss_b, long long ss_h, long long ss_r) {
    __shared__ __align__(16) unsigned char staged[kIndexWarps][kMaxItems][kItemBytes];
    const int b = blockIdx.z, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = (blockIdx.x * kIndexWarps + warp) * span;
    const int end = min(first + span, max_pages);
    const int items = first < max_pages ? (end - first + kItemPages - 1) / kItemPages : 0;
    if (!early) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int L = max(seq_lens[b], 0);
    const int np = min((L + LS_PAGE - 1) / LS_PAGE, table_stride);

    // Lane j fetches the block id of page first + j (-1: nothing to score).
    int ids = -1;
    {
        const int p = first + lane;
        bool need = p < end && p < np;
        if (!PER_HEAD) need = need && !(p == 0 || p >= np - recent);
        if (need) {
            const int id = block_tables[(long long)b * table_stride + p];
            if (id >= 0 && id < num_blocks) ids = id;
        }
    }
    const uint32_t mine = smem_u32(&staged[warp][0][0]) + lane * 8;
#pragma unroll
    for (int it = 0; it < kMaxItems; ++it) {
        if (it < items) {
#pragma unroll
            for (int k = 0; k < kItemPages; ++k) {
                const int blk = __shfl_sync(LS_FULL_MASK, ids, it * kItemPages + k);
                const long long off = blk >= 0 ? blk * sb_b + h * sb_h + lane * 4 : 0;
                const uint32_t dst = mine + it * kItemBytes + k * 512;
                cp_async_8(dst, kmin + off, blk >= 0 ? 8 : 0);          // an unscored page reads as zeros
                cp_async_8(dst + 256, kmax + off, blk >= 0 ? 8 : 0);
            }
        }
        cp_async_commit();
    }
    if (early) asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // q+ and q- of rows (2 rp, 2 rp + 1), channel j, packed; rows past n_rep are zero.
    f32x2 qp[4][4], qn[4][4];
#pragma unroll
    for (int rp = 0; rp < 4; ++rp) {
        float q0[4] = {0.f, 0.f, 0.f, 0.f}, q1[4] = {0.f, 0.f, 0.f, 0.f};
        if (2 * rp < n_rep)
            unpack4h(*reinterpret_cast<const uint2*>(q + b * sq_b + h * sq_h + (2 * rp) * sq_m + lane * 4), q0);
        if (2 * rp + 1 < n_rep)
            unpack4h(*reinterpret_cast<const uint2*>(q + b * sq_b + h * sq_h + (2 * rp + 1) * sq_m + lane * 4),
                     q1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            qp[rp][j] = pack2(fmaxf(q0[j], 0.f), fmaxf(q1[j], 0.f));
            qn[rp][j] = pack2(fminf(q0[j], 0.f), fminf(q1[j], 0.f));
        }
    }

    // Reduces group g of item `it` and writes its scores.
    auto reduce = [&](int it, int g) {
        uint2 lo_raw[kGroup], hi_raw[kGroup];
        const unsigned char* src = &staged[warp][it][g * kGroup * 512 + lane * 8];
#pragma unroll
        for (int k = 0; k < kGroup; ++k) {
            lo_raw[k] = *reinterpret_cast<const uint2*>(src + k * 512);
            hi_raw[k] = *reinterpret_cast<const uint2*>(src + k * 512 + 256);
        }
        float s = bounds_4x8(qp, qn, n_rep, lo_raw, hi_raw, lane);
        const int slot = it * kItemPages + g * kGroup + (lane >> 3);
        const int p = first + slot, r = lane & 7;
        const int blk = __shfl_sync(LS_FULL_MASK, ids, slot);
        if (PER_HEAD) {
            // Pages past the end get a finite 0: their token count of zero
            // removes them downstream, and a stale NaN here would not.
            if (p < end && r < n_rep) out[b * ss_b + h * ss_h + r * ss_r + p] = blk >= 0 ? s : 0.f;
        } else {
            if (r >= n_rep || blk < 0) s = neg_inf();
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) s = fmaxf(s, __shfl_xor_sync(LS_FULL_MASK, s, off));
            if (p >= np) s = neg_inf();                                  // past the end: never chosen
            else if (p == 0 || p >= np - recent) s = pos_inf();          // sink and recent: always kept
            if (r == 0 && p < end) out[b * ss_b + h * ss_h + p] = s;
        }
    };
    if (items > 0) {
        cp_async_wait<kMaxItems - 1>();
#pragma unroll
        for (int g = 0; g < kItemGroups; ++g) reduce(0, g);
    }
    if (items > 1) {
        cp_async_wait<kMaxItems - 2>();
#pragma unroll
        for (int g = 0; g < kItemGroups; ++g) reduce(1, g);
    }
    if (items > 2) {
        cp_async_wait<0>();
#pragma unroll
        for (int g = 0; g < kItemGroups; ++g) reduce(2, g);
    }
    // No early trigger for a programmatic successor: a CTA that has returned counts as
    // having triggered, so the next kernel's CTAs arrive while the last warps here
    // finish and never hold SM slots this kernel's single wave needs.
}

template <int E>
__global__ void __launch_bounds__(kSelectThreads)
select_pages_kernel(const float* __restrict__ scores, const int* __restrict__ seq_lens,
                    int* __restrict__ sel, int n, int k, int heads, float ratio, int recent,
                    long long ss_b, long long ss_h, long long sl_b, long long sl_h) {
    __shared__ SelectScratch sc;
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int bh = blockIdx.x, b = bh / heads, h = bh % heads;
    const int n_keep = pages_owed(seq_lens[b], ratio, recent, k, n);
    // Launched programmatically: everything above overlapped the end of the kernel
    // that writes the scores.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    select_row<kSelectThreads, E>(scores + b * ss_b + h * ss_h, sel + b * sl_b + h * sl_h, n, k, n_keep, sc);
}

}  // namespace ls

extern "C" {

static int launch_index(int per_head, const void* q, const void* kmin, const void* kmax,
                        const int32_t* block_tables, const int32_t* seq_lens, float* out, int batch,
                        int kv_heads, int n_rep, int head_dim, int page, int max_pages,
                        int table_stride, int num_blocks, int recent, int64_t sq_b, int64_t sq_h,
                        int64_t sq_m, int64_t sb_b, int64_t sb_h, int64_t ss_b, int64_t ss_h,
                        int64_t ss_r, void* stream, int flags = 0) {
    if (!q || !kmin || !kmax || !block_tables || !seq_lens || !out) return LS_ERR_NULL_POINTER;
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (batch <= 0 || kv_heads <= 0 || n_rep <= 0 || max_pages <= 0 || table_stride < max_pages ||
        num_blocks <= 0)
        return LS_ERR_BAD_SHAPE;
    if (n_rep > 8) return LS_ERR_UNSUPPORTED;
    if (batch > 65535 || kv_heads > 65535) return LS_ERR_TOO_LARGE;
    if ((sq_b % 4) || (sq_h % 4) || (sq_m % 4) || (sb_b % 4) || (sb_h % 4)) return LS_ERR_MISALIGNED;
    if (((uintptr_t)q & 7) || ((uintptr_t)kmin & 7) || ((uintptr_t)kmax & 7)) return LS_ERR_MISALIGNED;
    // Pages per warp: the smallest number of items that lets every CTA of the grid
    // be resident at once (no second wave), capped by what a warp can stage.
    static int sms_of[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    int sms = dev >= 0 && dev < 64 ? sms_of[dev] : 0;
    if (sms <= 0) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 1;
        if (dev >= 0 && dev < 64) sms_of[dev] = sms;
    }
    const long long resident = (long long)ls::kIndexCtasPerSm * sms;
    int span = ls::kItemPages;
    for (int items = 1; items <= ls::kMaxItems; ++items) {
        span = items * ls::kItemPages;
        const long long per_row = (max_pages + ls::kIndexWarps * span - 1) / (ls::kIndexWarps * span);
        if (per_row * kv_heads * batch <= resident) break;
    }
    const int per_cta = ls::kIndexWarps * span;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto kern = per_head ? ls::page_index_kernel<1> : ls::page_index_kernel<0>;
    static bool carveout_set[64][2] = {};
    const int slot = dev >= 0 && dev < 64 ? dev : 0;
    const int variant = per_head ? 1 : 0;
    if (!carveout_set[slot][variant]) {    // four 48 KB CTAs per SM need the large shared-memory split
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        carveout_set[slot][variant] = dev >= 0 && dev < 64;
    }
    // With LS_LAUNCH_PROGRAMMATIC the launch may begin while the previous kernel of the stream
    // drains; with LS_EARLY_PAGES on top of it the bounds are requested before the kernel
    // synchronises on that predecessor (see the kernel). Per-head bounds score a sequence's
    // last page too, and so does recent == 0: no early requests then.
    const bool programmatic = (flags & LS_LAUNCH_PROGRAMMATIC) != 0;
    const int early = programmatic && (flags & LS_EARLY_PAGES) && !per_head && recent >= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((max_pages + per_cta - 1) / per_cta, kv_heads, batch);
    cfg.blockDim = dim3(ls::kIndexWarps * 32);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    const long long a_sq_b = sq_b, a_sq_h = sq_h, a_sq_m = sq_m, a_sb_b = sb_b, a_sb_h = sb_h, a_ss_b = ss_b,
                    a_ss_h = ss_h, a_ss_r = ss_r;
    cudaError_t e = cudaLaunchKernelEx(
        &cfg, kern, static_cast<const __half*>(q), static_cast<const __half*>(kmin),
        static_cast<const __half*>(kmax), block_tables, seq_lens, out, n_rep, max_pages, span, table_stride,
        num_blocks, recent, early, a_sq_b, a_sq_h, a_sq_m, a_sb_b, a_sb_h, a_ss_b, a_ss_h, a_ss_r);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

int ls_page_index(const void* q, const void* kmin, const void* kmax, const int32_t* block_tables,
                  const int32_t* seq_lens, float* scores, int batch, int kv_heads, int n_rep,
                  int head_dim, int page, int max_pages, int table_stride, int num_blocks,
                  int recent, int64_t sq_b, int64_t sq_h, int64_t sq_m, int64_t sb_b, int64_t sb_h,
                  int64_t ss_b, int64_t ss_h, void* stream) {
    return launch_index(0, q, kmin, kmax, block_tables, seq_lens, scores, batch, kv_heads, n_rep,
                        head_dim, page, max_pages, table_stride, num_blocks, recent, sq_b, sq_h, sq_m,
                        sb_b, sb_h, ss_b, ss_h, 0, stream);
}

int ls_page_index_heads(const void* q, const void* kmin, const void* kmax,
                        const int32_t* block_tables, const int32_t* seq_lens, float* heads_out,
                        int batch, int kv_heads, int n_rep, int head_dim, int page, int max_pages,
                        int table_stride, int num_blocks, int64_t sq_b, int64_t sq_h, int64_t sq_m,
                        int64_t sb_b, int64_t sb_h, int64_t sh_b, int64_t sh_h, int64_t sh_r,
                        void* stream) {
    return launch_index(1, q, kmin, kmax, block_tables, seq_lens, heads_out, batch, kv_heads, n_rep,
                        head_dim, page, max_pages, table_stride, num_blocks, 0, sq_b, sq_h, sq_m, sb_b,
                        sb_h, sh_b, sh_h, sh_r, stream);
}

int ls_topk_pages(const float* scores, int32_t* sel, int batch, int kv_heads, int num_pages, int k,
                  int64_t ss_b, int64_t ss_h, int64_t sl_b, int64_t sl_h, void* stream) {
    if (!scores || !sel) return LS_ERR_NULL_POINTER;
    if (batch <= 0 || kv_heads <= 0 || num_pages <= 0 || k <= 0 || k > num_pages)
        return LS_ERR_BAD_SHAPE;
    int n_pow2 = 256;
    while (n_pow2 < num_pages) n_pow2 <<= 1;
    if (n_pow2 > ls::kTopkMaxRow || (long long)batch * kv_heads > 2147483647LL) return LS_ERR_TOO_LARGE;
    if (((uintptr_t)scores & 3) || ((uintptr_t)sel & 3)) return LS_ERR_MISALIGNED;
    const size_t smem = sizeof(unsigned long long) * (size_t)n_pow2;
    // Keys per thread: 4 measured best at 2048 keys (512 threads); 8 beyond 4096.
    const int per_thread = n_pow2 <= 4096 ? 4 : 8;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = batch * kv_heads;
#define LS_LAUNCH_TOPK(E)                                                                          \
    do {                                                                                           \
        cudaError_t e_ = cudaFuncSetAttribute(ls::topk_pages_kernel<E>,                            \
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e_ != cudaSuccess) return (int)e_;                                                     \
        ls::topk_pages_kernel<E><<<grid, n_pow2 / E, smem, st>>>(scores, sel, num_pages, n_pow2, k, \
                                                                 kv_heads, ss_b, ss_h, sl_b, sl_h); \
    } while (0)
    if (per_thread == 4) LS_LAUNCH_TOPK(4);
    else LS_LAUNCH_TOPK(8);
#undef LS_LAUNCH_TOPK
    return (int)cudaGetLastError();
}

int ls_select_pages(const float* scores, const int32_t* seq_lens, int32_t* sel, int batch, int kv_heads,
                    int num_pages, int k, float ratio, int recent, int64_t ss_b, int64_t ss_h,
                    int64_t sl_b, int64_t sl_h, void* stream) {
    if (!scores || !seq_lens || !sel) return LS_ERR_NULL_POINTER;
    if (batch <= 0 || kv_heads <= 0 || num_pages <= 0 || k <= 0 || k > num_pages || recent < 0)
        return LS_ERR_BAD_SHAPE;
    if (num_pages > ls::kTopkMaxRow || (long long)batch * kv_heads > 2147483647LL) return LS_ERR_TOO_LARGE;
    if (((uintptr_t)scores & 3) || ((uintptr_t)sel & 3)) return LS_ERR_MISALIGNED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = batch * kv_heads;
    // A programmatic launch: the CTAs may become resident while the kernel that writes
    // the scores drains (they wait for it before reading); after a kernel that never
    // triggers early this is an ordinary launch.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(ls::kSelectThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const long long a_ss_b = ss_b, a_ss_h = ss_h, a_sl_b = sl_b, a_sl_h = sl_h;
    cudaError_t e;
    if (num_pages <= 4 * ls::kSelectThreads)
        e = cudaLaunchKernelEx(&cfg, ls::select_pages_kernel<4>, scores, seq_lens, sel, num_pages, k,
                               kv_heads, ratio, recent, a_ss_b, a_ss_h, a_sl_b, a_sl_h);
    else
        e = cudaLaunchKernelEx(&cfg, ls::select_pages_kernel<16>, scores, seq_lens, sel, num_pages, k,
                               kv_heads, ratio, recent, a_ss_b, a_ss_h, a_sl_b, a_sl_h);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

int ls_page_index_select(const void* q, const void* kmin, const void* kmax, const int32_t* block_tables,
                         const int32_t* seq_lens, float* scores, int32_t* sel, int batch, int kv_heads,
                         int n_rep, int head_dim, int page, int max_pages, int table_stride,
                         int num_blocks, int recent, int k, float ratio, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sb_b, int64_t sb_h, int64_t ss_b, int64_t ss_h,
                         int64_t sl_b, int64_t sl_h, void* stream) {
    if (!sel) return LS_ERR_NULL_POINTER;
    if (flags & ~(LS_LAUNCH_PROGRAMMATIC | LS_EARLY_PAGES)) return LS_ERR_UNSUPPORTED;
    int rc = launch_index(0, q, kmin, kmax, block_tables, seq_lens, scores, batch, kv_heads, n_rep, head_dim,
                          page, max_pages, table_stride, num_blocks, recent, sq_b, sq_h, sq_m, sb_b, sb_h,
                          ss_b, ss_h, 0, stream, flags);
    if (rc) return rc;
    return ls_select_pages(scores, seq_lens, sel, batch, kv_heads, max_pages, k, ratio, recent, ss_b, ss_h,
                           sl_b, sl_h, stream);
}

}  // extern "C"
