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
// does that with a warp per page and an all-lanes butterfly per value. Here a
// LANE scores a page: the page's bounds wait in shared memory, the thirty-two
// per-lane partial sums of the reference become thirty-two values of one
// thread, and the butterfly becomes the same binary tree of additions walked in
// an order that keeps three partial results alive per query row. Same
// operands, same operations, no shuffles.
#include "ls_common.cuh"

namespace ls {

constexpr int kIndexWarps = 4;                 // warp pairs per CTA
constexpr int kItemPages = 32;               // pages a warp scores at a time: one per lane
constexpr int kItemBytes = kItemPages * 512; // a page's minimum and maximum rows, 256 bytes each
constexpr int kQFloats = 8 * 8 * 8 * 4;      // the CTA's query rows as q+ / q- pairs (see stage_query)
constexpr int kIndexSmem = kIndexWarps * kItemBytes + kQFloats * 4 + kIndexWarps * 8 * 32 * 4;
#ifndef LS_INDEX_CTAS
#define LS_INDEX_CTAS 2
#endif
constexpr int kIndexCtasPerSm = LS_INDEX_CTAS;   // resident CTAs of the index kernel (256 threads, 76 KB of shared memory each)

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
    int n_cand, bucket_count;                  // one-pass search: keys in the wanted bucket
};
constexpr int kMaxCandidates = 64;            // a wanted bucket with more keys goes to the bit-wise search

// How many pages a sequence attends: the rule of the attention kernel
// (kernels/cuda/paged_sparse_fp16.cu:242-247 in the reference).
__device__ __forceinline__ int pages_owed(int len, float ratio, int recent, int k, int n) {
    const int L = max(len, 0);
    const int np = (L + LS_PAGE - 1) / LS_PAGE;
    int want = np;
    if (ratio > 0.f && ratio < 1.f) want = max(recent + 1, (int)ceilf(ratio * (float)np));
    return min(min(want, np), min(k, n));
}

// Sum of the per-warp totals tot[0 .. warp) (column c of SelectScratch::warp_tot), by one
// scan inside the calling warp instead of a chain of dependent shared-memory reads.
template <int WARPS>
__device__ __forceinline__ int warps_before(const int (*tot)[2], int c, int warp, int lane) {
    static_assert(WARPS <= 32, "one lane per warp total");
    int v = lane < WARPS ? tot[lane][c] : 0;
#pragma unroll
    for (int off = 1; off < WARPS; off <<= 1) {
        const int u = __shfl_up_sync(LS_FULL_MASK, v, off);
        if (lane >= off) v += u;
    }
    const int incl = __shfl_sync(LS_FULL_MASK, v, warp);
    const int own = __shfl_sync(LS_FULL_MASK, lane < WARPS ? tot[lane][c] : 0, warp);
    return incl - own;
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
        // One pass over 2048 buckets of equal width between the smallest and the largest finite
        // key usually settles it: the bucket that holds the wanted key rarely holds more than a
        // handful, and among those the key is found by counting. (The bit-wise search below needs
        // three passes for scores that straddle a power of two.) Rows whose wanted bucket is
        // crowded -- many equal or nearly equal scores -- take the bit-wise search instead.
        if (top > kDigitBits) {
            const unsigned range = hi - lo;
            const int bshift = max(0, 32 - __clz(range) - kDigitBits);   // range >> bshift < kBins
#pragma unroll
            for (int e = 0; e < E; ++e) {
                if (key[e] != kPosInf && key[e] != kNegInf && tid * E + e < n)
                    atomicAdd(&sc.hist[(key[e] - lo) >> bshift], 1);
            }
            __syncthreads();
            int local[BPT], sum = 0;
#pragma unroll
            for (int j = 0; j < BPT; ++j) {
                const int bin = kBins - 1 - (BPT * tid + j);
                local[j] = sc.hist[bin];
                sum += local[j];
            }
            int incl = sum;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int v = __shfl_up_sync(LS_FULL_MASK, incl, off);
                if (lane >= off) incl += v;
            }
            if (lane == 31) sc.warp_tot[warp][0] = incl;
            if (tid == 0) sc.n_cand = 0;
            __syncthreads();
            int before = incl - sum + warps_before<THREADS / 32>(sc.warp_tot, 0, warp, lane);
            if (before < remaining && remaining <= before + sum) {
#pragma unroll
                for (int j = 0; j < BPT; ++j) {
                    if (before + local[j] >= remaining) {
                        sc.prefix = (unsigned)(kBins - 1 - (BPT * tid + j));     // the wanted bucket
                        sc.remaining = remaining - before;                       // rank inside it, from the top
                        sc.bucket_count = local[j];
                        break;
                    }
                    before += local[j];
                }
            }
            __syncthreads();
            const unsigned bucket = sc.prefix;
            const int want = sc.remaining, crowd = sc.bucket_count;
            // The histogram is needed again: by the bit-wise search (zeroed), or as the candidates' list.
            for (int i = tid; i < kBins; i += THREADS) sc.hist[i] = 0;
            __syncthreads();
            if (crowd <= kMaxCandidates) {
                unsigned* cand = reinterpret_cast<unsigned*>(sc.hist);
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    if (key[e] != kPosInf && key[e] != kNegInf && tid * E + e < n &&
                        ((key[e] - lo) >> bshift) == bucket)
                        cand[atomicAdd(&sc.n_cand, 1)] = key[e];
                }
                __syncthreads();
                if (tid < crowd) {
                    const unsigned x = cand[tid];
                    int gt = 0, ge = 0;
                    for (int i = 0; i < crowd; ++i) {
                        gt += cand[i] > x;
                        ge += cand[i] >= x;
                    }
                    if (gt < want && want <= ge) {          // equal candidates all write the same pair
                        sc.prefix = x;
                        sc.remaining = want - gt;
                    }
                }
                __syncthreads();
                prefix = sc.prefix;
                remaining = sc.remaining;
                top = 0;                                    // settled: no bit-wise pass
            }
        }
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
        int before = incl - sum + warps_before<THREADS / 32>(sc.warp_tot, 0, warp, lane);   // keys in bins above this thread's
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
    int eq_before = eq_incl - eq_local + warps_before<THREADS / 32>(sc.warp_tot, 0, warp, lane);
    int gt_before = gt_incl - gt_local + warps_before<THREADS / 32>(sc.warp_tot, 1, warp, lane);
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

// Shared-memory image of the CTA's query rows. max(q * lo, q * hi) with lo <= hi (a
// page's channel minimum and maximum) is q * hi for q > 0 and q * lo for q < 0. With
// q+ = max(q, 0) and q- = min(q, 0) that product is fma(q+, hi, q- * lo), bit for bit:
// one of the two factors is zero, so one term is a zero and the other is rounded
// exactly once. No compare, no select. The terms of channels c and c + 64 go through
// the two halves of packed fp32 instructions: c belongs to the reference's lane c / 4
// and c + 64 to lane c / 4 + 16, the two lanes whose partial sums are added first.
//
// Step j (0..7) of a page's evaluation covers the reference's lanes j, j + 8, j + 16 and
// j + 24, i.e. channels 4j + {0..3} + {0, 32, 64, 96}. Its operands for query row r are
// eight 16-byte entries (pp = 0..7): {q+[c], q+[c + 64], q-[c], q-[c + 64]} with
// c = 4j + pp for pp < 4 and c = 4j + 32 + (pp - 4) otherwise.
__device__ __forceinline__ int query_slot(int r, int c) {
    const int lane_ref = c >> 2, jj = c & 3;
    const int j = lane_ref & 7, m = lane_ref >> 3;          // reference lane = j + 8 m
    const int pp = jj + 4 * (m & 1), e = m >> 1;
    return (((j * 8 + r) * 8 + pp) << 2) + e;               // + 2 for q-
}

// Barrier of one warp pair (64 threads), with a constant id per pair so that the CTA
// holds five barriers, not sixteen.
__device__ __forceinline__ void pair_barrier(int pair) {
    switch (pair) {
        case 0: asm volatile("bar.sync 1, 64;\n" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 64;\n" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 64;\n" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;\n" ::: "memory"); break;
    }
}

// grid (ceil(max_pages / (4 * span)), H, B), block 256 = four PAIRS of warps: a pair
// scores `span` consecutive pages of one (sequence, KV head), thirty-two at a time. The
// bounds of those thirty-two pages are requested at once with 8-byte cp.async copies (a
// warp-wide copy is one 256-byte row; each warp of the pair requests sixteen of the pages)
// into the pair's 16 KB of shared memory, chunk u of page k at position u ^ (k & 15) so
// that the lanes, which then read one page each, hit different banks. Lane l evaluates
// page l: 128 channels x the group's query rows, the query operands broadcast from shared
// memory. The two warps of a pair each walk one half of the addition tree (the reference
// lanes with bit 0 clear / set: the operands of its last butterfly step) and the first warp
// adds the two halves, so a page's evaluation is two dependent chains of half the length.
//
// Launched programmatically with `early` set, the block ids and the first bounds are
// requested BEFORE the kernel synchronises on its predecessor: the pages whose bounds
// it reads are never a sequence's last page (page 0 and the `recent` last pages are
// not scored at all), and only a last page's bounds change between decode steps. The
// queries, which the predecessor usually wrote, are read after the wait.
//
// PER_HEAD = 0: scores [B,H,P]; PER_HEAD = 1: heads [B,H,R,P]. NREP: the group size when
// it is known at compile time (6), else 0 and the rows are tested against n_rep.
template <int PER_HEAD, int NREP>
__global__ void __launch_bounds__(kIndexWarps * 64, kIndexCtasPerSm)
page_index_kernel(const __half* __restrict__ q, const __half* __restrict__ kmin,
                  const __half* __restrict__ kmax, const int* __restrict__ block_tables,
                  const int* __restrict__ seq_lens, float* __restrict__ out, int n_rep_arg,
                  int max_pages, int span, int table_stride, int num_blocks, int recent, int early,
                  long long sq_b, long long sq_h, long long sq_m, long long sb_b, long long sb_h,
                  long long ss_b, long long ss_h, long long ss_r) {
    constexpr int ROWS = NREP ? NREP : 8;
    const int n_rep = NREP ? NREP : n_rep_arg;
    extern __shared__ __align__(16) unsigned char index_smem[];
    float* qs = reinterpret_cast<float*>(index_smem + kIndexWarps * kItemBytes);
    float* xch = qs + kQFloats;                              // [pair][row][lane]: the second warp's half sums
    const int b = blockIdx.z, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = warp >> 1, side = warp & 1;
    const int first = (blockIdx.x * kIndexWarps + pair) * span;
    const int end = min(first + span, max_pages);
    const int items = first < max_pages ? (end - first + kItemPages - 1) / kItemPages : 0;
    if (!early) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int L = max(seq_lens[b], 0);
    const int np = min((L + LS_PAGE - 1) / LS_PAGE, table_stride);
    const uint32_t mine = smem_u32(index_smem + pair * kItemBytes);
    const long long lane_off = h * sb_h + lane * 4;

    // Requests this warp's sixteen pages of item `it`; returns the lane's block id for page
    // `lane` of the item (-1: nothing to score).
    auto request = [&](int it) -> int {
        int id = -1;
        const int p = first + it * kItemPages + lane;
        bool need = p < end && p < np;
        if (!PER_HEAD) need = need && !(p == 0 || p >= np - recent);
        if (need) {
            const int got = block_tables[(long long)b * table_stride + p];
            if (got >= 0 && got < num_blocks) id = got;
        }
#pragma unroll 4
        for (int kk = 0; kk < kItemPages / 2; ++kk) {
            const int k = side * (kItemPages / 2) + kk;
            const int blk = __shfl_sync(LS_FULL_MASK, id, k);
            const long long off = blk >= 0 ? blk * sb_b + lane_off : 0;
            const uint32_t dst = mine + k * 512 + ((lane ^ (k & 15)) << 3);
            cp_async_8(dst, kmin + off, blk >= 0 ? 8 : 0);              // an unscored page reads as zeros
            cp_async_8(dst + 256, kmax + off, blk >= 0 ? 8 : 0);
        }
        cp_async_commit();
        return id;
    };
    int id = items > 0 ? request(0) : -1;
    if (early) asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // The CTA's query rows, once: threads 0..127 take channel c of rows 0..3, the others of rows 4..7.
    {
        const int c = threadIdx.x & 127, r0 = (threadIdx.x >> 7) * 4;
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
            const int r = r0 + rr;
            float v = 0.f;
            if (r < n_rep) v = __half2float(q[b * sq_b + h * sq_h + r * sq_m + c]);
            const int slot = query_slot(r, c);
            qs[slot] = fmaxf(v, 0.f);
            qs[slot + 2] = fminf(v, 0.f);
        }
    }
    __syncthreads();

    const uint32_t page_base = mine + lane * 512;
    const int sw = lane & 15;
    for (int it = 0; it < items; ++it) {
        cp_async_wait<0>();
        pair_barrier(pair);                         // both warps' copies have landed
        float s4[ROWS];                             // this warp's half of every row's sum
        float hold3[ROWS];
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
            // Reference lanes ja and ja + 4 (and + 8, + 16, + 24 of each); this warp's ja: side, side + 2.
            const int ja = side + 2 * half;
            float s2a[ROWS];
#pragma unroll
            for (int sd = 0; sd < 2; ++sd) {
                const int j = ja + 4 * sd;
                // Channels 4j + {0..3} + {0, 32, 64, 96}: 8-byte chunks j, j + 8, j + 16, j + 24.
                f32x2 lo2[8], hi2[8];
                {
                    float2 lo[4][2], hi[4][2];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const uint32_t a = page_base + (((j + 8 * m) ^ sw) << 3);
                        uint32_t l0, l1, h0, h1;
                        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=r"(l0), "=r"(l1) : "r"(a));
                        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=r"(h0), "=r"(h1) : "r"(a + 256));
                        lo[m][0] = __half22float2(*reinterpret_cast<const __half2*>(&l0));
                        lo[m][1] = __half22float2(*reinterpret_cast<const __half2*>(&l1));
                        hi[m][0] = __half22float2(*reinterpret_cast<const __half2*>(&h0));
                        hi[m][1] = __half22float2(*reinterpret_cast<const __half2*>(&h1));
                    }
                    // pp < 4: (chunk j, chunk j + 16); pp >= 4: (chunk j + 8, chunk j + 24)
                    lo2[0] = pack2(lo[0][0].x, lo[2][0].x); hi2[0] = pack2(hi[0][0].x, hi[2][0].x);
                    lo2[1] = pack2(lo[0][0].y, lo[2][0].y); hi2[1] = pack2(hi[0][0].y, hi[2][0].y);
                    lo2[2] = pack2(lo[0][1].x, lo[2][1].x); hi2[2] = pack2(hi[0][1].x, hi[2][1].x);
                    lo2[3] = pack2(lo[0][1].y, lo[2][1].y); hi2[3] = pack2(hi[0][1].y, hi[2][1].y);
                    lo2[4] = pack2(lo[1][0].x, lo[3][0].x); hi2[4] = pack2(hi[1][0].x, hi[3][0].x);
                    lo2[5] = pack2(lo[1][0].y, lo[3][0].y); hi2[5] = pack2(hi[1][0].y, hi[3][0].y);
                    lo2[6] = pack2(lo[1][1].x, lo[3][1].x); hi2[6] = pack2(hi[1][1].x, hi[3][1].x);
                    lo2[7] = pack2(lo[1][1].y, lo[3][1].y); hi2[7] = pack2(hi[1][1].y, hi[3][1].y);
                }
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    if (NREP || r < n_rep) {
                        const float4* qrow = reinterpret_cast<const float4*>(qs + ((j * 8 + r) << 5));
                        f32x2 acc_a = pack2(0.f, 0.f), acc_b = pack2(0.f, 0.f);
#pragma unroll
                        for (int pp = 0; pp < 8; ++pp) {
                            const float4 qv = qrow[pp];                  // the same address in every lane
                            const f32x2 t = fma2(pack2(qv.x, qv.y), hi2[pp], mul2(pack2(qv.z, qv.w), lo2[pp]));
                            if (pp < 4) acc_a = add2(acc_a, t);
                            else acc_b = add2(acc_b, t);
                        }
                        float a0, a1, b0, b1;
                        unpack2(acc_a, a0, a1);                          // lanes j, j + 16
                        unpack2(acc_b, b0, b1);                          // lanes j + 8, j + 24
                        const float s2 = __fadd_rn(__fadd_rn(a0, a1), __fadd_rn(b0, b1));   // distances 16, 8
                        if (sd == 0) s2a[r] = s2;
                        else {
                            const float s3 = __fadd_rn(s2a[r], s2);      // distance 4
                            if (half == 0) hold3[r] = s3;
                            else s4[r] = __fadd_rn(hold3[r], s3);        // distance 2
                        }
                    }
                }
            }
        }
        if (side == 1) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (NREP || r < n_rep) xch[(pair * 8 + r) * 32 + lane] = s4[r];
        }
        pair_barrier(pair);                         // half sums written; bounds read
        if (side == 0) {
            const int p = first + it * kItemPages + lane;
            float s = neg_inf();
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (NREP || r < n_rep) {
                    const float total = __fadd_rn(s4[r], xch[(pair * 8 + r) * 32 + lane]);   // distance 1
                    // Pages past the end get a finite 0 per head: their token count of zero
                    // removes them downstream, and a stale NaN here would not.
                    if (PER_HEAD) {
                        if (p < end) out[b * ss_b + h * ss_h + r * ss_r + p] = id >= 0 ? total : 0.f;
                    } else {
                        s = fmaxf(s, total);
                    }
                }
            }
            if (!PER_HEAD) {
                if (id < 0) s = neg_inf();
                if (p >= np) s = neg_inf();                              // past the end: never chosen
                else if (p == 0 || p >= np - recent) s = pos_inf();      // sink and recent: always kept
                if (p < end) out[b * ss_b + h * ss_h + p] = s;
            }
        }
        if (it + 1 < items) id = request(it + 1);
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
    for (int items = 1; items <= 256; ++items) {
        span = items * ls::kItemPages;
        const long long per_row = (max_pages + ls::kIndexWarps * span - 1) / (ls::kIndexWarps * span);
        if (per_row * kv_heads * batch <= resident) break;
    }
    const int per_cta = ls::kIndexWarps * span;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool six = n_rep == 6;
    auto kern = per_head ? (six ? ls::page_index_kernel<1, 6> : ls::page_index_kernel<1, 0>)
                         : (six ? ls::page_index_kernel<0, 6> : ls::page_index_kernel<0, 0>);
    static bool smem_set[64][4] = {};
    const int slot = dev >= 0 && dev < 64 ? dev : 0;
    const int variant = (per_head ? 1 : 0) + (six ? 2 : 0);
    if (!smem_set[slot][variant]) {        // 76 KB of dynamic shared memory per CTA, two CTAs per SM
        cudaError_t ea = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ls::kIndexSmem);
        if (ea != cudaSuccess) return (int)ea;
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        smem_set[slot][variant] = dev >= 0 && dev < 64;
    }
    // With LS_LAUNCH_PROGRAMMATIC the launch may begin while the previous kernel of the stream
    // drains; with LS_EARLY_PAGES on top of it the bounds are requested before the kernel
    // synchronises on that predecessor (see the kernel). Per-head bounds score a sequence's
    // last page too, and so does recent == 0: no early requests then.
    const bool programmatic = (flags & LS_LAUNCH_PROGRAMMATIC) != 0;
    const int early = programmatic && (flags & LS_EARLY_PAGES) && !per_head && recent >= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((max_pages + per_cta - 1) / per_cta, kv_heads, batch);
    cfg.blockDim = dim3(ls::kIndexWarps * 64);
    cfg.dynamicSmemBytes = ls::kIndexSmem;
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
