// Paged GQA decode attention for B200 (sm_100a): dense fp16, dense INT8 and
// page-sparse (fp16 and INT8), plus the log-sum-exp merge of the split partials.
//
// Replaces the reference's one-warp-per-program CUDA-core kernels
//   kernels/cuda/paged_decode_fp16.cu:55-200   (dense fp16)
//   kernels/cuda/paged_decode_int8.cu:87-280   (INT8 pools, fp16 K residual)
//   kernels/cuda/paged_sparse_fp16.cu:205-364  (attention over selected pages)
// and the Triton merge kernels/gqa/paged_decode.py:421-471.
//
// Design (see decode_sched.cuh for the partitioning):
//   * grid = (chunks, KV heads); a CTA of W warps owns one chunk of the
//     batch's page axis for one KV head, so every CTA streams the same number
//     of bytes whatever the sequence lengths are.
//   * each warp is its own load pipeline over its pages (fp16 page-head =
//     16 K rows + 16 V rows of 256 B): STAGES-deep ring in shared memory, rows
//     stored with a 16-byte-chunk XOR swizzle so that shared-memory reads are
//     free of bank conflicts. Two load sides fill the same tiles: per-lane
//     cp.async (groups complete on their own, nothing spins), and TMA tile
//     copies issued by one lane (tensor maps with the 128-byte swizzle,
//     completion counted on an mbarrier per stage, waits bounded). The INT8
//     kernel is instruction-issue bound and uses TMA by default; the fp16
//     kernels are memory bound and use cp.async. No warp waits on another warp
//     inside the page loop.
//   * with programmatic dependent launch the prologue (prefix sums, block ids)
//     and, on request, the first page requests run before the kernel
//     synchronises on its predecessor: everything but a sequence's last page
//     is immutable between decode steps.
//   * all query heads of the GQA group share each page load: scores are
//     S[16 tokens x 8 rows] = K_page . Q^T on the tensor cores (m16n8k16,
//     fp32 accumulation), the page's weights are transposed in registers
//     (movmatrix) and O^T[128 x 8] += V_page^T . P^T accumulates in fp32.
//     The CUDA-core variant (LS_IMPL_SIMT) does the same arithmetic with fp32
//     FMAs and is kept to show where the issue-slot limit sits.
//   * INT8 pages are expanded to fp16 in registers (exactly: |x| <= 128) on
//     their way into the MMA fragments; K's per-(block, head, channel) scale
//     is folded into the query once per page, V's per-token scale into the
//     softmax weight, so neither pool is ever dequantised element by element.
//     V comes in through ldmatrix.trans on byte pairs and enters its MMA as
//     1152 + v (the byte permute's raw result); one more MMA per page sums the
//     weights, and 1152 x that sum comes off every output dim at the end.
//   * rows past a sequence's end are zero-filled on the way in (cp.async with
//     a zero source size; the TMA variants clear or neutralise them after
//     arrival) and their scores forced to -inf: stale pool bytes, NaN patterns
//     included, never reach the arithmetic.
//   * at the end of a segment the CTA's warps merge their states through
//     shared memory and write ONE partial (m, l, acc) per (chunk, sequence,
//     head); every slot a sequence owns is written, so nothing is pre-filled.
//   * the CTA that delivers a sequence's last outstanding partial (an atomic
//     arrival count per (sequence, head), no waiting) merges them and writes
//     the fp16 output, so a layer call is ONE launch.
#include <cuda.h>

#include "decode_sched.cuh"

#include <mutex>
#include <type_traits>

namespace ls {

#define LS_IMPL_MMA 0
#define LS_IMPL_SIMT 1

#ifndef LS_STAGES
#define LS_STAGES 3                 // cp.async ring depth per warp
#endif
#ifndef LS_INT8_STAGES
#define LS_INT8_STAGES 3            // ring depth of the INT8 kernel (4.6 KB stages, 3 CTAs per SM)
#endif
#ifndef LS_INT8_TMA_STAGES
#define LS_INT8_TMA_STAGES 3        // 5 KB stages of the TMA-loading INT8 kernel (74 KB per CTA, three per SM)
#endif
#define LS_INT8_STAGES_ASYM 2       // 5.1 KB stages: a third one would cost the third CTA
#define LS_INT8_TMA_STAGES_ASYM 2   // 6 KB stages with the zero points: the same
#ifndef LS_INT8_CTAS
#define LS_INT8_CTAS 3              // resident CTAs per SM the INT8 kernel is compiled for (168 registers)
#endif
constexpr int kWarps = 4;
// Tensor maps of the TMA-loading variants (unused and zero for the others).
struct TmaMaps {
    CUtensorMap k, v, ks, kz;
    CUtensorMap kv;                 // INT8: K and V pools as one 5-d tensor (see build_int8_maps)
};
constexpr int kMbarSpinLimit = 1 << 22;   // probes of an mbarrier phase before a warp gives up
constexpr int kStages = LS_STAGES;
constexpr int kThreads = kWarps * 32;
constexpr int kMergeStride = LS_HEAD_DIM + 4;   // floats per merged row (bank-conflict pad)
constexpr int kRP = 8;                          // query rows held per partial


// What the load side knows about the page it is about to fetch.
struct PageItem {
    int blk;
    int valid;      // tokens of the page that exist (0 = skip)
    int last;       // bit 0: the sequence's last page; bit 1: a page the step before this
                    // launch may still be writing (never requested ahead of the dependency wait)
    int vl;         // valid | last << 8: equals LS_PAGE for a full page of a sequence's interior
};

// Lookahead over a warp's page sequence. Lane j of the warp holds the block id
// and extent of the j-th upcoming page of the current segment (up to 32 pages),
// fetched with one round of independent loads (two for the sparse kernel:
// selection entry, then block-table entry) instead of a dependent scalar load
// per page. The next window is fetched while the last two pages of the current
// one are still being handed out, so its latency hides behind compute.
template <int MODE>
struct PageWindow {
    Cursor c;                       // first page of the current window
    int n, i;                       // pages in the window, next one to hand out
    int blk, vl;                    // lane j: page j's block id, and valid tokens | last-page bits << 8
    Cursor nc;                      // the window after this one
    int nn, nblk, nvl;
    bool have_next;
    int cached_b, cached_len;

    __device__ __forceinline__ void fill(const DecodeParams& p, const Cursor& cur, int h, int lane,
                                         int& cnt, int& b_, int& vl_) {
        cnt = 0; b_ = 0; vl_ = 0;
        if (cur.done) return;
        if (cur.b != cached_b) {
            cached_b = cur.b;
            cached_len = max(p.seq_lens[cur.b], 0);
        }
        const int np = min((cached_len + LS_PAGE - 1) / LS_PAGE, p.max_pages);
        cnt = min(32, (cur.hi - cur.u + kWarps - 1) / kWarps);
        const int u = cur.u + kWarps * lane;
        const bool in = lane < cnt;
        int page = u;
        if (MODE == LS_MODE_SPARSE && in) page = p.sel[cur.b * p.sl_b + h * p.sl_h + u];
        if (in && page >= 0 && page < np) {
            const int id = p.block_tables[(long long)cur.b * p.max_pages + page];
            if (id >= 0 && id < p.num_blocks) {
                b_ = id;
                // INT8 pools: the page before the last is rewritten (K bytes and K scales,
                // by the page-finalize kernel) in the step whose new token opened the last
                // page, so it counts as mutable too; every earlier page is final.
                const int last = (page == np - 1 ? 1 : 0) | ((p.k_scale != nullptr && page >= np - 2) ? 2 : 0);
                vl_ = min(LS_PAGE, cached_len - page * LS_PAGE) | (last << 8);
            } else {
                p.seg_range[2 * p.batch] = 1;      // corrupt table: read nothing, flag it
            }
        }
    }

    __device__ __forceinline__ void begin(const DecodeParams& p, const Cursor& first, int h,
                                          int lane) {
        cached_b = -1;
        cached_len = 0;
        c = first;
        fill(p, c, h, lane, n, blk, vl);
        i = 0;
        have_next = false;
    }

    __device__ __forceinline__ void prefetch(const DecodeParams& p, const int* cum, int h, int warp,
                                             int lane) {
        nc = c;
        nc.u += kWarps * n;
        cursor_normalize<kWarps>(nc, cum, p.batch, warp);
        fill(p, nc, h, lane, nn, nblk, nvl);
        have_next = true;
    }

    // Next page of this warp; false when the chunk is exhausted. `b` is its sequence.
    __device__ __forceinline__ bool next(const DecodeParams& p, const int* cum, int h, int warp,
                                         int lane, PageItem& it, int& b) {
        if (i == n) {
            // The window after this one was fetched when its last pages were handed out
            // (below): every non-empty window reaches i + 2 >= n before it reaches i == n.
            if (n == 0 || !have_next) return false;
            c = nc; n = nn; blk = nblk; vl = nvl;
            have_next = false;
            i = 0;
            if (n == 0) return false;
        }
        it.blk = __shfl_sync(LS_FULL_MASK, blk, i);
        const int v = __shfl_sync(LS_FULL_MASK, vl, i);
        it.vl = v;
        it.valid = v & 255;
        it.last = v >> 8;
        b = c.b;
        ++i;
        // Once per window, when its last two pages are about to be handed out (i + 2 >= n
        // for the first time): one compare instead of three tests per page.
        if (i == max(n - 2, 1)) prefetch(p, cum, h, warp, lane);
        return true;
    }
};

// ---------------------------------------------------------------------------
// Online softmax on MMA accumulator fragments. Lane (g = lane / 4, t = lane % 4)
// holds scores of tokens g and g + 8 for query rows 2t and 2t + 1:
// s[0] = (g, 2t), s[1] = (g, 2t+1), s[2] = (g+8, 2t), s[3] = (g+8, 2t+1).
// On return s holds the weights 2^(s - m_new); m, l and the output
// accumulators o[8][4] are rescaled. Scores are in the log2 domain.
constexpr float kLazyMargin = 8.f;      // log2 units
template <int TILES>
__device__ __forceinline__ void softmax_update(float (&s)[4], float (&m)[2], float (&l)[2],
                                               float (&o)[TILES][4], float& a0, float& a1) {
    // Usual case after a segment's first pages: no score of the page rises more
    // than 2^kLazyMargin above the running reference m. Then m is kept as it is
    // (any shared reference gives the same normalised result; weights stay below
    // 2^kLazyMargin, well inside fp16) and one vote replaces the six shuffles and
    // the rescale test. The choice depends on the data only, so results are
    // reproducible.
    {
        const float lim0 = m[0] + kLazyMargin, lim1 = m[1] + kLazyMargin;
        const bool ok = (m[0] != neg_inf()) & (m[1] != neg_inf()) & (s[0] <= lim0) & (s[2] <= lim0) &
                        (s[1] <= lim1) & (s[3] <= lim1);
        if (__all_sync(LS_FULL_MASK, ok)) {
            a0 = a1 = 1.f;
            s[0] = ex2(s[0] - m[0]);
            s[1] = ex2(s[1] - m[1]);
            s[2] = ex2(s[2] - m[0]);
            s[3] = ex2(s[3] - m[1]);
            l[0] += s[0] + s[2];
            l[1] += s[1] + s[3];
            return;
        }
    }
    float mx0 = fmaxf(s[0], s[2]);
    float mx1 = fmaxf(s[1], s[3]);
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(LS_FULL_MASK, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(LS_FULL_MASK, mx1, off));
    }
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    // A row that has seen no valid token keeps m = -inf; subtracting a finite
    // stand-in keeps exp2 away from (-inf) - (-inf).
    const float ms0 = (mn0 == neg_inf()) ? 0.f : mn0;
    const float ms1 = (mn1 == neg_inf()) ? 0.f : mn1;
    a0 = ex2(m[0] - ms0);
    a1 = ex2(m[1] - ms1);
    s[0] = ex2(s[0] - ms0);
    s[1] = ex2(s[1] - ms1);
    s[2] = ex2(s[2] - ms0);
    s[3] = ex2(s[3] - ms1);
    m[0] = mn0;
    m[1] = mn1;
    l[0] = l[0] * a0 + (s[0] + s[2]);
    l[1] = l[1] * a1 + (s[1] + s[3]);
    // Once a row's running maximum has settled (the usual case after the first
    // few pages) the factors are exactly 1 and the rescale is skipped.
    if (a0 != 1.f || a1 != 1.f) {
#pragma unroll
        for (int mt = 0; mt < TILES; ++mt) {
            o[mt][0] *= a0;
            o[mt][1] *= a1;
            o[mt][2] *= a0;
            o[mt][3] *= a1;
        }
    }
}

__device__ __forceinline__ void mask_and_scale(float (&s)[4], int valid, float scale_log2, int lane) {
    const int g = lane >> 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] *= scale_log2;
    if (g >= valid) s[0] = s[1] = neg_inf();
    if (g + 8 >= valid) s[2] = s[3] = neg_inf();
}

// S[16 tokens x 8 rows] += K_page(fp16, swizzled at `kaddr`) . Q^T, with Q^T
// given as B fragments over natural 16-dim k-steps.
template <bool TMA = false>
__device__ __forceinline__ void qk_fp16(float (&s)[4], uint32_t kaddr, const uint32_t (&qb)[8][2],
                                        int lane) {
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int sw = row & 7, hi = lane >> 4;
    if (TMA) {
        // Two 16 x 128-byte tiles (dims 0..63 | 64..127), each swizzled by row & 7.
        const uint32_t base = kaddr + row * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(base + (ks >> 2) * 2048 + (((2 * (ks & 3) + hi) ^ sw) << 4), a0, a1, a2, a3);
            mma_16816(s, a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
        }
    } else {
        const uint32_t base = kaddr + row * 256;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(base + (((2 * ks + hi) ^ sw) << 4), a0, a1, a2, a3);
            mma_16816(s, a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
        }
    }
}

__device__ __forceinline__ void load_q_fragments(const DecodeParams& p, int b, int h, int lane,
                                                 uint32_t (&qb)[8][2]) {
    const int g = lane >> 2, t = lane & 3;
    const __half* src = p.q + b * p.sq_b + h * p.sq_h + g * p.sq_m + 2 * t;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        uint32_t x0 = 0, x1 = 0;
        if (g < p.n_rep) {
            x0 = *reinterpret_cast<const uint32_t*>(src + ks * 16);
            x1 = *reinterpret_cast<const uint32_t*>(src + ks * 16 + 8);
        }
        qb[ks][0] = x0;
        qb[ks][1] = x1;
    }
}

// ---------------------------------------------------------------------------
// fp16 pools: page loads.
struct PoolFp16 {
    static constexpr bool kTma = false;
    static constexpr int STAGE_BYTES = 8192;       // K 4096 | V 4096

    // 256 16-byte chunks of K and of V per page-head, 8 + 8 per lane: lane l
    // takes chunk (l & 15) of rows 2i + (l >> 4), i = 0..7, so a warp-wide copy
    // covers two whole 256-byte rows. Row r lands at r * 256 with its chunks
    // XOR-swizzled by r & 7.
    static __device__ __forceinline__ int issue(const DecodeParams& p, int b, int h,
                                                const PageItem& it, uint32_t stage, int lane,
                                                uint64_t pol) {
        const int hi = lane >> 4, col = lane & 15;
        const long long lane_off = hi * p.sk_p + col * 8;
        const long long row2 = 2 * p.sk_p;
        const __half* kb = static_cast<const __half*>(p.k_pool) + it.blk * p.sk_b + h * p.sk_h + lane_off;
        const __half* vb = static_cast<const __half*>(p.v_pool) + it.blk * p.sk_b + h * p.sk_h + lane_off;
        const uint32_t dst0 = stage + hi * 256;
        const uint32_t c0 = (uint32_t)(col ^ hi) << 4;      // ((2i + hi) & 7) = (2i & 7) | hi
        if (__builtin_expect(it.vl == LS_PAGE, 1)) {
            // A full page of a sequence's interior, the case almost every page is: one test.
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t dst = dst0 + i * 512 + (c0 ^ (((2 * i) & 7) << 4));
                cp_async_16_stream(dst, kb + i * row2, pol);
                cp_async_16_stream(dst + 4096, vb + i * row2, pol);
            }
        } else if (p.k_new != nullptr && (it.last & 1) && it.valid > 0) {
            // The step's append rides on this launch: the sequence's newest token (the last
            // valid row of its last page) is not in the pool yet. Its K and V rows come from
            // the caller's new rows, the older rows from the pool, and the new rows are stored
            // to the pool for the steps to come. This warp is the only reader of that row in
            // this launch (a page-head is walked by one warp, and a last page is never shared).
            const int r_new = it.valid - 1;
            const __half* kn = p.k_new + b * p.sn_b + h * p.sn_h + col * 8;
            const __half* vn = p.v_new + b * p.svn_b + h * p.svn_h + col * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t dst = dst0 + i * 512 + (c0 ^ (((2 * i) & 7) << 4));
                const int row = 2 * i + hi;
                const int nbytes = row <= r_new ? 16 : 0;
                const bool fresh = row == r_new;
                cp_async_16(dst, fresh ? kn : (nbytes ? kb + i * row2 : static_cast<const __half*>(p.k_pool)), nbytes);
                cp_async_16(dst + 4096, fresh ? vn : (nbytes ? vb + i * row2 : static_cast<const __half*>(p.v_pool)),
                            nbytes);
            }
            const uint4 row_bits = *reinterpret_cast<const uint4*>(hi ? vn : kn);
            __half* pool = static_cast<__half*>(const_cast<void*>(hi ? p.v_pool : p.k_pool));
            *reinterpret_cast<uint4*>(pool + it.blk * p.sk_b + r_new * p.sk_p + h * p.sk_h + col * 8) = row_bits;
        } else if (it.valid == LS_PAGE) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t dst = dst0 + i * 512 + (c0 ^ (((2 * i) & 7) << 4));
                cp_async_16_stream(dst, kb + i * row2, pol);
                cp_async_16_stream(dst + 4096, vb + i * row2, pol);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t dst = dst0 + i * 512 + (c0 ^ (((2 * i) & 7) << 4));
                const int nbytes = 2 * i + hi < it.valid ? 16 : 0;
                cp_async_16(dst, nbytes ? kb + i * row2 : static_cast<const __half*>(p.k_pool), nbytes);
                cp_async_16(dst + 4096, nbytes ? vb + i * row2 : static_cast<const __half*>(p.v_pool),
                            nbytes);
            }
        }
        return it.valid;
    }
};

// fp16 pools loaded by TMA (on request: measured 3 % slower than the cp.async
// form on this memory-bound kernel, whose 256-byte rows each become two 128-byte
// tile rows; the INT8 kernel, which is issue-bound, gains 14 % from it). A
// page-head (16 rows of 256 bytes, strided in the pool) arrives as two 16 x
// 128-byte tiles per tensor -- dims 0..63 and 64..127, each with the 128-byte
// swizzle -- issued by one lane. Tiles always hold all 16
// rows; what lies past the sequence's end is stale pool memory: its scores are
// masked, and the compute side zeroes those V rows before using the tile.
struct PoolFp16Tma {
    static constexpr bool kTma = true;
    static constexpr int STAGE_BYTES = 8192;       // K lo 2048 | K hi 2048 | V lo 2048 | V hi 2048

    static __device__ __forceinline__ int issue(const DecodeParams&, const TmaMaps& maps, int, int h,
                                                const PageItem& it, uint32_t stage, uint32_t mbar,
                                                int lane, uint64_t pol) {
        if (lane == 0) {
            if (it.valid == 0) {
                mbar_arrive(mbar);
            } else {
                mbar_expect_tx(mbar, 8192u);
                tma_load_4d(stage, &maps.k, mbar, 0, h, 0, it.blk, pol);
                tma_load_4d(stage + 2048, &maps.k, mbar, 64, h, 0, it.blk, pol);
                tma_load_4d(stage + 4096, &maps.v, mbar, 0, h, 0, it.blk, pol);
                tma_load_4d(stage + 6144, &maps.v, mbar, 64, h, 0, it.blk, pol);
            }
        }
        return it.valid;
    }
};

// Tensor-core state for fp16 pools (TMA = tile layout of PoolFp16Tma).
template <bool TMA>
struct MmaFp16T {
    using Pool = typename std::conditional<TMA, PoolFp16Tma, PoolFp16>::type;
    static constexpr int kMinCtas = 2;
    uint32_t qb[8][2];
    float o[8][4];             // O^T: tile mt = dims 16 mt + g (+8), rows 2t, 2t+1
    float m[2], l[2];

    __device__ __forceinline__ void begin(const DecodeParams& p, int b, int h, int lane) {
        m[0] = m[1] = neg_inf();
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[mt][i] = 0.f;
        load_q_fragments(p, b, h, lane, qb);
    }

    __device__ __forceinline__ void compute(const DecodeParams& p, uint32_t stage, int meta,
                                            int lane, uint32_t /*scratch*/) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        if (TMA && meta < LS_PAGE) {
            // A sequence's last page: the tile's V rows past the end are stale pool
            // memory (possibly NaN patterns) and would meet zero weights: clear them.
            // The proxy fence orders these stores before the next TMA write to the stage.
            for (int i = lane; i < (LS_PAGE - meta) * 16; i += 32) {
                const int row = meta + (i >> 4), c = i & 15;
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(
                                 stage + 4096 + (c >> 3) * 2048 + row * 128 + ((c & 7) << 4)),
                             "r"(0)
                             : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
        }
        qk_fp16<TMA>(s, stage, qb, lane);
        mask_and_scale(s, meta, p.scale_log2, lane);
        float a0, a1;
        softmax_update(s, m, l, o, a0, a1);
        // (token g, rows 2t..2t+1) -> (tokens 2t..2t+1, row g): the B fragment
        // layout of P^T for the second MMA.
        const uint32_t pb0 = movmatrix_trans(pack_half2(s[0], s[1]));
        const uint32_t pb1 = movmatrix_trans(pack_half2(s[2], s[3]));
        const int j = lane >> 3;
        const int row = (lane & 7) + (j >> 1) * 8;
        const int sw = row & 7, odd = j & 1;
        if (TMA) {
            const uint32_t base = stage + 4096 + row * 128;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t a0r, a1r, a2r, a3r;
                ldmatrix_x4_trans(base + (mt >> 2) * 2048 + (((2 * (mt & 3) + odd) ^ sw) << 4), a0r, a1r,
                                  a2r, a3r);
                mma_16816(o[mt], a0r, a1r, a2r, a3r, pb0, pb1);
            }
        } else {
            const uint32_t base = stage + 4096 + row * 256;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t a0r, a1r, a2r, a3r;
                ldmatrix_x4_trans(base + (((2 * mt + odd) ^ sw) << 4), a0r, a1r, a2r, a3r);
                mma_16816(o[mt], a0r, a1r, a2r, a3r, pb0, pb1);
            }
        }
    }

    // Reduce row sums over the token lanes, then warp state -> shared memory.
    __device__ __forceinline__ void finish(float* mo, float* mm, float* ml, int n_rep, int lane) {
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l[0] += __shfl_xor_sync(LS_FULL_MASK, l[0], off);
            l[1] += __shfl_xor_sync(LS_FULL_MASK, l[1], off);
        }
        const int g = lane >> 2, t = lane & 3;
        const int r0 = 2 * t, r1 = r0 + 1;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            const int d = mt * 16 + g;
            if (r0 < n_rep) {
                mo[r0 * kMergeStride + d] = o[mt][0];
                mo[r0 * kMergeStride + d + 8] = o[mt][2];
            }
            if (r1 < n_rep) {
                mo[r1 * kMergeStride + d] = o[mt][1];
                mo[r1 * kMergeStride + d + 8] = o[mt][3];
            }
        }
        if (g == 0) {
            if (r0 < n_rep) { mm[r0] = m[0]; ml[r0] = l[0]; }
            if (r1 < n_rep) { mm[r1] = m[1]; ml[r1] = l[1]; }
        }
    }
};

using MmaFp16 = MmaFp16T<false>;
using MmaFp16Tma = MmaFp16T<true>;

// ---------------------------------------------------------------------------
// CUDA-core version of the same page step (fp16 pools only). A half-warp owns
// a token: 16 lanes x 8 dims; the two halves take alternate tokens. R is the
// compile-time bound on query rows.
template <int R>
struct SimtFp16 {
    using Pool = PoolFp16;
    static constexpr int kMinCtas = 2;
    float qf[R][8];
    float acc[R][8];
    float m[R], l[R];

    __device__ __forceinline__ void begin(const DecodeParams& p, int b, int h, int lane) {
        const int d0 = (lane & 15) * 8;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            m[r] = neg_inf();
            l[r] = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[r][j] = 0.f;
            if (r < p.n_rep) {
                const uint4 raw =
                    *reinterpret_cast<const uint4*>(p.q + b * p.sq_b + h * p.sq_h + r * p.sq_m + d0);
                const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(h2[i]);
                    qf[r][2 * i] = f.x * p.scale_log2;
                    qf[r][2 * i + 1] = f.y * p.scale_log2;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) qf[r][j] = 0.f;
            }
        }
    }

    static __device__ __forceinline__ void lds_row8(uint32_t addr, float (&f)[8]) {
        uint4 raw;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                     : "r"(addr));
        const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __half22float2(h2[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }

    __device__ __forceinline__ void compute(const DecodeParams&, uint32_t stage, int valid,
                                            int lane, uint32_t /*scratch*/) {
        const int half_id = lane >> 4, li = lane & 15;
        // Two rounds of four tokens per half keep the score registers modest.
#pragma unroll
        for (int round = 0; round < 2; ++round) {
            float s[4][R];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = 2 * (round * 4 + i) + half_id;
                float kf[8];
                lds_row8(stage + tok * 256 + ((li ^ (tok & 7)) << 4), kf);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float dot = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) dot = fmaf(qf[r][j], kf[j], dot);
                    s[i][r] = dot;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int r = 0; r < R; ++r) {
#pragma unroll
                    for (int off = 8; off > 0; off >>= 1)
                        s[i][r] += __shfl_xor_sync(LS_FULL_MASK, s[i][r], off);
                    if (2 * (round * 4 + i) + half_id >= valid) s[i][r] = neg_inf();
                }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float mx = m[r];
#pragma unroll
                for (int i = 0; i < 4; ++i) mx = fmaxf(mx, s[i][r]);
                const float ms = (mx == neg_inf()) ? 0.f : mx;
                const float a = ex2(m[r] - ms);
                m[r] = mx;
                l[r] *= a;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[r][j] *= a;
#pragma unroll
                for (int i = 0; i < 4; ++i) s[i][r] = ex2(s[i][r] - ms);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = 2 * (round * 4 + i) + half_id;
                float vf[8];
                lds_row8(stage + 4096 + tok * 256 + ((li ^ (tok & 7)) << 4), vf);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    l[r] += s[i][r];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[r][j] = fmaf(s[i][r], vf[j], acc[r][j]);
                }
            }
        }
    }

    // Fold the odd-token half into the even-token half, then store.
    __device__ __forceinline__ void finish(float* mo, float* mm, float* ml, int n_rep, int lane) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float mo_ = __shfl_xor_sync(LS_FULL_MASK, m[r], 16);
            const float lo_ = __shfl_xor_sync(LS_FULL_MASK, l[r], 16);
            const float mn = fmaxf(m[r], mo_);
            const float ms = (mn == neg_inf()) ? 0.f : mn;
            const float ea = ex2(m[r] - ms), eb = ex2(mo_ - ms);
            l[r] = l[r] * ea + lo_ * eb;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float ao = __shfl_xor_sync(LS_FULL_MASK, acc[r][j], 16);
                acc[r][j] = acc[r][j] * ea + ao * eb;
            }
            m[r] = mn;
        }
        if (lane >= 16) return;
        const int d0 = lane * 8;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r < n_rep) {
#pragma unroll
                for (int j = 0; j < 8; ++j) mo[r * kMergeStride + d0 + j] = acc[r][j];
                if (lane == 0) { mm[r] = m[r]; ml[r] = l[r]; }
            }
        }
    }
};

// ---------------------------------------------------------------------------
// INT8 pools. Stage layout (bytes):
//   [0, 4096)     K: int8 page = 16 rows x 128 B (8 swizzled 16-B chunks), or, for a
//                 sequence's last page, the fp16 residual rows (16 x 256 B)
//   [4096, 6144)  V: int8, 16 rows x 128 B
//   [6144, 6656)  K scale, 128 fp32     [6656, 7168)  K zero point (asymmetric only)
//   [7168, 7232)  V scale, 16 fp32      [7232, 7296)  V zero point (asymmetric only)
template <int ASYM>
struct PoolInt8 {
    static constexpr bool kTma = false;
    // K 2 KB | V 2 KB | K scales 512 B | V scales 64 B [| K zeros 512 B | V zeros 64 B].
    // The fp16 K of a sequence's last page does not pass through the ring: the
    // compute side reads it straight from the residual (once per sequence and head).
    static constexpr int STAGE_BYTES = ASYM ? 5248 : 4672;
    static constexpr int OFF_V = 2048, OFF_KS = 4096, OFF_VS = 4608, OFF_KZ = 4672, OFF_VZ = 5184;

    // meta = valid tokens | (K came from the residual) << 8
    static __device__ __forceinline__ int issue(const DecodeParams& p, int b, int h,
                                                const PageItem& it, uint32_t stage, int lane,
                                                uint64_t pol) {
        bool from_res = p.k_res != nullptr && (it.last & 1) && it.valid > 0;
        int rr = from_res ? p.res_rows[b] : 0;
        if (rr < 0 || rr >= p.num_res_rows) {             // corrupt row index: read nothing, flag it
            if (lane == 0) p.seg_range[2 * p.batch] = 1;
            rr = 0;
        }
        // int8 rows: lane l takes chunk (l & 7) of rows 4i + (l >> 3), i = 0..3; a
        // warp-wide copy covers four whole 128-byte rows.
        const int r0 = lane >> 3, col = lane & 7;
        const long long lane_off = r0 * p.sk_p + col * 16;
        const long long row4 = 4 * p.sk_p;
        const uint32_t dst0 = stage + r0 * 128;
        const uint32_t c0 = (uint32_t)(col ^ r0) << 4;          // ((4i + r0) & 7) = (4i & 7) | r0
        const signed char* kb =
            static_cast<const signed char*>(p.k_pool) + it.blk * p.sk_b + h * p.sk_h + lane_off;
        const signed char* vb =
            static_cast<const signed char*>(p.v_pool) + it.blk * p.sk_b + h * p.sk_h + lane_off;
        const bool full = it.valid == LS_PAGE;
        if (!from_res) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t dst = dst0 + i * 512 + (c0 ^ (((4 * i) & 7) << 4));
                if (full) {
                    cp_async_16_stream(dst, kb + i * row4, pol);
                } else {
                    const int nbytes = 4 * i + r0 < it.valid ? 16 : 0;
                    cp_async_16(dst, nbytes ? kb + i * row4 : static_cast<const signed char*>(p.k_pool),
                                nbytes);
                }
            }
            // K scales (and zero points): float4 f = lane goes to slot
            // (f & ~7) | ((f & 7) ^ (f >> 3)), so the four quarter-rows that one
            // shared load touches sit in different banks.
            const int nb = it.valid > 0 ? 16 : 0;
            const uint32_t slot = (uint32_t)((lane & ~7) | ((lane & 7) ^ (lane >> 3))) << 4;
            cp_async_16(stage + OFF_KS + slot,
                        p.k_scale + (nb ? it.blk * p.ks_b + h * p.ks_h + lane * 4 : 0), nb);
            if (ASYM)
                cp_async_16(stage + OFF_KZ + slot,
                            p.k_zero + (nb ? it.blk * p.ks_b + h * p.ks_h + lane * 4 : 0), nb);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t dst = dst0 + OFF_V + i * 512 + (c0 ^ (((4 * i) & 7) << 4));
            if (full) {
                cp_async_16_stream(dst, vb + i * row4, pol);
            } else {
                const int nbytes = 4 * i + r0 < it.valid ? 16 : 0;
                cp_async_16(dst, nbytes ? vb + i * row4 : static_cast<const signed char*>(p.v_pool),
                            nbytes);
            }
        }
        {
            const int tok = lane & 15;
            const int nbytes = tok < it.valid ? 4 : 0;
            const long long off = nbytes ? it.blk * p.vs_b + tok * p.vs_p + h * p.vs_h : 0;
            if (lane < 16)
                cp_async_4(stage + OFF_VS + tok * 4, p.v_scale + off, nbytes);
            else if (ASYM)
                cp_async_4(stage + OFF_VZ + tok * 4, p.v_zero + off, nbytes);
        }
        return it.valid | (from_res ? 256 : 0);
    }
};

// INT8 pools loaded by TMA: one lane issues the K tile, the V tile
// (tensor maps with the 128-byte swizzle, which is the chunk ^ (row & 7) layout
// the compute side reads), the block's K scales (a 4 x 128-byte tile, swizzled
// the same way) and the page's V scales for all heads (one contiguous piece),
// against ~220 instructions per page and lane for the cp.async form. Tiles
// always hold all 16 rows: rows past the sequence's end are stale pool bytes,
// which for int8 are finite numbers; their scores are masked and their V scales
// are replaced by zero on the compute side.
template <int ASYM>
struct PoolInt8Tma {
    static constexpr bool kTma = true;
    // K 2 KB | V 2 KB | K scales 512 B | V scales (16 x heads) [| K zeros 512 B | V zeros]; stages
    // and the two swizzled 512-byte tiles stay 1024-byte aligned.
    static constexpr int STAGE_BYTES = ASYM ? 6144 : 5120;
    static constexpr int OFF_V = 2048, OFF_KS = 4096, OFF_VS = 4608, OFF_KZ = 5120, OFF_VZ = 5632;

    static __device__ __forceinline__ int issue(const DecodeParams& p, const TmaMaps& maps, int b,
                                                int h, const PageItem& it, uint32_t stage,
                                                uint32_t mbar, int lane, uint64_t pol) {
        if (__builtin_expect(!ASYM && it.vl == LS_PAGE && p.kv_merged, 1)) {
            // A full page of a sequence's interior, the case almost every page is: one test,
            // then three copies with nothing to decide.
            if (lane == 0) {
                mbar_expect_tx(mbar, 4096u + 512u + 16u * (uint32_t)p.heads * (uint32_t)sizeof(float));
                tma_load_5d(stage, &maps.kv, mbar, 0, h, 0, it.blk, 0, pol);
                tma_load_4d(stage + OFF_KS, &maps.ks, mbar, 0, 0, h, it.blk, pol);
                bulk_load(stage + OFF_VS, p.v_scale + it.blk * p.vs_b, 16u * p.heads * sizeof(float), mbar);
            }
            return LS_PAGE;
        }
        // Everything else: a last page (K from the residual, rows past the end), a page to skip,
        // asymmetric pools, pools the merged map cannot span.
        const bool from_res = p.k_res != nullptr && (it.last & 1) && it.valid > 0;
        if (from_res) {
            const int rr = p.res_rows[b];
            if ((rr < 0 || rr >= p.num_res_rows) && lane == 0) p.seg_range[2 * p.batch] = 1;
        }
        if (lane == 0) {
            if (it.valid == 0) {
                mbar_arrive(mbar);                     // nothing to load: the phase completes at once
            } else {
                const uint32_t vs_bytes = 16u * p.heads * sizeof(float);
                mbar_expect_tx(mbar, 2048u + (ASYM ? 2u : 1u) * vs_bytes +
                                         (from_res ? 0u : 2048u + (ASYM ? 1024u : 512u)));
                if (!from_res) {
                    tma_load_4d(stage + OFF_KS, &maps.ks, mbar, 0, 0, h, it.blk, pol);
                    if (ASYM) tma_load_4d(stage + OFF_KZ, &maps.kz, mbar, 0, 0, h, it.blk, pol);
                }
                if (!from_res && p.kv_merged) {
                    tma_load_5d(stage, &maps.kv, mbar, 0, h, 0, it.blk, 0, pol);     // both tiles, 4 KB
                } else {
                    if (!from_res) tma_load_4d(stage + p.k_off, &maps.k, mbar, 0, h, 0, it.blk, pol);
                    tma_load_4d(stage + (2048 - p.k_off), &maps.v, mbar, 0, h, 0, it.blk, pol);
                }
                bulk_load(stage + OFF_VS, p.v_scale + it.blk * p.vs_b, vs_bytes, mbar);
                if (ASYM) bulk_load(stage + OFF_VZ, p.v_zero + it.blk * p.vs_b, vs_bytes, mbar);
            }
        }
        return it.valid | (from_res ? 256 : 0);
    }
};

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "r"(addr));
    return r;
}
__device__ __forceinline__ float lds32f(uint32_t addr) {
    float r;
    asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(r) : "r"(addr));
    return r;
}

// Tensor-core state for INT8 pools.
//
// The MMA's k index is a free permutation as long as both operands agree, so
// for the int8 K page lane (g, t) takes dims 32t .. 32t+31 of rows g and g+8
// (two 16-byte shared loads per row) and k-step ks uses dims 32t + 4ks .. +3;
// the query fragments are built in the same order. For V the m index (output
// dim) is permuted instead: the tile's 16-byte chunk mt comes in through
// ldmatrix.trans on byte pairs, and output tile mt holds dims 16mt + 2g (rows g)
// and 16mt + 2g + 1 (rows g + 8).
template <int ASYM, bool TMA = false>
struct MmaInt8 {
    using Pool = typename std::conditional<TMA, PoolInt8Tma<ASYM>, PoolInt8<ASYM>>::type;
    static constexpr int kMinCtas = LS_INT8_CTAS;
    uint32_t qh[16];           // Q[row g][32t .. 32t+31] as half2 pairs (row g < n_rep, else 0)
    float o[9][4];             // O^T: tile mt < 8 = dims 16mt + 2g (regs 0,1) and +1 (regs 2,3), with V
                               // still carrying its conversion bias; tile 8 = sum of the weights per row
                               // (what the bias has to be taken off with at the end)
    float m[2], l[2];
    float zacc[2];             // asymmetric V: sum_t w * zero_t, added to every dim
    int b_, h_;
    uint32_t vs_off;           // byte offset of this lane's first V scale inside a stage (TMA layout)
    uint32_t oneq[4];          // half2(1, 1) four times over: the constant A operand of the MMA that sums
                               // the weights, held in registers (not re-made per page)

    __device__ __forceinline__ void begin(const DecodeParams& p, int b, int h, int lane) {
        b_ = b;
        h_ = h;
        m[0] = m[1] = neg_inf();
        l[0] = l[1] = 0.f;
        zacc[0] = zacc[1] = 0.f;
        vs_off = (uint32_t)(((lane >> 2) * p.heads + h) * 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            asm volatile("mov.b32 %0, 0x3C003C00;\n" : "=r"(oneq[i]));
        }
#pragma unroll
        for (int mt = 0; mt < 9; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[mt][i] = 0.f;
        const int g = lane >> 2, t = lane & 3;
        const __half* src = p.q + b * p.sq_b + h * p.sq_h + g * p.sq_m + 32 * t;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (g < p.n_rep) raw = *reinterpret_cast<const uint4*>(src + 8 * i);
            qh[4 * i] = raw.x;
            qh[4 * i + 1] = raw.y;
            qh[4 * i + 2] = raw.z;
            qh[4 * i + 3] = raw.w;
        }
    }

    // A full page of a sequence's interior (all 16 tokens, K in the pool) takes the
    // straight-line form: no masks, no residual branch. Anything else -- a last page, a
    // page to skip -- takes the general one.
    // `scratch`: 320 bytes of the warp's own shared memory that nothing else uses while pages
    // are being walked (the start of its merge rows).
    __device__ __forceinline__ void compute(const DecodeParams& p, uint32_t stage, int meta,
                                            int lane, uint32_t scratch) {
        if (meta == LS_PAGE) compute_page<true>(p, stage, meta, lane, scratch);
        else compute_page<false>(p, stage, meta, lane, scratch);
    }

    template <bool FULL>
    __device__ __forceinline__ void compute_page(const DecodeParams& p, uint32_t stage, int meta,
                                                 int lane, uint32_t scratch) {
        const int valid = FULL ? LS_PAGE : (meta & 255);
        const int g = lane >> 2, t = lane & 3;
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        if (!FULL && (meta & 256)) {
            // Last page: K is exact fp16 in the residual, read from global memory in
            // the same dim order as the int8 path (dims 32t .. 32t+31 of rows g, g+8:
            // 64 contiguous bytes per row); the query needs no scale. Rows past
            // `valid` may hold anything: their scores are masked below.
            int rr = p.res_rows[b_];
            if (rr < 0 || rr >= p.num_res_rows) rr = 0;           // flagged by the load side
            const __half* kr = p.k_res + (long long)rr * p.sr_r + h_ * p.sr_h + 32 * t;
            const uint4* r0 = reinterpret_cast<const uint4*>(kr + g * p.sr_p);
            const uint4* r1 = reinterpret_cast<const uint4*>(kr + (g + 8) * p.sr_p);
            uint4 ka[4], kb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                ka[j] = __ldcg(r0 + j);
                kb[j] = __ldcg(r1 + j);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                mma_16816(s, ka[j].x, kb[j].x, ka[j].y, kb[j].y, qh[4 * j], qh[4 * j + 1]);
                mma_16816(s, ka[j].z, kb[j].z, ka[j].w, kb[j].w, qh[4 * j + 2], qh[4 * j + 3]);
            }
        } else {
            // q' = q * fp16(k_scale) in half precision (the query stays in half2 registers:
            // sixteen fewer than its fp32 form), in this lane's dim order. The page's 128
            // scales are rounded to fp16 once per warp -- each lane converts four of them
            // and leaves them in the warp's scratch, rows of 32 dims 80 bytes apart so that
            // the four rows the lanes then read together lie in different banks -- instead
            // of every lane converting the 32 it needs (eight lanes need the same 32).
            uint32_t qk[8][2];
            float zq = 0.f;
            if (!ASYM) {
                {
                    const int row = lane >> 3, ch = lane & 7;
                    const uint4 sc = lds128(stage + Pool::OFF_KS + ((uint32_t)(8 * row + (ch ^ row)) << 4));
                    const uint32_t h0 = pack_half2(__uint_as_float(sc.x), __uint_as_float(sc.y));
                    const uint32_t h1 = pack_half2(__uint_as_float(sc.z), __uint_as_float(sc.w));
                    asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(scratch + row * 80 + ch * 8), "r"(h0),
                                 "r"(h1)
                                 : "memory");
                }
                __syncwarp();
                // (No second barrier: the loads below feed this page's first MMAs, which no lane
                // executes before every lane's operands are there; the next page's stores come later.)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 hs = lds128(scratch + t * 80 + j * 16);
                    qk[2 * j][0] = hmul2_u32(qh[4 * j], hs.x);
                    qk[2 * j][1] = hmul2_u32(qh[4 * j + 1], hs.y);
                    qk[2 * j + 1][0] = hmul2_u32(qh[4 * j + 2], hs.z);
                    qk[2 * j + 1][1] = hmul2_u32(qh[4 * j + 3], hs.w);
                }
            } else {
                // Asymmetric pools: every lane converts the scales it needs and, in the same
                // pass over its dims, sums q . k_zero (registers are too few for the shared form).
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t slot = (uint32_t)(8 * t + (i ^ t)) << 4;   // see PoolInt8::issue
                    const uint4 sc = lds128(stage + Pool::OFF_KS + slot);
                    qk[i][0] = hmul2_u32(qh[2 * i], pack_half2(__uint_as_float(sc.x), __uint_as_float(sc.y)));
                    qk[i][1] = hmul2_u32(qh[2 * i + 1], pack_half2(__uint_as_float(sc.z), __uint_as_float(sc.w)));
                    const uint4 z = lds128(stage + Pool::OFF_KZ + slot);
                    const float2 qa = __half22float2(*reinterpret_cast<const __half2*>(&qh[2 * i]));
                    const float2 qb = __half22float2(*reinterpret_cast<const __half2*>(&qh[2 * i + 1]));
                    zq = fmaf(qa.x, __uint_as_float(z.x), zq);
                    zq = fmaf(qa.y, __uint_as_float(z.y), zq);
                    zq = fmaf(qb.x, __uint_as_float(z.z), zq);
                    zq = fmaf(qb.y, __uint_as_float(z.w), zq);
                }
            }
            const uint32_t kt = TMA ? stage + p.k_off : stage;              // the K tile
            const uint32_t r0 = kt + g * 128, r1 = kt + (g + 8) * 128;
            uint4 w0[2], w1[2];
            w0[0] = lds128(r0 + (((2 * t) ^ g) << 4));
            w0[1] = lds128(r0 + (((2 * t + 1) ^ g) << 4));
            w1[0] = lds128(r1 + (((2 * t) ^ g) << 4));
            w1[1] = lds128(r1 + (((2 * t + 1) ^ g) << 4));
            const uint32_t* k0 = reinterpret_cast<const uint32_t*>(w0);
            const uint32_t* k1 = reinterpret_cast<const uint32_t*>(w1);
            // int8 x -> fp16 exactly: 0x6400 | (x ^ 0x80) is 1024 + (x + 128), minus 1152.
            // (Leaving the bias in and taking it off with a second MMA against a constant was
            // measured too: eight more tensor-core instructions per page cost more, under the
            // power cap, than the thirty-two half2 subtractions they replace.)
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t x0 = k0[ks] ^ 0x80808080u, x1 = k1[ks] ^ 0x80808080u;
                uint32_t a0, a1, a2, a3;
                bytes4_to_half2x2(x0, a0, a2);
                bytes4_to_half2x2(x1, a1, a3);
                mma_16816(s, a0, a1, a2, a3, qk[ks][0], qk[ks][1]);
            }
            if (ASYM) {
                // + q . k_zero: the same for every token of the page, per row.
                zq += __shfl_xor_sync(LS_FULL_MASK, zq, 1);
                zq += __shfl_xor_sync(LS_FULL_MASK, zq, 2);      // lanes (g, *) hold row g's sum
                const float z0 = __shfl_sync(LS_FULL_MASK, zq, (2 * t) * 4);
                const float z1 = __shfl_sync(LS_FULL_MASK, zq, (2 * t + 1) * 4);
                s[0] += z0; s[1] += z1; s[2] += z0; s[3] += z1;
            }
        }
        if (FULL) {
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] *= p.scale_log2;
        } else {
            mask_and_scale(s, valid, p.scale_log2, lane);
        }
        float a0, a1;
        softmax_update(s, m, l, o, a0, a1);
        // V's per-token scale rides on the weight (zero for rows past the end:
        // the scale slots of those rows were zero-filled).
        float vs0, vs1;
        if (TMA) {
            // The page's scales for all heads, [token][head]; tokens past the end are stale.
            vs0 = lds32f(stage + Pool::OFF_VS + vs_off);
            vs1 = lds32f(stage + Pool::OFF_VS + vs_off + 32 * p.heads);
            if (!FULL && g >= valid) vs0 = 0.f;
            if (!FULL && g + 8 >= valid) vs1 = 0.f;
        } else {
            vs0 = lds32f(stage + Pool::OFF_VS + g * 4);
            vs1 = lds32f(stage + Pool::OFF_VS + (g + 8) * 4);
        }
        if (ASYM) {
            float vz0, vz1;
            if (TMA) {
                vz0 = (g < valid) ? lds32f(stage + Pool::OFF_VZ + vs_off) : 0.f;
                vz1 = (g + 8 < valid) ? lds32f(stage + Pool::OFF_VZ + vs_off + 32 * p.heads) : 0.f;
            } else {
                vz0 = lds32f(stage + Pool::OFF_VZ + g * 4);
                vz1 = lds32f(stage + Pool::OFF_VZ + (g + 8) * 4);
            }
            zacc[0] = zacc[0] * a0 + (s[0] * vz0 + s[2] * vz1);
            zacc[1] = zacc[1] * a1 + (s[1] * vz0 + s[3] * vz1);
        }
        const uint32_t pb0 = movmatrix_trans(pack_half2(s[0] * vs0, s[1] * vs0));
        const uint32_t pb1 = movmatrix_trans(pack_half2(s[2] * vs1, s[3] * vs1));

        // V^T fragments straight out of the int8 tile: ldmatrix.trans on 16-bit units
        // (a unit = two neighbouring dims of one token) hands lane (g, t) the unit g of
        // tokens 2t and 2t+1 in one register -- bytes [T.dA, T.dB, T+1.dA, T+1.dB] -- which
        // two byte permutes turn into the half2 pairs (tokens 2t, 2t+1) of dims A and B.
        // Matrices of one ldmatrix.x4: tokens 0-7 / 8-15 of 16-byte chunk 2q, then of 2q+1;
        // output tile mt = chunk mt holds dims 16mt + 2g (rows g) and 16mt + 2g + 1 (rows g+8).
        // As for K, the values enter as 1152 + v; tile 8 accumulates the weights alone
        // (A = all ones) and finish() takes 1152 x that off every dim.
        const uint32_t magic = 0x64646464u;
        mma_16816(o[8], oneq[0], oneq[1], oneq[2], oneq[3], pb0, pb1);
        const int mi = lane >> 3;                                   // the matrix this lane addresses
        const int vrow = (lane & 7) + (mi & 1) * 8;
        const uint32_t vaddr = stage + (TMA ? 2048 - p.k_off : Pool::OFF_V) + vrow * 128;
        const int sw = vrow & 7, hi = mi >> 1;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t m0, m1, m2, m3;
            ldmatrix_x4_trans(vaddr + (((2 * q + hi) ^ sw) << 4), m0, m1, m2, m3);
            m0 ^= 0x80808080u; m1 ^= 0x80808080u; m2 ^= 0x80808080u; m3 ^= 0x80808080u;
            mma_16816(o[2 * q], prmt(m0, magic, 0x4240u), prmt(m0, magic, 0x4341u), prmt(m1, magic, 0x4240u),
                      prmt(m1, magic, 0x4341u), pb0, pb1);
            mma_16816(o[2 * q + 1], prmt(m2, magic, 0x4240u), prmt(m2, magic, 0x4341u),
                      prmt(m3, magic, 0x4240u), prmt(m3, magic, 0x4341u), pb0, pb1);
        }
    }

    __device__ __forceinline__ void finish(float* mo, float* mm, float* ml, int n_rep, int lane) {
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l[0] += __shfl_xor_sync(LS_FULL_MASK, l[0], off);
            l[1] += __shfl_xor_sync(LS_FULL_MASK, l[1], off);
            if (ASYM) {
                zacc[0] += __shfl_xor_sync(LS_FULL_MASK, zacc[0], off);
                zacc[1] += __shfl_xor_sync(LS_FULL_MASK, zacc[1], off);
            }
        }
        const int g = lane >> 2, t = lane & 3;
        const int r0 = 2 * t, r1 = r0 + 1;
        // minus the conversion bias of V (tile 8 = the weights' sum), plus the zero points' share
        const float z0 = (ASYM ? zacc[0] : 0.f) - 1152.f * o[8][0];
        const float z1 = (ASYM ? zacc[1] : 0.f) - 1152.f * o[8][1];
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            const int d = 16 * mt + 2 * g;
            if (r0 < n_rep) {
                mo[r0 * kMergeStride + d] = o[mt][0] + z0;
                mo[r0 * kMergeStride + d + 1] = o[mt][2] + z0;
            }
            if (r1 < n_rep) {
                mo[r1 * kMergeStride + d] = o[mt][1] + z1;
                mo[r1 * kMergeStride + d + 1] = o[mt][3] + z1;
            }
        }
        if (g == 0) {
            if (r0 < n_rep) { mm[r0] = m[0]; ml[r0] = l[0]; }
            if (r1 < n_rep) { mm[r1] = m[1]; ml[r1] = l[1]; }
        }
    }
};

// ---------------------------------------------------------------------------
// Merge of a sequence's partials:
//   out = sum_s acc_s 2^(m_s - M) / max(sum_s l_s 2^(m_s - M), 1e-20),
// the reference combine (kernels/gqa/paged_decode.py:421-471, torch form
// :689-706) with m held in the log2 domain. Called by the 4 warps of a CTA:
// warp w takes query rows w, w + 4; lane s holds partial s's (m, l) and weight,
// and the 32 lanes cover the 128 dims as float4, so a row of one partial is one
// coalesced 512-byte load and the loads of a row's partials are independent
// (issued back to back, not one L2 round trip after another). Loads bypass L1
// because other CTAs of the same launch may have written the partials.
__device__ __forceinline__ void merge_partials(const float* part_acc, const float* part_m,
                                               const float* part_l, int first, int count,
                                               __half* out, int heads, int n_rep, int b, int h,
                                               int tid, long long so_b, long long so_h,
                                               long long so_m) {
    constexpr int kBatch = 8;                                // partial rows loaded per round
    const int warp = tid >> 5, lane = tid & 31;
    const long long step = (long long)heads * kRP;           // rows between partials
    // Warp w merges rows w and w + 4 together, so both rows' loads are in flight at once.
    const int r0 = warp, r1 = warp + kWarps;
    const bool has0 = r0 < n_rep, has1 = r1 < n_rep;
    if (!has0) return;
    const long long base0 = ((long long)first * heads + h) * kRP + r0;
    const long long base1 = base0 + kWarps;
    const float4* src0 = reinterpret_cast<const float4*>(part_acc + base0 * LS_HEAD_DIM) + lane;
    const float4* src1 = src0 + kWarps * (LS_HEAD_DIM / 4);
    const long long pstep = step * (LS_HEAD_DIM / 4);

    // One round trip for everything the usual case needs: lane s's (m, l) of partial s,
    // and the accumulator rows of the first kBatch partials (which do not depend on m).
    float pm0 = neg_inf(), pm1 = neg_inf(), pl0 = 0.f, pl1 = 0.f;
    if (lane < count) {
        pm0 = __ldcg(part_m + base0 + lane * step);
        pl0 = __ldcg(part_l + base0 + lane * step);
        if (has1) {
            pm1 = __ldcg(part_m + base1 + lane * step);
            pl1 = __ldcg(part_l + base1 + lane * step);
        }
    }
    float4 v0[kBatch], v1[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
        const bool ok = j < count;
        v0[j] = ok ? __ldcg(src0 + j * pstep) : make_float4(0.f, 0.f, 0.f, 0.f);
        v1[j] = (ok && has1) ? __ldcg(src1 + j * pstep) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float mg0 = pm0, mg1 = pm1;
    for (int s = lane + 32; s < count; s += 32) {            // more than 32 partials: rare
        mg0 = fmaxf(mg0, __ldcg(part_m + base0 + s * step));
        if (has1) mg1 = fmaxf(mg1, __ldcg(part_m + base1 + s * step));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        mg0 = fmaxf(mg0, __shfl_xor_sync(LS_FULL_MASK, mg0, off));
        mg1 = fmaxf(mg1, __shfl_xor_sync(LS_FULL_MASK, mg1, off));
    }
    const float ms0 = (mg0 == neg_inf()) ? 0.f : mg0;
    const float ms1 = (mg1 == neg_inf()) ? 0.f : mg1;
    float ls0 = 0.f, ls1 = 0.f;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    for (int s0 = 0; s0 < count; s0 += 32) {
        const int s = s0 + lane;
        float w0 = 0.f, w1 = 0.f;
        if (s < count) {
            if (s0 > 0) {
                pm0 = __ldcg(part_m + base0 + s * step);
                pl0 = __ldcg(part_l + base0 + s * step);
                if (has1) {
                    pm1 = __ldcg(part_m + base1 + s * step);
                    pl1 = __ldcg(part_l + base1 + s * step);
                }
            }
            w0 = ex2(pm0 - ms0);
            ls0 += w0 * pl0;
            if (has1) {
                w1 = ex2(pm1 - ms1);
                ls1 += w1 * pl1;
            }
        }
        const int n = min(32, count - s0);
        for (int j0 = 0; j0 < n; j0 += kBatch) {
            if (s0 + j0 > 0) {                               // the first batch is already here
#pragma unroll
                for (int j = 0; j < kBatch; ++j) {
                    const bool ok = j0 + j < n;
                    v0[j] = ok ? __ldcg(src0 + (s0 + j0 + j) * pstep) : make_float4(0.f, 0.f, 0.f, 0.f);
                    v1[j] = (ok && has1) ? __ldcg(src1 + (s0 + j0 + j) * pstep)
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                const float x0 = __shfl_sync(LS_FULL_MASK, w0, (j0 + j) & 31);
                const float x1 = __shfl_sync(LS_FULL_MASK, w1, (j0 + j) & 31);
                a0.x += x0 * v0[j].x; a0.y += x0 * v0[j].y; a0.z += x0 * v0[j].z; a0.w += x0 * v0[j].w;
                a1.x += x1 * v1[j].x; a1.y += x1 * v1[j].y; a1.z += x1 * v1[j].z; a1.w += x1 * v1[j].w;
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        ls0 += __shfl_xor_sync(LS_FULL_MASK, ls0, off);
        ls1 += __shfl_xor_sync(LS_FULL_MASK, ls1, off);
    }
    const float i0 = 1.f / fmaxf(ls0, 1e-20f), i1 = 1.f / fmaxf(ls1, 1e-20f);
    uint2 packed;
    packed.x = pack_half2(a0.x * i0, a0.y * i0);
    packed.y = pack_half2(a0.z * i0, a0.w * i0);
    *reinterpret_cast<uint2*>(out + b * so_b + h * so_h + r0 * so_m + lane * 4) = packed;
    if (has1) {
        packed.x = pack_half2(a1.x * i1, a1.y * i1);
        packed.y = pack_half2(a1.z * i1, a1.w * i1);
        *reinterpret_cast<uint2*>(out + b * so_b + h * so_h + r1 * so_m + lane * 4) = packed;
    }
}

// ---------------------------------------------------------------------------
template <class State, int MODE, int STAGES>
__global__ void __launch_bounds__(kThreads, State::kMinCtas)
decode_kernel(const DecodeParams p, const __grid_constant__ TmaMaps maps) {
    extern __shared__ __align__(1024) unsigned char smem[];
    using Pool = typename State::Pool;
    constexpr int STAGE_BYTES = Pool::STAGE_BYTES;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk_id = blockIdx.x, h = blockIdx.y;

    // After the ring: one mbarrier per (warp, stage) for the TMA-loading variants.
    const uint32_t mbar0 = smem_u32(smem + kWarps * STAGES * STAGE_BYTES) + warp * STAGES * 8;
    float* merge_o = reinterpret_cast<float*>(smem + kWarps * STAGES * STAGE_BYTES + kWarps * STAGES * 8);
    float* merge_m = merge_o + kWarps * p.n_rep * kMergeStride;
    float* merge_l = merge_m + kWarps * kRP;
    int* scan = reinterpret_cast<int*>(merge_l + kWarps * kRP);   // [kWarps]
    int* flag = scan + kWarps;                                    // [1]
    int* cum = flag + 1;                                          // [batch + 1]

    // Programmatic dependent launch: let the next kernel of the stream be
    // scheduled as this one drains, and -- when this launch was itself made
    // with the attribute -- do the part of the prologue that reads only
    // seq_lens and block_tables while the previous kernel is still finishing.
    // Without the attribute both instructions are no-ops.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (Pool::kTma) {
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < STAGES; ++s) mbar_init(mbar0 + 8 * s, 1);
            mbar_init_fence();
        }
        __syncwarp();
    }
    const int total = build_prefix<MODE, kThreads>(p, cum, scan);
    const int chunk = chunk_size(p, total);
    const int g0 = chunk_id * chunk;
    const int g1 = min(total, g0 + chunk);
    const bool has_work = g0 < total;
    const int b0 = has_work ? find_seq(cum, p.batch, g0) : 0;
    const uint32_t ring = smem_u32(smem + warp * (STAGES * STAGE_BYTES));
    const uint32_t warp_scratch = smem_u32(merge_o + warp * p.n_rep * kMergeStride);   // free while pages are walked

    // Load side. The dense walk needs nothing the previous kernel may have
    // written; the sparse walk reads the selection, which it usually did write.
    // With LS_EARLY_PAGES the first pages are requested before the dependency
    // wait as well: a decode step's predecessor (the KV append) writes only the
    // newest token, which lies in its sequence's last page, so every other page
    // is immutable; a warp waits before it requests a last page. An INT8 cache also
    // rewrites the page before the last one (its K page is quantised, by a kernel that
    // precedes the append, in the step after it filled up), so there the wait comes
    // before either of a sequence's two last pages.
    PageWindow<MODE> win;
    const bool early = MODE == LS_MODE_DENSE && p.early != 0;
    if (MODE == LS_MODE_DENSE && has_work)
        win.begin(p, cursor_begin<kWarps>(cum, p.batch, b0, g0, g1, warp), h, lane);
    bool waited = false;
    auto dep_wait = [&]() {
        if (!waited) asm volatile("griddepcontrol.wait;\n" ::: "memory");
        waited = true;
    };
    // KV pages are read once per step: evict-first keeps tables, lengths, queries and
    // partials in L2.
    const uint64_t pol = l2_policy_evict_first();
    // What the load side knows about the page in each ring slot (valid tokens, flags):
    // warp-uniform, indexed by compile-time slot numbers only, so it lives in registers.
    int slot_meta[STAGES];
#pragma unroll
    for (int s = 0; s < STAGES; ++s) slot_meta[s] = 0;
    auto issue = [&](int slot) {
        PageItem item;
        int lb;
        if (win.next(p, cum, h, warp, lane, item, lb)) {
            if (item.vl != LS_PAGE && item.last) dep_wait();
            int mt;
            if constexpr (Pool::kTma)
                mt = Pool::issue(p, maps, lb, h, item, ring + slot * STAGE_BYTES, mbar0 + 8 * slot, lane, pol);
            else
                mt = Pool::issue(p, lb, h, item, ring + slot * STAGE_BYTES, lane, pol);
#pragma unroll
            for (int q = 0; q < STAGES; ++q) slot_meta[q] = slot == q ? mt : slot_meta[q];
        }
        if (!Pool::kTma) cp_async_commit();
    };
    auto issue_first = [&]() {                               // STAGES - 1 pages ahead
#pragma unroll 1
        for (int s = 0; s < STAGES - 1; ++s) issue(s);       // one copy of the code, not STAGES - 1
    };
    if (early && has_work) issue_first();
    dep_wait();

    if (chunk_id == 0 && h == 0) write_seg_ranges<kThreads>(p, cum, chunk);
    if (chunk_id == 0 && p.out != nullptr) {
        // Sequences with nothing to attend produce zeros (nobody else writes them).
        for (int b = 0; b < p.batch; ++b) {
            if (cum[b + 1] != cum[b]) continue;
            for (int i = tid; i < p.n_rep * LS_HEAD_DIM; i += kThreads)
                p.out[b * p.so_b + h * p.so_h + (i >> 7) * p.so_m + (i & 127)] = __float2half_rn(0.f);
        }
    }
    if (!has_work) return;
    if (MODE != LS_MODE_DENSE)
        win.begin(p, cursor_begin<kWarps>(cum, p.batch, b0, g0, g1, warp), h, lane);
    if (!early) issue_first();

    // Compute side: segment by segment. One page step: wait for the slot, refill the slot
    // consumed one page ago, compute. (A copy of the step per ring slot, with the slot a
    // compile-time constant, was measured: the larger code cost more than the immediates saved.)
    State st;
    int stage = 0;         // ring slot of the page being consumed
    uint32_t phase = 0;    // parity of that slot's mbarrier phase (TMA variants)
    int b = b0;
    int first_u = g0 - cum[b0];
    for (int guard = 0; guard <= p.batch; ++guard) {
        const int hi = min(g1, cum[b + 1]) - cum[b];
        st.begin(p, b, h, lane);
        for (int u = first_u + warp; u < hi; u += kWarps) {
            {
                const uint32_t bar = mbar0 + 8 * stage;
                if constexpr (Pool::kTma) {
                    if (!mbar_wait_bounded(bar, phase, kMbarSpinLimit)) {
                        if (lane == 0) p.seg_range[2 * p.batch] = 2;
                    }
                } else {
                    cp_async_wait<STAGES - 2>();
                }
                __syncwarp();
                int meta_now = slot_meta[0];
#pragma unroll
                for (int q = 1; q < STAGES; ++q) meta_now = stage == q ? slot_meta[q] : meta_now;
                issue(stage == 0 ? STAGES - 1 : stage - 1);          // the slot consumed one page ago
#ifndef LS_LOADS_ONLY
                st.compute(p, ring + stage * STAGE_BYTES, meta_now, lane, warp_scratch);
#else
                (void)meta_now;                          // build flag: pages land, nothing is computed
#endif
            }
            if (++stage == STAGES) {
                stage = 0;
                phase ^= 1u;
            }
        }
        st.finish(merge_o + warp * p.n_rep * kMergeStride, merge_m + warp * kRP,
                  merge_l + warp * kRP, p.n_rep, lane);
        __syncthreads();
        const int slot = chunk_id + b;
        {
            // CTA merge: thread = one of the 128 dims, all rows.
            float* pa = p.part_acc + ((long long)slot * p.heads + h) * kRP * LS_HEAD_DIM;
            float* pm = p.part_m + ((long long)slot * p.heads + h) * kRP;
            float* pl = p.part_l + ((long long)slot * p.heads + h) * kRP;
            for (int r = 0; r < p.n_rep; ++r) {
                float mg = neg_inf();
#pragma unroll
                for (int w = 0; w < kWarps; ++w) mg = fmaxf(mg, merge_m[w * kRP + r]);
                const float ms = (mg == neg_inf()) ? 0.f : mg;
                float lsum = 0.f;
                float wgt[kWarps];
#pragma unroll
                for (int w = 0; w < kWarps; ++w) {
                    wgt[w] = ex2(merge_m[w * kRP + r] - ms);
                    lsum += wgt[w] * merge_l[w * kRP + r];
                }
                for (int d = tid; d < LS_HEAD_DIM; d += kThreads) {
                    float a = 0.f;
#pragma unroll
                    for (int w = 0; w < kWarps; ++w)
                        a += wgt[w] * merge_o[(w * p.n_rep + r) * kMergeStride + d];
                    pa[r * LS_HEAD_DIM + d] = a;
                }
                if (tid == 0) {
                    pm[r] = mg;
                    pl[r] = lsum;
                }
            }
        }
        if (p.out != nullptr) {
            // Whoever brings a sequence's last partial merges them all. Arrival is
            // counted with one atomic per segment; nobody waits for anybody.
            const int c_lo = cum[b] / chunk, c_hi = (cum[b + 1] - 1) / chunk;
            const int nseg = c_hi - c_lo + 1;
            int* counter = p.seg_range + 2 * p.batch + 2 + b * p.heads + h;
            __syncthreads();                                  // the CTA's partial is written
            if (tid == 0) {
                int last = 1;
                if (nseg > 1) {
                    // Release the CTA's partial (ordered before this by the barrier) and
                    // acquire the others' in one atomic; the merge reads them from L2.
                    int seen;
                    asm volatile("atom.add.acq_rel.gpu.s32 %0, [%1], 1;\n" : "=r"(seen) : "l"(counter) : "memory");
                    last = seen == nseg - 1;
                    if (last) *counter = 0;                  // ready for the next launch
                }
                *flag = last;
            }
            __syncthreads();
            if (*flag) {
                merge_partials(p.part_acc, p.part_m, p.part_l, c_lo + b, nseg, p.out, p.heads,
                               p.n_rep, b, h, tid, p.so_b, p.so_h, p.so_m);
            }
        }
        if (cum[b + 1] >= g1) break;
        __syncthreads();
        ++b;
        while (b < p.batch - 1 && cum[b + 1] == cum[b]) ++b;
        first_u = 0;
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------
// Stand-alone merge (see merge_partials). grid (B, H), thread = head dim.
__global__ void __launch_bounds__(LS_HEAD_DIM)
merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_m,
             const float* __restrict__ part_l, const int* __restrict__ seg_range,
             __half* __restrict__ out, int heads, int n_rep, long long so_b, long long so_h,
             long long so_m) {
    const int b = blockIdx.x, h = blockIdx.y;
    merge_partials(part_acc, part_m, part_l, seg_range[2 * b], seg_range[2 * b + 1], out, heads,
                   n_rep, b, h, threadIdx.x, so_b, so_h, so_m);
}

// ---------------------------------------------------------------------------
static int validate_common(const DecodeParams& p) {
    if (!p.q || !p.k_pool || !p.v_pool || !p.block_tables || !p.seq_lens || !p.part_acc ||
        !p.part_m || !p.part_l || !p.seg_range)
        return LS_ERR_NULL_POINTER;
    if (p.batch <= 0 || p.heads <= 0 || p.n_rep <= 0 || p.max_pages <= 0 || p.num_chunks <= 0 ||
        p.num_blocks <= 0 || p.min_chunk <= 0)
        return LS_ERR_BAD_SHAPE;
    if (p.batch > LS_MAX_BATCH || p.heads > 65535) return LS_ERR_TOO_LARGE;
    if (p.n_rep > kRP) return LS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(p.q) & 15) || (p.sq_b % 8) || (p.sq_h % 8) || (p.sq_m % 8))
        return LS_ERR_MISALIGNED;
    if (p.out && ((reinterpret_cast<uintptr_t>(p.out) & 7) || (p.so_b % 4) || (p.so_h % 4) || (p.so_m % 4)))
        return LS_ERR_MISALIGNED;
    return LS_OK;
}

template <class State, int MODE, int STAGES>
static int launch_decode(const DecodeParams& p, cudaStream_t stream, bool programmatic = false,
                         const TmaMaps* maps = nullptr) {
    static const TmaMaps no_maps = {};
    const size_t smem = (size_t)kWarps * STAGES * State::Pool::STAGE_BYTES + kWarps * STAGES * 8 +
                        sizeof(float) * ((size_t)kWarps * p.n_rep * kMergeStride + 2 * kWarps * kRP) +
                        sizeof(int) * ((size_t)kWarps + 1 + p.batch + 1);
    auto kern = decode_kernel<State, MODE, STAGES>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.num_chunks, p.heads);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, kern, p, maps ? *maps : no_maps);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

}  // namespace ls

// ---------------------------------------------------------------------------
// Tensor maps for the TMA-loading INT8 kernel, encoded per call (a host-side
// table fill, no device work). The driver entry point is looked up through the
// runtime, so the library does not link libcuda.
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// A 4-d map with the 128-byte swizzle: dims innermost first, strides (bytes) of dims 1..3.
bool encode_4d(CUtensorMap* map, CUtensorMapDataType type, const void* base, const cuuint64_t (&dims)[4],
               const cuuint64_t (&strides)[3], const cuuint32_t (&box)[4],
               CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint32_t ones[4] = {1, 1, 1, 1};
    return fn(map, type, 4, const_cast<void*>(base), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// True if the symmetric INT8 pools have the layout the TMA kernel takes and the maps were built.
bool build_int8_maps(ls::DecodeParams& p, ls::TmaMaps* maps, bool merge_kv) {
    // pools [blocks][16][H][128] int8 (any strides that are 16-byte multiples, innermost unit);
    // K scales [blocks][H][128] fp32; V scales [blocks][16][H] fp32 with tokens and heads dense.
    if (p.heads > 8 || p.vs_h != 1 || p.vs_p != p.heads || (p.vs_b % 4) ||
        (reinterpret_cast<uintptr_t>(p.v_scale) & 15))
        return false;
    const cuuint64_t nb = (cuuint64_t)p.num_blocks, H = (cuuint64_t)p.heads;
    const cuuint64_t pool_dims[4] = {128, H, 16, nb};
    const cuuint64_t pool_strides[3] = {(cuuint64_t)p.sk_h, (cuuint64_t)p.sk_p, (cuuint64_t)p.sk_b};
    const cuuint32_t pool_box[4] = {128, 1, 16, 1};
    const cuuint64_t ks_dims[4] = {32, 4, H, nb};
    const cuuint64_t ks_strides[3] = {128, (cuuint64_t)p.ks_h * 4, (cuuint64_t)p.ks_b * 4};
    const cuuint32_t ks_box[4] = {32, 4, 1, 1};
    if (p.k_zero != nullptr &&
        ((reinterpret_cast<uintptr_t>(p.v_zero) & 15) ||
         !encode_4d(&maps->kz, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.k_zero, ks_dims, ks_strides, ks_box)))
        return false;                                  // zero points share the scales' layout
    if (!(encode_4d(&maps->k, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.k_pool, pool_dims, pool_strides, pool_box) &&
          encode_4d(&maps->v, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.v_pool, pool_dims, pool_strides, pool_box) &&
          encode_4d(&maps->ks, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.k_scale, ks_dims, ks_strides, ks_box)))
        return false;
    // The two pools seen as ONE tensor [2][blocks][16][H][128] whose outermost stride is the
    // distance between them: a page's K and V tiles then arrive by a single copy, in address
    // order (k_off says where the K tile lands). Any two allocations qualify as long as the
    // distance is a multiple of 16 bytes below the 2^40 a tensor map's strides may hold.
    p.kv_merged = 0;
    p.k_off = 0;
    const uintptr_t ka = reinterpret_cast<uintptr_t>(p.k_pool), va = reinterpret_cast<uintptr_t>(p.v_pool);
    const uintptr_t lo = ka < va ? ka : va, dist = ka < va ? va - ka : ka - va;
    if (merge_kv && dist != 0 && (dist % 16) == 0 && dist < (uintptr_t(1) << 40)) {
        EncodeTiledFn fn = encode_tiled_fn();
        const cuuint64_t dims5[5] = {128, H, 16, nb, 2};
        const cuuint64_t strides5[4] = {(cuuint64_t)p.sk_h, (cuuint64_t)p.sk_p, (cuuint64_t)p.sk_b, (cuuint64_t)dist};
        const cuuint32_t box5[5] = {128, 1, 16, 1, 2};
        const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
        if (fn != nullptr &&
            fn(&maps->kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, reinterpret_cast<void*>(lo), dims5, strides5, box5, ones,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
            p.kv_merged = 1;
            p.k_off = ka < va ? 0 : 2048;
        }
    }
    return true;
}

// fp16 pools [blocks][16][H][128] (strides in elements): tiles of 16 tokens x 64 dims.
bool build_fp16_maps(const ls::DecodeParams& p, ls::TmaMaps* maps) {
    const cuuint64_t dims[4] = {128, (cuuint64_t)p.heads, 16, (cuuint64_t)p.num_blocks};
    const cuuint64_t strides[3] = {(cuuint64_t)p.sk_h * 2, (cuuint64_t)p.sk_p * 2, (cuuint64_t)p.sk_b * 2};
    const cuuint32_t box[4] = {64, 1, 16, 1};
    if (p.sk_h <= 0 || p.sk_p <= 0 || p.sk_b <= 0) return false;
    // A row is 256 bytes and arrives as two tile rows: with 256-byte L2 promotion the
    // first half's request brings the second half into L2 as well.
    const CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    return encode_4d(&maps->k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.k_pool, dims, strides, box, promo) &&
           encode_4d(&maps->v, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.v_pool, dims, strides, box, promo);
}

}  // namespace

using ls::DecodeParams;

static int check_pool_fp16(const DecodeParams& p) {
    if ((reinterpret_cast<uintptr_t>(p.k_pool) & 15) || (reinterpret_cast<uintptr_t>(p.v_pool) & 15) ||
        (p.sk_b % 8) || (p.sk_p % 8) || (p.sk_h % 8))
        return LS_ERR_MISALIGNED;
    return LS_OK;
}

extern "C" {

int ls_decode_slots(int batch, int num_chunks) { return batch + num_chunks; }

static int decode_fp16_impl(const void* q, const void* k_new, const void* v_new, int64_t sn_b, int64_t sn_h,
                            int64_t svn_b, int64_t svn_h, const void* k_pool, const void* v_pool,
                            const int32_t* block_tables, const int32_t* seq_lens, float* part_acc,
                            float* part_m, float* part_l, int32_t* seg_range, void* out, int batch,
                            int kv_heads, int n_rep, int head_dim, int page, int max_pages, int num_blocks,
                            int num_chunks, int min_chunk, int flags, int64_t sq_b, int64_t sq_h, int64_t sq_m,
                            int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t so_b, int64_t so_h, int64_t so_m,
                            float softmax_scale, void* stream) {
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    DecodeParams p = {};
    p.q = static_cast<const __half*>(q);
    p.k_new = static_cast<const __half*>(k_new);
    p.v_new = static_cast<const __half*>(v_new);
    p.sn_b = sn_b; p.sn_h = sn_h; p.svn_b = svn_b; p.svn_h = svn_h;
    p.k_pool = k_pool;
    p.v_pool = v_pool;
    p.block_tables = block_tables;
    p.seq_lens = seq_lens;
    p.part_acc = part_acc;
    p.part_m = part_m;
    p.part_l = part_l;
    p.seg_range = seg_range;
    p.out = static_cast<__half*>(out);
    p.so_b = so_b; p.so_h = so_h; p.so_m = so_m;
    p.batch = batch;
    p.heads = kv_heads;
    p.n_rep = n_rep;
    p.max_pages = max_pages;
    p.num_blocks = num_blocks;
    p.num_chunks = num_chunks;
    p.min_chunk = min_chunk;
    p.sq_b = sq_b; p.sq_h = sq_h; p.sq_m = sq_m;
    p.sk_b = sk_b; p.sk_p = sk_p; p.sk_h = sk_h;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    int rc = ls::validate_common(p);
    if (rc) return rc;
    rc = check_pool_fp16(p);
    if (rc) return rc;
    if (k_new != nullptr &&
        ((reinterpret_cast<uintptr_t>(k_new) & 15) || (reinterpret_cast<uintptr_t>(v_new) & 15) || (sn_b % 8) ||
         (sn_h % 8) || (svn_b % 8) || (svn_h % 8)))
        return LS_ERR_MISALIGNED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool pdl = (flags & LS_LAUNCH_PROGRAMMATIC) != 0;
    const int impl = flags & 0xff;
    if (flags & ~(0xff | LS_LAUNCH_PROGRAMMATIC | LS_LOAD_CP_ASYNC | LS_LOAD_TMA | LS_EARLY_PAGES))
        return LS_ERR_UNSUPPORTED;
    p.early = (flags & LS_EARLY_PAGES) != 0;
    ls::TmaMaps maps;
    // The append rides on the per-lane copies only: a TMA tile always comes whole out of the pool.
    if (impl == LS_IMPL_MMA && (flags & LS_LOAD_TMA) && k_new == nullptr && build_fp16_maps(p, &maps))
        return ls::launch_decode<ls::MmaFp16Tma, LS_MODE_DENSE, ls::kStages>(p, s, pdl, &maps);
    if (impl == LS_IMPL_SIMT) {
        if (n_rep <= 6)
            rc = ls::launch_decode<ls::SimtFp16<6>, LS_MODE_DENSE, ls::kStages>(p, s, pdl);
        else
            rc = ls::launch_decode<ls::SimtFp16<8>, LS_MODE_DENSE, ls::kStages>(p, s, pdl);
    } else if (impl == LS_IMPL_MMA) {
        rc = ls::launch_decode<ls::MmaFp16, LS_MODE_DENSE, ls::kStages>(p, s, pdl);
    } else {
        return LS_ERR_UNSUPPORTED;
    }
    return rc;
}

int ls_paged_decode_fp16(const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, float* part_acc,
                         float* part_m, float* part_l, int32_t* seg_range, void* out, int batch,
                         int kv_heads, int n_rep, int head_dim, int page, int max_pages,
                         int num_blocks, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h,
                         int64_t so_b, int64_t so_h, int64_t so_m, float softmax_scale,
                         void* stream) {
    return decode_fp16_impl(q, nullptr, nullptr, 0, 0, 0, 0, k_pool, v_pool, block_tables, seq_lens, part_acc,
                            part_m, part_l, seg_range, out, batch, kv_heads, n_rep, head_dim, page, max_pages,
                            num_blocks, num_chunks, min_chunk, flags, sq_b, sq_h, sq_m, sk_b, sk_p, sk_h, so_b,
                            so_h, so_m, softmax_scale, stream);
}

int ls_paged_decode_append_fp16(const void* q, const void* k_new, const void* v_new, void* k_pool,
                                void* v_pool, const int32_t* block_tables, const int32_t* seq_lens,
                                float* part_acc, float* part_m, float* part_l, int32_t* seg_range, void* out,
                                int batch, int kv_heads, int n_rep, int head_dim, int page, int max_pages,
                                int num_blocks, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                                int64_t sq_h, int64_t sq_m, int64_t sn_b, int64_t sn_h, int64_t svn_b,
                                int64_t svn_h, int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t so_b,
                                int64_t so_h, int64_t so_m, float softmax_scale, void* stream) {
    if (!k_new || !v_new) return LS_ERR_NULL_POINTER;
    return decode_fp16_impl(q, k_new, v_new, sn_b, sn_h, svn_b, svn_h, k_pool, v_pool, block_tables, seq_lens,
                            part_acc, part_m, part_l, seg_range, out, batch, kv_heads, n_rep, head_dim, page,
                            max_pages, num_blocks, num_chunks, min_chunk, flags, sq_b, sq_h, sq_m, sk_b, sk_p,
                            sk_h, so_b, so_h, so_m, softmax_scale, stream);
}

int ls_paged_sparse_fp16(const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, const int32_t* sel,
                         float ratio, int recent, float* part_acc, float* part_m, float* part_l,
                         int32_t* seg_range, void* out, int batch, int kv_heads, int n_rep,
                         int head_dim, int page, int max_pages, int num_blocks, int num_sel,
                         int num_chunks, int min_chunk, int flags, int64_t sq_b, int64_t sq_h,
                         int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t sl_b, int64_t sl_h,
                         int64_t so_b, int64_t so_h, int64_t so_m, float softmax_scale,
                         void* stream) {
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (!sel) return LS_ERR_NULL_POINTER;
    if (num_sel <= 0) return LS_ERR_BAD_SHAPE;
    DecodeParams p = {};
    p.q = static_cast<const __half*>(q);
    p.k_pool = k_pool;
    p.v_pool = v_pool;
    p.block_tables = block_tables;
    p.seq_lens = seq_lens;
    p.sel = sel;
    p.ratio = ratio;
    p.recent = recent;
    p.num_sel = num_sel;
    p.sl_b = sl_b; p.sl_h = sl_h;
    p.part_acc = part_acc;
    p.part_m = part_m;
    p.part_l = part_l;
    p.seg_range = seg_range;
    p.out = static_cast<__half*>(out);
    p.so_b = so_b; p.so_h = so_h; p.so_m = so_m;
    p.batch = batch;
    p.heads = kv_heads;
    p.n_rep = n_rep;
    p.max_pages = max_pages;
    p.num_blocks = num_blocks;
    p.num_chunks = num_chunks;
    p.min_chunk = min_chunk;
    p.sq_b = sq_b; p.sq_h = sq_h; p.sq_m = sq_m;
    p.sk_b = sk_b; p.sk_p = sk_p; p.sk_h = sk_h;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    int rc = ls::validate_common(p);
    if (rc) return rc;
    rc = check_pool_fp16(p);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (flags & ~(LS_LAUNCH_PROGRAMMATIC | LS_LOAD_CP_ASYNC | LS_LOAD_TMA)) return LS_ERR_UNSUPPORTED;
    const bool pdl = (flags & LS_LAUNCH_PROGRAMMATIC) != 0;
    ls::TmaMaps maps;
    if ((flags & LS_LOAD_TMA) && build_fp16_maps(p, &maps))
        return ls::launch_decode<ls::MmaFp16Tma, LS_MODE_SPARSE, ls::kStages>(p, s, pdl, &maps);
    return ls::launch_decode<ls::MmaFp16, LS_MODE_SPARSE, ls::kStages>(p, s, pdl);
}

static int int8_decode_impl(const int32_t* sel, float ratio, int recent, int num_sel, int64_t sl_b,
                            int64_t sl_h, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, const float* k_scale,
                         const float* v_scale, const float* k_zero, const float* v_zero,
                         const void* k_res, const int32_t* res_rows, float* part_acc, float* part_m,
                         float* part_l, int32_t* seg_range, void* out, int batch, int kv_heads,
                         int n_rep, int head_dim, int page, int max_pages, int num_blocks,
                         int num_res_rows, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t ks_b,
                         int64_t ks_h,
                         int64_t vs_b, int64_t vs_p, int64_t vs_h, int64_t sr_r, int64_t sr_p,
                         int64_t sr_h, int64_t so_b, int64_t so_h, int64_t so_m, float softmax_scale,
                         void* stream) {
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (!k_scale || !v_scale) return LS_ERR_NULL_POINTER;
    if ((k_zero == nullptr) != (v_zero == nullptr)) return LS_ERR_NULL_POINTER;
    if ((k_res == nullptr) != (res_rows == nullptr)) return LS_ERR_NULL_POINTER;
    DecodeParams p = {};
    p.sel = sel;
    p.ratio = ratio;
    p.recent = recent;
    p.num_sel = num_sel;
    p.sl_b = sl_b; p.sl_h = sl_h;
    p.q = static_cast<const __half*>(q);
    p.k_pool = k_pool;
    p.v_pool = v_pool;
    p.block_tables = block_tables;
    p.seq_lens = seq_lens;
    p.k_scale = k_scale;
    p.v_scale = v_scale;
    p.k_zero = k_zero;
    p.v_zero = v_zero;
    p.k_res = static_cast<const __half*>(k_res);
    p.res_rows = res_rows;
    p.num_res_rows = k_res ? num_res_rows : 1;
    if (k_res && num_res_rows <= 0) return LS_ERR_BAD_SHAPE;
    p.part_acc = part_acc;
    p.part_m = part_m;
    p.part_l = part_l;
    p.seg_range = seg_range;
    p.out = static_cast<__half*>(out);
    p.so_b = so_b; p.so_h = so_h; p.so_m = so_m;
    p.batch = batch;
    p.heads = kv_heads;
    p.n_rep = n_rep;
    p.max_pages = max_pages;
    p.num_blocks = num_blocks;
    p.num_chunks = num_chunks;
    p.min_chunk = min_chunk;
    p.sq_b = sq_b; p.sq_h = sq_h; p.sq_m = sq_m;
    p.sk_b = sk_b; p.sk_p = sk_p; p.sk_h = sk_h;
    p.ks_b = ks_b; p.ks_h = ks_h;
    p.vs_b = vs_b; p.vs_p = vs_p; p.vs_h = vs_h;
    p.sr_r = sr_r; p.sr_p = sr_p; p.sr_h = sr_h;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    int rc = ls::validate_common(p);
    if (rc) return rc;
    // 16-byte rows for the int8 pools, the K scales / zero points and the residual.
    if ((reinterpret_cast<uintptr_t>(k_pool) & 15) || (reinterpret_cast<uintptr_t>(v_pool) & 15) ||
        (sk_b % 16) || (sk_p % 16) || (sk_h % 16))
        return LS_ERR_MISALIGNED;
    if ((reinterpret_cast<uintptr_t>(k_scale) & 15) || (ks_b % 4) || (ks_h % 4)) return LS_ERR_MISALIGNED;
    if (k_zero && (reinterpret_cast<uintptr_t>(k_zero) & 15)) return LS_ERR_MISALIGNED;
    if (k_res && ((reinterpret_cast<uintptr_t>(k_res) & 15) || (sr_r % 8) || (sr_p % 8) || (sr_h % 8)))
        return LS_ERR_MISALIGNED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (flags & ~(LS_LAUNCH_PROGRAMMATIC | LS_LOAD_CP_ASYNC | LS_LOAD_TMA | LS_EARLY_PAGES | LS_LOAD_TMA_SPLIT_KV))
        return LS_ERR_UNSUPPORTED;
    const bool pdl = (flags & LS_LAUNCH_PROGRAMMATIC) != 0;
    p.early = (flags & LS_EARLY_PAGES) != 0;
    ls::TmaMaps maps;
    const bool tma = !(flags & LS_LOAD_CP_ASYNC) && build_int8_maps(p, &maps, !(flags & LS_LOAD_TMA_SPLIT_KV));
    if (sel != nullptr) {
        // Attention over the selected pages only (symmetric pools).
        if (k_zero) return LS_ERR_UNSUPPORTED;
        p.early = 0;
        if (tma)
            return ls::launch_decode<ls::MmaInt8<0, true>, LS_MODE_SPARSE, LS_INT8_TMA_STAGES>(p, s, pdl, &maps);
        return ls::launch_decode<ls::MmaInt8<0>, LS_MODE_SPARSE, LS_INT8_STAGES>(p, s, pdl);
    }
    if (k_zero && tma)
        rc = ls::launch_decode<ls::MmaInt8<1, true>, LS_MODE_DENSE, LS_INT8_TMA_STAGES_ASYM>(p, s, pdl, &maps);
    else if (k_zero)
        rc = ls::launch_decode<ls::MmaInt8<1>, LS_MODE_DENSE, LS_INT8_STAGES_ASYM>(p, s, pdl);
    else if (tma)
        rc = ls::launch_decode<ls::MmaInt8<0, true>, LS_MODE_DENSE, LS_INT8_TMA_STAGES>(p, s, pdl, &maps);
    else
        rc = ls::launch_decode<ls::MmaInt8<0>, LS_MODE_DENSE, LS_INT8_STAGES>(p, s, pdl);
    return rc;
}

int ls_paged_decode_int8(const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, const float* k_scale,
                         const float* v_scale, const float* k_zero, const float* v_zero,
                         const void* k_res, const int32_t* res_rows, float* part_acc, float* part_m,
                         float* part_l, int32_t* seg_range, void* out, int batch, int kv_heads,
                         int n_rep, int head_dim, int page, int max_pages, int num_blocks,
                         int num_res_rows, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t ks_b,
                         int64_t ks_h,
                         int64_t vs_b, int64_t vs_p, int64_t vs_h, int64_t sr_r, int64_t sr_p,
                         int64_t sr_h, int64_t so_b, int64_t so_h, int64_t so_m, float softmax_scale,
                         void* stream) {
    return int8_decode_impl(nullptr, 0.f, 0, 0, 0, 0, q, k_pool, v_pool, block_tables, seq_lens, k_scale, v_scale, k_zero, v_zero, k_res, res_rows, part_acc, part_m, part_l, seg_range, out, batch, kv_heads, n_rep, head_dim, page, max_pages, num_blocks, num_res_rows, num_chunks, min_chunk, flags, sq_b, sq_h, sq_m, sk_b, sk_p, sk_h, ks_b, ks_h, vs_b, vs_p, vs_h, sr_r, sr_p, sr_h, so_b, so_h, so_m, softmax_scale, stream);
}

int ls_paged_sparse_int8(const int32_t* sel, float ratio, int recent, int num_sel, int64_t sl_b,
                         int64_t sl_h, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* seq_lens, const float* k_scale,
                         const float* v_scale, const float* k_zero, const float* v_zero,
                         const void* k_res, const int32_t* res_rows, float* part_acc, float* part_m,
                         float* part_l, int32_t* seg_range, void* out, int batch, int kv_heads,
                         int n_rep, int head_dim, int page, int max_pages, int num_blocks,
                         int num_res_rows, int num_chunks, int min_chunk, int flags, int64_t sq_b,
                         int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t ks_b,
                         int64_t ks_h,
                         int64_t vs_b, int64_t vs_p, int64_t vs_h, int64_t sr_r, int64_t sr_p,
                         int64_t sr_h, int64_t so_b, int64_t so_h, int64_t so_m, float softmax_scale,
                         void* stream) {
    if (!sel) return LS_ERR_NULL_POINTER;
    if (num_sel <= 0) return LS_ERR_BAD_SHAPE;
    return int8_decode_impl(sel, ratio, recent, num_sel, sl_b, sl_h, q, k_pool, v_pool, block_tables, seq_lens, k_scale, v_scale, k_zero, v_zero, k_res, res_rows, part_acc, part_m, part_l, seg_range, out, batch, kv_heads, n_rep, head_dim, page, max_pages, num_blocks, num_res_rows, num_chunks, min_chunk, flags, sq_b, sq_h, sq_m, sk_b, sk_p, sk_h, ks_b, ks_h, vs_b, vs_p, vs_h, sr_r, sr_p, sr_h, so_b, so_h, so_m, softmax_scale, stream);
}

int ls_combine(const float* part_acc, const float* part_m, const float* part_l,
               const int32_t* seg_range, void* out, int batch, int kv_heads, int n_rep,
               int64_t so_b, int64_t so_h, int64_t so_m, void* stream) {
    if (!part_acc || !part_m || !part_l || !seg_range || !out) return LS_ERR_NULL_POINTER;
    if (batch <= 0 || kv_heads <= 0 || n_rep <= 0 || n_rep > ls::kRP) return LS_ERR_BAD_SHAPE;
    if (kv_heads > 65535) return LS_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(out) & 7) || (so_b % 4) || (so_h % 4) || (so_m % 4))
        return LS_ERR_MISALIGNED;
    ls::merge_kernel<<<dim3(batch, kv_heads), LS_HEAD_DIM, 0, static_cast<cudaStream_t>(stream)>>>(
        part_acc, part_m, part_l, seg_range, static_cast<__half*>(out), kv_heads, n_rep, so_b, so_h,
        so_m);
    return (int)cudaGetLastError();
}

}  // extern "C"

// ---------------------------------------------------------------------------
// ls_paged_decode_fp16_noalloc: dense fp16 decode for callers that cannot
// allocate device memory.
//
// Who that is: a host that embeds this library from C, Go or Java through its
// foreign-function interface and owns no device allocator of its own; or a
// serving process whose device memory was handed out in full at start-up (KV
// pools sized to fill the GPU), where a later cudaMalloc can simply fail, and
// would in any case stall every stream of the device while it runs. Such a
// caller can still provide its inputs and its output, but has nowhere to put
// the partial softmax states the split-KV kernel needs between its CTAs.
//
// This entry point keeps that scratch inside the library image instead: a
// fixed array in device global memory, LS_NOALLOC_SCRATCH_BYTES (about 4.1 MiB)
// on every GPU that loads the library, held until the process exits. The price
// of a fixed array is a fixed ceiling:
//     batch <= LS_NOALLOC_MAX_BATCH (64)   and
//     (batch + num_chunks) * kv_heads <= LS_NOALLOC_MAX_ROWS (1024);
// anything larger is refused with LS_ERR_NOALLOC_LIMIT and nothing is launched.
//
// The array's name is only a handle on the host side, not a device address.
// The first call on each device (with that device current) asks the runtime
// for the address with cudaGetSymbolAddress and remembers it; make that first
// call before any stream capture begins. Every later call does no set-up.
//
// All calls on a device share the one array, and it keeps whatever the last
// call left in it. The bookkeeping part (slot ranges, error flag, arrival
// counters, whose positions depend on the batch size) is therefore cleared on
// the caller's stream at the start of every call; the partial states need no
// clearing because every slot that is read has been written by the same
// launch. Two calls whose kernels overlap on the GPU (different streams, no
// ordering between them) race on the array: keep calls on one device ordered.
//
// No cudaMalloc, cudaFree or allocating library routine is called here.
#define LS_NOALLOC_MAX_BATCH 64
#define LS_NOALLOC_MAX_ROWS 1024
#define LS_ERR_NOALLOC_LIMIT (-8)

namespace ls {

constexpr size_t kNaAccBytes = (size_t)LS_NOALLOC_MAX_ROWS * kRP * LS_HEAD_DIM * sizeof(float);
constexpr size_t kNaMlBytes = (size_t)LS_NOALLOC_MAX_ROWS * kRP * sizeof(float);
constexpr size_t kNaSegInts = 2 * LS_NOALLOC_MAX_BATCH + 2 + LS_NOALLOC_MAX_ROWS;
constexpr size_t kNaSegBytes = (kNaSegInts * sizeof(int) + 255) / 256 * 256;
constexpr size_t kNaTotalBytes = kNaAccBytes + 2 * kNaMlBytes + kNaSegBytes;

static_assert(kNaTotalBytes == 4264704, "keep LS_NOALLOC_SCRATCH_BYTES in the header in step");

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaTotalBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_noalloc_mutex;
static unsigned char* g_noalloc_base[kMaxDevices] = {};

// Device address of the scratch array on the current device (looked up once).
static int noalloc_scratch_base(unsigned char** base) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return LS_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_base[dev] == nullptr) {
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (ptr == nullptr) return LS_ERR_NULL_POINTER;
        g_noalloc_base[dev] = ptr;
    }
    *base = g_noalloc_base[dev];
    return LS_OK;
}

}  // namespace ls

extern "C" {

int ls_paged_decode_fp16_noalloc(const void* q, const void* k_pool, const void* v_pool,
                                 const int32_t* block_tables, const int32_t* seq_lens, void* out,
                                 int batch, int kv_heads, int n_rep, int head_dim, int page,
                                 int max_pages, int num_blocks, int num_chunks, int min_chunk,
                                 int64_t sq_b, int64_t sq_h, int64_t sq_m, int64_t sk_b, int64_t sk_p,
                                 int64_t sk_h, int64_t so_b, int64_t so_h, int64_t so_m,
                                 float softmax_scale, void* stream) {
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (!out) return LS_ERR_NULL_POINTER;
    if (batch <= 0 || kv_heads <= 0 || num_chunks <= 0) return LS_ERR_BAD_SHAPE;
    if (batch > LS_NOALLOC_MAX_BATCH ||
        ((long long)batch + num_chunks) * kv_heads > LS_NOALLOC_MAX_ROWS)
        return LS_ERR_NOALLOC_LIMIT;
    unsigned char* base = nullptr;
    int rc = ls::noalloc_scratch_base(&base);
    if (rc) return rc;
    DecodeParams p = {};
    p.q = static_cast<const __half*>(q);
    p.k_pool = k_pool;
    p.v_pool = v_pool;
    p.block_tables = block_tables;
    p.seq_lens = seq_lens;
    p.part_acc = reinterpret_cast<float*>(base);
    p.part_m = reinterpret_cast<float*>(base + ls::kNaAccBytes);
    p.part_l = reinterpret_cast<float*>(base + ls::kNaAccBytes + ls::kNaMlBytes);
    p.seg_range = reinterpret_cast<int*>(base + ls::kNaAccBytes + 2 * ls::kNaMlBytes);
    p.out = static_cast<__half*>(out);
    p.so_b = so_b; p.so_h = so_h; p.so_m = so_m;
    p.batch = batch;
    p.heads = kv_heads;
    p.n_rep = n_rep;
    p.max_pages = max_pages;
    p.num_blocks = num_blocks;
    p.num_chunks = num_chunks;
    p.min_chunk = min_chunk;
    p.sq_b = sq_b; p.sq_h = sq_h; p.sq_m = sq_m;
    p.sk_b = sk_b; p.sk_p = sk_p; p.sk_h = sk_h;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    rc = ls::validate_common(p);
    if (rc) return rc;
    rc = check_pool_fp16(p);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Bookkeeping of the previous call (possibly another batch size) must not
    // be mistaken for this call's arrival counters.
    const size_t seg_bytes = sizeof(int) * (2 * (size_t)batch + 2 + (size_t)batch * kv_heads);
    cudaError_t e = cudaMemsetAsync(p.seg_range, 0, seg_bytes, s);
    if (e != cudaSuccess) return (int)e;
    return ls::launch_decode<ls::MmaFp16, LS_MODE_DENSE, ls::kStages>(p, s);
}

}  // extern "C"
