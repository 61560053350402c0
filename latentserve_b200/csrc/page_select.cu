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
// lane l sums channels 4l..4l+3 left to right starting from 0, then an xor
// butterfly over lanes with offsets 16, 8, 4, 2, 1 -- so that scores, and with
// them the selected indices, are reproducible bit for bit on a CPU.
#include "ls_common.cuh"

namespace ls {

constexpr int kIndexWarps = 4;
constexpr int kPagesPerWarp = 4;

__device__ __forceinline__ void unpack4h(uint2 raw, float (&f)[4]) {
    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
    const float2 a = __half22float2(h2[0]), b = __half22float2(h2[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// Bounds of all 8 (padded) query rows for one page. Every row keeps the order
// "lane sum of 4 channels from 0, then xor butterfly 16, 8, 4, 2, 1"; the rows'
// butterflies are interleaved so their shuffle latencies overlap.
__device__ __forceinline__ void bound_rows(const float (&q)[8][4], const float (&lo)[4],
                                           const float (&hi)[4], float (&s)[8]) {
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            t = __fadd_rn(t, fmaxf(__fmul_rn(q[r][j], lo[j]), __fmul_rn(q[r][j], hi[j])));
        s[r] = t;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int r = 0; r < 8; ++r) s[r] = __fadd_rn(s[r], __shfl_xor_sync(LS_FULL_MASK, s[r], off));
}

// grid (ceil(max_pages / 16), H, B), block 128. PER_HEAD = 0: scores [B,H,P];
// PER_HEAD = 1: heads [B,H,R,P].
template <int PER_HEAD>
__global__ void __launch_bounds__(kIndexWarps * 32)
page_index_kernel(const __half* __restrict__ q, const __half* __restrict__ kmin,
                  const __half* __restrict__ kmax, const int* __restrict__ block_tables,
                  const int* __restrict__ seq_lens, float* __restrict__ out, int n_rep,
                  int max_pages, int table_stride, int num_blocks, int recent, long long sq_b,
                  long long sq_h, long long sq_m, long long sb_b, long long sb_h, long long ss_b,
                  long long ss_h, long long ss_r) {
    const int b = blockIdx.z, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = (blockIdx.x * kIndexWarps + warp) * kPagesPerWarp;
    if (first >= max_pages) return;
    const int L = max(seq_lens[b], 0);
    const int np = min((L + LS_PAGE - 1) / LS_PAGE, table_stride);

    float qf[8][4];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        if (r < n_rep) {
            unpack4h(*reinterpret_cast<const uint2*>(q + b * sq_b + h * sq_h + r * sq_m + lane * 4),
                     qf[r]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) qf[r][j] = 0.f;
        }
    }

    // Issue every page's loads before any arithmetic.
    uint2 lo_raw[kPagesPerWarp], hi_raw[kPagesPerWarp];
    bool scored[kPagesPerWarp];
#pragma unroll
    for (int k = 0; k < kPagesPerWarp; ++k) {
        const int p = first + k;
        bool need = p < max_pages && p < np;
        if (!PER_HEAD) need = need && !(p == 0 || p >= np - recent);
        int blk = 0;
        if (need) {
            blk = block_tables[(long long)b * table_stride + p];
            need = blk >= 0 && blk < num_blocks;
        }
        scored[k] = need;
        lo_raw[k] = make_uint2(0, 0);
        hi_raw[k] = make_uint2(0, 0);
        if (need) {
            lo_raw[k] = *reinterpret_cast<const uint2*>(kmin + blk * sb_b + h * sb_h + lane * 4);
            hi_raw[k] = *reinterpret_cast<const uint2*>(kmax + blk * sb_b + h * sb_h + lane * 4);
        }
    }
#pragma unroll
    for (int k = 0; k < kPagesPerWarp; ++k) {
        const int p = first + k;
        if (p >= max_pages) break;
        float lo[4], hi[4];
        unpack4h(lo_raw[k], lo);
        unpack4h(hi_raw[k], hi);
        float s[8];
        if (scored[k]) {                                // warp-uniform
            bound_rows(qf, lo, hi, s);
        } else {
#pragma unroll
            for (int r = 0; r < 8; ++r) s[r] = 0.f;
        }
        if (PER_HEAD) {
            // Pages past the end get a finite 0: their token count of zero
            // removes them downstream, and a stale NaN here would not.
#pragma unroll
            for (int r = 0; r < 8; ++r)
                if (r < n_rep && lane == 0) out[b * ss_b + h * ss_h + r * ss_r + p] = s[r];
        } else {
            float best;
            if (p >= np) {
                best = neg_inf();                       // past the end: never chosen
            } else if (p == 0 || p >= np - recent) {
                best = pos_inf();                       // sink and recent pages: always kept
            } else {
                best = neg_inf();
                if (scored[k]) {
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        if (r < n_rep) best = fmaxf(best, s[r]);
                }
            }
            if (lane == 0) out[b * ss_b + h * ss_h + p] = best;
        }
    }
}

// Monotone map from fp32 to uint32: a > b as floats <=> key(a) > key(b).
// -0 is folded onto +0 first so the two compare equal, as they do as floats.
__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t u = __float_as_uint(x + 0.f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kTopkThreads = 128;
constexpr int kTopkPerThread = 2;
constexpr int kTopkTile = kTopkThreads * kTopkPerThread;

// Rank by counting: rank(i) = #{j : s_j > s_i} + #{j < i : s_j == s_i}. The
// entry of rank r < k lands at sel[r], which is the stable descending order.
// grid (ceil(n / 256), B*H); a thread ranks two candidates (i and i + 128 of
// the CTA's 256-entry tile) against the whole row held in shared memory, so
// each 16-byte broadcast read of four keys serves eight comparisons.
// O(n^2 / grid) compares; n is a block-table width (2048 pages at 32K context).
__global__ void __launch_bounds__(kTopkThreads)
topk_pages_kernel(const float* __restrict__ scores, int* __restrict__ sel, int n, int k, int heads,
                  long long ss_b, long long ss_h, long long sl_b, long long sl_h) {
    extern __shared__ uint32_t keys[];
    const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
    const float* row = scores + b * ss_b + h * ss_h;
    const int n4 = (n + 3) & ~3;
    for (int j = threadIdx.x; j < n4; j += kTopkThreads) keys[j] = j < n ? order_key(row[j]) : 0u;
    __syncthreads();
    const int tile_lo = blockIdx.x * kTopkTile, tile_hi = min(n4, tile_lo + kTopkTile);
    const int i0 = tile_lo + threadIdx.x, i1 = i0 + kTopkThreads;
    const uint32_t m0 = i0 < n ? keys[i0] : 0xffffffffu;
    const uint32_t m1 = i1 < n ? keys[i1] : 0xffffffffu;
    int rank0 = 0, rank1 = 0;
    const uint4* k4 = reinterpret_cast<const uint4*>(keys);
    // Entries before this CTA's tile precede every candidate of the tile: ties count.
#pragma unroll 4
    for (int j = 0; j < tile_lo / 4; ++j) {
        const uint4 v = k4[j];
        rank0 += (v.x >= m0) + (v.y >= m0) + (v.z >= m0) + (v.w >= m0);
        rank1 += (v.x >= m1) + (v.y >= m1) + (v.z >= m1) + (v.w >= m1);
    }
    for (int j = tile_lo; j < tile_hi; ++j) {
        const uint32_t v = keys[j];
        rank0 += (v > m0) || (v == m0 && j < i0);
        rank1 += (v > m1) || (v == m1 && j < i1);
    }
#pragma unroll 4
    for (int j = tile_hi / 4; j < n4 / 4; ++j) {
        const uint4 v = k4[j];
        rank0 += (v.x > m0) + (v.y > m0) + (v.z > m0) + (v.w > m0);
        rank1 += (v.x > m1) + (v.y > m1) + (v.z > m1) + (v.w > m1);
    }
    // Padding keys (0) never outrank a real entry: key(x) >= 1 for every
    // float except NaN patterns with the sign bit set, which sort last.
    if (i0 < n && rank0 < k) sel[b * sl_b + h * sl_h + rank0] = i0;
    if (i1 < n && rank1 < k) sel[b * sl_b + h * sl_h + rank1] = i1;
}

}  // namespace ls

extern "C" {

static int launch_index(int per_head, const void* q, const void* kmin, const void* kmax,
                        const int32_t* block_tables, const int32_t* seq_lens, float* out, int batch,
                        int kv_heads, int n_rep, int head_dim, int page, int max_pages,
                        int table_stride, int num_blocks, int recent, int64_t sq_b, int64_t sq_h,
                        int64_t sq_m, int64_t sb_b, int64_t sb_h, int64_t ss_b, int64_t ss_h,
                        int64_t ss_r, void* stream) {
    if (!q || !kmin || !kmax || !block_tables || !seq_lens || !out) return LS_ERR_NULL_POINTER;
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (batch <= 0 || kv_heads <= 0 || n_rep <= 0 || max_pages <= 0 || table_stride < max_pages ||
        num_blocks <= 0)
        return LS_ERR_BAD_SHAPE;
    if (n_rep > 8) return LS_ERR_UNSUPPORTED;
    if (batch > 65535 || kv_heads > 65535) return LS_ERR_TOO_LARGE;
    if ((sq_b % 4) || (sq_h % 4) || (sq_m % 4) || (sb_b % 4) || (sb_h % 4)) return LS_ERR_MISALIGNED;
    if (((uintptr_t)q & 7) || ((uintptr_t)kmin & 7) || ((uintptr_t)kmax & 7)) return LS_ERR_MISALIGNED;
    const int per_cta = ls::kIndexWarps * ls::kPagesPerWarp;
    dim3 grid((max_pages + per_cta - 1) / per_cta, kv_heads, batch);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (per_head)
        ls::page_index_kernel<1><<<grid, ls::kIndexWarps * 32, 0, s>>>(
            static_cast<const __half*>(q), static_cast<const __half*>(kmin),
            static_cast<const __half*>(kmax), block_tables, seq_lens, out, n_rep, max_pages,
            table_stride, num_blocks, recent, sq_b, sq_h, sq_m, sb_b, sb_h, ss_b, ss_h, ss_r);
    else
        ls::page_index_kernel<0><<<grid, ls::kIndexWarps * 32, 0, s>>>(
            static_cast<const __half*>(q), static_cast<const __half*>(kmin),
            static_cast<const __half*>(kmax), block_tables, seq_lens, out, n_rep, max_pages,
            table_stride, num_blocks, recent, sq_b, sq_h, sq_m, sb_b, sb_h, ss_b, ss_h, ss_r);
    return (int)cudaGetLastError();
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
    const size_t smem = sizeof(uint32_t) * (size_t)((num_pages + 3) & ~3);
    if (smem > 200 * 1024 || (long long)batch * kv_heads > 65535) return LS_ERR_TOO_LARGE;
    if (((uintptr_t)scores & 3) || ((uintptr_t)sel & 3)) return LS_ERR_MISALIGNED;
    cudaError_t e = cudaFuncSetAttribute(ls::topk_pages_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((num_pages + ls::kTopkTile - 1) / ls::kTopkTile, batch * kv_heads);
    ls::topk_pages_kernel<<<grid, ls::kTopkThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        scores, sel, num_pages, k, kv_heads, ss_b, ss_h, sl_b, sl_h);
    return (int)cudaGetLastError();
}

}  // extern "C"
