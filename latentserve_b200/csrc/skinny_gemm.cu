// Decode-step projections: out[M, N] = f(x)[M, K] . W[N, K]^T for a batch of
// M <= 32 token rows, where W (fp16, row-major, K contiguous) is tens of MB and
// x is tens of KB. At these shapes the product is a stream of weights through
// HBM, so the kernel is built around that stream:
//
//   * Lane (g, t) of a warp takes 16 contiguous bytes of weight row g at
//     k = 32 c + 8 t: the B fragments of two mma.sync.m16n8k16 once the k index
//     is permuted (the MMA does not care in which order k is summed as long as
//     A uses the same order; A is read with the same 16-byte pattern). The
//     bytes travel by cp.async into a per-warp ring in shared memory -- each
//     lane's piece at the address that lane reads back, an asynchronous
//     register spill: no swizzle, no ldmatrix, no barrier -- six 2 KB chunks
//     deep, 192 KB in flight per SM.
//   * A tile is 32 rows of W (4 n-tiles) by a slice of K; the 8 warps of a CTA
//     take the slice's 32-wide k chunks round-robin, each keeping several chunks
//     of loads in flight, and add their accumulators through shared memory. A
//     warp's activation fragments (at most six chunks) are read, normalised and
//     kept in registers once: they are the same for every tile. The grid is sized
//     to what the device holds at once and a CTA walks several tiles, its warps'
//     rings already filling with the next tile's weights while the current one
//     is reduced.
//   * K is cut across CTAs (`splits`) where 32-row tiles alone would leave SMs
//     idle. Partials go to an fp32 scratch and the CTA that arrives last at a
//     tile's counter adds them in split order (deterministic), exactly as the
//     decode kernel merges its partials; nobody waits.
//   * The weight loads of the first chunks are issued BEFORE
//     griddepcontrol.wait: weights do not depend on the previous kernel, so with
//     programmatic dependent launch the stream of the next projection starts
//     while the previous kernel drains.
//
// Fused around the product, with the rounding sequence of the unfused model
// code (and of the reference's kernels/fused_elementwise.py:75-107):
//   PRO_NORM    x <- RMSNorm(x [+ residual]) * gamma, rounded to fp16 where HF
//               rounds; the CTA (0, 0) also stores x + residual for the next
//               residual add. Replaces a norm launch.
//   EPI_SWIGLU  W = [gate; up] stacked ([2 I, K]); a CTA takes 16 gate rows and
//               the 16 matching up rows and writes fp16(silu(gate)) * up
//               ([M, I]). Replaces the SiLU * up launch and the [M, 2 I] round trip.
//   bias        out += bias (QKV projection).
//   EPI_ROPE    the fused QKV projection of a decode step: a CTA takes 16 dims of a
//               head and the 16 dims 64 further on (the rotation partners), adds the
//               bias, rotates q and k heads by the position's cos / sin row, and
//               stores q to the query buffer and k, v to the fp16 cache pools at the
//               sequence's slot (+ the page's K bounds). Replaces the RoPE + append
//               launch and the [M, N] round trip, with the same roundings.
//   add_res     out = fp16(fp16(product) + residual): the residual add that follows
//               o_proj and down_proj. With sumsq_out the same epilogue leaves each
//               row's sum of squares over the tile's 32 columns, and the next
//               PRO_NORM projection takes those partials (sumsq_in) instead of
//               reading whole rows again for its statistics.
#include "ls_common.cuh"

namespace ls {

constexpr int kGemmThreads = 256;
constexpr int kGemmWarps = 8;
constexpr int kTileRows = 32;           // rows of W per CTA
enum { PRO_NONE = 0, PRO_NORM = 1 };
enum { EPI_NONE = 0, EPI_SWIGLU = 1, EPI_ROPE = 2 };

struct GemmParams {
    const __half* x;        // [M, K]
    const __half* res;      // [M, K] added to x before the norm, or null (PRO_NORM)
    const __half* gamma;    // [K] (PRO_NORM)
    __half* res_out;        // [M, K] <- x + res when res is given
    const float* sumsq_in;  // [64][sumsq_tiles] per-row partial sums of x^2, or null (PRO_NORM)
    const __half* w;        // [N, K]
    const __half* bias;     // [N] or null
    const __half* add_res;  // [M, N] added to the rounded product (EPI_NONE), or null
    float* sumsq_out;       // [64][tiles] <- per-row sums of out^2 over the tile's 32 columns, or null
    __half* out;            // [M, N], or [M, N / 2] with EPI_SWIGLU
    float* part;            // [tiles * splits][M_pad * 32] fp32, splits > 1
    int* counters;          // [tiles], zero before first use, left at zero
    int m, n, k, splits, sumsq_tiles;
    float eps;
    long long sx, sres, sres_out, sw, sadd, sout;
    // EPI_ROPE: heads of 128 in q, k, v order; cos / sin [max_pos][128] (halves duplicated).
    const __half* cos_t;
    const __half* sin_t;
    const long long* positions;   // [M]
    const long long* slots;       // [M] flat token slots of the pools
    __half* q_out;                // [M][hq * 128]
    __half* k_pool;               // [num_slots][hk][128]
    __half* v_pool;
    __half* kmin;                 // [num_blocks][hk][128] or null
    __half* kmax;
    int hq, hk;
    long long max_pos, num_slots, s_cos, sq_b, sp_t, sp_h, sb_b, sb_h;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p, uint64_t pol) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(pol));
    return v;
}

// Activations: L2 hits. A plain load, so the compiler keeps it behind the
// griddepcontrol.wait barrier and is free to batch independent ones.
__device__ __forceinline__ uint4 ldg_l2(const __half* p) {
    return __ldcg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ uint4 lds128g(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}

__device__ __forceinline__ void sts128g(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w));
}

__device__ __forceinline__ float round_h(float f) { return __half2float(__float2half_rn(f)); }

// s = fp16(fp32(x) + fp32(r)), eight at a time: the fp32 sum is rounded first, as
// in the separate residual + norm kernel (an fp16 add would round once and could
// differ on a tie).
__device__ __forceinline__ uint4 add8(uint4 a, uint4 b) {
    uint4 o;
    const __half2* ah = reinterpret_cast<const __half2*>(&a);
    const __half2* bh = reinterpret_cast<const __half2*>(&b);
    uint32_t* oo = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fa = __half22float2(ah[i]), fb = __half22float2(bh[i]);
        oo[i] = pack_half2(fa.x + fb.x, fa.y + fb.y);
    }
    return o;
}

// RMSNorm is x * inv_rms(row) * gamma, and the row factor commutes with the
// product: (x * inv * gamma) W^T = inv * ((x * gamma) W^T). So the A operand is
// fp16(x * gamma * 2^-8) -- available as soon as x is, without waiting for the
// row statistics -- and the epilogue multiplies the fp32 sums by inv * 2^8. The
// fixed 2^-8 keeps x * gamma inside fp16 for un-normalised activations up to
// 1.6e7 (a residual stream's outlier channels reach thousands); what it pushes
// into the subnormal range keeps an absolute error of 2^-25 * 2^8, below the
// rounding error of any element of ordinary size.
constexpr float kPreScale = 1.f / 256.f, kPostScale = 256.f;
// gamma * 2^-8, exact in fp16 for |gamma| >= 2^-6 (smaller weights keep an absolute error
// below 2^-17).
__device__ __forceinline__ uint4 prescale8(uint4 gamma) {
    uint4 o;
    const __half2* gh = reinterpret_cast<const __half2*>(&gamma);
    __half2* oh = reinterpret_cast<__half2*>(&o);
    const __half2 c = __floats2half2_rn(kPreScale, kPreScale);
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __hmul2(gh[i], c);
    return o;
}
// fp16(x * gamma'), eight at a time: one rounding of the exact product.
__device__ __forceinline__ uint4 scale8(uint4 s, uint4 gamma_scaled) {
    uint4 o;
    const __half2* sh = reinterpret_cast<const __half2*>(&s);
    const __half2* gh = reinterpret_cast<const __half2*>(&gamma_scaled);
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __hmul2(sh[i], gh[i]);
    return o;
}

__device__ __forceinline__ float sumsq8(uint4 v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        acc += f.x * f.x + f.y * f.y;
    }
    return acc;
}

// Halves between rows of the staged activations: the slice plus a pad that puts
// consecutive rows 64 bytes apart modulo 128, so the eight rows a quarter-warp
// reads (16 bytes per lane, four lanes per row) fall on distinct banks.
__host__ __device__ inline int a_stride_halves(int slice_k) {
    return slice_k + ((slice_k % 64 == 0) ? 32 : 0);
}

#ifndef LS_GEMM_CONTIG
#define LS_GEMM_CONTIG 1
#endif
constexpr int kRing = 6;                // chunks of W a warp keeps in flight (2 KB each)
constexpr int kMaxCpw = 6;              // chunks of a tile a warp may own (its A fragments stay in registers)

// MT = 16-row tiles of the batch (M <= 16 MT). grid (CTAs per split, splits): a
// CTA walks the tiles blockIdx.x, + gridDim.x, ... of its split.
template <int MT, int PRO, int EPI>
__global__ void __launch_bounds__(kGemmThreads, MT == 1 ? 2 : 1) skinny_gemm_kernel(const GemmParams p) {
    // [kGemmWarps][kRing][4][32] x 16 bytes: the warps' rings of W chunks, each lane's
    // 16 bytes where that lane will read them back (an asynchronous register spill, no
    // swizzle or warp barrier needed); then [kGemmWarps][ROWS][32] fp32 for the reduction.
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int ROWS = MT * 16;
    __shared__ float inv_rms[ROWS];
    __shared__ int is_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.y;
    const int chunks = p.k >> 5;
    const int per_split = (chunks + p.splits - 1) / p.splits;
    const int c_begin = split * per_split;
    const int c_end = min(chunks, c_begin + per_split);
    const uint32_t ring = smem_u32(smem_raw) + warp * (kRing * 2048) + lane * 16;
    float* red = reinterpret_cast<float*>(smem_raw + kGemmWarps * kRing * 2048);
    const int n_tiles = p.n / kTileRows;
#if LS_GEMM_CONTIG
    // Chunks of a tile's slice this warp takes: cpw <= kMaxCpw consecutive ones from
    // w_first, so the warp's back-to-back requests walk along each row of W.
    const int c_share = (c_end - c_begin + kGemmWarps - 1) / kGemmWarps;
    const int w_first = c_begin + warp * c_share;
    const int cpw = max(0, min(c_share, c_end - w_first));
    constexpr int kChunkStep = 1;
#else
    // Chunks of a tile's slice this warp takes: c_begin + warp + 8 i, i < cpw <= kMaxCpw.
    const int w_first = c_begin + warp;
    const int cpw = max(0, (c_end - c_begin - warp + kGemmWarps - 1) / kGemmWarps);
    constexpr int kChunkStep = kGemmWarps;
#endif
    const int my_tiles = (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int items = my_tiles * cpw;   // (tile, chunk) pairs this warp streams, tile-major

    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // Rows of W behind this lane's four B fragments, at the warp's first chunk of tile 0.
    const __half* wrow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = (EPI == EPI_SWIGLU)
                            ? (i < 2 ? 0 : (p.n >> 1)) + (i & 1) * 8 + g
                            : (EPI == EPI_ROPE) ? (i < 2 ? 0 : 64) + (i & 1) * 8 + g : i * 8 + g;
        wrow[i] = p.w + (long long)row * p.sw + 8 * t + 32 * w_first;
    }
    // First row of W behind tile t (EPI_ROPE: four tiles per head of 128).
    auto tile_off = [&](int t) -> long long {
        const int row = (EPI == EPI_SWIGLU) ? 16 * t : (EPI == EPI_ROPE) ? (t >> 2) * 128 + (t & 3) * 16
                                                                         : kTileRows * t;
        return (long long)row * p.sw;
    };
    const uint64_t pol = l2_policy_evict_first();

    // Load side: item q of the warp's stream goes to ring slot q % kRing.
    int ld_tile = blockIdx.x, ld_ci = 0, ld_slot = 0, ld_q = 0;
    auto issue = [&]() {
        if (ld_q < items) {
            const long long off = tile_off(ld_tile) + 32 * kChunkStep * ld_ci;
            const uint32_t dst = ring + ld_slot * 2048;
#pragma unroll
            for (int i = 0; i < 4; ++i) cp_async_16_stream(dst + i * 512, wrow[i] + off, pol);
            if (++ld_ci == cpw) {
                ld_ci = 0;
                ld_tile += gridDim.x;
            }
            ++ld_q;
        }
        cp_async_commit();
        if (++ld_slot == kRing) ld_slot = 0;
    };
#pragma unroll
    for (int s = 0; s < kRing - 1; ++s) issue();        // weights do not depend on the previous kernel

    // Everything below reads what the previous kernel wrote.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // Row sums of squares left by the kernel that produced x (one partial per 32
    // columns, a row's partials contiguous): a warp takes ROWS / 8 rows, 256 / ROWS
    // lanes per row take interleaved shares, so a row's request is one or two
    // 64-byte segments. Requested here so that they travel with the activations.
    constexpr int LPR = kGemmThreads / ROWS;                 // lanes per row: 16 or 8
    const int st_row = warp * (ROWS / kGemmWarps) + lane / LPR, st_part = lane % LPR;
    float st[4] = {0.f, 0.f, 0.f, 0.f};
    if (PRO == PRO_NORM && p.sumsq_in != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = st_part + j * LPR;
            if (i < p.sumsq_tiles) st[j] = __ldcg(p.sumsq_in + st_row * p.sumsq_tiles + i);
        }
    }

    // This lane's A fragments for the warp's chunks (rows g, g + 8 of each 16-row tile, 16
    // bytes at 8 t).
    uint4 areg[kMaxCpw][MT][2];
    uint4 gam[PRO == PRO_NORM ? kMaxCpw : 1];
#pragma unroll
    for (int ci = 0; ci < kMaxCpw; ++ci) {
        if (ci < cpw) {
            const int k = 32 * (w_first + kChunkStep * ci) + 8 * t;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int rr = min(mt * 16 + hh * 8 + g, p.m - 1);
                    uint4 a = ldg_l2(p.x + rr * p.sx + k);
                    if (PRO == PRO_NORM && p.res != nullptr) a = add8(a, ldg_l2(p.res + rr * p.sres + k));
                    areg[ci][mt][hh] = a;
                }
            if (PRO == PRO_NORM) gam[ci] = *reinterpret_cast<const uint4*>(p.gamma + k);
        }
    }
    // Applied in a second pass so that every request above is in flight before the
    // first one is waited for.
    if (PRO == PRO_NORM) {
#pragma unroll
        for (int ci = 0; ci < kMaxCpw; ++ci) {
            if (ci < cpw) {
                const uint4 gs = prescale8(gam[ci]);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) areg[ci][mt][hh] = scale8(areg[ci][mt][hh], gs);
            }
        }
    }

    if (PRO == PRO_NORM && p.sumsq_in == nullptr) {
        // Whole rows once: x (+ residual) -> sum of squares. 16 threads per row.
        const int sub = tid & 15;
        constexpr int B = 4;
        for (int r0 = 0; r0 < ROWS; r0 += 16) {
            const int row = r0 + (tid >> 4);
            const int rr = min(row, p.m - 1);
            float acc = 0.f;
            for (int i0 = sub * 8; i0 < p.k; i0 += 128 * B) {
                uint4 v[B], r[B];
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    const int i = i0 + 128 * j;
                    v[j] = make_uint4(0, 0, 0, 0);
                    r[j] = v[j];
                    if (i < p.k) {
                        v[j] = ldg_l2(p.x + rr * p.sx + i);
                        if (p.res != nullptr) r[j] = ldg_l2(p.res + rr * p.sres + i);
                    }
                }
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    const int i = i0 + 128 * j;
                    if (i >= p.k) continue;
                    if (p.res != nullptr) {
                        v[j] = add8(v[j], r[j]);
                        if (blockIdx.x == 0 && split == 0 && row < p.m)
                            *reinterpret_cast<uint4*>(p.res_out + rr * p.sres_out + i) = v[j];
                    }
                    acc += sumsq8(v[j]);
                }
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(LS_FULL_MASK, acc, off);
            if (sub == 0) inv_rms[row] = rsqrtf(acc / (float)p.k + p.eps);
        }
        __syncthreads();
    }
    // With statistics from the previous kernel, the shares requested above are added up
    // after the first tile's products (below): no warp waits for them here.
    bool stats_pending = PRO == PRO_NORM && p.sumsq_in != nullptr;

    int slot = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        float acc[4][MT][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][mt][j] = 0.f;
        // What the epilogue will add to this thread's elements, requested now.
        constexpr int EPT = ROWS * 32 / kGemmThreads;
        float pre_bias = 0.f, pre_res[EPT];
        if (EPI == EPI_NONE) {
            if (p.bias != nullptr) pre_bias = __half2float(p.bias[tile * kTileRows + lane]);
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const int row = (tid >> 5) + j * kGemmWarps;
                pre_res[j] = (p.add_res != nullptr && row < p.m)
                                 ? __half2float(p.add_res[row * p.sadd + tile * kTileRows + lane])
                                 : 0.f;
            }
        }
        // EPI_ROPE: this thread's pair of dims (r_d, r_d + 64) of head r_head, for rows
        // (tid >> 4) + 16 j: bias, position and the position's cos / sin, requested now.
        constexpr int EPR = ROWS * 16 / kGemmThreads;
        const int r_head = tile >> 2, r_d = (tile & 3) * 16 + (tid & 15);
        float rb_lo = 0.f, rb_hi = 0.f, rc1[EPR], rs1[EPR], rc2[EPR], rs2[EPR];
        bool r_ok[EPR];
        if (EPI == EPI_ROPE) {
            if (p.bias != nullptr) {
                rb_lo = __half2float(p.bias[r_head * 128 + r_d]);
                rb_hi = __half2float(p.bias[r_head * 128 + r_d + 64]);
            }
#pragma unroll
            for (int j = 0; j < EPR; ++j) {
                const int row = (tid >> 4) + 16 * j;
                rc1[j] = rc2[j] = 1.f;
                rs1[j] = rs2[j] = 0.f;
                r_ok[j] = row < p.m;
                if (r_ok[j] && r_head < p.hq + p.hk) {          // q and k heads are rotated
                    const long long pos = p.positions[row];
                    r_ok[j] = pos >= 0 && pos < p.max_pos;
                    if (r_ok[j]) {
                        rc1[j] = __half2float(p.cos_t[pos * p.s_cos + r_d]);
                        rc2[j] = __half2float(p.cos_t[pos * p.s_cos + r_d + 64]);
                        rs1[j] = __half2float(p.sin_t[pos * p.s_cos + r_d]);
                        rs2[j] = __half2float(p.sin_t[pos * p.s_cos + r_d + 64]);
                    }
                }
            }
        }

#pragma unroll
        for (int ci = 0; ci < kMaxCpw; ++ci) {
            if (ci < cpw) {
                cp_async_wait<kRing - 2>();             // this item's 16-byte pieces have landed
                issue();                                // refill the slot consumed one item ago
                const uint32_t src = ring + slot * 2048;
                if (++slot == kRing) slot = 0;
                uint4 w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) w[i] = lds128g(src + i * 512);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        mma_16816(acc[i][mt], areg[ci][mt][0].x, areg[ci][mt][1].x, areg[ci][mt][0].y,
                                  areg[ci][mt][1].y, w[i].x, w[i].y);
                        mma_16816(acc[i][mt], areg[ci][mt][0].z, areg[ci][mt][1].z, areg[ci][mt][0].w,
                                  areg[ci][mt][1].w, w[i].z, w[i].w);
                    }
            }
        }

        if (PRO == PRO_NORM && stats_pending) {
            // Row statistics: this lane's shares, the rest of a long row, a shuffle tree.
            // The epilogue reads inv_rms after the barrier below.
            float acc = (st[0] + st[1]) + (st[2] + st[3]);
            for (int i = st_part + 4 * LPR; i < p.sumsq_tiles; i += LPR)
                acc += __ldcg(p.sumsq_in + st_row * p.sumsq_tiles + i);
#pragma unroll
            for (int off = LPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(LS_FULL_MASK, acc, off);
            if (st_part == 0) inv_rms[st_row] = rsqrtf(acc / (float)p.k + p.eps);
            stats_pending = false;
        }
        // Warps -> CTA: red[warp][row][col], col = 8 i + 2 t + {0, 1} of the tile's 32 rows of W.
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float* dst = red + ((warp * ROWS + mt * 16 + g) * 32 + i * 8 + 2 * t);
                *reinterpret_cast<float2*>(dst) = make_float2(acc[i][mt][0], acc[i][mt][1]);
                *reinterpret_cast<float2*>(dst + 8 * 32) = make_float2(acc[i][mt][2], acc[i][mt][3]);
            }
        __syncthreads();

        auto cta_sum = [&](int e) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kGemmWarps; ++w) s += red[w * ROWS * 32 + e];
            return s;
        };

        // The sum for element e goes to red[e] (warp 0's slot): only the thread that owns
        // e reads or writes that address, so no barrier is needed in between.
        bool finish = true;
        if (p.splits > 1) {
            float* mine = p.part + ((long long)tile * p.splits + split) * (ROWS * 32);
            for (int e = tid; e < ROWS * 32; e += kGemmThreads) mine[e] = cta_sum(e);
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                const int seen = atomicAdd(p.counters + tile, 1);
                is_last = (seen == p.splits - 1);
                if (is_last) {
                    p.counters[tile] = 0;               // ready for the next launch
                    __threadfence();
                }
            }
            __syncthreads();
            finish = is_last != 0;
            if (finish) {
                // Split order, whoever arrives last: the sum does not depend on timing.
                const float* base = p.part + (long long)tile * p.splits * (ROWS * 32);
                for (int e = tid; e < ROWS * 32; e += kGemmThreads) {
                    float s = 0.f;
                    for (int sp = 0; sp < p.splits; ++sp) s += __ldcg(base + sp * (ROWS * 32) + e);
                    red[e] = s;
                }
            }
        } else {
            for (int e = tid; e < ROWS * 32; e += kGemmThreads) red[e] = cta_sum(e);
        }
        __syncthreads();

        // Epilogue on red[row][col].
        if (finish && EPI == EPI_SWIGLU) {
            for (int e = tid; e < ROWS * 16; e += kGemmThreads) {
                const int row = e >> 4, j = e & 15;
                if (row >= p.m) continue;
                const float f = (PRO == PRO_NORM) ? inv_rms[row] * kPostScale : 1.f;
                const float gate = round_h(red[row * 32 + j] * f);
                const float up = round_h(red[row * 32 + 16 + j] * f);
                const float act = round_h(gate / (1.f + expf(-gate)));
                p.out[row * p.sout + tile * 16 + j] = __float2half_rn(act * up);
            }
        } else if (finish && EPI == EPI_ROPE) {
            // red[row][c] is dim r_d of the head, red[row][16 + c] its partner r_d + 64.
#pragma unroll
            for (int j = 0; j < EPR; ++j) {
                const int row = (tid >> 4) + 16 * j, c = tid & 15;
                if (!r_ok[j]) continue;
                const float f = (PRO == PRO_NORM) ? inv_rms[row] * kPostScale : 1.f;
                const float a = round_h(__fmaf_rn(red[row * 32 + c], f, rb_lo));        // the projection's fp16 output
                const float b = round_h(__fmaf_rn(red[row * 32 + 16 + c], f, rb_hi));
                float y_lo = a, y_hi = b;
                if (r_head < p.hq + p.hk) {                     // the rounding sequence of rope_append_kernel
                    y_lo = round_h(round_h(a * rc1[j]) + round_h(-(b * rs1[j])));
                    y_hi = round_h(round_h(b * rc2[j]) + round_h(a * rs2[j]));
                }
                if (r_head < p.hq) {
                    __half* dst = p.q_out + row * p.sq_b + r_head * 128 + r_d;
                    dst[0] = __float2half_rn(y_lo);
                    dst[64] = __float2half_rn(y_hi);
                    continue;
                }
                const long long slot = p.slots[row];
                if (slot < 0 || slot >= p.num_slots) continue;
                const bool is_k = r_head < p.hq + p.hk;
                const int kvh = is_k ? r_head - p.hq : r_head - p.hq - p.hk;
                __half* dst = (is_k ? p.k_pool : p.v_pool) + slot * p.sp_t + kvh * p.sp_h + r_d;
                dst[0] = __float2half_rn(y_lo);
                dst[64] = __float2half_rn(y_hi);
                if (is_k && p.kmin != nullptr) {
                    // Page bounds of K: reset by the page's first row, else widened. One
                    // thread owns a (page, head, dim), and no two sequences write one page.
                    const long long bi = (slot / LS_PAGE) * p.sb_b + kvh * p.sb_h + r_d;
                    const bool first = slot % LS_PAGE == 0;
#pragma unroll
                    for (int part = 0; part < 2; ++part) {
                        const float v = part ? y_hi : y_lo;
                        __half* mn = p.kmin + bi + 64 * part;
                        __half* mx = p.kmax + bi + 64 * part;
                        *mn = __float2half_rn(first ? v : fminf(__half2float(*mn), v));
                        *mx = __float2half_rn(first ? v : fmaxf(__half2float(*mx), v));
                    }
                }
            }
        } else if (finish) {
            // A warp covers one row's 32 columns per sweep (256 threads = 8 rows).
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const int e = tid + j * kGemmThreads;
                const int row = e >> 5, col = tile * kTileRows + (e & 31);
                const float f = (PRO == PRO_NORM) ? inv_rms[row] * kPostScale : 1.f;
                float v = round_h(__fmaf_rn(red[e], f, pre_bias));
                if (p.add_res != nullptr) v = round_h(v + pre_res[j]);
                if (row < p.m) p.out[row * p.sout + col] = __float2half_rn(v);
                if (p.sumsq_out != nullptr) {
                    float sq = (row < p.m) ? v * v : 0.f;
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(LS_FULL_MASK, sq, off);
                    if (lane == 0) p.sumsq_out[row * n_tiles + tile] = sq;
                }
            }
        }
        __syncthreads();                                // red is free for the next tile
    }
}

template <int MT, int PRO, int EPI>
static int launch_gemm(const GemmParams& p, int tiles, cudaStream_t stream, bool programmatic) {
    const int per_split = ((p.k >> 5) + p.splits - 1) / p.splits;
    if (per_split > kGemmWarps * kMaxCpw) return LS_ERR_TOO_LARGE;     // cut K into more splits
    const size_t smem = (size_t)kGemmWarps * kRing * 2048 + sizeof(float) * kGemmWarps * MT * 16 * 32;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int resident = (MT == 1 ? 2 : 1) * sms;      // CTAs the device holds at once
    int per = resident / p.splits;
    per = per < 1 ? 1 : (per > tiles ? tiles : per);
    auto kern = skinny_gemm_kernel<MT, PRO, EPI>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(per, p.splits);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

template <int PRO, int EPI>
static int launch_gemm_m(const GemmParams& p, int tiles, cudaStream_t stream, bool programmatic) {
    if (p.m <= 16) return launch_gemm<1, PRO, EPI>(p, tiles, stream, programmatic);
    return launch_gemm<2, PRO, EPI>(p, tiles, stream, programmatic);
}

}  // namespace ls

extern "C" int ls_skinny_gemm(const void* x, const void* res, const void* gamma, void* res_out,
                              const float* sumsq_in, int sumsq_tiles, const void* w, const void* bias,
                              const void* add_res, float* sumsq_out, void* out, float* part,
                              int32_t* counters, int m, int n, int k, int splits, int mode, float eps,
                              int64_t sx, int64_t sres, int64_t sres_out, int64_t sw, int64_t sadd,
                              int64_t sout, void* stream) {
    using namespace ls;
    const bool norm = mode & LS_GEMM_NORM, swiglu = mode & LS_GEMM_SWIGLU;
    if (!x || !w || !out || (norm && !gamma) || (res && !res_out)) return LS_ERR_NULL_POINTER;
    if ((res && !norm) || (sumsq_in && (!norm || res)) || (swiglu && (bias || add_res || sumsq_out)))
        return LS_ERR_UNSUPPORTED;
    if (m <= 0 || n <= 0 || k <= 0 || splits <= 0 || (sumsq_in && sumsq_tiles <= 0))
        return LS_ERR_BAD_SHAPE;
    if (m > 32) return LS_ERR_TOO_LARGE;
    if ((k % 32) || (n % 32) || splits > k / 32) return LS_ERR_UNSUPPORTED;
    if (splits > 1 && (!part || !counters)) return LS_ERR_NULL_POINTER;
    auto bad = [](const void* ptr, int64_t stride) {
        return (reinterpret_cast<uintptr_t>(ptr) & 15) || (stride % 8);
    };
    if (bad(x, sx) || bad(w, sw) || (res && (bad(res, sres) || bad(res_out, sres_out))) ||
        (norm && bad(gamma, 8)))
        return LS_ERR_MISALIGNED;
    GemmParams p = {};
    p.x = static_cast<const __half*>(x);
    p.res = static_cast<const __half*>(res);
    p.gamma = static_cast<const __half*>(gamma);
    p.res_out = static_cast<__half*>(res_out);
    p.sumsq_in = sumsq_in;
    p.sumsq_tiles = sumsq_tiles;
    p.w = static_cast<const __half*>(w);
    p.bias = static_cast<const __half*>(bias);
    p.add_res = static_cast<const __half*>(add_res);
    p.sumsq_out = sumsq_out;
    p.out = static_cast<__half*>(out);
    p.part = part;
    p.counters = counters;
    p.m = m; p.n = n; p.k = k; p.splits = splits; p.eps = eps;
    p.sx = sx; p.sres = sres; p.sres_out = sres_out; p.sw = sw; p.sadd = sadd; p.sout = sout;
    const int tiles = n / kTileRows;                    // with SWIGLU: 16 gate + 16 up rows each
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool pdl = mode & LS_LAUNCH_PROGRAMMATIC;
    if (norm && swiglu) return launch_gemm_m<PRO_NORM, EPI_SWIGLU>(p, tiles, st, pdl);
    if (norm) return launch_gemm_m<PRO_NORM, EPI_NONE>(p, tiles, st, pdl);
    if (swiglu) return launch_gemm_m<PRO_NONE, EPI_SWIGLU>(p, tiles, st, pdl);
    return launch_gemm_m<PRO_NONE, EPI_NONE>(p, tiles, st, pdl);
}

extern "C" int ls_qkv_rope_append_fp16(const void* x, const void* gamma, const float* sumsq_in,
                                       int sumsq_tiles, const void* w, const void* bias, const void* cos,
                                       const void* sin, const int64_t* positions, const int64_t* slots,
                                       void* q_out, void* k_pool, void* v_pool, void* kmin, void* kmax,
                                       float* part, int32_t* counters, int m, int q_heads, int kv_heads,
                                       int head_dim, int page, int k, int splits, int mode, float eps,
                                       int64_t max_pos, int64_t num_slots, int64_t sx, int64_t sw,
                                       int64_t s_cos, int64_t sq_b, int64_t sp_t, int64_t sp_h,
                                       int64_t sb_b, int64_t sb_h, void* stream) {
    using namespace ls;
    const bool norm = mode & LS_GEMM_NORM;
    if (!x || !w || !cos || !sin || !positions || !slots || !q_out || !k_pool || !v_pool ||
        (norm && !gamma))
        return LS_ERR_NULL_POINTER;
    if ((kmin == nullptr) != (kmax == nullptr)) return LS_ERR_NULL_POINTER;
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE || (mode & LS_GEMM_SWIGLU) || (sumsq_in && !norm))
        return LS_ERR_UNSUPPORTED;
    if (m <= 0 || q_heads <= 0 || kv_heads <= 0 || k <= 0 || splits <= 0 || max_pos <= 0 ||
        num_slots <= 0 || (sumsq_in && sumsq_tiles <= 0))
        return LS_ERR_BAD_SHAPE;
    if (m > 32) return LS_ERR_TOO_LARGE;
    if ((k % 32) || splits > k / 32) return LS_ERR_UNSUPPORTED;
    if (splits > 1 && (!part || !counters)) return LS_ERR_NULL_POINTER;
    auto bad = [](const void* ptr, int64_t stride) {
        return (reinterpret_cast<uintptr_t>(ptr) & 15) || (stride % 8);
    };
    if (bad(x, sx) || bad(w, sw) || (norm && bad(gamma, 8))) return LS_ERR_MISALIGNED;
    const void* halves[] = {bias, cos, sin, q_out, k_pool, v_pool, kmin, kmax};
    for (const void* ptr : halves)
        if (reinterpret_cast<uintptr_t>(ptr) & 1) return LS_ERR_MISALIGNED;
    GemmParams p = {};
    p.x = static_cast<const __half*>(x);
    p.gamma = static_cast<const __half*>(gamma);
    p.sumsq_in = sumsq_in;
    p.sumsq_tiles = sumsq_tiles;
    p.w = static_cast<const __half*>(w);
    p.bias = static_cast<const __half*>(bias);
    p.part = part;
    p.counters = counters;
    p.m = m; p.n = (q_heads + 2 * kv_heads) * LS_HEAD_DIM; p.k = k; p.splits = splits; p.eps = eps;
    p.sx = sx; p.sw = sw;
    p.cos_t = static_cast<const __half*>(cos);
    p.sin_t = static_cast<const __half*>(sin);
    p.positions = reinterpret_cast<const long long*>(positions);
    p.slots = reinterpret_cast<const long long*>(slots);
    p.q_out = static_cast<__half*>(q_out);
    p.k_pool = static_cast<__half*>(k_pool);
    p.v_pool = static_cast<__half*>(v_pool);
    p.kmin = static_cast<__half*>(kmin);
    p.kmax = static_cast<__half*>(kmax);
    p.hq = q_heads; p.hk = kv_heads;
    p.max_pos = max_pos; p.num_slots = num_slots; p.s_cos = s_cos; p.sq_b = sq_b;
    p.sp_t = sp_t; p.sp_h = sp_h; p.sb_b = sb_b; p.sb_h = sb_h;
    const int tiles = p.n / kTileRows;                  // four per head: 16 dims and their partners
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool pdl = mode & LS_LAUNCH_PROGRAMMATIC;
    if (norm) return launch_gemm_m<PRO_NORM, EPI_ROPE>(p, tiles, st, pdl);
    return launch_gemm_m<PRO_NONE, EPI_ROPE>(p, tiles, st, pdl);
}
