// The small per-layer kernels around decode attention: RMSNorm (+ residual
// add), SiLU(gate) * up, and RoPE fused with the KV append.
//
// The reference has these as Triton kernels (kernels/fused_elementwise.py:
// `_rms_norm_kernel` :118-137, `_silu_mul_kernel` :140-151, `_rope_kernel`
// :154-182) whose point is to keep the Hugging Face fp16 rounding sequence
// while removing launches; the torch forms they match are `rms_norm_ref`,
// `fused_add_rms_norm_ref`, `silu_and_mul_ref`, `rope_qk_ref` (:75-107). The
// same rounding sequences are kept here:
//   RMSNorm   s = fp16(x + r); y = fp16(w * fp16(s * rsqrt(mean(s^2) + eps)))
//   SiLU*up   out = fp16(fp16(g * sigmoid(g)) * u)
//   RoPE      o1 = fp16(fp16(x1 c1) + fp16(-(x2 s1))), o2 = fp16(fp16(x2 c2) + fp16(x1 s2))
// RoPE goes one step further than the reference: it reads q, k, v straight out
// of the fused QKV projection row and, in the same launch, writes the rotated
// query, appends the rotated K row and the V row to the paged cache (fp16:
// scatter + page bounds; INT8: V quantised on write, K into the fp16 residual),
// so "RoPE + cache.write" is one launch instead of the reference's two or three.
//
// All of them are latency-sized at decode batch sizes (tens of rows).
#include "ls_common.cuh"

namespace ls {

__device__ __forceinline__ float h2f(__half h) { return __half2float(h); }
__device__ __forceinline__ __half f2h(float f) { return __float2half_rn(f); }
// Round to fp16 and come back: where the unfused model code rounds.
__device__ __forceinline__ float rh(float f) { return __half2float(__float2half_rn(f)); }

// ---------------------------------------------------------------------------
// grid (rows), block 256: thread handles 8 consecutive elements per sweep.
__global__ void __launch_bounds__(256)
rms_norm_kernel(const __half* __restrict__ x, const __half* __restrict__ res,
                const __half* __restrict__ w, __half* __restrict__ y, __half* __restrict__ res_out,
                int n, float eps, long long sx, long long sr, long long sy, long long sro) {
    extern __shared__ __align__(16) __half row_s[];          // the (summed) row, n halves
    __shared__ float warp_sum[8];
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // let a programmatic successor start its prologue
    const int row = blockIdx.x, tid = threadIdx.x;
    const __half* xr = x + row * sx;
    float acc = 0.f;
    for (int i = tid * 8; i < n; i += 256 * 8) {
        uint4 raw = *reinterpret_cast<const uint4*>(xr + i);
        __half* h = reinterpret_cast<__half*>(&raw);
        if (res != nullptr) {
            const uint4 rraw = *reinterpret_cast<const uint4*>(res + row * sr + i);
            const __half* r = reinterpret_cast<const __half*>(&rraw);
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = f2h(h2f(h[j]) + h2f(r[j]));   // fp32 add, one rounding
            *reinterpret_cast<uint4*>(res_out + row * sro + i) = raw;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float f = h2f(h[j]);
            acc += f * f;
        }
        *reinterpret_cast<uint4*>(row_s + i) = raw;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(LS_FULL_MASK, acc, off);
    if ((tid & 31) == 0) warp_sum[tid >> 5] = acc;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += warp_sum[i];
    const float inv = rsqrtf(total / (float)n + eps);
    for (int i = tid * 8; i < n; i += 256 * 8) {
        uint4 raw = *reinterpret_cast<const uint4*>(row_s + i);
        const uint4 wraw = *reinterpret_cast<const uint4*>(w + i);
        __half* h = reinterpret_cast<__half*>(&raw);
        const __half* wh = reinterpret_cast<const __half*>(&wraw);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = f2h(h2f(wh[j]) * rh(h2f(h[j]) * inv));
        *reinterpret_cast<uint4*>(y + row * sy + i) = raw;
    }
}

// grid (ceil(inter / 2048), rows), block 256: 8 elements per thread.
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half* __restrict__ gu, __half* __restrict__ out, int inter, long long sgu,
                long long sout) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // let a programmatic successor start its prologue
    const int row = blockIdx.y;
    const int i = (blockIdx.x * 256 + threadIdx.x) * 8;
    if (i >= inter) return;
    const uint4 graw = *reinterpret_cast<const uint4*>(gu + row * sgu + i);
    const uint4 uraw = *reinterpret_cast<const uint4*>(gu + row * sgu + inter + i);
    const __half* g = reinterpret_cast<const __half*>(&graw);
    const __half* u = reinterpret_cast<const __half*>(&uraw);
    uint4 oraw;
    __half* o = reinterpret_cast<__half*>(&oraw);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float gf = h2f(g[j]);
        const float act = rh(gf / (1.f + expf(-gf)));
        o[j] = f2h(act * h2f(u[j]));
    }
    *reinterpret_cast<uint4*>(out + row * sout + i) = oraw;
}

// ---------------------------------------------------------------------------
// RoPE of one 128-wide head held by a warp: lane l owns dims 2l, 2l+1 (first
// half) and 64+2l, 64+2l+1 (second half), i.e. both members of two rotation
// pairs. Returns the rotated values in place.
__device__ __forceinline__ void rope_head(float (&lo)[2], float (&hi)[2], const __half* cos_row,
                                          const __half* sin_row, int lane) {
    const float2 c1 = __half22float2(*reinterpret_cast<const __half2*>(cos_row + 2 * lane));
    const float2 c2 = __half22float2(*reinterpret_cast<const __half2*>(cos_row + 64 + 2 * lane));
    const float2 s1 = __half22float2(*reinterpret_cast<const __half2*>(sin_row + 2 * lane));
    const float2 s2 = __half22float2(*reinterpret_cast<const __half2*>(sin_row + 64 + 2 * lane));
    const float a0 = lo[0], a1 = lo[1], b0 = hi[0], b1 = hi[1];
    lo[0] = rh(rh(a0 * c1.x) + rh(-(b0 * s1.x)));
    lo[1] = rh(rh(a1 * c1.y) + rh(-(b1 * s1.y)));
    hi[0] = rh(rh(b0 * c2.x) + rh(a0 * s2.x));
    hi[1] = rh(rh(b1 * c2.y) + rh(a1 * s2.y));
}

// Page bounds of K for the sparse indexer: the block's per-channel minimum and
// maximum over its written rows (reset by the first row of a page). One warp,
// lane l owning dims 2l, 2l+1 and 64+2l, 64+2l+1 of the new row.
__device__ __forceinline__ void update_page_bounds(__half* kmin, __half* kmax, long long bi, bool first,
                                                   int lane, const float (&lo)[2], const float (&hi)[2],
                                                   uint32_t plo, uint32_t phi) {
    if (first) {
        *reinterpret_cast<uint32_t*>(kmin + bi + 2 * lane) = plo;
        *reinterpret_cast<uint32_t*>(kmin + bi + 64 + 2 * lane) = phi;
        *reinterpret_cast<uint32_t*>(kmax + bi + 2 * lane) = plo;
        *reinterpret_cast<uint32_t*>(kmax + bi + 64 + 2 * lane) = phi;
        return;
    }
#pragma unroll
    for (int part = 0; part < 2; ++part) {
        const int d = part * 64 + 2 * lane;
        const float2 mn = __half22float2(*reinterpret_cast<__half2*>(kmin + bi + d));
        const float2 mx = __half22float2(*reinterpret_cast<__half2*>(kmax + bi + d));
        const float v0 = part ? hi[0] : lo[0], v1 = part ? hi[1] : lo[1];
        *reinterpret_cast<uint32_t*>(kmin + bi + d) = pack_half2(fminf(mn.x, v0), fminf(mn.y, v1));
        *reinterpret_cast<uint32_t*>(kmax + bi + d) = pack_half2(fmaxf(mx.x, v0), fmaxf(mx.y, v1));
    }
}

struct RopeQuant {
    int asym;
    float eps, qmax, inv_qmax, levels, inv_levels, offset;
};

__device__ __forceinline__ float wmax(float x) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) x = fmaxf(x, __shfl_xor_sync(LS_FULL_MASK, x, off));
    return x;
}

// grid (ceil(B * (HQ + 2 HK) / 4)), block 128: one warp per (sequence, head of
// the fused QKV row). INT8 = 0: fp16 pools (+ optional page bounds);
// INT8 = 1: V quantised per (token, head), K row into the fp16 residual.
template <int INT8>
__global__ void __launch_bounds__(128)
rope_append_kernel(const __half* __restrict__ qkv, const __half* __restrict__ cos_t,
                   const __half* __restrict__ sin_t, const long long* __restrict__ positions,
                   const long long* __restrict__ slots, const long long* __restrict__ res_idx,
                   __half* __restrict__ q_out, void* __restrict__ k_dst, void* __restrict__ v_dst,
                   __half* __restrict__ kmin, __half* __restrict__ kmax,
                   float* __restrict__ v_scale, float* __restrict__ v_zero, int batch, int hq, int hk,
                   long long max_pos, long long num_slots, long long num_res, long long s_qkv,
                   long long s_cos, long long sq_b, long long sp_t, long long sp_h, long long sb_b,
                   long long sb_h, RopeQuant qc) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // let a programmatic successor start its prologue
    const int heads = hq + 2 * hk;
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= batch * heads) return;
    const int b = item / heads, head = item % heads;
    const __half* src = qkv + b * s_qkv + head * LS_HEAD_DIM;
    const __half2 l2 = *reinterpret_cast<const __half2*>(src + 2 * lane);
    const __half2 h2 = *reinterpret_cast<const __half2*>(src + 64 + 2 * lane);
    float lo[2] = {__low2float(l2), __high2float(l2)}, hi[2] = {__low2float(h2), __high2float(h2)};
    const long long pos = positions[b];
    if (head < hq + hk) {                         // q and k heads are rotated
        if (pos < 0 || pos >= max_pos) return;
        rope_head(lo, hi, cos_t + pos * s_cos, sin_t + pos * s_cos, lane);
    }
    const uint32_t plo = pack_half2(lo[0], lo[1]), phi = pack_half2(hi[0], hi[1]);
    if (head < hq) {
        __half* dst = q_out + b * sq_b + head * LS_HEAD_DIM;
        *reinterpret_cast<uint32_t*>(dst + 2 * lane) = plo;
        *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = phi;
        return;
    }
    const long long slot = slots[b];
    if (slot < 0 || slot >= num_slots) return;
    const bool is_k = head < hq + hk;
    const int kvh = is_k ? head - hq : head - hq - hk;
    if (!INT8) {
        __half* pool = static_cast<__half*>(is_k ? k_dst : v_dst) + slot * sp_t + kvh * sp_h;
        *reinterpret_cast<uint32_t*>(pool + 2 * lane) = plo;
        *reinterpret_cast<uint32_t*>(pool + 64 + 2 * lane) = phi;
        if (is_k && kmin != nullptr)
            update_page_bounds(kmin, kmax, (slot / LS_PAGE) * sb_b + kvh * sb_h, slot % LS_PAGE == 0, lane, lo,
                               hi, plo, phi);
        return;
    }
    if (is_k) {                                   // INT8 cache: rotated K stays exact in the residual
        const long long ridx = res_idx[b];
        if (ridx < 0 || ridx >= num_res) return;
        __half* dst = static_cast<__half*>(k_dst) + (ridx * hk + kvh) * LS_HEAD_DIM;
        *reinterpret_cast<uint32_t*>(dst + 2 * lane) = plo;
        *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = phi;
        if (kmin != nullptr)                      // bounds of the exact fp16 K, as for the fp16 cache
            update_page_bounds(kmin, kmax, (slot / LS_PAGE) * sb_b + kvh * sb_h, slot % LS_PAGE == 0, lane, lo,
                               hi, plo, phi);
        return;
    }
    // INT8 V: the reference's quantiser (kernels/cuda/int8_write.cu:45-78), per (token, head).
    const float x[4] = {lo[0], lo[1], hi[0], hi[1]};
    const long long out_row = slot * hk + kvh;
    int q[4];
    if (!qc.asym) {
        const float amax = wmax(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
        const float step = __fmul_rn(fmaxf(amax, qc.eps), qc.inv_qmax);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            q[j] = (int)fminf(fmaxf(rintf(__fdiv_rn(x[j], step)), -qc.qmax), qc.qmax);
        if (lane == 0) v_scale[out_row] = step;
    } else {
        const float mx = wmax(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])));
        const float mn = -wmax(fmaxf(fmaxf(-x[0], -x[1]), fmaxf(-x[2], -x[3])));
        const float step = fmaxf(__fmul_rn(__fsub_rn(mx, mn), qc.inv_levels), qc.eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float u = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(x[j], mn), step)), 0.f), qc.levels);
            q[j] = (int)__fsub_rn(u, qc.offset);
        }
        if (lane == 0) {
            v_scale[out_row] = step;
            v_zero[out_row] = __fadd_rn(mn, __fmul_rn(qc.offset, step));
        }
    }
    signed char* dst = static_cast<signed char*>(v_dst) + out_row * LS_HEAD_DIM;
    *reinterpret_cast<uint16_t*>(dst + 2 * lane) = (uint16_t)((q[0] & 0xff) | ((q[1] & 0xff) << 8));
    *reinterpret_cast<uint16_t*>(dst + 64 + 2 * lane) = (uint16_t)((q[2] & 0xff) | ((q[3] & 0xff) << 8));
}

}  // namespace ls

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" {

int ls_rms_norm(const void* x, const void* residual, const void* weight, void* y, void* res_out,
                int rows, int n, float eps, int64_t sx, int64_t sr, int64_t sy, int64_t sro,
                void* stream) {
    if (!x || !weight || !y) return LS_ERR_NULL_POINTER;
    if ((residual == nullptr) != (res_out == nullptr)) return LS_ERR_NULL_POINTER;
    if (rows <= 0 || n <= 0 || n % 8) return LS_ERR_BAD_SHAPE;
    if (n > 16384) return LS_ERR_TOO_LARGE;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(y) || !aligned16(residual) ||
        !aligned16(res_out) || (sx % 8) || (sy % 8) || (sr % 8) || (sro % 8))
        return LS_ERR_MISALIGNED;
    ls::rms_norm_kernel<<<rows, 256, (size_t)n * 2, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(residual),
        static_cast<const __half*>(weight), static_cast<__half*>(y), static_cast<__half*>(res_out), n,
        eps, sx, sr, sy, sro);
    return (int)cudaGetLastError();
}

int ls_silu_mul(const void* gate_up, void* out, int rows, int inter, int64_t sgu, int64_t sout,
                void* stream) {
    if (!gate_up || !out) return LS_ERR_NULL_POINTER;
    if (rows <= 0 || inter <= 0 || inter % 8) return LS_ERR_BAD_SHAPE;
    if (rows > 65535) return LS_ERR_TOO_LARGE;
    if (!aligned16(gate_up) || !aligned16(out) || (sgu % 8) || (sout % 8)) return LS_ERR_MISALIGNED;
    dim3 grid((inter + 2047) / 2048, rows);
    ls::silu_mul_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(gate_up), static_cast<__half*>(out), inter, sgu, sout);
    return (int)cudaGetLastError();
}

int ls_rope_append_fp16(const void* qkv, const void* cos, const void* sin, const int64_t* positions,
                        const int64_t* slots, void* q_out, void* k_pool, void* v_pool, void* kmin,
                        void* kmax, int batch, int q_heads, int kv_heads, int head_dim, int page,
                        int64_t max_pos, int64_t num_slots, int64_t s_qkv, int64_t s_cos, int64_t sq_b,
                        int64_t sp_t, int64_t sp_h, int64_t sb_b, int64_t sb_h, void* stream) {
    if (!qkv || !cos || !sin || !positions || !slots || !q_out || !k_pool || !v_pool)
        return LS_ERR_NULL_POINTER;
    if ((kmin == nullptr) != (kmax == nullptr)) return LS_ERR_NULL_POINTER;
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || max_pos <= 0 || num_slots <= 0)
        return LS_ERR_BAD_SHAPE;
    const int64_t st[] = {s_qkv, s_cos, sq_b, sp_t, sp_h, sb_b, sb_h};
    for (int64_t v : st)
        if (v % 2) return LS_ERR_MISALIGNED;
    const void* ptrs[] = {qkv, cos, sin, q_out, k_pool, v_pool, kmin, kmax};
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) & 3) return LS_ERR_MISALIGNED;
    const int items = batch * (q_heads + 2 * kv_heads);
    ls::RopeQuant qc = {};
    ls::rope_append_kernel<0><<<(items + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(qkv), static_cast<const __half*>(cos),
        static_cast<const __half*>(sin), reinterpret_cast<const long long*>(positions),
        reinterpret_cast<const long long*>(slots), nullptr, static_cast<__half*>(q_out), k_pool, v_pool,
        static_cast<__half*>(kmin), static_cast<__half*>(kmax), nullptr, nullptr, batch, q_heads,
        kv_heads, max_pos, num_slots, 0, s_qkv, s_cos, sq_b, sp_t, sp_h, sb_b, sb_h, qc);
    return (int)cudaGetLastError();
}

int ls_rope_append_int8(const void* qkv, const void* cos, const void* sin, const int64_t* positions,
                        const int64_t* slots, const int64_t* res_idx, void* q_out, void* flat_v,
                        float* flat_v_scale, float* flat_v_zero, void* k_res, void* kmin, void* kmax,
                        int batch, int q_heads, int kv_heads, int head_dim, int64_t max_pos,
                        int64_t num_slots, int64_t num_res, int64_t s_qkv, int64_t s_cos, int64_t sq_b,
                        int64_t sb_b, int64_t sb_h, int asym, float eps, float qmax, float inv_qmax,
                        float levels, float inv_levels, float offset, void* stream) {
    if (!qkv || !cos || !sin || !positions || !slots || !res_idx || !q_out || !flat_v ||
        !flat_v_scale || !k_res)
        return LS_ERR_NULL_POINTER;
    if ((kmin == nullptr) != (kmax == nullptr)) return LS_ERR_NULL_POINTER;
    if (kmin && ((reinterpret_cast<uintptr_t>(kmin) & 3) || (reinterpret_cast<uintptr_t>(kmax) & 3) ||
                 (sb_b % 2) || (sb_h % 2)))
        return LS_ERR_MISALIGNED;
    if (asym && !flat_v_zero) return LS_ERR_NULL_POINTER;
    if (head_dim != LS_HEAD_DIM) return LS_ERR_UNSUPPORTED;
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || max_pos <= 0 || num_slots <= 0 || num_res <= 0)
        return LS_ERR_BAD_SHAPE;
    if ((s_qkv % 2) || (s_cos % 2) || (sq_b % 2)) return LS_ERR_MISALIGNED;
    const void* ptrs[] = {qkv, cos, sin, q_out, k_res};
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) & 3) return LS_ERR_MISALIGNED;
    if (reinterpret_cast<uintptr_t>(flat_v) & 1) return LS_ERR_MISALIGNED;
    const int items = batch * (q_heads + 2 * kv_heads);
    ls::RopeQuant qc = {asym, eps, qmax, inv_qmax, levels, inv_levels, offset};
    ls::rope_append_kernel<1><<<(items + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(qkv), static_cast<const __half*>(cos),
        static_cast<const __half*>(sin), reinterpret_cast<const long long*>(positions),
        reinterpret_cast<const long long*>(slots), reinterpret_cast<const long long*>(res_idx),
        static_cast<__half*>(q_out), k_res, flat_v, static_cast<__half*>(kmin), static_cast<__half*>(kmax),
        flat_v_scale, flat_v_zero, batch, q_heads, kv_heads, max_pos, num_slots, num_res, s_qkv, s_cos, sq_b,
        0, 0, sb_b, sb_h, qc);
    return (int)cudaGetLastError();
}

}  // extern "C"
