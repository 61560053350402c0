// Decode-step KV append kernels (one new token per sequence per layer).
//
//   ls_kv_append_fp16        fp16 cache: scatter the K and V rows into the pools
//                            and keep the page's per-channel K min/max, one launch
//                            (reference: two index_copy_ scatters + page_bounds_update,
//                            cache/paged_cache.py:398-417, kernels/cuda/paged_sparse_fp16.cu:54-72)
//   ls_int8_decode_write     INT8 cache: V quantised per (token, head) and scattered,
//                            K row copied into the fp16 residual
//                            (reference: kernels/cuda/int8_write.cu:45-78)
//   ls_int8_finalize_blocks  INT8 cache: a completed 16-token K page quantised per
//                            (block, head, channel) out of the residual
//                            (reference: Int8PagedKVCache._finalize_blocks,
//                            cache/int8_paged_cache.py:670-699, torch ops on the GPU)
//
// The two INT8 kernels are bit-exact against the reference's GPU arithmetic:
// fp32 throughout, round-half-to-even, every multiply / subtract / divide
// rounded on its own (no FMA contraction), and "divide by a Python number"
// done as torch does it on a GPU: a multiplication by the fp32 reciprocal that
// the host computed.
//
// All three are launch-latency sized (a few hundred rows), so they use one
// warp per (token, head) row and nothing cleverer.
#include "ls_common.cuh"

namespace ls {

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) x = fmaxf(x, __shfl_xor_sync(LS_FULL_MASK, x, off));
    return x;
}

__device__ __forceinline__ void unpack4(uint2 raw, float (&f)[4]) {
    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
    const float2 a = __half22float2(h2[0]), b = __half22float2(h2[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// grid (ceil(B*H / warps)), one warp per (sequence, head); lane owns 4 channels.
__global__ void __launch_bounds__(128)
kv_append_fp16_kernel(const __half* __restrict__ k, const __half* __restrict__ v,
                      const long long* __restrict__ slots, __half* __restrict__ k_pool,
                      __half* __restrict__ v_pool, __half* __restrict__ kmin,
                      __half* __restrict__ kmax, int batch, int heads, long long num_slots,
                      long long sk_b, long long sk_h, long long sv_b, long long sv_h,
                      long long sp_t, long long sp_h, long long sb_b, long long sb_h) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // let a programmatic successor start its prologue
    // Launched programmatically itself: the launch overlaps the end of the previous
    // kernel (in a layer loop, the previous layer's attention), and nothing is read or
    // written before that kernel has completed.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= batch * heads) return;
    const int b = row / heads, h = row % heads;
    const long long slot = slots[b];
    if (slot < 0 || slot >= num_slots) return;          // never write outside the pool
    const uint2 kraw = *reinterpret_cast<const uint2*>(k + b * sk_b + h * sk_h + lane * 4);
    if (k_pool != nullptr) {                            // null pools: bounds only
        const uint2 vraw = *reinterpret_cast<const uint2*>(v + b * sv_b + h * sv_h + lane * 4);
        const long long dst = slot * sp_t + h * sp_h + lane * 4;
        *reinterpret_cast<uint2*>(k_pool + dst) = kraw;
        *reinterpret_cast<uint2*>(v_pool + dst) = vraw;
    }
    if (kmin != nullptr) {
        const long long blk = slot / LS_PAGE;
        const int off = (int)(slot % LS_PAGE);
        const long long bi = blk * sb_b + h * sb_h + lane * 4;
        if (off == 0) {                                   // first token of a page: reset
            *reinterpret_cast<uint2*>(kmin + bi) = kraw;
            *reinterpret_cast<uint2*>(kmax + bi) = kraw;
        } else {                                          // later tokens widen (exact in fp32)
            float nf[4], lo[4], hi[4];
            unpack4(kraw, nf);
            unpack4(*reinterpret_cast<const uint2*>(kmin + bi), lo);
            unpack4(*reinterpret_cast<const uint2*>(kmax + bi), hi);
            uint2 olo, ohi;
            olo.x = pack_half2(fminf(lo[0], nf[0]), fminf(lo[1], nf[1]));
            olo.y = pack_half2(fminf(lo[2], nf[2]), fminf(lo[3], nf[3]));
            ohi.x = pack_half2(fmaxf(hi[0], nf[0]), fmaxf(hi[1], nf[1]));
            ohi.y = pack_half2(fmaxf(hi[2], nf[2]), fmaxf(hi[3], nf[3]));
            *reinterpret_cast<uint2*>(kmin + bi) = olo;
            *reinterpret_cast<uint2*>(kmax + bi) = ohi;
        }
    }
}

struct QuantConsts {
    int asym;
    float eps, qmax, inv_qmax, levels, inv_levels, offset;
};

// One value through the reference's quantiser, given the row's fitted step.
__device__ __forceinline__ int quant_sym(float x, float step, float qmax) {
    return (int)fminf(fmaxf(rintf(__fdiv_rn(x, step)), -qmax), qmax);
}
__device__ __forceinline__ int quant_asym(float x, float lo, float step, float levels,
                                          float offset) {
    const float u = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(x, lo), step)), 0.f), levels);
    return (int)__fsub_rn(u, offset);
}

// grid (ceil(B*H / 4)), one warp per (sequence, head); lane owns 4 channels.
__global__ void __launch_bounds__(128)
int8_decode_write_kernel(const __half* __restrict__ k, const __half* __restrict__ v,
                         const long long* __restrict__ slots,
                         const long long* __restrict__ res_idx, signed char* __restrict__ flat_v,
                         float* __restrict__ flat_v_scale, float* __restrict__ flat_v_zero,
                         __half* __restrict__ k_res, int batch, int heads, long long num_slots,
                         long long num_res, long long sk_b, long long sk_h, long long sv_b,
                         long long sv_h, QuantConsts c) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // let a programmatic successor start its prologue
    asm volatile("griddepcontrol.wait;\n" ::: "memory");                // launched programmatically, as the fp16 append
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= batch * heads) return;
    const int b = row / heads, h = row % heads;
    const long long slot = slots[b];
    const long long ridx = res_idx[b];
    if (slot < 0 || slot >= num_slots || ridx < 0 || ridx >= num_res) return;
    float x[4];
    unpack4(*reinterpret_cast<const uint2*>(v + b * sv_b + h * sv_h + lane * 4), x);
    const long long out_row = slot * heads + h;
    int q[4];
    if (!c.asym) {
        const float amax = warp_max(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
        const float step = __fmul_rn(fmaxf(amax, c.eps), c.inv_qmax);
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = quant_sym(x[j], step, c.qmax);
        if (lane == 0) flat_v_scale[out_row] = step;
    } else {
        const float hi = warp_max(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])));
        const float lo = -warp_max(fmaxf(fmaxf(-x[0], -x[1]), fmaxf(-x[2], -x[3])));
        const float step = fmaxf(__fmul_rn(__fsub_rn(hi, lo), c.inv_levels), c.eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = quant_asym(x[j], lo, step, c.levels, c.offset);
        if (lane == 0) {
            flat_v_scale[out_row] = step;
            flat_v_zero[out_row] = __fadd_rn(lo, __fmul_rn(c.offset, step));
        }
    }
    const uint32_t packed = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) |
                            ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    *reinterpret_cast<uint32_t*>(flat_v + out_row * LS_HEAD_DIM + lane * 4) = packed;
    // K stays exact in the fp16 residual until its page completes.
    *reinterpret_cast<uint2*>(k_res + (ridx * heads + h) * LS_HEAD_DIM + lane * 4) =
        *reinterpret_cast<const uint2*>(k + b * sk_b + h * sk_h + lane * 4);
}

// One residual row (a sequence's completed K page, exact fp16) quantised into one
// pool block, per (head, channel): thread = channel, loop over the page's 16 tokens.
__device__ __forceinline__ void finalize_page(const __half* __restrict__ k_res,
                                              signed char* __restrict__ k_pool,
                                              float* __restrict__ k_scale, float* __restrict__ k_zero,
                                              long long rr, long long blk, int h, int d, long long sr_r,
                                              long long sr_p, long long sr_h, long long sk_b,
                                              long long sk_p, long long sk_h, long long ss_b,
                                              long long ss_h, const QuantConsts& c) {
    const __half* src = k_res + rr * sr_r + h * sr_h + d;
    float f[LS_PAGE];
#pragma unroll
    for (int t = 0; t < LS_PAGE; ++t) f[t] = __half2float(src[t * sr_p]);
    signed char* dst = k_pool + blk * sk_b + h * sk_h + d;
    if (!c.asym) {
        float amax = 0.f;
#pragma unroll
        for (int t = 0; t < LS_PAGE; ++t) amax = fmaxf(amax, fabsf(f[t]));
        const float step = __fmul_rn(fmaxf(amax, c.eps), c.inv_qmax);
#pragma unroll
        for (int t = 0; t < LS_PAGE; ++t) dst[t * sk_p] = (signed char)quant_sym(f[t], step, c.qmax);
        k_scale[blk * ss_b + h * ss_h + d] = step;
    } else {
        float lo = f[0], hi = f[0];
#pragma unroll
        for (int t = 1; t < LS_PAGE; ++t) {
            lo = fminf(lo, f[t]);
            hi = fmaxf(hi, f[t]);
        }
        const float step = fmaxf(__fmul_rn(__fsub_rn(hi, lo), c.inv_levels), c.eps);
#pragma unroll
        for (int t = 0; t < LS_PAGE; ++t)
            dst[t * sk_p] = (signed char)quant_asym(f[t], lo, step, c.levels, c.offset);
        k_scale[blk * ss_b + h * ss_h + d] = step;
        k_zero[blk * ss_b + h * ss_h + d] = __fadd_rn(lo, __fmul_rn(c.offset, step));
    }
}

// grid (N, H, layers), block 128. Layers are the same tensors `s*_l` elements apart
// (0 for a single layer).
__global__ void __launch_bounds__(LS_HEAD_DIM)
int8_finalize_blocks_kernel(const __half* __restrict__ k_res, const long long* __restrict__ res_rows,
                            const long long* __restrict__ block_ids,
                            signed char* __restrict__ k_pool, float* __restrict__ k_scale,
                            float* __restrict__ k_zero, long long num_rows, long long num_blocks,
                            long long sr_r, long long sr_p, long long sr_h, long long sk_b,
                            long long sk_p, long long sk_h, long long ss_b, long long ss_h,
                            long long sr_l, long long sk_l, long long ss_l, QuantConsts c) {
    const int n = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const long long layer = blockIdx.z;
    const long long rr = res_rows[n], blk = block_ids[n];
    if (rr < 0 || rr >= num_rows || blk < 0 || blk >= num_blocks) return;
    finalize_page(k_res + layer * sr_l, k_pool + layer * sk_l, k_scale + layer * ss_l,
                  k_zero != nullptr ? k_zero + layer * ss_l : nullptr, rr, blk, h, d, sr_r, sr_p, sr_h,
                  sk_b, sk_p, sk_h, ss_b, ss_h, c);
}

// The same work with the page list's LENGTH on the device, so that the launch can be
// a fixed node of a captured decode step: grid (gx, H, layers) is set at capture, the
// CTAs stride over the first state[0] entries of res_rows / block_ids, and a step
// with nothing to finalise costs one read per CTA. The list is consumed once: the
// last CTA to arrive (state[1] counts arrivals; nobody waits) sets state[0] back to
// zero, so replaying the step again without a new list -- capture warm-ups, timing
// loops -- does not quantise a residual row that the append has since started to
// overwrite.
__global__ void __launch_bounds__(LS_HEAD_DIM)
int8_finalize_pending_kernel(const __half* __restrict__ k_res, const long long* __restrict__ res_rows,
                             const long long* __restrict__ block_ids, int* __restrict__ state,
                             signed char* __restrict__ k_pool, float* __restrict__ k_scale,
                             float* __restrict__ k_zero, int max_count, long long num_rows,
                             long long num_blocks, long long sr_r, long long sr_p, long long sr_h,
                             long long sk_b, long long sk_p, long long sk_h, long long ss_b,
                             long long ss_h, long long sr_l, long long sk_l, long long ss_l,
                             QuantConsts c) {
    __shared__ int s_count;
    if (threadIdx.x == 0) s_count = *reinterpret_cast<volatile int*>(state);
    __syncthreads();
    const int count = min(s_count, max_count);
    if (count <= 0) return;                              // the usual step: nothing completed
    const int h = blockIdx.y, d = threadIdx.x;
    const long long layer = blockIdx.z;
    for (int n = blockIdx.x; n < count; n += gridDim.x) {
        const long long rr = res_rows[n], blk = block_ids[n];
        if (rr < 0 || rr >= num_rows || blk < 0 || blk >= num_blocks) continue;
        finalize_page(k_res + layer * sr_l, k_pool + layer * sk_l, k_scale + layer * ss_l,
                      k_zero != nullptr ? k_zero + layer * ss_l : nullptr, rr, blk, h, d, sr_r, sr_p,
                      sr_h, sk_b, sk_p, sk_h, ss_b, ss_h, c);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // Every CTA has read the count before it arrives here, so the last arrival may clear it.
        __threadfence();
        const int total = (int)(gridDim.x * gridDim.y * gridDim.z);
        if (atomicAdd(state + 1, 1) == total - 1) {
            state[1] = 0;
            state[0] = 0;
        }
    }
}

}  // namespace ls

extern "C" {

int ls_kv_append_fp16(const void* k, const void* v, const int64_t* slots, void* k_pool, void* v_pool,
                      void* kmin, void* kmax, int batch, int kv_heads, int head_dim, int page,
                      int64_t num_slots, int64_t sk_b, int64_t sk_h, int64_t sv_b, int64_t sv_h,
                      int64_t sp_t, int64_t sp_h, int64_t sb_b, int64_t sb_h, void* stream) {
    if (!k || !slots) return LS_ERR_NULL_POINTER;
    if ((k_pool == nullptr) != (v_pool == nullptr) || (k_pool != nullptr && !v)) return LS_ERR_NULL_POINTER;
    if ((kmin == nullptr) != (kmax == nullptr)) return LS_ERR_NULL_POINTER;
    if (!k_pool && !kmin) return LS_ERR_NULL_POINTER;   // nothing to do
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (batch <= 0 || kv_heads <= 0 || num_slots <= 0) return LS_ERR_BAD_SHAPE;
    const int64_t strides[] = {sk_b, sk_h, sv_b, sv_h, sp_t, sp_h, sb_b, sb_h};
    for (int64_t s : strides)
        if (s % 4) return LS_ERR_MISALIGNED;
    const uintptr_t ptrs[] = {(uintptr_t)k, (uintptr_t)v, (uintptr_t)k_pool, (uintptr_t)v_pool,
                              (uintptr_t)kmin, (uintptr_t)kmax};
    for (uintptr_t a : ptrs)
        if (a & 7) return LS_ERR_MISALIGNED;
    const int rows = batch * kv_heads;
    // A programmatic launch (the kernel waits for its predecessor before it touches
    // memory); after a kernel that never triggers early this is an ordinary launch.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((rows + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const long long a_ns = num_slots, a_sk_b = sk_b, a_sk_h = sk_h, a_sv_b = sv_b, a_sv_h = sv_h,
                    a_sp_t = sp_t, a_sp_h = sp_h, a_sb_b = sb_b, a_sb_h = sb_h;
    cudaError_t e = cudaLaunchKernelEx(
        &cfg, ls::kv_append_fp16_kernel, static_cast<const __half*>(k), static_cast<const __half*>(v),
        reinterpret_cast<const long long*>(slots), static_cast<__half*>(k_pool),
        static_cast<__half*>(v_pool), static_cast<__half*>(kmin), static_cast<__half*>(kmax), batch,
        kv_heads, a_ns, a_sk_b, a_sk_h, a_sv_b, a_sv_h, a_sp_t, a_sp_h, a_sb_b, a_sb_h);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

int ls_int8_decode_write(const void* k, const void* v, const int64_t* slots, const int64_t* res_idx,
                         void* flat_v, float* flat_v_scale, float* flat_v_zero, void* k_res,
                         int batch, int kv_heads, int head_dim, int64_t num_slots, int64_t num_res,
                         int64_t sk_b, int64_t sk_h, int64_t sv_b, int64_t sv_h, int asym, float eps,
                         float qmax, float inv_qmax, float levels, float inv_levels, float offset,
                         void* stream) {
    if (!k || !v || !slots || !res_idx || !flat_v || !flat_v_scale || !k_res)
        return LS_ERR_NULL_POINTER;
    if (asym && !flat_v_zero) return LS_ERR_NULL_POINTER;
    if (head_dim != LS_HEAD_DIM) return LS_ERR_UNSUPPORTED;
    if (batch <= 0 || kv_heads <= 0 || num_slots <= 0 || num_res <= 0) return LS_ERR_BAD_SHAPE;
    if ((sk_b % 4) || (sk_h % 4) || (sv_b % 4) || (sv_h % 4)) return LS_ERR_MISALIGNED;
    if (((uintptr_t)k & 7) || ((uintptr_t)v & 7) || ((uintptr_t)flat_v & 3) || ((uintptr_t)k_res & 7))
        return LS_ERR_MISALIGNED;
    ls::QuantConsts c = {asym, eps, qmax, inv_qmax, levels, inv_levels, offset};
    const int rows = batch * kv_heads;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((rows + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const long long a_ns = num_slots, a_nr = num_res, a_sk_b = sk_b, a_sk_h = sk_h, a_sv_b = sv_b,
                    a_sv_h = sv_h;
    cudaError_t e = cudaLaunchKernelEx(
        &cfg, ls::int8_decode_write_kernel, static_cast<const __half*>(k), static_cast<const __half*>(v),
        reinterpret_cast<const long long*>(slots), reinterpret_cast<const long long*>(res_idx),
        static_cast<signed char*>(flat_v), flat_v_scale, flat_v_zero, static_cast<__half*>(k_res),
        batch, kv_heads, a_ns, a_nr, a_sk_b, a_sk_h, a_sv_b, a_sv_h, c);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

int ls_int8_finalize_layers(const void* k_res, const int64_t* res_rows, const int64_t* block_ids,
                            void* k_pool, float* k_scale, float* k_zero, int count, int layers,
                            int kv_heads, int head_dim, int page, int64_t num_rows, int64_t num_blocks,
                            int64_t sr_l, int64_t sr_r, int64_t sr_p, int64_t sr_h, int64_t sk_l,
                            int64_t sk_b, int64_t sk_p, int64_t sk_h, int64_t ss_l, int64_t ss_b,
                            int64_t ss_h, int asym, float eps, float qmax, float inv_qmax, float levels,
                            float inv_levels, float offset, void* stream) {
    if (!k_res || !res_rows || !block_ids || !k_pool || !k_scale) return LS_ERR_NULL_POINTER;
    if (asym && !k_zero) return LS_ERR_NULL_POINTER;
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (count < 0 || layers <= 0 || layers > 65535 || kv_heads <= 0 || kv_heads > 65535)
        return LS_ERR_BAD_SHAPE;
    if (count == 0) return LS_OK;
    ls::QuantConsts c = {asym, eps, qmax, inv_qmax, levels, inv_levels, offset};
    ls::int8_finalize_blocks_kernel<<<dim3(count, kv_heads, layers), LS_HEAD_DIM, 0,
                                      static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(k_res), reinterpret_cast<const long long*>(res_rows),
        reinterpret_cast<const long long*>(block_ids), static_cast<signed char*>(k_pool), k_scale,
        k_zero, num_rows, num_blocks, sr_r, sr_p, sr_h, sk_b, sk_p, sk_h, ss_b, ss_h, sr_l, sk_l, ss_l, c);
    return (int)cudaGetLastError();
}

int ls_int8_finalize_pending(const void* k_res, const int64_t* res_rows, const int64_t* block_ids,
                             int32_t* state, void* k_pool, float* k_scale, float* k_zero,
                             int max_count, int layers, int kv_heads, int head_dim, int page,
                             int64_t num_rows, int64_t num_blocks, int64_t sr_l, int64_t sr_r,
                             int64_t sr_p, int64_t sr_h, int64_t sk_l, int64_t sk_b, int64_t sk_p,
                             int64_t sk_h, int64_t ss_l, int64_t ss_b, int64_t ss_h, int asym, float eps,
                             float qmax, float inv_qmax, float levels, float inv_levels, float offset,
                             void* stream) {
    if (!k_res || !res_rows || !block_ids || !state || !k_pool || !k_scale) return LS_ERR_NULL_POINTER;
    if (asym && !k_zero) return LS_ERR_NULL_POINTER;
    if (head_dim != LS_HEAD_DIM || page != LS_PAGE) return LS_ERR_UNSUPPORTED;
    if (max_count <= 0 || layers <= 0 || layers > 65535 || kv_heads <= 0 || kv_heads > 65535)
        return LS_ERR_BAD_SHAPE;
    if ((uintptr_t)state & 3) return LS_ERR_MISALIGNED;
    ls::QuantConsts c = {asym, eps, qmax, inv_qmax, levels, inv_levels, offset};
    const int gx = max_count < 16 ? max_count : 16;
    ls::int8_finalize_pending_kernel<<<dim3(gx, kv_heads, layers), LS_HEAD_DIM, 0,
                                       static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(k_res), reinterpret_cast<const long long*>(res_rows),
        reinterpret_cast<const long long*>(block_ids), state, static_cast<signed char*>(k_pool), k_scale,
        k_zero, max_count, num_rows, num_blocks, sr_r, sr_p, sr_h, sk_b, sk_p, sk_h, ss_b, ss_h, sr_l, sk_l,
        ss_l, c);
    return (int)cudaGetLastError();
}

int ls_int8_finalize_blocks(const void* k_res, const int64_t* res_rows, const int64_t* block_ids,
                            void* k_pool, float* k_scale, float* k_zero, int count, int kv_heads,
                            int head_dim, int page, int64_t num_rows, int64_t num_blocks,
                            int64_t sr_r, int64_t sr_p, int64_t sr_h, int64_t sk_b, int64_t sk_p,
                            int64_t sk_h, int64_t ss_b, int64_t ss_h, int asym, float eps, float qmax,
                            float inv_qmax, float levels, float inv_levels, float offset,
                            void* stream) {
    return ls_int8_finalize_layers(k_res, res_rows, block_ids, k_pool, k_scale, k_zero, count, 1, kv_heads,
                                   head_dim, page, num_rows, num_blocks, 0, sr_r, sr_p, sr_h, 0, sk_b, sk_p,
                                   sk_h, 0, ss_b, ss_h, asym, eps, qmax, inv_qmax, levels, inv_levels,
                                   offset, stream);
}

}  // extern "C"
