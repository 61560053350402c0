// Shared device helpers for the paged decode-attention kernels (sm_100a).
//
// Everything here is warp-synchronous, register- or shared-memory-level
// plumbing: cp.async (16-byte global->shared copies with zero-fill), ldmatrix,
// the m16n8k16 fp16 tensor-core MMA with fp32 accumulation, the 8x8 register
// transpose (movmatrix), ex2, and the status codes the C-ABI returns.
//
// None of the kernels built on this header spin on a flag, an mbarrier or a
// peer: data arrives through cp.async groups, which complete on their own, so
// there is no wait that could hang a GPU.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// L2 prefetch granularity asked of the 16-byte page loads (rows are 256 B
// contiguous for fp16 pools, 128 B for INT8 pools).
#ifndef LS_CP_L2_HINT
#define LS_CP_L2_HINT ".L2::128B"
#endif

#define LS_HEAD_DIM 128
#define LS_PAGE 16
#define LS_FULL_MASK 0xffffffffu

// Status codes returned by every extern "C" entry point (0 = ok, > 0 is a
// cudaError_t from the launch, < 0 is an argument-validation failure).
#define LS_OK 0
#define LS_ERR_NULL_POINTER (-1)
#define LS_ERR_BAD_SHAPE (-2)
#define LS_ERR_BAD_STRIDE (-3)
#define LS_ERR_MISALIGNED (-4)
#define LS_ERR_TOO_LARGE (-5)
#define LS_ERR_UNSUPPORTED (-6)
#define LS_ERR_SCRATCH_TOO_SMALL (-7)
#ifndef LS_LAUNCH_PROGRAMMATIC
#define LS_LAUNCH_PROGRAMMATIC 0x100
#endif
#define LS_LOAD_CP_ASYNC 0x200
#define LS_LOAD_TMA 0x400
#define LS_EARLY_PAGES 0x800
#define LS_LOAD_TMA_SPLIT_KV 0x1000
#define LS_GEMM_NORM 1
#define LS_GEMM_SWIGLU 2

namespace ls {

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }
__device__ __forceinline__ float pos_inf() { return __int_as_float(0x7f800000); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous copy, L1-bypassing. src_bytes == 0 writes 16 zero bytes
// and reads nothing, which is how rows past a sequence's end are kept free of
// whatever bit patterns (NaN included) the pool holds there.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global" LS_CP_L2_HINT " [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
                 "r"(src_bytes)
                 : "memory");
}

// The same copy for rows known to exist (no source-size operand).
__device__ __forceinline__ void cp_async_16_full(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global" LS_CP_L2_HINT " [%0], [%1], 16;\n" ::"r"(dst), "l"(src)
                 : "memory");
}

// KV pages are read once per decode step: marking them evict-first keeps the
// small, re-read inputs (block tables, lengths, queries, partials) in L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void cp_async_16_stream(uint32_t dst, const void* src, uint64_t pol) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint" LS_CP_L2_HINT " [%0], [%1], 16, 16, %2;\n" ::"r"(dst),
                 "l"(src), "l"(pol)
                 : "memory");
}

// 8-byte copy with zero-fill: `src_bytes` (0 or 8) are read, the rest of the 8 are zeros.
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(dst), "l"(src),
                 "r"(src_bytes)
                 : "memory");
}

// 4-byte asynchronous copy (scalars such as a per-token V scale).
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src),
                 "r"(src_bytes)
                 : "memory");
}

__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}

template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Packed fp32 pairs (sm_100 has two-wide fp32 add / mul / fma on 64-bit
// registers; each half is an ordinary IEEE operation).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// ---------------------------------------------------------------------------
// TMA (bulk asynchronous copies into shared memory, completion counted in bytes
// on an mbarrier). One lane issues a whole tile; nobody computes addresses per
// 16 bytes. No cluster multicast is used anywhere.
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(mbar) : "memory");
}
// One probe of the phase with the given parity; the instruction itself waits a
// bounded, implementation-defined time before it answers "not yet".
__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(mbar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false if the phase did not complete within `limit` probes. The first
// probe, which usually finds the data there, is inline; the loop is kept out of line.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t mbar, uint32_t parity, int limit) {
    for (int i = 1; i < limit; ++i)
        if (mbar_try_wait(mbar, parity)) return true;
    return false;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity, int limit) {
    if (mbar_try_wait(mbar, parity)) return true;
    return mbar_wait_slow(mbar, parity, limit);
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t mbar, int c0,
                                            int c1, int c2, int c3, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;\n" ::"r"(dst),
        "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(mbar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void* tmap, uint32_t mbar, int c0,
                                            int c1, int c2, int c3, int c4, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;\n" ::"r"(dst),
        "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(mbar), "l"(policy)
        : "memory");
}
// Untiled bulk copy: both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
            "r"(dst),
        "l"(src), "r"(bytes), "r"(mbar)
        : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D = A(16x16, fp16, row) * B(16x8, fp16, col) + D, fp32 accumulators.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Transpose an 8x8 matrix of 16-bit values held one row-pair per lane.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Four bytes already biased to unsigned (x ^ 0x80) -> two half2 registers
// holding the signed values exactly: bytes (0,1) and bytes (2,3).
// 0x6400 | u is the fp16 number 1024 + u; subtracting 1152 = 1024 + 128
// undoes the bias. Every step is exact.
__device__ __forceinline__ void bytes4_to_half2x2(uint32_t biased, uint32_t& lo, uint32_t& hi) {
    const uint32_t magic = 0x64646464u;
    uint32_t a = prmt(biased, magic, 0x4140u);   // [b0, 0x64, b1, 0x64]
    uint32_t b = prmt(biased, magic, 0x4342u);   // [b2, 0x64, b3, 0x64]
    const __half2 off = __floats2half2_rn(1152.f, 1152.f);
    __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), off);
    __half2 hb = __hsub2(*reinterpret_cast<__half2*>(&b), off);
    lo = *reinterpret_cast<uint32_t*>(&ha);
    hi = *reinterpret_cast<uint32_t*>(&hb);
}

}  // namespace ls
