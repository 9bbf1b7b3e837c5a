// Streaming primitives for the persistent weight-streaming kernels.
//
// Every warp owns a private ring of shared-memory stages.  One lane fills a stage with
// bulk asynchronous copies (cp.async.bulk, completion counted in bytes on an mbarrier);
// all lanes of the same warp wait on that mbarrier, consume the stage with 128-bit
// shared loads, and the lane refills it.  No block-level synchronisation is involved
// and the bytes in flight are bounded by shared memory, not by registers.
//
// Waits are bounded: after kWaitLimit failed polls the warp records a flag and stops.
#pragma once

#include "common.cuh"

namespace lemoq {

constexpr uint32_t kWaitLimit = 1u << 22;  // try_wait polls before a warp gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false = gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// Global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned),
// completing `bytes` transaction units on `bar`.  Local memory only, no multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_half(uint32_t addr) {
    unsigned short h;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
    return __half2float(__ushort_as_half(h));
}

// ---- int8 -> floating point without the conversion unit ------------------------------
// A code c in [-128, 127] is stored as byte b; b ^ 0x80 = c + 128 = u in [0, 255].
//
// DOT_F32_MAGIC  u dropped into byte 1 of the fp32 pattern 0x47000000 is exactly 32768 + u, so
//                sum c_j x_j = sum (32768 + u_j) x_j - 32896 * sum x_j: one PRMT + one FFMA per
//                code, but the products carry 9 extra magnitude bits (~15 significant bits left).
// DOT_F16_CVT    two codes per PRMT into the fp16 pattern 0x6400 | u = 1024 + u (exact), one HSUB2
//                by 1152 gives the exact codes as half2, widened to fp32 and FFMA'd: exact.
// DOT_F16_FOLD   the fp16 patterns 1024 + u are widened to fp32 as they are and the constant 1152 is
//                folded out: sum c_j x_j = sum (1024 + u_j) x_j - 1152 * sum x_j.  Products are exact
//                in fp32 (11 x 11 bits); the accumulation carries ~4 extra magnitude bits (~1e-6).
// DOT_F16_MIXED  same exact half2 codes, multiplied with the fp16 activations by the mixed
//                precision fma.rn.f32.f16 (fp32 accumulate): exact, activations stay packed fp16.
constexpr int DOT_F32_MAGIC = 0, DOT_F16_CVT = 1, DOT_F16_MIXED = 2, DOT_F16_FOLD = 3;
constexpr float kMagicOffset = 32896.0f;

__device__ __forceinline__ float magic_dot16(const uint4& w, const float* __restrict__ x) {
    const uint32_t u[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        a0 = fmaf(__uint_as_float(__byte_perm(u[i], 0x47000000u, 0x7404)), x[4 * i + 0], a0);
        a1 = fmaf(__uint_as_float(__byte_perm(u[i], 0x47000000u, 0x7414)), x[4 * i + 1], a1);
        a2 = fmaf(__uint_as_float(__byte_perm(u[i], 0x47000000u, 0x7424)), x[4 * i + 2], a2);
        a3 = fmaf(__uint_as_float(__byte_perm(u[i], 0x47000000u, 0x7434)), x[4 * i + 3], a3);
    }
    return (a0 + a1) + (a2 + a3);
}
__device__ __forceinline__ float sum16(const float* __restrict__ x) {
    float s0 = (x[0] + x[1]) + (x[2] + x[3]);
    float s1 = (x[4] + x[5]) + (x[6] + x[7]);
    float s2 = (x[8] + x[9]) + (x[10] + x[11]);
    float s3 = (x[12] + x[13]) + (x[14] + x[15]);
    return (s0 + s1) + (s2 + s3);
}

// Exact half2 pair of codes (bytes lo, lo+1 of the offset word u): (1024 + u) - 1152.
__device__ __forceinline__ __half2 codes_half2(uint32_t u, uint32_t sel) {
    const uint32_t bits = __byte_perm(u, 0x64646464u, sel);
    const uint32_t off = 0x64806480u;  // (1152, 1152)
    return __hsub2(*reinterpret_cast<const __half2*>(&bits), *reinterpret_cast<const __half2*>(&off));
}
__device__ __forceinline__ float exact_dot16_cvt(const uint4& w, const float* __restrict__ x) {
    const uint32_t u[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 lo = __half22float2(codes_half2(u[i], 0x4140));
        const float2 hi = __half22float2(codes_half2(u[i], 0x4342));
        a0 = fmaf(lo.x, x[4 * i + 0], a0);
        a1 = fmaf(lo.y, x[4 * i + 1], a1);
        a2 = fmaf(hi.x, x[4 * i + 2], a2);
        a3 = fmaf(hi.y, x[4 * i + 3], a3);
    }
    return (a0 + a1) + (a2 + a3);
}
constexpr float kFoldOffset = 1152.0f;
__device__ __forceinline__ float fold_dot16(const uint4& w, const float* __restrict__ x) {
    const uint32_t u[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t b0 = __byte_perm(u[i], 0x64646464u, 0x4140);
        const uint32_t b1 = __byte_perm(u[i], 0x64646464u, 0x4342);
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&b0));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&b1));
        a0 = fmaf(lo.x, x[4 * i + 0], a0);
        a1 = fmaf(lo.y, x[4 * i + 1], a1);
        a2 = fmaf(hi.x, x[4 * i + 2], a2);
        a3 = fmaf(hi.y, x[4 * i + 3], a3);
    }
    return (a0 + a1) + (a2 + a3);
}
// acc0 += c.lo * x.lo, acc1 += c.hi * x.hi with fp16 inputs and fp32 accumulation.
__device__ __forceinline__ void fma2_mixed(float& acc0, float& acc1, __half2 c, uint32_t x2) {
    const uint32_t cb = *reinterpret_cast<const uint32_t*>(&c);
    asm("{\n\t.reg .f16 cl, ch, xl, xh;\n\t"
        "mov.b32 {cl, ch}, %2;\n\t"
        "mov.b32 {xl, xh}, %3;\n\t"
        "fma.rn.f32.f16 %0, cl, xl, %0;\n\t"
        "fma.rn.f32.f16 %1, ch, xh, %1;\n\t}"
        : "+f"(acc0), "+f"(acc1)
        : "r"(cb), "r"(x2));
}
// x: 8 packed half2 words (16 activations).
__device__ __forceinline__ float exact_dot16_mixed(const uint4& w, const uint32_t* __restrict__ x) {
    const uint32_t u[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        fma2_mixed(a0, a1, codes_half2(u[i], 0x4140), x[2 * i]);
        fma2_mixed(a2, a3, codes_half2(u[i], 0x4342), x[2 * i + 1]);
    }
    return (a0 + a1) + (a2 + a3);
}

// ---- per-warp stage ring ---------------------------------------------------------------
// Shared layout (dynamic shared memory, 128-byte aligned):
//   [warp 0: STAGES x STAGE_BYTES][warp 1: ...] ... [barriers: warps x STAGES x 8 bytes]
template <int STAGES>
struct WarpRing {
    uint32_t data;   // shared address of this warp's stage 0
    uint32_t bars;   // shared address of this warp's barrier 0
    uint32_t stage_bytes;

    __device__ __forceinline__ void init(unsigned char* smem, int warp, int warps, uint32_t stage_bytes_, int lane) {
        stage_bytes = stage_bytes_;
        data = smem_u32(smem) + static_cast<uint32_t>(warp) * STAGES * stage_bytes;
        bars = smem_u32(smem) + static_cast<uint32_t>(warps) * STAGES * stage_bytes + static_cast<uint32_t>(warp) * STAGES * 8u;
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < STAGES; ++s) mbar_init(bars + 8u * s, 1u);
            mbar_fence_init();
        }
        __syncwarp();
    }
    __device__ __forceinline__ uint32_t stage(int s) const { return data + static_cast<uint32_t>(s) * stage_bytes; }
    __device__ __forceinline__ uint32_t bar(int s) const { return bars + 8u * static_cast<uint32_t>(s); }
    static __host__ __device__ size_t smem_bytes(int warps, size_t stage_bytes_) {
        return static_cast<size_t>(warps) * STAGES * stage_bytes_ + static_cast<size_t>(warps) * STAGES * 8;
    }
};

}  // namespace lemoq
