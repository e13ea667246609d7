// Shared device/host helpers for the B200 quantized-matmul kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../../include/garnet_b200.h"

namespace gb200 {

// Records a message for garnet_b200_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* where);

#define GB_CUDA(expr)                                             \
    do {                                                          \
        cudaError_t e__ = (expr);                                 \
        if (e__ != cudaSuccess) return gb200::cuda_fail(e__, #expr); \
    } while (0)

constexpr int kSmCount = 148;

#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier (shared::cta) ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Nanoseconds of the GPU's global timer (the same clock for every SM).
__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Default limit of every device-side wait: far longer than any copy or kernel of
// this library takes, short enough that a protocol error ends in a fault word
// and not in a hung GPU.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

// Bounded wait: returns false (and the caller records a fault) if the phase does
// not complete within `limit_ns` of the global timer.  The timer is read once
// per 256 polls, so the fast path costs nothing extra.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns = kWaitLimitNs)
{
    for (int spin = 0; spin < 256; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int spin = 0; spin < 256; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Programmatic dependent launch: wait for the producer grid's memory, and let
// the dependent grid start its own prologue early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t r;   // (a & b) ^ c : truth table 0x6a
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// Two int4 codes (two's complement) -> exact bf16x2 integers in [-8, 7].
// Nibble j (bits 4j) lands in the low half and nibble j+4 (bits 4j+16) in the
// high half: 0x4300 | (nibble ^ 8) is the bf16 number 128 + (q + 8); subtracting
// 136 leaves q.
__device__ __forceinline__ uint32_t int4x2_to_bf16x2(uint32_t word_shifted)
{
    const uint32_t t = lop3_and_xor(word_shifted, 0x000F000Fu, 0x43084308u);
    uint32_t r;
    const uint32_t bias = 0x43084308u;   // bf16x2 {136, 136}
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(t), "r"(bias));
    return r;
}

// One byte holding two e2m1 codes (low nibble first) -> f16x2, by the sm_100a
// conversion instruction; all 16 codes are exact in fp16.  `word` must come from
// a 32-bit (or wider) load: when the operand is a zero-extended byte load, the
// byte unpack below was observed to yield zero with nvcc 12.9.
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t word, int byte_index)
{
    uint32_t r;
    switch (byte_index) {
        case 0: asm("{ .reg .b8 b0,b1,b2,b3; mov.b32 {b0,b1,b2,b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b0; }" : "=r"(r) : "r"(word)); break;
        case 1: asm("{ .reg .b8 b0,b1,b2,b3; mov.b32 {b0,b1,b2,b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b1; }" : "=r"(r) : "r"(word)); break;
        case 2: asm("{ .reg .b8 b0,b1,b2,b3; mov.b32 {b0,b1,b2,b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b2; }" : "=r"(r) : "r"(word)); break;
        default: asm("{ .reg .b8 b0,b1,b2,b3; mov.b32 {b0,b1,b2,b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b3; }" : "=r"(r) : "r"(word)); break;
    }
    return r;
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                              const float (&c)[4])
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]),
          "f"(c[3]));
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                             const float (&c)[4])
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]),
          "f"(c[3]));
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ float bf16_round_f(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

#endif  // __CUDACC__

}  // namespace gb200
