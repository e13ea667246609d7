// Helpers shared by the block-scaled (tcgen05.mma kind::mxf8f6f4) MoE kernels.
#pragma once
#include "tc_common.cuh"

namespace gb200 {

constexpr int kMxSlab = 128;         // K elements per pipeline stage (4 MMAs of K = 32 per piece)
constexpr int kMxAtom = 512;         // bytes of one scale atom: 128 rows x 4 blocks
constexpr int kMxMaxExperts = 1024;

#if defined(__CUDACC__)

// K-major operand without swizzle: 8-row core matrices of 128 contiguous bytes,
// `sbo` bytes apart (the source format of the scale-atom copies).
__device__ __forceinline__ uint64_t umma_desc_k_plain(uint32_t smem_addr, uint32_t sbo)
{
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
    d |= uint64_t(sbo >> 4) << 32;
    d |= uint64_t(1) << 46;   // version
    return d;
}

// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated to
// the four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Instruction descriptor of kind::mxf8f6f4, both operands K-major, e8m0 scales; operand
// formats: 0 = e4m3, 5 = e2m1; `sf` selects which of the four blocks of the scale atoms
// this MMA uses.
constexpr uint32_t kMxFmtE4M3 = 0, kMxFmtE2M1 = 5;
__device__ __forceinline__ uint32_t mx_idesc_fmt(uint32_t a_fmt, uint32_t b_fmt, int m, int n, uint32_t sf)
{
    return (sf << 4) | (a_fmt << 7) | (b_fmt << 10) | (uint32_t(n >> 3) << 17) | (1u << 23) | (uint32_t(m >> 4) << 24) | (sf << 29);
}

__device__ __forceinline__ void umma_mx(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa,
                                        uint32_t sfb, bool accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)), "r"(sfa), "r"(sfb)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}


#endif  // __CUDACC__

}  // namespace gb200
