// Tensor-core (tcgen05 / TMEM) tile kernel of the int4 linear, for batches above
// the streaming kernel's 16 rows.
//
// The weights are the A operand: a CTA owns kATiles x 128 weight rows (8 strips per
// A tile) and up to 128 batch rows (the UMMA N dimension).  Per 64 columns of K:
//   producer warp   bulk-copies the packed strip-chunks (codes + scales) and issues
//                   the TMA load of the activation tile (128-byte swizzle);
//   8 dequant warps expand int4 -> bf16, multiply by the group scale and store the
//                   16-byte rows into the 128-byte-swizzled K-major A tile
//                   (the row interleave of the packed layout makes those stores
//                   bank-conflict free);
//   MMA warp        one thread issues 4 x kATiles tcgen05.mma (M=128, N=batch tile,
//                   K=16) into the TMEM accumulator and commits to the stage barrier;
//   4 epilogue warps read the accumulator with tcgen05.ld, round to bf16 and store
//                   y[m, n]; accumulators are double buffered so the next tile's
//                   main loop overlaps the epilogue.
// Numerics: w = bf16(q * s) (one rounding of the dequantised weight), products
// exact, fp32 accumulation in TMEM, bf16 output.
#include <algorithm>
#include <cstdlib>

#include "layout.h"
#include "tc_common.cuh"
#include "w4a16.h"

namespace gb200 {

constexpr int kTcTokens = 128;            // batch rows per tile (UMMA N, multiple of 16)
// Ring depths.  A (expanded weights) only has to cover the dequant -> MMA hand-off;
// B (activations, from L2 through TMA) has to cover about a microsecond of L2
// latency at ~0.4 us per 64-column tile; the packed ring is fed from L2 as well,
// because the producer prefetches packed chunks into L2 well ahead of their use.
__host__ __device__ constexpr int tc_a_stages(int atiles) { return atiles == 2 ? 3 : 4; }
__host__ __device__ constexpr int tc_b_stages(int atiles) { return atiles == 2 ? 4 : 6; }
constexpr int kTcPrefetchChunks = 8;      // packed chunks prefetched into L2 ahead of the ring
// Packed ring depth, in 128-column chunks.  The codes come from HBM (microseconds
// of latency against ~0.3 us per 64-column tile), so this ring is the deep one.
__host__ __device__ constexpr int tc_pack_stages(int atiles) { return atiles == 2 ? 3 : 4; }
// One dequant warp per strip of the CTA tile (8 per 128-row A tile): the expansion
// of a 64-column tile is then one 16-byte unit per lane, and the 16 warps of a
// 256-row tile keep all four schedulers busy.
__host__ __device__ constexpr int tc_dequant_warps(int atiles) { return 8 * atiles; }
constexpr int kTcEpilogueWarps = 4;
constexpr int kTcFirstDequantWarp = 3;    // warp 0: packed producer, 1: MMA, 2: activation producer
__host__ __device__ constexpr int tc_threads(int atiles)
{
    return (kTcFirstDequantWarp + tc_dequant_warps(atiles) + kTcEpilogueWarps) * 32;
}
constexpr int kTcChunkBytes = 1024 + 32;  // int4 strip-chunk
constexpr int kTcTileBytes = 128 * 128;   // one 128-row x 64-column 16-bit tile

struct TcParams {
    const uint8_t* packed;
    __nv_bfloat16* y;
    int* fault;
    int m, n, k;
    int ldy;
    int strips_padded, chunks;
    int panels, token_tiles;
    int kslices, chunks_per_slice;   // the K dimension of a tile may be cut into slices handled by different CTAs
    float* partial;                  // [kslices][m][n] fp32 partial sums (kslices > 1), else nullptr
    int scale_dtype;
};

// Work item -> (panel, batch tile, K slice) and the slice's chunk range.
struct TcItem {
    int panel, tt, c0, c1;
    int slice;
};
__device__ __forceinline__ TcItem tc_decode(const TcParams& p, int item)
{
    TcItem it;
    const int per_panel = p.token_tiles * p.kslices;
    it.panel = item / per_panel;
    const int rem = item - it.panel * per_panel;
    it.tt = rem / p.kslices;
    it.slice = rem - it.tt * p.kslices;
    it.c0 = it.slice * p.chunks_per_slice;
    it.c1 = min(p.chunks, it.c0 + p.chunks_per_slice);
    return it;
}

template <int kATiles>
struct TcSmem {
    static constexpr int a = 0;
    static constexpr int b = a + tc_a_stages(kATiles) * kATiles * kTcTileBytes;
    static constexpr int pk = b + tc_b_stages(kATiles) * kTcTileBytes;
    static constexpr int bars = pk + tc_pack_stages(kATiles) * kATiles * 8 * kTcChunkBytes;
    static constexpr int total = bars + 256 + 1024;   // barriers + slack for 1024-byte alignment
};

// One int4 word (8 codes of one row, pair-interleaved) times a scale -> 8 bf16.
__device__ __forceinline__ uint4 int4_word_to_bf16x8(uint32_t w, uint32_t scale_bf16x2)
{
    uint4 r;
    const uint32_t p0 = int4x2_to_bf16x2(w), p1 = int4x2_to_bf16x2(w >> 4), p2 = int4x2_to_bf16x2(w >> 8),
                   p3 = int4x2_to_bf16x2(w >> 12);
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r.x) : "r"(p0), "r"(scale_bf16x2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r.y) : "r"(p1), "r"(scale_bf16x2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r.z) : "r"(p2), "r"(scale_bf16x2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r.w) : "r"(p3), "r"(scale_bf16x2));
    return r;
}
// Same with an fp32 scale (fp16-scaled artifacts): q * s rounded once to bf16.
__device__ __forceinline__ uint4 int4_word_to_bf16x8_f32(uint32_t w, float s)
{
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t p = int4x2_to_bf16x2(w >> (4 * j));
        const float lo = __uint_as_float(p << 16) * s, hi = __uint_as_float(p & 0xffff0000u) * s;
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        out[j] = *reinterpret_cast<const uint32_t*>(&v);
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

template <int kATiles>
__global__ void __launch_bounds__(tc_threads(kATiles), 1)
w4a16_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap x_map,
                const __grid_constant__ CUtensorMap w_map)
{
    using S = TcSmem<kATiles>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_ring = smem + S::a;
    uint8_t* b_ring = smem + S::b;
    uint8_t* pk_ring = smem + S::pk;
    constexpr int kTcPackStages = tc_pack_stages(kATiles);
    constexpr int kAStages = tc_a_stages(kATiles);
    constexpr int kBStages = tc_b_stages(kATiles);
    constexpr int kTcDequantWarps = tc_dequant_warps(kATiles);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::bars);
    uint64_t* pk_full = bars;                          // [kTcPackStages]
    uint64_t* pk_empty = pk_full + kTcPackStages;      // [kTcPackStages]
    uint64_t* a_full = pk_empty + kTcPackStages;       // [kAStages]
    uint64_t* a_empty = a_full + kAStages;             // [kAStages]
    uint64_t* b_full = a_empty + kAStages;             // [kBStages]
    uint64_t* b_empty = b_full + kBStages;             // [kBStages]
    uint64_t* acc_full = b_empty + kBStages;           // [2]
    uint64_t* acc_empty = acc_full + 2;                // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    constexpr int kStripsPerPanel = 8 * kATiles;
    constexpr int kPackStageBytes = kStripsPerPanel * kTcChunkBytes;
    constexpr uint32_t kTmemCols = 2 * kATiles * 128;   // two accumulator buffers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcPackStages; ++s) {
            mbar_init(&pk_full[s], 1);
            mbar_init(&pk_empty[s], kTcDequantWarps);
        }
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&a_full[s], kTcDequantWarps);
            mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < kBStages; ++s) {
            mbar_init(&b_full[s], 1);
            mbar_init(&b_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], kTcEpilogueWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    const int items = p.panels * p.token_tiles * p.kslices;

    if (warp == 0) {
        // ------------------------------------- producer of packed codes + scales
        // Weights are constants: this stream starts before the previous kernel in the
        // stream has finished, and runs as far ahead as its ring allows.
        if (lane == 0) {
            // One thread feeds the ring, so its loop carries no divisions: the stage index, the
            // ring's wrap count and the prefetch cursor advance by increments.
            uint32_t ps = 0, round = 0, issued = 0, prefetched = 0;
            int pf_item = blockIdx.x;
            TcItem pf = pf_item < items ? tc_decode(p, pf_item) : TcItem{};
            int pf_c = pf.c0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const TcItem it = tc_decode(p, item);
                const int strip0 = it.panel * kStripsPerPanel;
                for (int c = it.c0; c < it.c1; ++c, ++issued) {
                    // keep the L2 prefetch kTcPrefetchChunks ahead of the ring, across items
                    while (pf_item < items && prefetched < issued + kTcPrefetchChunks) {
                        tma_prefetch_2d(&w_map, pf_c * (kTcChunkBytes / 8), pf.panel * kStripsPerPanel);
                        ++prefetched;
                        if (++pf_c == pf.c1) {
                            pf_item += gridDim.x;
                            if (pf_item < items) {
                                pf = tc_decode(p, pf_item);
                                pf_c = pf.c0;
                            }
                        }
                    }
                    if (round > 0 && !mbar_wait_bounded(&pk_empty[ps], (round - 1) & 1)) {
                        atomicExch(p.fault, 11);
                        *abort_flag = 1;
                        break;
                    }
                    // one TMA operation fetches chunk c of all the panel's strips (rows
                    // past the last strip are filled with zeros and count as bytes)
                    mbar_expect_tx(&pk_full[ps], kPackStageBytes);
                    tma_load_2d(pk_ring + ps * kPackStageBytes, &w_map, c * (kTcChunkBytes / 8), strip0, &pk_full[ps]);
                    if (++ps == kTcPackStages) {
                        ps = 0;
                        ++round;
                    }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------ producer of activation tiles
        if (lane == 0) {
            uint32_t ab_n = 0;
            pdl_wait();   // activations come from the previous kernel in the stream
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const TcItem it = tc_decode(p, item);
                const int tt = it.tt;
                for (int kt = 2 * it.c0; kt < 2 * it.c1; ++kt) {
                    const uint32_t s = ab_n % kBStages;
                    if (ab_n >= kBStages && !mbar_wait_bounded(&b_empty[s], ((ab_n / kBStages) - 1) & 1)) {
                        atomicExch(p.fault, 12);
                        *abort_flag = 1;
                        break;
                    }
                    mbar_expect_tx(&b_full[s], kTcTileBytes);
                    tma_load_2d(b_ring + s * kTcTileBytes, &x_map, kt * 64, tt * kTcTokens, &b_full[s]);
                    ++ab_n;
                }
            }
        }
    } else if (warp == 1) {
        // ----------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t ab_n = 0, it_n = 0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
                                // UMMA M = 128 batch rows (TMEM lanes), N = the tile's weight rows (TMEM columns)
                const uint32_t idesc = umma_idesc_f16(1, kTcTokens, kATiles * 128);
                const uint32_t buf = it_n & 1;
                if (it_n >= 2 && !mbar_wait_bounded(&acc_empty[buf], ((it_n >> 1) - 1) & 1)) {
                    atomicExch(p.fault, 13);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const TcItem it = tc_decode(p, item);
                const int ktiles = 2 * (it.c1 - it.c0);
                for (int kt = 0; kt < ktiles; ++kt) {
                    const uint32_t s = ab_n % kAStages, sb = ab_n % kBStages;
                    if (!mbar_wait_bounded(&a_full[s], (ab_n / kAStages) & 1) ||
                        !mbar_wait_bounded(&b_full[sb], (ab_n / kBStages) & 1)) {
                        atomicExch(p.fault, 14);
                        *abort_flag = 1;
                        break;
                    }
                    tc_fence_after();
                    // The activation tile is the UMMA A operand; the expanded weight tiles of
                    // the stage are contiguous and form one B operand of kATiles*128 rows.  One
                    // instruction per 16 columns of K reads 4 KiB + kATiles*4 KiB of shared memory.
                    const uint32_t x_addr = smem_u32(b_ring + sb * kTcTileBytes);
                    const uint32_t w_addr = smem_u32(a_ring + s * kATiles * kTcTileBytes);
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)
                        umma_f16(tmem_base + buf * (kATiles * 128), umma_desc_k_sw128(x_addr + k16 * 32),
                                 umma_desc_k_sw128(w_addr + k16 * 32), idesc, kt > 0 || k16 > 0);
                    umma_commit(&a_empty[s]);    // stages reusable once these MMAs have read them
                    umma_commit(&b_empty[sb]);
                    ++ab_n;
                }
                if (*abort_flag) break;
                umma_commit(&acc_full[buf]);
            }
        }
    } else if (warp < kTcFirstDequantWarp + kTcDequantWarps) {
        // -------------------------------------------------------------- dequant
        const int dq = warp - kTcFirstDequantWarp;
        const int g = lane >> 2, t = lane & 3;
        uint32_t pk_n = 0, ab_n = 0;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
            const TcItem it = tc_decode(p, item);
            const int panel = it.panel;
            const int valid = min(kStripsPerPanel, p.strips_padded - panel * kStripsPerPanel);
            for (int c = it.c0; c < it.c1 && !*abort_flag; ++c) {
                const uint32_t ps = pk_n % kTcPackStages;
                if (!mbar_wait_bounded(&pk_full[ps], (pk_n / kTcPackStages) & 1)) {
                    atomicExch(p.fault, 15);
                    *abort_flag = 1;
                    break;
                }
                const uint8_t* pk = pk_ring + ps * kPackStageBytes;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t s = ab_n % kAStages;
                    if (ab_n >= kAStages && !mbar_wait_bounded(&a_empty[s], ((ab_n / kAStages) - 1) & 1)) {
                        atomicExch(p.fault, 16);
                        *abort_flag = 1;
                        break;
                    }
                    tc_fence_after();
                    {
                        const int sidx = dq, at = dq >> 3;   // this warp's strip, and the A tile it belongs to
                        if (sidx < valid) {
                            const uint8_t* sc = pk + sidx * kTcChunkBytes;
                            const uint4 u = *reinterpret_cast<const uint4*>(sc + half * 512 + lane * 16);
                            const uint32_t sw = *reinterpret_cast<const uint32_t*>(sc + 1024 + g * 4);
                            uint4 v0, v1, v2, v3;
                            if (p.scale_dtype == GARNET_B200_BF16) {
                                const uint32_t s_lo = (sw & 0xffffu) * 0x10001u, s_hi = (sw >> 16) * 0x10001u;
                                v0 = int4_word_to_bf16x8(u.x, s_lo);
                                v1 = int4_word_to_bf16x8(u.y, s_hi);
                                v2 = int4_word_to_bf16x8(u.z, s_lo);
                                v3 = int4_word_to_bf16x8(u.w, s_hi);
                            } else {
                                const float f_lo = __half2float(__ushort_as_half(uint16_t(sw & 0xffffu)));
                                const float f_hi = __half2float(__ushort_as_half(uint16_t(sw >> 16)));
                                v0 = int4_word_to_bf16x8_f32(u.x, f_lo);
                                v1 = int4_word_to_bf16x8_f32(u.y, f_hi);
                                v2 = int4_word_to_bf16x8_f32(u.z, f_lo);
                                v3 = int4_word_to_bf16x8_f32(u.w, f_hi);
                            }
                            // rows R(g), R(g)+8 of strip dq; 16-byte chunks t and t+4, XOR-swizzled by row % 8
                            uint8_t* tile = a_ring + (s * kATiles + at) * kTcTileBytes;
                            const int r0 = (dq & 7) * 16 + row_of_g(g), r1 = r0 + 8;
                            const int x0 = r0 & 7;   // == r1 & 7
                            *reinterpret_cast<uint4*>(tile + r0 * 128 + ((t ^ x0) << 4)) = v0;
                            *reinterpret_cast<uint4*>(tile + r1 * 128 + ((t ^ x0) << 4)) = v1;
                            *reinterpret_cast<uint4*>(tile + r0 * 128 + (((t + 4) ^ x0) << 4)) = v2;
                            *reinterpret_cast<uint4*>(tile + r1 * 128 + (((t + 4) ^ x0) << 4)) = v3;
                        }
                    }
                    fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[s]);
                    ++ab_n;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&pk_empty[ps]);
                ++pk_n;
            }
        }
    } else {
        // ------------------------------------------------------------- epilogue
        const int quarter = warp & 3;   // TMEM lanes 32*quarter .. +31 belong to this warp
        uint32_t it_n = 0;
        bool waited = false;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
            const TcItem it = tc_decode(p, item);
            const int panel = it.panel, tt = it.tt;
            const uint32_t buf = it_n & 1;
            if (!mbar_wait_bounded(&acc_full[buf], (it_n >> 1) & 1)) {
                atomicExch(p.fault, 17);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            if (!waited) {
                pdl_wait();   // y may still be read by the previous kernel in the stream
                waited = true;
            }
            // TMEM lane = batch row of the tile, column = weight row of the panel: a thread
            // reads 32 consecutive outputs of its row and stores them as 64 contiguous bytes.
            const int m = tt * kTcTokens + quarter * 32 + lane;
            __nv_bfloat16* yrow = p.y + size_t(min(m, p.m - 1)) * p.ldy;
            const bool vec_ok = (p.ldy & 7) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15) == 0;
            for (int c0 = 0; c0 < kATiles * 128; c0 += 32) {
                const int n0 = panel * (kATiles * 128) + c0;
                if (n0 >= p.n) break;   // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + buf * (kATiles * 128) + c0, r);
                tmem_ld_wait();
                if (m >= p.m) continue;
                if (p.partial) {
                    // a K slice: fp32 partial sums, added up in slice order by the reduction kernel
                    float* prow = p.partial + (size_t(it.slice) * p.m + m) * p.n;
                    if (n0 + 32 <= p.n && (p.n & 3) == 0) {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            *reinterpret_cast<uint4*>(prow + n0 + 4 * q) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + j < p.n) prow[n0 + j] = __uint_as_float(r[j]);
                    }
                    continue;
                }
                if (vec_ok && n0 + 32 <= p.n) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * j]),
                                                                           __uint_as_float(r[8 * q + 2 * j + 1]));
                            w[j] = *reinterpret_cast<const uint32_t*>(&v);
                        }
                        *reinterpret_cast<uint4*>(yrow + n0 + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n0 + j < p.n) yrow[n0 + j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }

    // ---- teardown: every role arrives here, also after a wait that gave up
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// y[m, n] = bf16(sum of the K slices' partial sums, in slice order).  Four outputs per thread.
__global__ void w4a16_splitk_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ y, int m, int n, int ldy,
                                           int slices)
{
    pdl_wait();   // the partial sums come from the kernel before this one
    const size_t total = size_t(m) * n;
    const size_t idx = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (idx >= total) return;
    if ((n & 3) == 0 && (ldy & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 7) == 0) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < slices; ++s) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + size_t(s) * total + idx));
            sum.x += v.x;
            sum.y += v.y;
            sum.z += v.z;
            sum.w += v.w;
        }
        const __nv_bfloat162 a = __floats2bfloat162_rn(sum.x, sum.y), b = __floats2bfloat162_rn(sum.z, sum.w);
        *reinterpret_cast<uint2*>(y + (idx / n) * ldy + idx % n) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
    } else {
        for (size_t j = idx; j < min(idx + 4, total); ++j) {
            float sum = 0.f;
            for (int s = 0; s < slices; ++s) sum += partial[size_t(s) * total + j];
            y[(j / n) * ldy + j % n] = __float2bfloat16_rn(sum);
        }
    }
}

// ------------------------------------------------------------------ host side

// How the tile kernel cuts the work for a batch of m rows: 256-row panels when they
// already fill the machine, else 128-row panels, and K slices until there are about
// as many work items as SMs.
TcPlan tc_plan(const PackGeom& geo, int m)
{
    TcPlan t;
    t.token_tiles = (m + kTcTokens - 1) / kTcTokens;
    const int panels256 = (geo.strips_padded + 15) / 16;
    t.atiles = panels256 * t.token_tiles >= 2 * kSmCount ? 2 : 1;
    t.panels = t.atiles == 2 ? panels256 : geo.strips_padded / 8;
    const int tiles = t.panels * t.token_tiles;
    int want = tiles >= kSmCount ? 1 : (kSmCount + tiles - 1) / tiles;
    want = std::min(want, std::min(geo.chunks, 16));
    // every slice writes and the last one re-reads m x n fp32 partial sums: beyond a few MB per
    // slice that costs more than the idle SMs it saves
    const size_t plane = size_t(m) * geo.rows * sizeof(float);
    want = int(std::max<size_t>(1, std::min<size_t>(size_t(want), (size_t(6) << 20) / std::max<size_t>(plane, 1))));

    t.chunks_per_slice = (geo.chunks + want - 1) / want;
    t.kslices = (geo.chunks + t.chunks_per_slice - 1) / t.chunks_per_slice;
    t.workspace = t.kslices > 1 ? size_t(t.kslices) * m * geo.rows * sizeof(float) : 0;
    return t;
}

TensorMapEncodeFn tensor_map_encoder()
{
    static TensorMapEncodeFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<TensorMapEncodeFn>(ptr);
    }();
    return fn;
}

int make_tensor_map_2d_16bit(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return fail(GARNET_B200_NOT_SUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GARNET_B200_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code %d", int(r));
    return GARNET_B200_OK;
}

int make_tensor_map_2d_bytes(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                             uint64_t stride_bytes, uint32_t box_bytes, uint32_t box_rows)
{
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return fail(GARNET_B200_NOT_SUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {row_bytes / 8, rows};
    const cuuint64_t strides[1] = {stride_bytes};
    const cuuint32_t box[2] = {box_bytes / 8, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GARNET_B200_CUDA_ERROR, "cuTensorMapEncodeTiled (bytes) failed with code %d", int(r));
    return GARNET_B200_OK;
}

int W4A16::init_tc()
{
    static_assert(sizeof(tc_packed_map[0]) == sizeof(CUtensorMap), "tensor map storage size");
    for (int at = 1; at <= 2; ++at)
        if (int rc = make_tensor_map_2d_bytes(reinterpret_cast<CUtensorMap*>(&tc_packed_map[at - 1]), packed,
                                              uint64_t(geo.strips_padded), geo.strip_bytes(), geo.strip_bytes(),
                                              kTcChunkBytes, 8 * at))
            return rc;
    GB_CUDA(cudaFuncSetAttribute(w4a16_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<1>::total));
    GB_CUDA(cudaFuncSetAttribute(w4a16_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<2>::total));
    return GARNET_B200_OK;
}

int W4A16::launch_tc(const __nv_bfloat16* x, __nv_bfloat16* y, int m, void* ws, size_t ws_bytes, unsigned flags, cudaStream_t stream)
{
    CUtensorMap map;
    if (int rc = make_tensor_map_2d_16bit(&map, x, uint64_t(m), uint64_t(geo.cols), kTcTokens)) return rc;
    TcParams p;
    p.packed = packed;
    p.y = y;
    p.fault = fault_dev;
    p.m = m;
    p.n = geo.rows;
    p.k = geo.cols;
    p.ldy = geo.rows;
    p.strips_padded = geo.strips_padded;
    p.chunks = geo.chunks;
    const TcPlan plan = tc_plan(geo, m);
    p.token_tiles = plan.token_tiles;
    p.scale_dtype = scale_dtype;
    const int atiles = plan.atiles;
    p.panels = plan.panels;
    // K slices need the caller's workspace for their partial sums; without one the tiles keep all of K
    const bool sliced = plan.kslices > 1 && ws && ws_bytes >= plan.workspace && (reinterpret_cast<uintptr_t>(ws) & 15) == 0;
    p.kslices = sliced ? plan.kslices : 1;
    p.chunks_per_slice = sliced ? plan.chunks_per_slice : geo.chunks;
    p.partial = sliced ? static_cast<float*>(ws) : nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(std::min(p.panels * p.token_tiles * p.kslices, kSmCount)));
    cfg.blockDim = dim3(tc_threads(atiles));
    cfg.dynamicSmemBytes = atiles == 2 ? TcSmem<2>::total : TcSmem<1>::total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & 1u) ? 1 : 0;
    if (atiles == 2)
        GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_tc_kernel<2>, p, map, *reinterpret_cast<const CUtensorMap*>(&tc_packed_map[1])));
    else
        GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_tc_kernel<1>, p, map, *reinterpret_cast<const CUtensorMap*>(&tc_packed_map[0])));
    if (sliced) {
        const size_t quads = (size_t(m) * geo.rows + 3) / 4;
        cudaLaunchConfig_t rc = {};
        rc.gridDim = dim3(unsigned((quads + 255) / 256));
        rc.blockDim = dim3(256);
        rc.stream = stream;
        rc.attrs = attr;
        rc.numAttrs = 1;   // starts while the tile kernel drains; waits for its results on the device
        GB_CUDA(cudaLaunchKernelEx(&rc, w4a16_splitk_reduce_kernel, (const float*)p.partial, y, m, geo.rows, geo.rows, p.kslices));
    }
    return GARNET_B200_OK;
}

}  // namespace gb200
