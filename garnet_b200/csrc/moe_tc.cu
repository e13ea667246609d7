// Tensor-core (tcgen05 / TMEM) grouped GEMM of the gpt-oss MXFP4 experts, used when
// experts receive many rows (prefill).  It replaces, at those sizes, the reference's
// grouped WMMA kernel (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:843-906) and its Marlin
// adapter (plugins/gpt_oss/cuda/gpt_oss_marlin.cu:586-648).
//
// Rows are first gathered into expert order (slot list sorted by expert, as the
// reference does for Marlin, gpt_oss_marlin.cu:239-277), so that the rows of one
// expert are contiguous and a TMA box fetches a tile of them.  A work item is
// (expert, tile of up to 128 rows, panel of 256 weight rows).  Per 64 columns of K:
//   producers      one TMA operation for the 16 packed strip-chunks (codes + e8m0
//                  scales) of the panel, one TMA operation for the activation tile;
//   16 dequant warps   cvt.rn.f16x2.e2m1x2 + one fp16 multiply by 2^(e - ref) per
//                  pair, stored into the 128-byte-swizzled K-major A tiles;
//   MMA warp       8 tcgen05.mma (M=128, N=rows, K=16, fp16 in, fp32 accumulate in TMEM);
//   4 epilogue warps   tcgen05.ld, undo the exponent offsets, then either bias +
//                  clamped SwiGLU -> fp16 activation rows (gate/up projection) or
//                  bias -> per-slot values for the combine (down projection).
// Exponent bookkeeping: weights enter as code * 2^(e - ref) with ref = (largest scale
// byte of the matrix kind) - 12, exact in fp16 when the scale bytes span at most 24
// binades (checked at create time; otherwise this path is not used); activations
// are the per-token normalised fp16 rows.  The epilogue multiplies the fp32
// accumulator by 2^(ref - 127 + xshift[row]), an exact power of two.
#include <algorithm>

#include "layout.h"
#include "moe.h"
#include "tc_common.cuh"

namespace gb200 {

constexpr int kMtTokens = 128;                 // rows per tile (UMMA N)
constexpr int kMtATiles = 2;                   // 256 weight rows per CTA tile
constexpr int kMtStrips = 8 * kMtATiles;
constexpr int kMtAStages = 3, kMtBStages = 4, kMtPackStages = 6;
constexpr int kMtPrefetch = 12;                // packed k-tiles prefetched into L2 ahead of the ring
constexpr int kMtDequantWarps = kMtStrips;
constexpr int kMtFirstDequantWarp = 3;
constexpr int kMtThreads = (kMtFirstDequantWarp + kMtDequantWarps + 4) * 32;
constexpr int kMtChunkBytes = 512 + 32;
constexpr int kMtTileBytes = 128 * 128;
constexpr int kMtPackStageBytes = kMtStrips * kMtChunkBytes;
constexpr int kMtMaxExperts = 1024;

struct MtSmem {
    static constexpr int a = 0;
    static constexpr int b = a + kMtAStages * kMtATiles * kMtTileBytes;
    static constexpr int pk = b + kMtBStages * kMtTileBytes;
    static constexpr int prefix = pk + kMtPackStages * kMtPackStageBytes;   // int[kMtMaxExperts + 1]
    static constexpr int bars = prefix + (kMtMaxExperts + 1) * 4 + 12;
    static constexpr int total = bars + 512 + 1024;
};

struct MtParams {
    const int* offsets;        // [experts + 1] start of every expert's rows in sorted order
    const int* sorted;         // [slots] slot ids in expert order
    const int* xshift_g;       // [slots] exponent of the fp16 row (up) or null (down)
    const float* bias;         // [experts(local or global), rows] original row order
    __half* act_out;           // up: [slots, inter] in sorted order
    float* vals_out;           // down: [slots(by slot id), hidden]
    int* fault;
    int experts;               // global expert count
    int rows;                  // logical rows of the weight matrix (2I or H)
    int strips_padded;
    int chunks;                // 64-column tiles along K
    int panels;                // 256-row panels per expert
    int expert_base, expert_div, bias_by_global;
    int expert_lo, expert_hi, interleave_world, interleave_rank;   // which experts are local
    int ref_exp;               // weights carry 2^(e - ref_exp)
    float limit;
};

__device__ __forceinline__ bool mt_expert_local(const MtParams& p, int e)
{
    if (p.interleave_world > 1) return (e % p.interleave_world) == p.interleave_rank;
    return e >= p.expert_lo && e < p.expert_hi;
}

// Item -> (expert, row tile, panel): items are numbered expert by expert, row tile
// by row tile, panels fastest, so that CTAs running side by side share the
// activation tile (L2) while the expert's weights stream once from HBM.
struct MtItem {
    int expert, tile, panel, row0, rows;
};
__device__ __forceinline__ MtItem mt_decode(const MtParams& p, const int* tile_prefix, const int* offsets, int item,
                                            int& cursor)
{
    const int t = item / p.panels;
    while (tile_prefix[cursor + 1] <= t) ++cursor;
    MtItem it;
    it.expert = cursor;
    it.tile = t - tile_prefix[cursor];
    it.panel = item % p.panels;
    it.row0 = offsets[cursor] + it.tile * kMtTokens;
    it.rows = min(kMtTokens, offsets[cursor + 1] - it.row0);
    return it;
}

// One e2m1 word (8 codes of one row) times 2^(e - ref) -> 8 fp16.
__device__ __forceinline__ uint4 e2m1_word_to_f16x8(uint32_t w, uint32_t scale_f16x2)
{
    uint4 r;
    const uint32_t p0 = e2m1x2_to_f16x2(w, 0), p1 = e2m1x2_to_f16x2(w, 1), p2 = e2m1x2_to_f16x2(w, 2),
                   p3 = e2m1x2_to_f16x2(w, 3);
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r.x) : "r"(p0), "r"(scale_f16x2));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r.y) : "r"(p1), "r"(scale_f16x2));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r.z) : "r"(p2), "r"(scale_f16x2));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r.w) : "r"(p3), "r"(scale_f16x2));
    return r;
}

// fp16x2 {2^(e - ref), 2^(e - ref)}; the exponent field is clamped to the normal
// range so that padding scales (whose codes are zero) cannot produce inf or NaN.
__device__ __forceinline__ uint32_t e8m0_to_f16x2_rel(uint32_t e, int ref)
{
    const int field = max(1, min(30, int(e) - ref + 15));
    return uint32_t(field << 10) * 0x10001u;
}

template <bool kUp>
__global__ void __launch_bounds__(kMtThreads, 1)
moe_tc_kernel(const MtParams p, const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map)
{
    using S = MtSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_ring = smem + S::a;
    uint8_t* b_ring = smem + S::b;
    uint8_t* pk_ring = smem + S::pk;
    int* tile_prefix = reinterpret_cast<int*>(smem + S::prefix);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::bars);
    uint64_t* pk_full = bars;
    uint64_t* pk_empty = pk_full + kMtPackStages;
    uint64_t* a_full = pk_empty + kMtPackStages;
    uint64_t* a_empty = a_full + kMtAStages;
    uint64_t* b_full = a_empty + kMtAStages;
    uint64_t* b_empty = b_full + kMtBStages;
    uint64_t* acc_full = b_empty + kMtBStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    constexpr uint32_t kTmemCols = 2 * kMtATiles * 128;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kMtPackStages; ++s) {
            mbar_init(&pk_full[s], 1);
            mbar_init(&pk_empty[s], kMtDequantWarps);
        }
        for (int s = 0; s < kMtAStages; ++s) {
            mbar_init(&a_full[s], kMtDequantWarps);
            mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < kMtBStages; ++s) {
            mbar_init(&b_full[s], 1);
            mbar_init(&b_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    pdl_wait();   // offsets and rows come from the earlier kernels of this call
    if (warp == 2) {
        // prefix of row tiles per expert: tile_prefix[e] = sum_{q<e} ceil(count_q / 128)
        int run = 0;
        for (int e0 = 0; e0 < p.experts; e0 += 32) {
            const int e = e0 + lane;
            int tiles = 0;
            if (e < p.experts) tiles = (p.offsets[e + 1] - p.offsets[e] + kMtTokens - 1) / kMtTokens;
            int incl = tiles;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += v;
            }
            if (e < p.experts) tile_prefix[e] = run + incl - tiles;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) tile_prefix[p.experts] = run;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int items = tile_prefix[p.experts] * p.panels;
    const int ktiles = p.chunks;

    if (warp == 0) {
        // ------------------------------------- producer of packed codes + scales
        if (lane == 0) {
            uint32_t pk_n = 0, pf_n = 0;
            int cur = 0, pf_cur = 0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const MtItem it = mt_decode(p, tile_prefix, p.offsets, item, cur);
                const int se = (it.expert - p.expert_base) / p.expert_div;
                const int strip0 = se * p.strips_padded + it.panel * kMtStrips;
                for (int c = 0; c < ktiles; ++c) {
                    while (pf_n < pk_n + kMtPrefetch) {
                        const int pf_item = blockIdx.x + int(pf_n / ktiles) * gridDim.x;
                        if (pf_item >= items) break;
                        const MtItem pi = mt_decode(p, tile_prefix, p.offsets, pf_item, pf_cur);
                        const int pse = (pi.expert - p.expert_base) / p.expert_div;
                        tma_prefetch_2d(&w_map, int(pf_n % ktiles) * (kMtChunkBytes / 8),
                                        pse * p.strips_padded + pi.panel * kMtStrips);
                        ++pf_n;
                    }
                    const uint32_t ps = pk_n % kMtPackStages;
                    if (pk_n >= kMtPackStages && !mbar_wait_bounded(&pk_empty[ps], ((pk_n / kMtPackStages) - 1) & 1)) {
                        atomicExch(p.fault, 21);
                        *abort_flag = 1;
                        break;
                    }
                    mbar_expect_tx(&pk_full[ps], kMtPackStageBytes);
                    tma_load_2d(pk_ring + ps * kMtPackStageBytes, &w_map, c * (kMtChunkBytes / 8), strip0, &pk_full[ps]);
                    ++pk_n;
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------ producer of activation tiles
        if (lane == 0) {
            uint32_t ab_n = 0;
            int cur = 0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const MtItem it = mt_decode(p, tile_prefix, p.offsets, item, cur);
                for (int kt = 0; kt < ktiles; ++kt) {
                    const uint32_t s = ab_n % kMtBStages;
                    if (ab_n >= kMtBStages && !mbar_wait_bounded(&b_empty[s], ((ab_n / kMtBStages) - 1) & 1)) {
                        atomicExch(p.fault, 22);
                        *abort_flag = 1;
                        break;
                    }
                    mbar_expect_tx(&b_full[s], kMtTileBytes);
                    tma_load_2d(b_ring + s * kMtTileBytes, &x_map, kt * 64, it.row0, &b_full[s]);
                    ++ab_n;
                }
            }
        }
    } else if (warp == 1) {
        // ----------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t ab_n = 0, it_n = 0;
            int cur = 0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
                const MtItem it = mt_decode(p, tile_prefix, p.offsets, item, cur);
                // UMMA M = 128 rows (TMEM lanes), N = 256 weight rows of the panel (TMEM columns)
                const uint32_t idesc = umma_idesc_f16(0, kMtTokens, kMtATiles * 128);
                const uint32_t buf = it_n & 1;
                if (it_n >= 2 && !mbar_wait_bounded(&acc_empty[buf], ((it_n >> 1) - 1) & 1)) {
                    atomicExch(p.fault, 23);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                for (int kt = 0; kt < ktiles; ++kt) {
                    const uint32_t s = ab_n % kMtAStages, sb = ab_n % kMtBStages;
                    if (!mbar_wait_bounded(&a_full[s], (ab_n / kMtAStages) & 1) ||
                        !mbar_wait_bounded(&b_full[sb], (ab_n / kMtBStages) & 1)) {
                        atomicExch(p.fault, 24);
                        *abort_flag = 1;
                        break;
                    }
                    tc_fence_after();
                    // rows are the UMMA A operand; the two expanded weight tiles of the stage
                    // are contiguous and form one 256-row B operand
                    const uint32_t x_addr = smem_u32(b_ring + sb * kMtTileBytes);
                    const uint32_t w_addr = smem_u32(a_ring + s * kMtATiles * kMtTileBytes);
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)
                        umma_f16(tmem_base + buf * (kMtATiles * 128), umma_desc_k_sw128(x_addr + k16 * 32),
                                 umma_desc_k_sw128(w_addr + k16 * 32), idesc, kt > 0 || k16 > 0);
                    umma_commit(&a_empty[s]);
                    umma_commit(&b_empty[sb]);
                    ++ab_n;
                }
                if (*abort_flag) break;
                umma_commit(&acc_full[buf]);
            }
        }
    } else if (warp < kMtFirstDequantWarp + kMtDequantWarps) {
        // -------------------------------------------------------------- dequant
        const int dq = warp - kMtFirstDequantWarp;   // strip of the panel
        const int at = dq >> 3;
        const int g = lane >> 2, t = lane & 3;
        const int r0 = (dq & 7) * 16 + row_of_g(g), r1 = r0 + 8, x0 = r0 & 7;
        uint32_t pk_n = 0, ab_n = 0;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
            for (int c = 0; c < ktiles && !*abort_flag; ++c) {
                const uint32_t ps = pk_n % kMtPackStages;
                if (!mbar_wait_bounded(&pk_full[ps], (pk_n / kMtPackStages) & 1)) {
                    atomicExch(p.fault, 25);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t s = ab_n % kMtAStages;
                if (ab_n >= kMtAStages && !mbar_wait_bounded(&a_empty[s], ((ab_n / kMtAStages) - 1) & 1)) {
                    atomicExch(p.fault, 26);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint8_t* sc = pk_ring + ps * kMtPackStageBytes + dq * kMtChunkBytes;
                const uint4 u = *reinterpret_cast<const uint4*>(sc + lane * 16);
                const uint32_t sw = *reinterpret_cast<const uint32_t*>(sc + 512 + g * 4);
                // words: x = (row R, octet t), y = (R+8, t), z = (R, t+4), w = (R+8, t+4);
                // scale bytes: (R, group 0), (R+8, group 0), (R, group 1), (R+8, group 1)
                const uint4 v0 = e2m1_word_to_f16x8(u.x, e8m0_to_f16x2_rel(sw & 0xff, p.ref_exp));
                const uint4 v1 = e2m1_word_to_f16x8(u.y, e8m0_to_f16x2_rel((sw >> 8) & 0xff, p.ref_exp));
                const uint4 v2 = e2m1_word_to_f16x8(u.z, e8m0_to_f16x2_rel((sw >> 16) & 0xff, p.ref_exp));
                const uint4 v3 = e2m1_word_to_f16x8(u.w, e8m0_to_f16x2_rel(sw >> 24, p.ref_exp));
                uint8_t* tile = a_ring + (s * kMtATiles + at) * kMtTileBytes;
                *reinterpret_cast<uint4*>(tile + r0 * 128 + ((t ^ x0) << 4)) = v0;
                *reinterpret_cast<uint4*>(tile + r1 * 128 + ((t ^ x0) << 4)) = v1;
                *reinterpret_cast<uint4*>(tile + r0 * 128 + (((t + 4) ^ x0) << 4)) = v2;
                *reinterpret_cast<uint4*>(tile + r1 * 128 + (((t + 4) ^ x0) << 4)) = v3;
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&a_full[s]);
                    mbar_arrive(&pk_empty[ps]);
                }
                ++ab_n;
                ++pk_n;
            }
        }
    } else {
        // ------------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        const int l = quarter * 32 + lane;        // TMEM lane = row of the 128-row A tile
        uint32_t it_n = 0;
        int cur = 0;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
            const MtItem it = mt_decode(p, tile_prefix, p.offsets, item, cur);
            const uint32_t buf = it_n & 1;
            if (!mbar_wait_bounded(&acc_full[buf], (it_n >> 1) & 1)) {
                atomicExch(p.fault, 27);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const int ebias = p.bias_by_global ? it.expert : (it.expert - p.expert_base) / p.expert_div;
            // TMEM lane = row of the tile (a routed slot), column = weight row of the panel.
            const bool live = l < it.rows;
            const int pos = it.row0 + min(l, it.rows - 1);
            const float* bias = p.bias + size_t(ebias) * p.rows;
            if (kUp) {
                // 32 columns = two strips; in a strip, columns 0..7 are the gates and 8..15 the
                // ups of channels 8*strip .. 8*strip+7 (the repacker's row order).
                const float f = __uint_as_float(uint32_t(p.ref_exp + p.xshift_g[pos]) << 23);
                __half* arow = p.act_out + size_t(pos) * (p.rows / 2);
                for (int c0 = 0; c0 < kMtATiles * 128; c0 += 32) {
                    const int strip0 = it.panel * kMtStrips + (c0 >> 4);
                    if (strip0 * 16 >= p.rows) break;   // warp-uniform
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + buf * (kMtATiles * 128) + c0, r);
                    tmem_ld_wait();
                    if (!live) continue;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int i0 = (strip0 + h) * 8;
                        if (2 * i0 >= p.rows) break;
                        uint32_t packed[4];
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            float gate = __uint_as_float(r[16 * h + q]) * f;
                            float up = __uint_as_float(r[16 * h + 8 + q]) * f;
                            gate = fminf(bf16_round_f(bf16_round_f(gate) + bias[2 * (i0 + q)]), p.limit);
                            up = fminf(p.limit, fmaxf(-p.limit, bf16_round_f(bf16_round_f(up) + bias[2 * (i0 + q) + 1])));
                            const float sig = bf16_round_f(1.f / (1.f + expf(-bf16_round_f(1.702f * gate))));
                            const float glu = bf16_round_f(gate * sig);
                            const uint32_t hv = __half_as_ushort(__float2half_rn(bf16_round_f(glu * bf16_round_f(up + 1.f))));
                            if (q & 1) packed[q >> 1] |= hv << 16;
                            else packed[q >> 1] = hv;
                        }
                        *reinterpret_cast<uint4*>(arow + i0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    }
                }
            } else {
                const float f = __uint_as_float(uint32_t(p.ref_exp) << 23);
                float* vrow = p.vals_out + size_t(p.sorted[pos]) * p.rows;
                for (int c0 = 0; c0 < kMtATiles * 128; c0 += 32) {
                    const int d0 = it.panel * (kMtATiles * 128) + c0;
                    if (d0 >= p.rows) break;   // warp-uniform
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + buf * (kMtATiles * 128) + c0, r);
                    tmem_ld_wait();
                    if (!live) continue;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float4 v;
                        float* vp = reinterpret_cast<float*>(&v);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int d = d0 + 4 * q + j;
                            vp[j] = d < p.rows ? bf16_round_f(bf16_round_f(__uint_as_float(r[4 * q + j]) * f) + bias[d]) : 0.f;
                        }
                        if (d0 + 4 * q + 3 < p.rows) *reinterpret_cast<float4*>(vrow + d0 + 4 * q) = v;
                        else
                            for (int j = 0; j < 4; ++j)
                                if (d0 + 4 * q + j < p.rows) vrow[d0 + 4 * q + j] = vp[j];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Rows in expert order: xg[pos, :] = xh[sorted[pos] / top_k, :] and its exponent.
__global__ void moe_gather_rows_kernel(const __half* __restrict__ xh, const int* __restrict__ xshift,
                                       const int* __restrict__ sorted, const int* __restrict__ offsets, int experts,
                                       int topk, int hidden, __half* __restrict__ xg, int* __restrict__ xshift_g)
{
    const int pos = blockIdx.x;
    if (pos >= offsets[experts]) return;
    const int token = sorted[pos] / topk;
    const uint4* src = reinterpret_cast<const uint4*>(xh + size_t(token) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(xg + size_t(pos) * hidden);
    for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) dst[v] = src[v];
    if (threadIdx.x == 0) xshift_g[pos] = xshift[token];
}

// Smallest and largest e8m0 byte of a scale tensor (device reduction for create()).
__global__ void mx_scale_range_kernel(const uint8_t* __restrict__ scales, size_t count, int* lo, int* hi)
{
    int mn = 255, mx = 0;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x) {
        const int e = scales[i];
        mn = min(mn, e);
        mx = max(mx, e);
    }
    for (int off = 16; off; off >>= 1) {
        mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, off));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMin(lo, mn);
        atomicMax(hi, mx);
    }
}

// ------------------------------------------------------------------ host side

bool moe_tc_eligible(const garnet_b200_moe_options& o, int tokens)
{
    const int world = o.ep_world > 1 ? o.ep_world : 1;
    const long long local = std::max(1, o.experts / world);
    return (long long)tokens * o.top_k >= 16LL * local && o.experts <= kMtMaxExperts;
}

int Moe::init_tc(int lo_up, int hi_up, int lo_dn, int hi_dn)
{
    tc_ok = false;
    if (careful_scales) return GARNET_B200_OK;                       // bytes 0 / 255 need the exact decode
    if (hi_up - lo_up > 24 || hi_dn - lo_dn > 24) return GARNET_B200_OK;   // would leave the fp16 normal range
    ref_up = hi_up - 12;
    ref_down = hi_dn - 12;
    if (ref_up < 40 || ref_up > 200 || ref_down < 40 || ref_down > 200) return GARNET_B200_OK;
    if (!tensor_map_encoder()) return GARNET_B200_OK;
    static_assert(sizeof(TensorMapStorage) == sizeof(CUtensorMap), "tensor map storage size");
    for (int pass = 0; pass < 2; ++pass) {
        const PackGeom& geo = pass == 0 ? geo_up : geo_down;
        if (int rc = make_tensor_map_2d_bytes(reinterpret_cast<CUtensorMap*>(&tc_w_map[pass]),
                                              pass == 0 ? packed_up : packed_down,
                                              uint64_t(stored_experts) * geo.strips_padded, geo.strip_bytes(),
                                              geo.strip_bytes(), kMtChunkBytes, kMtStrips))
            return rc;
    }
    GB_CUDA(cudaFuncSetAttribute(moe_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MtSmem::total));
    GB_CUDA(cudaFuncSetAttribute(moe_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MtSmem::total));
    tc_ok = true;
    return GARNET_B200_OK;
}

int Moe::gather_rows(const MoeWorkspacePtrs& w, int slots, int topk, cudaStream_t stream)
{
    moe_gather_rows_kernel<<<slots, 128, 0, stream>>>(w.xh, w.xshift, w.sorted, w.offsets, opt.experts, topk, opt.hidden,
                                                      w.xg, w.xshift_g);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int Moe::launch_tc(bool up, const MoeWorkspacePtrs& w, int slots, cudaStream_t stream)
{
    const PackGeom& geo = up ? geo_up : geo_down;
    const MoeShard sh = shard();
    CUtensorMap x_map;
    if (int rc = make_tensor_map_2d_16bit(&x_map, up ? static_cast<const void*>(w.xg) : static_cast<const void*>(w.act),
                                          uint64_t(slots), uint64_t(geo.cols), kMtTokens))
        return rc;
    MtParams p;
    p.offsets = w.offsets;
    p.sorted = w.sorted;
    p.xshift_g = up ? w.xshift_g : nullptr;
    p.bias = up ? up_bias_ptr : down_bias_ptr;
    p.act_out = w.act;
    p.vals_out = w.vals;
    p.fault = fault_dev;
    p.experts = opt.experts;
    p.rows = geo.rows;
    p.strips_padded = geo.strips_padded;
    p.chunks = geo.chunks;
    p.panels = (geo.strips_padded + kMtStrips - 1) / kMtStrips;
    p.expert_base = (sh.world > 1 && !sh.interleaved) ? sh.lo : (sh.world > 1 ? sh.rank : 0);
    p.expert_div = (sh.world > 1 && sh.interleaved) ? sh.world : 1;
    p.bias_by_global = (!opt.expert_weights_sharded && sh.world > 1) ? 1 : 0;
    p.expert_lo = sh.lo;
    p.expert_hi = sh.hi;
    p.interleave_world = sh.interleaved ? sh.world : 1;
    p.interleave_rank = sh.rank;
    p.ref_exp = up ? ref_up : ref_down;
    p.limit = opt.limit;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kSmCount);
    cfg.blockDim = dim3(kMtThreads);
    cfg.dynamicSmemBytes = MtSmem::total;
    cfg.stream = stream;
    const CUtensorMap& wm = *reinterpret_cast<const CUtensorMap*>(&tc_w_map[up ? 0 : 1]);
    if (up)
        GB_CUDA(cudaLaunchKernelEx(&cfg, moe_tc_kernel<true>, p, x_map, wm));
    else
        GB_CUDA(cudaLaunchKernelEx(&cfg, moe_tc_kernel<false>, p, x_map, wm));
    return GARNET_B200_OK;
}

}  // namespace gb200
