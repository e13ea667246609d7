// Block-scaled tensor-core path of the gpt-oss MXFP4 experts: the e2m1 codes and
// their e8m0 scales go to the tensor core as they are stored (tcgen05.mma
// kind::mxf8f6f4 with block scales), so no thread ever expands a weight.  It
// replaces, at every batch size, the reference's grouped WMMA kernel
// (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:843-906) and its Marlin adapter
// (plugins/gpt_oss/cuda/gpt_oss_marlin.cu:586-648).
//
// Operands.
//   A (UMMA M side, 128 rows per tile): expert weights as contiguous 8 KiB tiles of
//     128 rows x 128 columns of e2m1 codes (K padded to a multiple of 128).  The MMA reads 4-bit operands from 16-byte slots whose low
//     8 bytes hold 16 codes.  TMA can write that format itself (element type
//     16U4_ALIGN16B), but was measured at 8 packed bytes per cycle per SM (2.3 TB/s
//     over the GPU), so the packed bytes are fetched as plain bytes and four warps
//     spread them into the slots - a copy, no arithmetic.  Scales: 512-byte atoms of
//     128 rows x 4 blocks, copied to tensor memory with tcgen05.cp (32x128b,
//     replicated to the four lane quarters).
//   B (UMMA N side, 16..128 routed rows per tile): activations.  The MMA takes
//     8-bit floats there, so every bf16 activation is split into two e4m3 numbers
//     that share the e8m0 scale of their 32-block: hi = e4m3(v), lo = e4m3(v - hi),
//     v = x / 2^s with the block maximum scaled into [128, 256).  hi + lo equals v
//     exactly for elements within 2^-9 of the block maximum and to 2^-18 of it
//     otherwise, far below the bf16 rounding of the result.  Both pieces multiply
//     the same weight tile and accumulate into the same fp32 accumulator.
//   D: fp32 in tensor memory, lane = weight row, column = routed row.
//
// Rows are grouped by expert (the stable slot order of moe_fill_kernel); tiles of
// `nt` rows never span two experts, and the quantiser writes rows and scale atoms
// at tile-aligned positions, so a tile's operands are plain TMA boxes.
#include <algorithm>

#include "layout.h"
#include "moe.h"
#include "tc_common.cuh"
#include "mx_common.cuh"

namespace gb200 {

constexpr int kMxM = 128;            // weight rows per tile
constexpr int kMxEpiWarps = 8;       // two per 32-lane quarter of tensor memory
constexpr int kMxUnpackWarps = 4;
constexpr int kMxFirstUnpack = 3, kMxFirstEpi = kMxFirstUnpack + kMxUnpackWarps;
constexpr int kMxThreads = (kMxFirstEpi + kMxEpiWarps) * 32;   // 2 producers, MMA issuer, unpack and epilogue warps
constexpr int kMxPkStages = 4;       // ring of packed weight tiles (8 KiB each)
constexpr int kMxPkBytes = kMxM * kMxSlab / 2;
constexpr uint32_t kMxATileBytes = kMxM * 128;       // shared-memory footprint of a weight tile

// Two ways to feed the two e4m3 pieces of a tile's rows:
//   joined (tiles of up to 120 rows): one N = 2 nt operand, accumulator columns [0, nt)
//     and [nt, 2 nt) added in the epilogue - one MMA per K block;
//   split (tiles of 160 rows): two MMAs per K block, N = the live rows in sixteens, into
//     the same accumulator.
__host__ __device__ constexpr bool mx_joined(int nt) { return nt <= 120; }
__host__ __device__ constexpr int mx_sfb_atoms(int nt) { return ((mx_joined(nt) ? 2 : 1) * nt + 127) / 128; }
// An MMA of this kind (M = 128, K = 32) was measured to occupy the tensor pipe for about
// 130 cycles however small its N - the time to stream its 4 KiB A tile - and only an
// N near 256 has that much math: the instruction count, not the math, sets the pace of
// small tiles, hence the joined form wherever the tile is short enough.
__host__ __device__ constexpr int mx_stage_bytes(int nt)
{
    return int(kMxATileBytes) + 2 * nt * 128 + 1024 * ((kMxAtom * (1 + mx_sfb_atoms(nt)) + 1023) / 1024);
}
__host__ __device__ constexpr int mx_stages(int nt)
{
    const int s = (188 * 1024) / mx_stage_bytes(nt);
    return s > 8 ? 8 : s;
}
__host__ __device__ constexpr int mx_tmem_cols(int nt)
{
    const int need = (mx_joined(nt) ? 4 : 2) * nt + 4 + 4 * mx_sfb_atoms(nt);
    return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
}
// dynamic shared memory: 1 KiB alignment slack, the stages, tile prefix, barriers
__host__ __device__ constexpr int mx_smem_total(int nt)
{
    return 1024 + mx_stages(nt) * mx_stage_bytes(nt) + kMxPkStages * kMxPkBytes + (kMxMaxExperts + 1) * 4 + 512;
}

struct MxParams {
    const int* offsets;        // [experts + 1] start of every expert's rows in sorted order
    const int* sorted;         // [slots] slot ids in expert order
    const int* tile_prefix;    // [experts + 1] row tiles before each expert
    const float* bias;         // [experts(local or global), rows] original row order
    const uint8_t* w;          // [stored experts][mtiles][kslabs][8 KiB] weight tiles
    const uint8_t* sfa;        // [stored experts][mtiles][kslabs][512] weight scale atoms
    const uint8_t* sfb;        // [row tiles][kslabs][atoms per tile][512] activation scale atoms
    __half* act_out;           // up: [sorted position, intermediate]
    float* vals_out;           // down: [slot id, hidden]
    int* fault;
    int experts;               // global expert count
    int rows;                  // logical rows of the weight matrix (2I or H)
    int mtiles;                // 128-row tiles of the weight matrix
    int kslabs;                // 128-column slabs along K
    int expert_base, expert_div, bias_by_global;
    float limit;
};

// 16 accumulator columns of this thread's lane; in the joined form the two pieces'
// columns, kN apart, are added.
template <int kN>
__device__ __forceinline__ void mx_load_acc(uint32_t taddr, uint32_t (&r)[16])
{
    tmem_ld_32x16(taddr, r);
    if (mx_joined(kN)) {
        uint32_t r2[16];
        tmem_ld_32x16(taddr + kN, r2);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
    } else {
        tmem_ld_wait();
    }
}

struct MxItem {
    int expert, tile, mtile, rows;   // tile: global row-tile index; rows: live rows of it
    int row0;                        // sorted position of the tile's first row
};
template <int kN>
__device__ __forceinline__ MxItem mx_decode(const MxParams& p, const int* tile_prefix, int item, int& cursor)
{
    const int t = item / p.mtiles;
    while (tile_prefix[cursor + 1] <= t) ++cursor;
    MxItem it;
    it.expert = cursor;
    it.tile = t;
    it.mtile = item % p.mtiles;
    const int local = t - tile_prefix[cursor];
    it.row0 = p.offsets[cursor] + local * kN;
    it.rows = min(kN, p.offsets[cursor + 1] - it.row0);
    return it;
}

template <bool kUp, int kN>
__global__ void __launch_bounds__(kMxThreads, 1)
moe_mx_kernel(const MxParams p, const __grid_constant__ CUtensorMap q_map, const int q_rows)
{
    constexpr int kStages = mx_stages(kN);
    constexpr int kStageBytes = mx_stage_bytes(kN);
    constexpr uint32_t kTmemCols = mx_tmem_cols(kN);
    constexpr int kSfbAtoms = mx_sfb_atoms(kN);
    constexpr bool kJoined = mx_joined(kN);
    constexpr uint32_t kAccCols = kJoined ? 2 * kN : kN;   // accumulator columns per buffer
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    uint8_t* pk_ring = smem + kStages * kStageBytes;
    int* tile_prefix = reinterpret_cast<int*>(pk_ring + kMxPkStages * kMxPkBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(tile_prefix) + (kMxMaxExperts + 1) * 4 + 4);
    uint64_t* pk_full = bars;
    uint64_t* pk_empty = pk_full + kMxPkStages;
    uint64_t* full = pk_empty + kMxPkStages;      // activation tiles and scale atoms have landed
    uint64_t* a_ready = full + kStages;           // the weight tile has been spread into its slots
    uint64_t* empty = a_ready + kStages;
    uint64_t* acc_full = empty + kStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kMxPkStages; ++s) {
            mbar_init(&pk_full[s], 1);
            mbar_init(&pk_empty[s], kMxUnpackWarps);
        }
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&a_ready[s], kMxUnpackWarps);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], kMxEpiWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    pdl_launch_dependents();
    pdl_wait();   // row order, tile prefix and quantised rows come from earlier kernels of this call
    for (int e = threadIdx.x; e <= p.experts; e += blockDim.x) tile_prefix[e] = p.tile_prefix[e];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfa = tmem_base + 2 * kAccCols, tmem_sfb = tmem_sfa + 4;
    const int items = tile_prefix[p.experts] * p.mtiles;

    if (warp == 0) {
        // ------------------------------------- producer of packed weight tiles
        if (lane == 0) {
            uint32_t n = 0;
            int cur = 0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const MxItem it = mx_decode<kN>(p, tile_prefix, item, cur);
                const int se = (it.expert - p.expert_base) / p.expert_div;
                const uint8_t* wt = p.w + (size_t(se) * p.mtiles + it.mtile) * p.kslabs * kMxPkBytes;
                for (int ks = 0; ks < p.kslabs; ++ks, ++n) {
                    const uint32_t s = n % kMxPkStages;
                    const bool okw = !(n >= kMxPkStages && !mbar_wait_bounded(&pk_empty[s], ((n / kMxPkStages) - 1) & 1));
                    if (!okw) {
                        atomicExch(p.fault, 30);
                        *abort_flag = 1;
                        break;
                    }
                    mbar_expect_tx(&pk_full[s], kMxPkBytes);
                    bulk_g2s(pk_ring + s * kMxPkBytes, wt + size_t(ks) * kMxPkBytes, kMxPkBytes, &pk_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------- producer of activation tiles and scale atoms
        if (lane == 0) {
            uint32_t n = 0;
            int cur = 0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const MxItem it = mx_decode<kN>(p, tile_prefix, item, cur);
                const int se = (it.expert - p.expert_base) / p.expert_div;
                const uint8_t* sfa = p.sfa + (size_t(se) * p.mtiles + it.mtile) * p.kslabs * kMxAtom;
                const uint8_t* sfb = p.sfb + size_t(it.tile) * p.kslabs * (kSfbAtoms * kMxAtom);
                constexpr uint32_t tx = uint32_t(2 * kN * 128) + uint32_t((1 + kSfbAtoms) * kMxAtom);
                for (int ks = 0; ks < p.kslabs; ++ks, ++n) {
                    const uint32_t s = n % kStages;
                    const bool okw = !(n >= kStages && !mbar_wait_bounded(&empty[s], ((n / kStages) - 1) & 1));
                    if (!okw) {
                        atomicExch(p.fault, 31);
                        *abort_flag = 1;
                        break;
                    }
                    uint8_t* st = ring + s * kStageBytes;
                    uint8_t* sf_s = st + kMxATileBytes + 2 * kN * 128;
                    mbar_expect_tx(&full[s], tx);
                    tma_load_2d(st + kMxATileBytes, &q_map, ks * kMxSlab, it.tile * kN, &full[s]);
                    tma_load_2d(st + kMxATileBytes + kN * 128, &q_map, ks * kMxSlab, q_rows + it.tile * kN, &full[s]);
                    bulk_g2s(sf_s, sfa + size_t(ks) * kMxAtom, kMxAtom, &full[s]);
                    bulk_g2s(sf_s + kMxAtom, sfb + size_t(ks) * (kSfbAtoms * kMxAtom), kSfbAtoms * kMxAtom, &full[s]);
                }
            }
        }
    } else if (warp >= kMxFirstUnpack && warp < kMxFirstEpi) {
        // ------------------------------------------------------------- unpack
        // Packed tile: 128 rows x 64 bytes.  Operand tile: 128 rows x 128 bytes with the
        // 128-byte swizzle, 16 codes in the low 8 bytes of every 16-byte slot.  Lane l of
        // a pass handles 16 bytes (two slots) of row l / 4: loads are conflict-free.
        const int uw = warp - kMxFirstUnpack;
        uint32_t n = 0;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
            for (int ks = 0; ks < p.kslabs && !*abort_flag; ++ks, ++n) {
                const uint32_t ps = n % kMxPkStages, s = n % kStages;
                if (!mbar_wait_bounded(&pk_full[ps], (n / kMxPkStages) & 1) ||
                    (n >= kStages && !mbar_wait_bounded(&empty[s], ((n / kStages) - 1) & 1))) {
                    atomicExch(p.fault, 35);
                    *abort_flag = 1;
                    break;
                }
                const uint8_t* src = pk_ring + ps * kMxPkBytes;
                uint8_t* dst = ring + s * kStageBytes;
#pragma unroll
                for (int pass = 0; pass < 4; ++pass) {
                    const int row = uw * 32 + pass * 8 + (lane >> 2), c16 = lane & 3;
                    const uint4 v = *reinterpret_cast<const uint4*>(src + row * 64 + c16 * 16);
                    uint8_t* drow = dst + row * 128;
                    *reinterpret_cast<uint2*>(drow + (((2 * c16) ^ (row & 7)) << 4)) = make_uint2(v.x, v.y);
                    *reinterpret_cast<uint2*>(drow + (((2 * c16 + 1) ^ (row & 7)) << 4)) = make_uint2(v.z, v.w);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&a_ready[s]);
                    mbar_arrive(&pk_empty[ps]);
                }
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t n = 0, it_n = 0;
            int cur = 0;
            const uint32_t ring_addr = smem_u32(ring);
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
                const MxItem it = mx_decode<kN>(p, tile_prefix, item, cur);
                const int n16 = (it.rows + 15) & ~15;   // split form: UMMA N = the live rows, in sixteens
                const uint32_t idesc0 = mx_idesc_fmt(kMxFmtE2M1, kMxFmtE4M3, kMxM, kJoined ? 2 * kN : n16, 0);
                const uint32_t buf = it_n & 1;
                if (it_n >= 2 && !mbar_wait_bounded(&acc_empty[buf], ((it_n >> 1) - 1) & 1)) {
                    atomicExch(p.fault, 32);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                for (int ks = 0; ks < p.kslabs; ++ks, ++n) {
                    const uint32_t s = n % kStages;
                    if (!mbar_wait_bounded(&full[s], (n / kStages) & 1) ||
                        !mbar_wait_bounded(&a_ready[s], (n / kStages) & 1)) {
                        atomicExch(p.fault, 33);
                        *abort_flag = 1;
                        break;
                    }
                    // One thread issues everything, so the loop is kept to a few instructions per
                    // MMA: descriptors advance by adding to the start-address field (32 bytes =
                    // 2 units per K block), the scale selectors by adding to the two id fields.
                    const uint32_t a_addr = ring_addr + s * kStageBytes;
                    const uint64_t a_d = umma_desc_k_sw128(a_addr), b_d = umma_desc_k_sw128(a_addr + kMxATileBytes);
                    const uint32_t sfa_addr = a_addr + kMxATileBytes + 2 * kN * 128;
                    tmem_cp_32x128b_warpx4(tmem_sfa, umma_desc_k_plain(sfa_addr, 128));
#pragma unroll
                    for (int at = 0; at < kSfbAtoms; ++at)
                        tmem_cp_32x128b_warpx4(tmem_sfb + 4 * at, umma_desc_k_plain(sfa_addr + (1 + at) * kMxAtom, 128));

                    const uint32_t d_addr = tmem_base + buf * kAccCols;
#pragma unroll
                    for (uint32_t kb = 0; kb < 4; ++kb) {
                        const uint32_t idesc = idesc0 + kb * ((1u << 4) | (1u << 29));
                        umma_mx(d_addr, a_d + 2 * kb, b_d + 2 * kb, idesc, tmem_sfa, tmem_sfb, ks > 0 || kb > 0);
                        if (!kJoined)
                            umma_mx(d_addr, a_d + 2 * kb, b_d + (kN * 128 >> 4) + 2 * kb, idesc, tmem_sfa, tmem_sfb, true);
                    }
                    umma_commit(&empty[s]);
                }
                if (*abort_flag) break;
                umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        // Warp w serves the 32-lane quarter w % 4 (a warp may only read its own quarter of
        // tensor memory); the two warps of a quarter take alternate 16-column groups.
        const int quarter = warp & 3, half = (warp - kMxFirstEpi) >> 2;
        const int l = quarter * 32 + lane;   // TMEM lane = weight row of the tile
        uint32_t it_n = 0;
        int cur = 0;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
            const MxItem it = mx_decode<kN>(p, tile_prefix, item, cur);
            const uint32_t buf = it_n & 1;
            if (!mbar_wait_bounded(&acc_full[buf], (it_n >> 1) & 1)) {
                atomicExch(p.fault, 34);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const int ebias = p.bias_by_global ? it.expert : (it.expert - p.expert_base) / p.expert_div;
            const int row = it.mtile * kMxM + l;
            const bool row_ok = row < p.rows;
            const float b_mine = row_ok ? p.bias[size_t(ebias) * p.rows + row] : 0.f;
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kAccCols;
            if (kUp) {
                // Weight rows 2i (gate) and 2i+1 (up) sit in neighbouring lanes.  Per pair of
                // columns the lanes swap one value, after which the even lane holds gate and
                // up of column j and the odd lane those of column j + 1: every lane finishes
                // one output.
                const float b_other = __shfl_xor_sync(0xffffffffu, b_mine, 1);
                const float b_gate = (lane & 1) ? b_other : b_mine, b_up = (lane & 1) ? b_mine : b_other;
                const int ch = row >> 1;
                const int inter = p.rows >> 1;
                for (int c0 = half * 16; c0 < it.rows; c0 += 32) {
                    uint32_t r[16];
                    mx_load_acc<kN>(taddr + c0, r);
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float send = __uint_as_float((lane & 1) ? r[j] : r[j + 1]);
                        const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
                        const float g_raw = (lane & 1) ? recv : __uint_as_float(r[j]);
                        const float u_raw = (lane & 1) ? __uint_as_float(r[j + 1]) : recv;
                        const int col = c0 + j + (lane & 1);
                        if (row_ok && col < it.rows) {
                            const float gate = fminf(bf16_round_f(bf16_round_f(g_raw) + b_gate), p.limit);
                            const float up = fminf(p.limit, fmaxf(-p.limit, bf16_round_f(bf16_round_f(u_raw) + b_up)));
                            const float sig = bf16_round_f(1.f / (1.f + expf(-bf16_round_f(1.702f * gate))));
                            const float glu = bf16_round_f(gate * sig);
                            p.act_out[size_t(it.row0 + col) * inter + ch] =
                                __float2half_rn(bf16_round_f(glu * bf16_round_f(up + 1.f)));
                        }
                    }
                }
            } else {
                for (int c0 = half * 16; c0 < it.rows; c0 += 32) {
                    uint32_t r[16];
                    mx_load_acc<kN>(taddr + c0, r);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (row_ok && c0 + j < it.rows) {
                            const int slot = p.sorted[it.row0 + c0 + j];
                            p.vals_out[size_t(slot) * p.rows + row] =
                                bf16_round_f(bf16_round_f(__uint_as_float(r[j])) + b_mine);
                        }
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
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------ create-time kernels

// Weight tiles: dst[e][mtile][kslab][128 rows][64 bytes], i.e. every (128 rows x 128
// columns) tile of an expert matrix is one contiguous 8 KiB block (a k-slab of a
// row-major matrix would be 128 separate 64-byte pieces, which DRAM serves at a
// fraction of its bandwidth).  Rows and columns beyond the matrix hold zero codes.
__global__ void mx_tile_weights_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int experts, int rows,
                                       int k, int mtiles, int kslabs)
{
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one 16-byte piece of the output
    const long long total = (long long)experts * mtiles * kslabs * (kMxPkBytes / 16);
    if (idx >= total) return;
    const int piece = int(idx % 4);
    const int r = int((idx / 4) % kMxM);
    const long long tile = idx / (4 * kMxM);
    const int ks = int(tile % kslabs);
    const int mt = int((tile / kslabs) % mtiles);
    const int e = int(tile / ((long long)kslabs * mtiles));
    const int row = mt * kMxM + r, col = ks * kMxSlab + piece * 32;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows && col < k) v = *reinterpret_cast<const uint4*>(src + (size_t(e) * rows + row) * (k / 2) + col / 2);
    *reinterpret_cast<uint4*>(dst + idx * 16) = v;
}

// Scale atoms of the weights: dst[e][mtile][kslab][512], byte (r % 32) * 16 + (r / 32) * 4 + kb
// holds the e8m0 scale of row mtile * 128 + r, block kslab * 4 + kb; rows and blocks
// beyond the matrix get 127 (1.0; their codes are zero).
__global__ void mx_weight_atoms_kernel(const uint8_t* __restrict__ scales, uint8_t* __restrict__ dst, int experts, int rows,
                                       int blocks, int mtiles, int kslabs)
{
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)experts * mtiles * kslabs * kMxAtom;
    if (idx >= total) return;
    const int byte = int(idx % kMxAtom);
    const long long atom = idx / kMxAtom;
    const int ks = int(atom % kslabs);
    const int mt = int((atom / kslabs) % mtiles);
    const int e = int(atom / (kslabs * (long long)mtiles));
    const int r = (byte >> 4) + 32 * ((byte >> 2) & 3), kb = byte & 3;
    const int row = mt * kMxM + r, blk = ks * 4 + kb;
    uint8_t v = 127;
    if (row < rows && blk < blocks) v = scales[(size_t(e) * rows + row) * blocks + blk];
    dst[idx] = v;
}

// ------------------------------------------------------------- per-call kernels

__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t v)
{
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(uint16_t(v)));
    const __half2 h = *reinterpret_cast<const __half2*>(&h2);
    return make_float2(__low2float(h), __high2float(h));
}

// 32 consecutive elements of a row as bf16-valued floats.
__device__ __forceinline__ void mx_load32(const float* p, float (&v)[32])
{
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 f = *reinterpret_cast<const float4*>(p + 4 * i);
        v[4 * i] = bf16_round_f(f.x);
        v[4 * i + 1] = bf16_round_f(f.y);
        v[4 * i + 2] = bf16_round_f(f.z);
        v[4 * i + 3] = bf16_round_f(f.w);
    }
}
__device__ __forceinline__ void mx_load32(const __nv_bfloat16* p, float (&v)[32])
{
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 u = *reinterpret_cast<const uint4*>(p + 8 * i);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            v[8 * i + 2 * q] = __uint_as_float(w[q] << 16);
            v[8 * i + 2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u);
        }
    }
}
__device__ __forceinline__ void mx_load32(const __half* p, float (&v)[32])
{
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 u = *reinterpret_cast<const uint4*>(p + 8 * i);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
            v[8 * i + 2 * q] = f.x;
            v[8 * i + 2 * q + 1] = f.y;
        }
    }
}

// One routed row per CTA, one 32-block per thread: the row (bf16-valued) becomes two
// e4m3 rows sharing one e8m0 scale per block, written at the row's tile-aligned
// position; blocks behind column K are zero with scale 1.
//   src row of sorted position pos: src[(sorted[pos] / div) * k]  (div = top_k for the
//   layer input, and the caller passes sorted = nullptr for rows already in sorted order)
template <typename T>
__global__ void mx_quant_rows_kernel(const T* __restrict__ src, const int* __restrict__ sorted, int div,
                                     const int* __restrict__ offsets, const int* __restrict__ tile_prefix, int experts,
                                     int nt, int k, int kp, int q_rows, uint8_t* __restrict__ q,
                                     uint8_t* __restrict__ sf)
{
    pdl_launch_dependents();
    pdl_wait();
    const int pos = blockIdx.x;
    if (pos >= offsets[experts]) return;
    __shared__ int s_expert;
    if (threadIdx.x == 0) {
        int lo = 0, hi = experts;   // largest e with offsets[e] <= pos
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (offsets[mid] <= pos) lo = mid;
            else hi = mid;
        }
        s_expert = lo;
    }
    __syncthreads();
    const int e = s_expert;
    const int idx = pos - offsets[e];
    const int tile = tile_prefix[e] + idx / nt, r = idx % nt;
    const T* row = src + size_t(sorted ? sorted[pos] / div : pos) * k;
    const int kslabs = kp / kMxSlab, atoms = mx_sfb_atoms(nt);
    for (int b = threadIdx.x; b < kp / 32; b += blockDim.x) {
        float v[32];
        float amax = 0.f;
        if (b * 32 < k) {
            mx_load32(row + b * 32, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        int sbyte = 127;
        if (amax > 0.f && isfinite(amax)) sbyte = int((__float_as_uint(amax) >> 23) & 0xff) - 7;   // max lands in [128, 256)
        sbyte = max(1, min(254, sbyte));
        const float inv = __uint_as_float(uint32_t(254 - sbyte) << 23);   // 2^(127 - sbyte)
        uint32_t hi_w[8], lo_w[8];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            uint32_t hw = 0, lw = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float a = v[i + 2 * h] * inv, c = v[i + 2 * h + 1] * inv;
                const uint32_t hp = f32x2_to_e4m3x2(a, c);
                const float2 back = e4m3x2_to_f32x2(hp);
                const uint32_t lp = f32x2_to_e4m3x2(a - back.x, c - back.y);
                hw |= hp << (16 * h);
                lw |= lp << (16 * h);
            }
            hi_w[i >> 2] = hw;
            lo_w[i >> 2] = lw;
        }
        uint8_t* dst_hi = q + (size_t(tile) * nt + r) * kp + b * 32;
        uint8_t* dst_lo = dst_hi + size_t(q_rows) * kp;
        *reinterpret_cast<uint4*>(dst_hi) = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
        *reinterpret_cast<uint4*>(dst_hi + 16) = make_uint4(hi_w[4], hi_w[5], hi_w[6], hi_w[7]);
        *reinterpret_cast<uint4*>(dst_lo) = make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
        *reinterpret_cast<uint4*>(dst_lo + 16) = make_uint4(lo_w[4], lo_w[5], lo_w[6], lo_w[7]);
        // operand rows r (first piece) and nt + r (second piece) carry the same scale
        uint8_t* atom0 = sf + (size_t(tile) * kslabs + (b >> 2)) * atoms * kMxAtom;
#pragma unroll
        for (int piece = 0; piece < (mx_joined(nt) ? 2 : 1); ++piece) {
            const int rr = r + piece * nt;
            atom0[(rr >> 7) * kMxAtom + (rr & 31) * 16 + ((rr >> 5) & 3) * 4 + (b & 3)] = uint8_t(sbyte);
        }
    }
}

// ------------------------------------------------------------------ host side

// GARNET_B200_MOE_MX: 0 keeps the expert GEMMs on the kernels that expand the weights
// in registers, 2 uses the block-scaled path at every size (for tests), 3 selects the
// orientation with the weights as the M operand (this file's kernel; the default is the
// rows-as-M kernel of moe_mxr.cu), anything else lets the row count per expert decide.
// Read once.
static int moe_mx_mode()
{
    static const int mode = [] {
        const char* e = getenv("GARNET_B200_MOE_MX");
        return (e && e[0] == '0') ? 0 : (e && e[0] == '2') ? 2 : (e && e[0] == '3') ? 3 : 1;
    }();
    return mode;
}
bool moe_mx_enabled() { return moe_mx_mode() != 0; }
bool moe_mx_forced() { return moe_mx_mode() == 2; }
bool moe_mx_weights_as_m() { return moe_mx_mode() == 3; }

// Rows per tile: no expert can get more rows than there are tokens; beyond 64 the
// average decides between 120-row joined tiles and 160-row split tiles.
int moe_mx_nt(int tokens, int slots, int local_experts)
{
    if (!moe_mx_weights_as_m()) return 128;   // rows-as-M kernel: 128-row tiles
    if (tokens <= 16) return 16;
    if (tokens <= 32) return 32;
    if (tokens <= 64) return 64;
    return slots / std::max(1, local_experts) <= 100 ? 120 : 160;
}

MoeMxPlan moe_mx_plan(const garnet_b200_moe_options& o, int tokens, int slots)
{
    MoeMxPlan m;
    const int world = o.ep_world > 1 ? o.ep_world : 1;
    m.nt = moe_mx_nt(tokens, slots, std::max(1, o.experts / world));
    m.tiles_max = slots / m.nt + std::min(slots, o.experts) + 1;   // full tiles + one partial tile per expert that has rows
    m.q_rows = m.tiles_max * m.nt;
    const int kmax = std::max(o.hidden, o.intermediate);
    m.kp_max = (kmax + kMxSlab - 1) / kMxSlab * kMxSlab;
    m.q_bytes = size_t(2) * m.q_rows * m.kp_max;
    m.sf_bytes = size_t(m.tiles_max) * (m.kp_max / kMxSlab) * mx_sfb_atoms(m.nt) * kMxAtom;
    return m;
}

static int mx_encode(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base, const cuuint64_t* dims,
                     const cuuint64_t* strides, const cuuint32_t* box,
                     CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B)
{
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return fail(GARNET_B200_NOT_SUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(map, dt, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GARNET_B200_CUDA_ERROR, "cuTensorMapEncodeTiled (block-scaled path) failed with code %d", int(r));
    return GARNET_B200_OK;
}

template <bool U, int N>
static cudaError_t mx_set_attr()
{
    return cudaFuncSetAttribute(moe_mx_kernel<U, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, mx_smem_total(N));
}

// Second copy of the expert weights in the block-scaled path's layout.  `blocks` and
// `scales` are the tensors of the stored experts, in stored order.
int Moe::init_mx(int pass, const uint8_t* blocks, const uint8_t* scales, int first_stored, int count, cudaStream_t stream)
{
    const PackGeom& geo = pass == 0 ? geo_up : geo_down;
    const int k = geo.cols, rows = geo.rows;
    const int kp = (k + kMxSlab - 1) / kMxSlab * kMxSlab;
    const int mtiles = (rows + kMxM - 1) / kMxM, kslabs = kp / kMxSlab;
    mx_kp[pass] = kp;
    mx_mtiles[pass] = mtiles;
    mx_kslabs[pass] = kslabs;
    if (!moe_mx_weights_as_m()) return init_mxr(pass, blocks, scales, first_stored, count, stream);
    if (!mx_w[pass]) {
        GB_CUDA(cudaMalloc(&mx_w[pass], size_t(stored_experts) * mtiles * kslabs * kMxPkBytes));
        GB_CUDA(cudaMalloc(&mx_sfa[pass], size_t(stored_experts) * mtiles * kslabs * kMxAtom));
        mx_kp[pass] = kp;
        mx_mtiles[pass] = mtiles;
        mx_kslabs[pass] = kslabs;
    }
    const long long pieces = (long long)count * mtiles * kslabs * (kMxPkBytes / 16);
    mx_tile_weights_kernel<<<unsigned((pieces + 255) / 256), 256, 0, stream>>>(
        blocks, mx_w[pass] + size_t(first_stored) * mtiles * kslabs * kMxPkBytes, count, rows, k, mtiles, kslabs);
    const long long bytes = (long long)count * mtiles * kslabs * kMxAtom;
    mx_weight_atoms_kernel<<<unsigned((bytes + 255) / 256), 256, 0, stream>>>(
        scales, mx_sfa[pass] + size_t(first_stored) * mtiles * kslabs * kMxAtom, count, rows, k / 32, mtiles, kslabs);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int Moe::finish_mx()
{
    mx_ok = false;
    if (!tensor_map_encoder() || opt.experts > kMxMaxExperts) return GARNET_B200_OK;
    if ((opt.hidden % 32) || (opt.intermediate % 32)) return GARNET_B200_OK;
    if (int rc = finish_mxr()) return rc;
    GB_CUDA((mx_set_attr<true, 16>()));
    GB_CUDA((mx_set_attr<true, 32>()));
    GB_CUDA((mx_set_attr<true, 64>()));
    GB_CUDA((mx_set_attr<true, 120>()));
    GB_CUDA((mx_set_attr<true, 160>()));
    GB_CUDA((mx_set_attr<false, 160>()));
    GB_CUDA((mx_set_attr<false, 16>()));
    GB_CUDA((mx_set_attr<false, 32>()));
    GB_CUDA((mx_set_attr<false, 64>()));
    GB_CUDA((mx_set_attr<false, 120>()));
    mx_ok = true;
    return GARNET_B200_OK;
}

template <bool kUp, int kN>
static cudaError_t mx_launch(const MxParams& p, const CUtensorMap& qm, int q_rows, int grid, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(kMxThreads);
    cfg.dynamicSmemBytes = mx_smem_total(kN);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, moe_mx_kernel<kUp, kN>, p, qm, q_rows);
}

// Quantises the rows (layer input for the gate/up projection, activations for the
// down projection) and runs the grouped GEMM of one projection.
//   x: layer input [tokens, hidden] in the operator's io dtype (gate/up only)
int Moe::launch_mx(bool up, const MoeWorkspacePtrs& w, const void* x, int x_is_sorted, int tokens, int slots, int topk,
                   cudaStream_t stream)
{
    const int pass = up ? 0 : 1;
    const PackGeom& geo = up ? geo_up : geo_down;
    const MoeShard sh = shard();
    const MoeMxPlan plan = moe_mx_plan(opt, tokens, slots);
    const int nt = plan.nt, kp = mx_kp[pass], k = geo.cols;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.stream = stream;
    cfg.gridDim = dim3(unsigned(slots));
    cfg.blockDim = dim3(96);
    const int* sorted = (up && !x_is_sorted) ? w.sorted : nullptr;
    if (!up)
        GB_CUDA(cudaLaunchKernelEx(&cfg, mx_quant_rows_kernel<__half>, (const __half*)w.act, (const int*)nullptr, 1,
                                   (const int*)w.offsets, (const int*)w.mx_tp, opt.experts, nt, k, kp, plan.q_rows,
                                   w.mx_q, w.mx_sf));
    else if (opt.io_dtype == GARNET_B200_FP32)
        GB_CUDA(cudaLaunchKernelEx(&cfg, mx_quant_rows_kernel<float>, static_cast<const float*>(x), sorted, topk,
                                   (const int*)w.offsets, (const int*)w.mx_tp, opt.experts, nt, k, kp, plan.q_rows,
                                   w.mx_q, w.mx_sf));
    else
        GB_CUDA(cudaLaunchKernelEx(&cfg, mx_quant_rows_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(x), sorted,
                                   topk, (const int*)w.offsets, (const int*)w.mx_tp, opt.experts, nt, k, kp, plan.q_rows,
                                   w.mx_q, w.mx_sf));

    CUtensorMap q_map;
    {
        const cuuint64_t dims[2] = {cuuint64_t(kp), cuuint64_t(2) * plan.q_rows};
        const cuuint64_t strides[1] = {cuuint64_t(kp)};
        const cuuint32_t box[2] = {kMxSlab, cuuint32_t(nt)};
        if (int rc = mx_encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.mx_q, dims, strides, box)) return rc;
    }
    if (!moe_mx_weights_as_m()) return launch_mxr_gemm(up, w, &q_map, plan.q_rows, plan.tiles_max, stream);
    MxParams p;
    p.offsets = w.offsets;
    p.sorted = w.sorted;
    p.tile_prefix = w.mx_tp;
    p.bias = up ? up_bias_ptr : down_bias_ptr;
    p.w = mx_w[pass];
    p.sfa = mx_sfa[pass];
    p.sfb = w.mx_sf;
    p.act_out = w.act;
    p.vals_out = w.vals;
    p.fault = fault_dev;
    p.experts = opt.experts;
    p.rows = geo.rows;
    p.mtiles = mx_mtiles[pass];
    p.kslabs = mx_kslabs[pass];
    p.expert_base = (sh.world > 1 && !sh.interleaved) ? sh.lo : (sh.world > 1 ? sh.rank : 0);
    p.expert_div = (sh.world > 1 && sh.interleaved) ? sh.world : 1;
    p.bias_by_global = (!opt.expert_weights_sharded && sh.world > 1) ? 1 : 0;
    p.limit = opt.limit;
    // upper bound of the item count: every tile of every expert
    const long long max_items = (long long)plan.tiles_max * p.mtiles;
    const int grid = int(std::min<long long>(kSmCount, max_items));
#define GB_MX_LAUNCH(N_)                                                                       \
    GB_CUDA(up ? (mx_launch<true, N_>(p, q_map, plan.q_rows, grid, stream))                \
               : (mx_launch<false, N_>(p, q_map, plan.q_rows, grid, stream)))
    if (nt == 16) GB_MX_LAUNCH(16);
    else if (nt == 32) GB_MX_LAUNCH(32);
    else if (nt == 64) GB_MX_LAUNCH(64);
    else if (nt == 120) GB_MX_LAUNCH(120);
    else GB_MX_LAUNCH(160);
#undef GB_MX_LAUNCH
    return GARNET_B200_OK;
}

}  // namespace gb200
