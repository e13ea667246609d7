// Block-scaled grouped GEMM of the gpt-oss MXFP4 experts with the routed rows as the
// UMMA M operand and 240 weight rows as the N operand.
//
// Why this orientation.  A tcgen05.mma of kind::mxf8f6f4 with M = 128, K = 32 keeps the
// tensor pipe busy for about 130 cycles whatever its N (the time to stream its 128 x
// 32-byte A tile), and an N near 256 has that much math.  With the weights as A and a
// tile's rows as N (moe_mx.cu) an expert with 130 rows runs at half the pipe's rate;
// here every MMA is 240 wide, and what a partly filled row tile wastes is M, not N.
// 240 = the widest N for which two accumulators (2 x 240 columns) and the scale copies
// (4 + 8 columns) fit the 512 columns of tensor memory; it divides the gpt-oss
// matrices (5760 = 24 x 240, 2880 = 12 x 240).
//
// Operands per pipeline stage (128 columns of K):
//   A  two e4m3 pieces of 128 routed rows (mx_quant_rows_kernel, tiles of 128 rows that
//      never span two experts), fetched by TMA with the 128-byte swizzle; their e8m0
//      scales as one 512-byte atom;
//   B  240 weight rows as one contiguous 15 KiB block of e2m1 codes (own layout:
//      [expert][240-row tile][k slab][240][64 B]), fetched by TMA with the element type
//      16U4_ALIGN16B, which writes 16 codes into the low 8 bytes of every 16-byte slot -
//      the format the MMA reads 4-bit operands in (spreading them with warps instead
//      costs shared-memory bandwidth, which is what bounds this kernel: the MMAs alone
//      read 85 bytes per cycle of the 128 the SM has); their e8m0 scales as two
//      512-byte atoms;
//   D  fp32 in tensor memory, lane = routed row, column = weight row, double-buffered.
// Each K block of 32 takes two MMAs (first piece, second piece) into the same D.
// Epilogue: a thread owns one routed row: gate and up of a channel are neighbouring
// columns, outputs leave as 16-byte stores.
#include <algorithm>

#include "layout.h"
#include "moe.h"
#include "moe_pack.h"
#include "mx_common.cuh"

namespace gb200 {

constexpr int kRxRows = 128;          // routed rows per tile (UMMA M)
constexpr int kRxN = kMxBlockRows;    // weight rows per tile (UMMA N): 240
constexpr int kRxEpiWarps = 8;
constexpr int kRxFirstEpi = 3;                          // warp 0: producer, warp 1: MMA issuer, warp 2: spare
constexpr int kRxThreads = (kRxFirstEpi + kRxEpiWarps) * 32;
constexpr int kRxPkBytes = kMxBlockBytes;               // 15360: packed weight block of a stage
constexpr int kRxPrefetch = 8;                          // weight blocks requested into L2 ahead of the ring
constexpr int kRxMaxExperts = 1024;                     // tile prefix kept in shared memory
constexpr int kRxATile = kRxRows * 128;                 // one e4m3 piece of a stage
constexpr int kRxBTile = kRxN * 128;                    // expanded weight tile of a stage
constexpr int kRxSfBytes = 2048;                        // 1 activation atom + 2 weight atoms, padded
constexpr int kRxStageBytes = 2 * kRxATile + kRxBTile + kRxSfBytes;   // 65536
constexpr int kRxStages = 3;
constexpr uint32_t kRxTmemCols = 512;
constexpr int kRxSmemTotal = 1024 + kRxStages * kRxStageBytes + (kRxMaxExperts + 1) * 4 + 512;
static_assert(kRxSmemTotal <= 227 * 1024, "shared memory budget");

struct RxParams {
    const int* offsets;        // [experts + 1] start of every expert's rows in sorted order
    const int* sorted;         // [slots] slot ids in expert order
    const int* tile_prefix;    // [experts + 1] 128-row tiles before each expert
    const float* bias;         // [experts(local or global), rows] original row order
    const uint8_t* w;          // [stored experts][ntiles][kslabs][15 KiB] weight blocks
    const uint8_t* sfw;        // [stored experts][ntiles][kslabs][2][512] weight scale atoms
    const uint8_t* sfx;        // [row tiles][kslabs][512] activation scale atoms
    __half* act_out;           // up: [sorted position, intermediate]
    float* vals_out;           // down: [slot id, hidden]
    int vals_bf16;             // vals_out holds bf16
    int* fault;
    int experts, rows, ntiles, kslabs;
    int expert_base, expert_div, bias_by_global;
    float limit;
};

// Ask L2 for a byte range (no shared-memory destination, no barrier).
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

struct RxItem {
    int expert, tile, ntile, rows, row0;
};
__device__ __forceinline__ RxItem rx_decode(const RxParams& p, const int* tile_prefix, int item, int& cursor)
{
    const int t = item / p.ntiles;
    while (tile_prefix[cursor + 1] <= t) ++cursor;
    RxItem it;
    it.expert = cursor;
    it.tile = t;
    it.ntile = item % p.ntiles;
    it.row0 = p.offsets[cursor] + (t - tile_prefix[cursor]) * kRxRows;
    it.rows = min(kRxRows, p.offsets[cursor + 1] - it.row0);
    return it;
}

template <bool kUp>
__global__ void __launch_bounds__(kRxThreads, 1)
moe_mxr_kernel(const RxParams p, const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap q_map,
               const int q_rows)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    int* tile_prefix = reinterpret_cast<int*>(smem + kRxStages * kRxStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(tile_prefix) + (kRxMaxExperts + 1) * 4 + 4);
    uint64_t* full = bars;                        // a stage's operands and scale atoms have landed
    uint64_t* empty = full + kRxStages;
    uint64_t* acc_full = empty + kRxStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kRxStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], kRxEpiWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kRxTmemCols);
        tmem_relinquish();
    }
    pdl_launch_dependents();
    pdl_wait();   // row order, tile prefix and quantised rows come from earlier kernels of this call
    for (int e = threadIdx.x; e <= p.experts; e += blockDim.x) tile_prefix[e] = p.tile_prefix[e];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfx = tmem_base + 2 * kRxN, tmem_sfw = tmem_sfx + 4;
    const int items = tile_prefix[p.experts] * p.ntiles;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            // One thread feeds the whole pipeline, so its loop carries no divisions: the stage
            // index, its parity and the prefetch cursor advance by increments.
            uint32_t s = 0, round = 0;          // stage and how many times the ring has wrapped
            uint32_t issued = 0, prefetched = 0;
            int cur = 0, pf_cur = 0;
            int pf_item = blockIdx.x, pf_ks = 0;
            const uint8_t* pf_base = nullptr;
            if (pf_item < items) {
                const RxItem pi = rx_decode(p, tile_prefix, pf_item, pf_cur);
                pf_base = p.w + (size_t((pi.expert - p.expert_base) / p.expert_div) * p.ntiles + pi.ntile) * p.kslabs * kRxPkBytes;
            }
            constexpr uint32_t tx = kRxPkBytes + 2 * kRxATile + 3 * kMxAtom;   // the 4-bit TMA counts packed bytes
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const RxItem it = rx_decode(p, tile_prefix, item, cur);
                const int se = (it.expert - p.expert_base) / p.expert_div;
                const size_t wblock = (size_t(se) * p.ntiles + it.ntile) * p.kslabs;
                const uint8_t* sfw = p.sfw + wblock * (2 * kMxAtom);
                const uint8_t* sfx = p.sfx + size_t(it.tile) * p.kslabs * kMxAtom;
                int wrow = int(wblock * kRxN);
                const int arow = it.tile * kRxRows;
                for (int ks = 0; ks < p.kslabs; ++ks, ++issued) {
                    // ask L2 for the weight blocks a few stages ahead (also across the item boundary)
                    while (pf_base && prefetched < issued + kRxPrefetch) {
                        bulk_prefetch_l2(pf_base + size_t(pf_ks) * kRxPkBytes, kRxPkBytes);
                        ++prefetched;
                        if (++pf_ks == p.kslabs) {
                            pf_ks = 0;
                            pf_item += gridDim.x;
                            pf_base = nullptr;
                            if (pf_item < items) {
                                const RxItem pi = rx_decode(p, tile_prefix, pf_item, pf_cur);
                                pf_base = p.w + (size_t((pi.expert - p.expert_base) / p.expert_div) * p.ntiles + pi.ntile) *
                                                    p.kslabs * kRxPkBytes;
                            }
                        }
                    }
                    if (round > 0 && !mbar_wait_bounded(&empty[s], (round - 1) & 1)) {
                        atomicExch(p.fault, 41);
                        *abort_flag = 1;
                        break;
                    }
                    uint8_t* st = ring + s * kRxStageBytes;
                    uint8_t* sf_s = st + 2 * kRxATile + kRxBTile;
                    mbar_expect_tx(&full[s], tx);
                    tma_load_2d(st + 2 * kRxATile, &w_map, 0, wrow, &full[s]);
                    tma_load_2d(st, &q_map, ks * kMxSlab, arow, &full[s]);
                    tma_load_2d(st + kRxATile, &q_map, ks * kMxSlab, q_rows + arow, &full[s]);
                    bulk_g2s(sf_s, sfx, kMxAtom, &full[s]);
                    bulk_g2s(sf_s + kMxAtom, sfw, 2 * kMxAtom, &full[s]);
                    wrow += kRxN;
                    sfx += kMxAtom;
                    sfw += 2 * kMxAtom;
                    if (++s == kRxStages) {
                        s = 0;
                        ++round;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t s = 0, phase = 0, it_n = 0;
            // The issuing thread shares its scheduler with two epilogue warps, so its loop is
            // kept to a few instructions per MMA: every descriptor is the stage-0 descriptor
            // plus a stage offset and a K-block offset in the start-address field (16-byte
            // units), and the four instruction descriptors differ only in the scale selectors.
            const uint32_t ring_addr = smem_u32(ring);
            const uint64_t hi_d0 = umma_desc_k_sw128(ring_addr), lo_d0 = umma_desc_k_sw128(ring_addr + kRxATile),
                           w_d0 = umma_desc_k_sw128(ring_addr + 2 * kRxATile);
            const uint64_t sfx_d0 = umma_desc_k_plain(ring_addr + 2 * kRxATile + kRxBTile, 128);
            constexpr uint32_t kStageUnits = kRxStageBytes >> 4, kAtomUnits = kMxAtom >> 4;
            // A = e4m3 pieces (rows), B = e2m1 weights
            const uint32_t idesc0 = mx_idesc_fmt(kMxFmtE4M3, kMxFmtE2M1, kRxRows, kRxN, 0);
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
                const uint32_t buf = it_n & 1;
                if (it_n >= 2 && !mbar_wait_bounded(&acc_empty[buf], ((it_n >> 1) - 1) & 1)) {
                    atomicExch(p.fault, 42);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d_addr = tmem_base + buf * kRxN;
                for (int ks = 0; ks < p.kslabs; ++ks) {
                    if (!mbar_wait_bounded(&full[s], phase)) {
                        atomicExch(p.fault, 43);
                        *abort_flag = 1;
                        break;
                    }
                    const uint64_t off = uint64_t(s * kStageUnits);
                    const uint64_t hi_d = hi_d0 + off, lo_d = lo_d0 + off, w_d = w_d0 + off, sf_d = sfx_d0 + off;
                    tmem_cp_32x128b_warpx4(tmem_sfx, sf_d);
                    tmem_cp_32x128b_warpx4(tmem_sfw, sf_d + kAtomUnits);
                    tmem_cp_32x128b_warpx4(tmem_sfw + 4, sf_d + 2 * kAtomUnits);
#pragma unroll
                    for (uint32_t kb = 0; kb < 4; ++kb) {
                        const uint32_t idesc = idesc0 + kb * ((1u << 4) | (1u << 29));
                        umma_mx(d_addr, hi_d + 2 * kb, w_d + 2 * kb, idesc, tmem_sfx, tmem_sfw, ks > 0 || kb > 0);
                        umma_mx(d_addr, lo_d + 2 * kb, w_d + 2 * kb, idesc, tmem_sfx, tmem_sfw, true);
                    }
                    umma_commit(&empty[s]);
                    if (++s == kRxStages) {
                        s = 0;
                        phase ^= 1;
                    }
                }
                if (*abort_flag) break;
                umma_commit(&acc_full[buf]);
            }
        }
    } else if (warp < kRxFirstEpi) {
        // spare warp: keeps the epilogue warps' numbering aligned with the lane quarters
    } else {
        // ------------------------------------------------------------ epilogue
        // Warp w serves the 32-lane quarter w % 4 (a warp may only read its own quarter of
        // tensor memory); the two warps of a quarter take alternate 16-column groups.
        const int quarter = warp & 3, half = (warp - kRxFirstEpi) >> 2;
        const int l = quarter * 32 + lane;   // TMEM lane = routed row of the tile
        uint32_t it_n = 0;
        int cur = 0;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
            const RxItem it = rx_decode(p, tile_prefix, item, cur);
            const uint32_t buf = it_n & 1;
            if (!mbar_wait_bounded(&acc_full[buf], (it_n >> 1) & 1)) {
                atomicExch(p.fault, 45);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const int ebias = p.bias_by_global ? it.expert : (it.expert - p.expert_base) / p.expert_div;
            const float* bias = p.bias + size_t(ebias) * p.rows;
            const bool live = l < it.rows;
            const int pos = it.row0 + min(l, it.rows - 1);
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kRxN;
            const int n0 = it.ntile * kRxN;
            if (kUp) {
                __half* arow = p.act_out + size_t(pos) * (p.rows >> 1) + (n0 >> 1);
                for (int c0 = half * 16; c0 < kRxN; c0 += 32) {
                    if (n0 + c0 >= p.rows) break;   // warp-uniform
                    uint32_t r[16];
                    tmem_ld_32x16(taddr + c0, r);
                    tmem_ld_wait();
                    if (!live) continue;
                    uint32_t packed[4];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {   // columns 2q (gate), 2q + 1 (up) of channel (n0 + c0) / 2 + q
                        const int nrow = n0 + c0 + 2 * q;
                        float gate = 0.f, up = 0.f;
                        if (nrow + 1 < p.rows) {
                            gate = fminf(bf16_round_f(bf16_round_f(__uint_as_float(r[2 * q])) + bias[nrow]), p.limit);
                            up = fminf(p.limit, fmaxf(-p.limit, bf16_round_f(bf16_round_f(__uint_as_float(r[2 * q + 1])) + bias[nrow + 1])));
                        }
                        const float sig = bf16_round_f(1.f / (1.f + expf(-bf16_round_f(1.702f * gate))));
                        const float glu = bf16_round_f(gate * sig);
                        const uint32_t hv = __half_as_ushort(__float2half_rn(bf16_round_f(glu * bf16_round_f(up + 1.f))));
                        if (q & 1) packed[q >> 1] |= hv << 16;
                        else packed[q >> 1] = hv;
                    }
                    if (n0 + c0 + 16 <= p.rows) {
                        *reinterpret_cast<uint4*>(arow + (c0 >> 1)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    } else {
                        for (int q = 0; q < 8; ++q)
                            if (n0 + c0 + 2 * q + 1 < p.rows)
                                arow[(c0 >> 1) + q] = __ushort_as_half(uint16_t(packed[q >> 1] >> (16 * (q & 1))));
                    }
                }
            } else {
                float* vrow = p.vals_out + size_t(p.sorted[pos]) * p.rows + n0;
                for (int c0 = half * 16; c0 < kRxN; c0 += 32) {
                    if (n0 + c0 >= p.rows) break;   // warp-uniform
                    uint32_t r[16];
                    tmem_ld_32x16(taddr + c0, r);
                    tmem_ld_wait();
                    if (!live) continue;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float4 v;
                        float* vp = reinterpret_cast<float*>(&v);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int d = n0 + c0 + 4 * q + j;
                            vp[j] = d < p.rows ? bf16_round_f(bf16_round_f(__uint_as_float(r[4 * q + j])) + bias[d]) : 0.f;
                        }
                        if (p.vals_bf16) {   // the values are bf16-valued: the conversions below are exact
                            __nv_bfloat16* vb = reinterpret_cast<__nv_bfloat16*>(p.vals_out) + size_t(p.sorted[pos]) * p.rows + n0 + c0 + 4 * q;
                            if (n0 + c0 + 4 * q + 3 < p.rows) {
                                const __nv_bfloat162 lo = __floats2bfloat162_rn(vp[0], vp[1]), hi = __floats2bfloat162_rn(vp[2], vp[3]);
                                *reinterpret_cast<uint2*>(vb) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
                            } else {
                                for (int j = 0; j < 4; ++j)
                                    if (n0 + c0 + 4 * q + j < p.rows) vb[j] = __float2bfloat16_rn(vp[j]);
                            }
                        } else if (n0 + c0 + 4 * q + 3 < p.rows) *reinterpret_cast<float4*>(vrow + c0 + 4 * q) = v;
                        else
                            for (int j = 0; j < 4; ++j)
                                if (n0 + c0 + 4 * q + j < p.rows) vrow[c0 + 4 * q + j] = vp[j];
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
        tmem_dealloc(tmem_base, kRxTmemCols);
    }
}

// ------------------------------------------------------------ create-time kernels

// Weight blocks: dst[e][ntile][kslab][240 rows][64 bytes]; rows and columns beyond the
// matrix hold zero codes (moe_pack.h says where each 16-byte piece comes from).
__global__ void mxr_tile_weights_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int experts, MxBlockGeom g)
{
    const size_t per_expert = g.code_bytes() / 16;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;   // one 16-byte piece of the output
    if (idx >= per_expert * experts) return;
    const size_t e = idx / per_expert;
    size_t sb;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (mx_block_piece(g, idx % per_expert, &sb))
        v = *reinterpret_cast<const uint4*>(src + e * g.rows * size_t(g.k / 2) + sb);
    *reinterpret_cast<uint4*>(dst + idx * 16) = v;
}

// Weight scale atoms: dst[e][ntile][kslab][2][512]; rows and groups beyond the matrix get 127.
__global__ void mxr_weight_atoms_kernel(const uint8_t* __restrict__ scales, uint8_t* __restrict__ dst, int experts, MxBlockGeom g)
{
    const size_t per_expert = g.atom_bytes();
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= per_expert * experts) return;
    const size_t e = idx / per_expert;
    size_t sb;
    uint8_t v = 127;
    if (mx_block_atom(g, idx % per_expert, &sb)) v = scales[e * g.rows * size_t(g.k / 32) + sb];
    dst[idx] = v;
}

// fp32 value of every element of one stored expert matrix, decoded from the 15 KiB
// blocks and scale atoms above (the operands the tensor core reads), in the
// original row order.  Subnormal (0) and NaN (255) scale bytes decode as in the
// reference (gpt_oss_kernels.cu:55-56).
__global__ void mxr_dequant_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ sf, float* __restrict__ out,
                                   int expert, int rows, int k, int ntiles, int kslabs)
{
    const size_t total = size_t(rows) * k / 2;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int row = int(idx / (k / 2)), col = int(idx % (k / 2)) * 2;
    const int nt = row / kRxN, r = row % kRxN, ks = col / kMxSlab, c = col % kMxSlab;
    const size_t block = (size_t(expert) * ntiles + nt) * kslabs + ks;
    // the conversion is fed from an aligned 32-bit word, as everywhere else
    const size_t byte = block * kRxPkBytes + size_t(r) * (kMxSlab / 2) + c / 2;
    const uint32_t word = *reinterpret_cast<const uint32_t*>(w + (byte & ~size_t(3)));
    const uint32_t pair = e2m1x2_to_f16x2(word >> (8 * (byte & 3)), 0);
    const int rr = r & 127;
    const uint32_t e = sf[(block * 2 + (r >> 7)) * kMxAtom + (rr & 31) * 16 + (rr >> 5) * 4 + (c >> 5)];
    const float s = e == 0 ? __uint_as_float(0x00400000u) : e == 255 ? __uint_as_float(0x7fc00000u) : __uint_as_float(e << 23);
    const __half2 hv = *reinterpret_cast<const __half2*>(&pair);
    out[size_t(row) * k + col] = __half2float(__low2half(hv)) * s;
    out[size_t(row) * k + col + 1] = __half2float(__high2half(hv)) * s;
}

// ------------------------------------------------------------------ host side

int Moe::dequant_block_scaled(int pass, int stored_expert, float* out, cudaStream_t stream)
{
    if (!mx_ok || !mxr_w[pass]) return fail(GARNET_B200_NOT_SUPPORTED, "moe_dequant: this handle holds no block-scaled weight copy");
    const PackGeom& geo = pass == 0 ? geo_up : geo_down;
    const size_t total = size_t(geo.rows) * geo.cols / 2;
    mxr_dequant_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(mxr_w[pass], mxr_sf[pass], out, stored_expert, geo.rows,
                                                                        geo.cols, mxr_ntiles[pass], mx_kslabs[pass]);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int Moe::init_mxr(int pass, const uint8_t* blocks, const uint8_t* scales, int first_stored, int count, cudaStream_t stream)
{
    const PackGeom& geo = pass == 0 ? geo_up : geo_down;
    const MxBlockGeom g = make_block_geom(geo.rows, geo.cols);
    if (!mxr_w[pass]) {
        // one allocation: all blocks, then all scale atoms (the form garnet_b200_moe_pack_host writes)
        GB_CUDA(cudaMalloc(&mxr_w[pass], size_t(stored_experts) * (g.code_bytes() + g.atom_bytes())));
        mxr_sf[pass] = mxr_w[pass] + size_t(stored_experts) * g.code_bytes();
        mxr_ntiles[pass] = g.ntiles;
    }
    const size_t pieces = size_t(count) * (g.code_bytes() / 16);
    mxr_tile_weights_kernel<<<unsigned((pieces + 255) / 256), 256, 0, stream>>>(
        blocks, mxr_w[pass] + size_t(first_stored) * g.code_bytes(), count, g);
    const size_t bytes = size_t(count) * g.atom_bytes();
    mxr_weight_atoms_kernel<<<unsigned((bytes + 255) / 256), 256, 0, stream>>>(
        scales, mxr_sf[pass] + size_t(first_stored) * g.atom_bytes(), count, g);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int Moe::finish_mxr()
{
    if (opt.experts > kRxMaxExperts) return fail(GARNET_B200_NOT_SUPPORTED, "moe: more than %d experts", kRxMaxExperts);
    GB_CUDA(cudaFuncSetAttribute(moe_mxr_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRxSmemTotal));
    GB_CUDA(cudaFuncSetAttribute(moe_mxr_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRxSmemTotal));
    if (!mxr_w[0] || !mxr_w[1]) return GARNET_B200_OK;   // this handle uses the other orientation
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return fail(GARNET_B200_NOT_SUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    for (int pass = 0; pass < 2; ++pass) {
        // all weight blocks of a projection as one matrix of 128-code rows: block b = rows [240 b, 240 b + 240)
        const cuuint64_t dims[2] = {cuuint64_t(kMxSlab), cuuint64_t(stored_experts) * mxr_ntiles[pass] * mx_kslabs[pass] * kRxN};
        const cuuint64_t strides[1] = {kMxSlab / 2};
        const cuuint32_t box[2] = {kMxSlab, kRxN};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = enc(reinterpret_cast<CUtensorMap*>(&mxr_w_map[pass]), CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2,
                               mxr_w[pass], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GARNET_B200_CUDA_ERROR, "cuTensorMapEncodeTiled (4-bit weight blocks) failed with code %d", int(r));
    }
    return GARNET_B200_OK;
}

int Moe::launch_mxr_gemm(bool up, const MoeWorkspacePtrs& w, const void* q_map_ptr, int q_rows, int tiles_max,
                         cudaStream_t stream)
{
    const int pass = up ? 0 : 1;
    const PackGeom& geo = up ? geo_up : geo_down;
    const MoeShard sh = shard();
    RxParams p;
    p.offsets = w.offsets;
    p.sorted = w.sorted;
    p.tile_prefix = w.mx_tp;
    p.bias = up ? up_bias_ptr : down_bias_ptr;
    p.w = mxr_w[pass];
    p.sfw = mxr_sf[pass];
    p.sfx = w.mx_sf;
    p.act_out = w.act;
    p.vals_out = w.vals;
    p.vals_bf16 = w.vals_bf16;
    p.fault = fault_dev;
    p.experts = opt.experts;
    p.rows = geo.rows;
    p.ntiles = mxr_ntiles[pass];
    p.kslabs = mx_kslabs[pass];
    p.expert_base = (sh.world > 1 && !sh.interleaved) ? sh.lo : (sh.world > 1 ? sh.rank : 0);
    p.expert_div = (sh.world > 1 && sh.interleaved) ? sh.world : 1;
    p.bias_by_global = (!opt.expert_weights_sharded && sh.world > 1) ? 1 : 0;
    p.limit = opt.limit;
    const long long max_items = (long long)tiles_max * p.ntiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(std::min<long long>(kSmCount, max_items)));
    cfg.blockDim = dim3(kRxThreads);
    cfg.dynamicSmemBytes = kRxSmemTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const CUtensorMap& qm = *static_cast<const CUtensorMap*>(q_map_ptr);
    const CUtensorMap& wm = *reinterpret_cast<const CUtensorMap*>(&mxr_w_map[pass]);
    if (up) GB_CUDA(cudaLaunchKernelEx(&cfg, moe_mxr_kernel<true>, p, wm, qm, q_rows));
    else GB_CUDA(cudaLaunchKernelEx(&cfg, moe_mxr_kernel<false>, p, wm, qm, q_rows));
    return GARNET_B200_OK;
}

}  // namespace gb200
