// Block-scaled tensor-core path of the gpt-oss MXFP4 experts: the e2m1 codes and
// their e8m0 scales go to the tensor core as they are stored (tcgen05.mma
// kind::mxf8f6f4 with block scales), so no thread ever expands a weight.  It
// replaces, at every batch size, the reference's grouped WMMA kernel
// (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:843-906) and its Marlin adapter
// (plugins/gpt_oss/cuda/gpt_oss_marlin.cu:586-648).
//
// Operands.
//   A (UMMA M side, 128 rows per tile): expert weights, row-major e2m1 with K padded
//     to a multiple of 128, fetched by TMA with the 16U4_ALIGN16B element type (16
//     codes land in the low 8 bytes of every 16-byte slot, the layout the MMA reads
//     4-bit operands in).  Scales: 512-byte atoms of 128 rows x 4 blocks, copied to
//     tensor memory with tcgen05.cp (32x128b, replicated to the four lane quarters).
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

namespace gb200 {

constexpr int kMxM = 128;            // weight rows per tile
constexpr int kMxSlab = 128;         // K elements per pipeline stage (4 MMAs of K = 32 per piece)
constexpr int kMxAtom = 512;         // bytes of one scale atom: 128 rows x 4 blocks
constexpr int kMxThreads = 6 * 32;   // producer, MMA issuer, 4 epilogue warps
constexpr int kMxMaxExperts = 1024;
constexpr uint32_t kMxATileBytes = kMxM * 128;       // shared-memory footprint of a weight tile
constexpr uint32_t kMxATxBytes = kMxM * kMxSlab / 2;   // bytes the weight tile's TMA transfers

__host__ __device__ constexpr int mx_stage_bytes(int nt) { return int(kMxATileBytes) + 2 * nt * 128 + 2 * kMxAtom; }
__host__ __device__ constexpr int mx_stages(int nt)
{
    const int s = (200 * 1024) / mx_stage_bytes(nt);
    return s > 8 ? 8 : s;
}
__host__ __device__ constexpr int mx_tmem_cols(int nt)
{
    const int need = 2 * nt + 8;
    return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
}
// dynamic shared memory: 1 KiB alignment slack, the stages, tile prefix, barriers
__host__ __device__ constexpr int mx_smem_total(int nt)
{
    return 1024 + mx_stages(nt) * mx_stage_bytes(nt) + (kMxMaxExperts + 1) * 4 + 256;
}

struct MxParams {
    const int* offsets;        // [experts + 1] start of every expert's rows in sorted order
    const int* sorted;         // [slots] slot ids in expert order
    const int* tile_prefix;    // [experts + 1] row tiles before each expert
    const float* bias;         // [experts(local or global), rows] original row order
    const uint8_t* sfa;        // [stored experts][mtiles][kslabs][512] weight scale atoms
    const uint8_t* sfb;        // [row tiles][kslabs][512] activation scale atoms
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

// 3-D tiled TMA load (innermost coordinate first).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}

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

// Instruction descriptor of kind::mxf8f6f4: A = e2m1, B = e4m3, both K-major, e8m0
// scales; `sf` selects which of the four blocks of the scale atoms this MMA uses.
__device__ __forceinline__ uint32_t mx_idesc(int m, int n, uint32_t sf)
{
    return (sf << 4) | (5u << 7) | (0u << 10) | (uint32_t(n >> 3) << 17) | (1u << 23) | (uint32_t(m >> 4) << 24) |
           (sf << 29);
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
moe_mx_kernel(const MxParams p, const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap q_map,
              const int q_rows)
{
    constexpr int kStages = mx_stages(kN);
    constexpr int kStageBytes = mx_stage_bytes(kN);
    constexpr uint32_t kTmemCols = mx_tmem_cols(kN);
    constexpr uint32_t kStageTx = kMxATxBytes + 2 * kN * 128 + 2 * kMxAtom;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    int* tile_prefix = reinterpret_cast<int*>(smem + kStages * kStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + (kMxMaxExperts + 1) * 4 + 4);
    uint64_t* full = bars;
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
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
    pdl_launch_dependents();
    pdl_wait();   // row order, tile prefix and quantised rows come from earlier kernels of this call
    for (int e = threadIdx.x; e <= p.experts; e += blockDim.x) tile_prefix[e] = p.tile_prefix[e];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfa = tmem_base + 2 * kN, tmem_sfb = tmem_sfa + 4;
    const int items = tile_prefix[p.experts] * p.mtiles;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t n = 0;
            int cur = 0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const MxItem it = mx_decode<kN>(p, tile_prefix, item, cur);
                const int se = (it.expert - p.expert_base) / p.expert_div;
                const uint8_t* sfa = p.sfa + (size_t(se) * p.mtiles + it.mtile) * p.kslabs * kMxAtom;
                const uint8_t* sfb = p.sfb + size_t(it.tile) * p.kslabs * kMxAtom;
                for (int ks = 0; ks < p.kslabs; ++ks, ++n) {
                    const uint32_t s = n % kStages;
                    if (n >= kStages && !mbar_wait_bounded(&empty[s], ((n / kStages) - 1) & 1)) {
                        atomicExch(p.fault, 31);
                        *abort_flag = 1;
                        break;
                    }
                    uint8_t* st = ring + s * kStageBytes;
                    mbar_expect_tx(&full[s], kStageTx);
                    tma_load_3d(st, &w_map, ks * kMxSlab, it.mtile * kMxM, se, &full[s]);
                    tma_load_2d(st + kMxATileBytes, &q_map, ks * kMxSlab, it.tile * kN, &full[s]);
                    tma_load_2d(st + kMxATileBytes + kN * 128, &q_map, ks * kMxSlab, q_rows + it.tile * kN, &full[s]);
                    bulk_g2s(st + kMxATileBytes + 2 * kN * 128, sfa + size_t(ks) * kMxAtom, kMxAtom, &full[s]);
                    bulk_g2s(st + kMxATileBytes + 2 * kN * 128 + kMxAtom, sfb + size_t(ks) * kMxAtom, kMxAtom, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t n = 0, it_n = 0;
            for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++it_n) {
                const uint32_t buf = it_n & 1;
                if (it_n >= 2 && !mbar_wait_bounded(&acc_empty[buf], ((it_n >> 1) - 1) & 1)) {
                    atomicExch(p.fault, 32);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                for (int ks = 0; ks < p.kslabs; ++ks, ++n) {
                    const uint32_t s = n % kStages;
                    if (!mbar_wait_bounded(&full[s], (n / kStages) & 1)) {
                        atomicExch(p.fault, 33);
                        *abort_flag = 1;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(ring + s * kStageBytes);
                    const uint32_t hi_addr = a_addr + kMxATileBytes, lo_addr = hi_addr + kN * 128;
                    const uint32_t sfa_addr = lo_addr + kN * 128, sfb_addr = sfa_addr + kMxAtom;
                    tmem_cp_32x128b_warpx4(tmem_sfa, umma_desc_k_plain(sfa_addr, 128));
                    tmem_cp_32x128b_warpx4(tmem_sfb, umma_desc_k_plain(sfb_addr, 128));
#pragma unroll
                    for (uint32_t kb = 0; kb < 4; ++kb) {
                        const uint32_t idesc = mx_idesc(kMxM, kN, kb);
                        const uint64_t a_desc = umma_desc_k_sw128(a_addr + kb * 32);
                        umma_mx(tmem_base + buf * kN, a_desc, umma_desc_k_sw128(hi_addr + kb * 32), idesc, tmem_sfa,
                                tmem_sfb, ks > 0 || kb > 0);
                        umma_mx(tmem_base + buf * kN, a_desc, umma_desc_k_sw128(lo_addr + kb * 32), idesc, tmem_sfa,
                                tmem_sfb, true);
                    }
                    umma_commit(&empty[s]);
                }
                if (*abort_flag) break;
                umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;
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
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kN;
            if (kUp) {
                // rows 2i (gate) and 2i+1 (up) sit in neighbouring lanes
                const float b_other = __shfl_xor_sync(0xffffffffu, b_mine, 1);
                const int ch = row >> 1;
                const int inter = p.rows >> 1;
                for (int c0 = 0; c0 < kN && c0 < it.rows; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld_32x16(taddr + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float mine = __uint_as_float(r[j]);
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        if (!(lane & 1) && row_ok && c0 + j < it.rows) {
                            const float gate = fminf(bf16_round_f(bf16_round_f(mine) + b_mine), p.limit);
                            const float up = fminf(p.limit, fmaxf(-p.limit, bf16_round_f(bf16_round_f(other) + b_other)));
                            const float sig = bf16_round_f(1.f / (1.f + expf(-bf16_round_f(1.702f * gate))));
                            const float glu = bf16_round_f(gate * sig);
                            p.act_out[size_t(it.row0 + c0 + j) * inter + ch] =
                                __float2half_rn(bf16_round_f(glu * bf16_round_f(up + 1.f)));
                        }
                    }
                }
            } else {
                for (int c0 = 0; c0 < kN && c0 < it.rows; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld_32x16(taddr + c0, r);
                    tmem_ld_wait();
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
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------ create-time kernels

// Row-major e2m1 rows padded with zero codes to `kp` columns: dst[e][row][kp / 2].
__global__ void mx_pad_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long rows_total,
                                   int k, int kp)
{
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one 16-byte piece of a padded row
    const int per_row = kp / 32;
    if (idx >= rows_total * per_row) return;
    const long long row = idx / per_row;
    const int piece = int(idx % per_row);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (piece * 32 < k) v = *reinterpret_cast<const uint4*>(src + row * (k / 2) + piece * 16);
    *reinterpret_cast<uint4*>(dst + row * (kp / 2) + piece * 16) = v;
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

// tile_prefix[e] = number of nt-row tiles of the experts before e; one warp.
__global__ void mx_tile_prefix_kernel(const int* __restrict__ offsets, int experts, int nt, int* __restrict__ tile_prefix)
{
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x;
    int run = 0;
    for (int e0 = 0; e0 < experts; e0 += 32) {
        const int e = e0 + lane;
        int tiles = 0;
        if (e < experts) tiles = (offsets[e + 1] - offsets[e] + nt - 1) / nt;
        int incl = tiles;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += v;
        }
        if (e < experts) tile_prefix[e] = run + incl - tiles;
        run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) tile_prefix[experts] = run;
}

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

template <typename T>
__device__ __forceinline__ float mx_load(const T* p);
template <>
__device__ __forceinline__ float mx_load<float>(const float* p) { return bf16_round_f(*p); }
template <>
__device__ __forceinline__ float mx_load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float mx_load<__half>(const __half* p) { return __half2float(*p); }

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
    const int kslabs = kp / kMxSlab;
    for (int b = threadIdx.x; b < kp / 32; b += blockDim.x) {
        float v[32];
        float amax = 0.f;
        if (b * 32 < k) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                v[i] = mx_load<T>(row + b * 32 + i);
                amax = fmaxf(amax, fabsf(v[i]));
            }
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
        sf[(size_t(tile) * kslabs + (b >> 2)) * kMxAtom + (r & 31) * 16 + (r >> 5) * 4 + (b & 3)] = uint8_t(sbyte);
    }
}

// ------------------------------------------------------------------ host side

bool moe_mx_enabled()
{
    // GARNET_B200_MOE_MX=0 keeps the expert GEMMs on the kernels that expand the
    // weights in registers (A/B switch, read once).
    static const bool on = [] {
        const char* e = getenv("GARNET_B200_MOE_MX");
        return !(e && e[0] == '0');
    }();
    return on;
}

int moe_mx_nt(int rows_per_expert_max)
{
    return rows_per_expert_max <= 16 ? 16 : rows_per_expert_max <= 32 ? 32 : rows_per_expert_max <= 64 ? 64 : 128;
}

MoeMxPlan moe_mx_plan(const garnet_b200_moe_options& o, int tokens, int slots)
{
    MoeMxPlan m;
    m.nt = moe_mx_nt(tokens);
    m.tiles_max = slots / m.nt + std::min(slots, o.experts) + 1;   // full tiles + one partial tile per expert that has rows
    m.q_rows = m.tiles_max * m.nt;
    const int kmax = std::max(o.hidden, o.intermediate);
    m.kp_max = (kmax + kMxSlab - 1) / kMxSlab * kMxSlab;
    m.q_bytes = size_t(2) * m.q_rows * m.kp_max;
    m.sf_bytes = size_t(m.tiles_max) * (m.kp_max / kMxSlab) * kMxAtom;
    return m;
}

static int mx_encode(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base, const cuuint64_t* dims,
                     const cuuint64_t* strides, const cuuint32_t* box)
{
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return fail(GARNET_B200_NOT_SUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(map, dt, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
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
    if (!mx_w[pass]) {
        // one spare row: the last tile's TMA box may start inside the matrix and is clipped, never read past it
        GB_CUDA(cudaMalloc(&mx_w[pass], size_t(stored_experts) * rows * (kp / 2)));
        GB_CUDA(cudaMalloc(&mx_sfa[pass], size_t(stored_experts) * mtiles * kslabs * kMxAtom));
        mx_kp[pass] = kp;
        mx_mtiles[pass] = mtiles;
        mx_kslabs[pass] = kslabs;
    }
    const long long rows_total = (long long)count * rows;
    const long long pieces = rows_total * (kp / 32);
    mx_pad_rows_kernel<<<unsigned((pieces + 255) / 256), 256, 0, stream>>>(
        blocks, mx_w[pass] + size_t(first_stored) * rows * (kp / 2), rows_total, k, kp);
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
    static_assert(sizeof(TensorMapStorage) == sizeof(CUtensorMap), "tensor map storage size");
    for (int pass = 0; pass < 2; ++pass) {
        const PackGeom& geo = pass == 0 ? geo_up : geo_down;
        const cuuint64_t dims[3] = {cuuint64_t(mx_kp[pass]), cuuint64_t(geo.rows), cuuint64_t(stored_experts)};
        const cuuint64_t strides[2] = {cuuint64_t(mx_kp[pass] / 2), cuuint64_t(geo.rows) * (mx_kp[pass] / 2)};
        const cuuint32_t box[3] = {kMxSlab, kMxM, 1};
        if (int rc = mx_encode(reinterpret_cast<CUtensorMap*>(&mx_w_map[pass]), CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3,
                               mx_w[pass], dims, strides, box))
            return rc;
    }
    GB_CUDA((mx_set_attr<true, 16>()));
    GB_CUDA((mx_set_attr<true, 32>()));
    GB_CUDA((mx_set_attr<true, 64>()));
    GB_CUDA((mx_set_attr<true, 128>()));
    GB_CUDA((mx_set_attr<false, 16>()));
    GB_CUDA((mx_set_attr<false, 32>()));
    GB_CUDA((mx_set_attr<false, 64>()));
    GB_CUDA((mx_set_attr<false, 128>()));
    mx_ok = true;
    return GARNET_B200_OK;
}

template <bool kUp, int kN>
static cudaError_t mx_launch(const MxParams& p, const CUtensorMap& wm, const CUtensorMap& qm, int q_rows, int grid,
                             cudaStream_t stream)
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
    return cudaLaunchKernelEx(&cfg, moe_mx_kernel<kUp, kN>, p, wm, qm, q_rows);
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
    if (up) {
        cfg.gridDim = dim3(1);
        cfg.blockDim = dim3(32);
        GB_CUDA(cudaLaunchKernelEx(&cfg, mx_tile_prefix_kernel, (const int*)w.offsets, opt.experts, nt, w.mx_tp));
    }
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
    MxParams p;
    p.offsets = w.offsets;
    p.sorted = w.sorted;
    p.tile_prefix = w.mx_tp;
    p.bias = up ? up_bias_ptr : down_bias_ptr;
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
    const CUtensorMap& wm = *reinterpret_cast<const CUtensorMap*>(&mx_w_map[pass]);
    // upper bound of the item count: every tile of every expert
    const long long max_items = (long long)plan.tiles_max * p.mtiles;
    const int grid = int(std::min<long long>(kSmCount, max_items));
#define GB_MX_LAUNCH(N_)                                                                       \
    GB_CUDA(up ? (mx_launch<true, N_>(p, wm, q_map, plan.q_rows, grid, stream))                \
               : (mx_launch<false, N_>(p, wm, q_map, plan.q_rows, grid, stream)))
    if (nt == 16) GB_MX_LAUNCH(16);
    else if (nt == 32) GB_MX_LAUNCH(32);
    else if (nt == 64) GB_MX_LAUNCH(64);
    else GB_MX_LAUNCH(128);
#undef GB_MX_LAUNCH
    return GARNET_B200_OK;
}

}  // namespace gb200
