// Per-call side of the block-scaled tensor-core path of the gpt-oss MXFP4 experts
// (the grouped GEMM itself is moe_mxr.cu): the routed rows are quantised for the
// tensor core, and the two projections are launched.
//
// The MMA (tcgen05.mma kind::mxf8f6f4 with block scales) takes the e2m1 weights and
// their e8m0 scales as they are stored; on the activation side it takes 8-bit
// floats, so every bf16 activation is split into two e4m3 numbers that share the
// e8m0 scale of their 32-block: hi = e4m3(v), lo = e4m3(v - hi), v = x / 2^s with the
// block maximum scaled into [128, 256).  hi + lo equals v exactly for elements
// within 2^-9 of the block maximum and to 2^-17 of it otherwise, far below the bf16
// rounding of the result.  Both pieces multiply the same weight tile and
// accumulate into the same fp32 accumulator.
//
// Rows are grouped by expert (the stable slot order of moe_fill_kernel); tiles of
// 128 rows never span two experts, and the quantiser writes rows and scale atoms
// at tile-aligned positions, so a tile's operands are plain TMA boxes.  Replaces the
// reference's per-call preparation for its grouped GEMM
// (plugins/gpt_oss/cuda/gpt_oss_marlin.cu:586-648).
#include <algorithm>
#include <cstdlib>

#include "layout.h"
#include "moe.h"
#include "tc_common.cuh"
#include "mx_common.cuh"

namespace gb200 {

constexpr int kMxRowsPerTile = 128;   // routed rows per tile (the UMMA M of moe_mxr.cu)

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

// One 32-block of a row (bf16-valued floats, largest magnitude `amax`) -> 32 e4m3 codes
// of the first piece, 32 of the second, and the e8m0 byte they share.  The block is
// scaled by a power of two so that its maximum lands in [128, 256); hi = e4m3(v),
// lo = e4m3(v - hi).  A block that holds an infinity or a NaN gets the scale byte 255,
// which the tensor core reads as NaN: non-finite activations give NaN outputs (the
// reference's fp32 arithmetic gives an infinity or a NaN there).
__device__ __forceinline__ int mx_split_block(const float (&v)[32], float amax, uint32_t (&hi_w)[8], uint32_t (&lo_w)[8])
{
    int sbyte = 127;
    const bool finite = isfinite(amax);
    if (amax > 0.f && finite) sbyte = int((__float_as_uint(amax) >> 23) & 0xff) - 7;   // max lands in [128, 256)
    sbyte = max(1, min(254, sbyte));
    const float inv = __uint_as_float(uint32_t(254 - sbyte) << 23);   // 2^(127 - sbyte)
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        uint32_t hw = 0, lw = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float a = finite ? v[i + 2 * h] * inv : 0.f, c = finite ? v[i + 2 * h + 1] * inv : 0.f;
            const uint32_t hp = f32x2_to_e4m3x2(a, c);
            const float2 back = e4m3x2_to_f32x2(hp);
            const uint32_t lp = f32x2_to_e4m3x2(a - back.x, c - back.y);
            hw |= hp << (16 * h);
            lw |= lp << (16 * h);
        }
        hi_w[i >> 2] = hw;
        lo_w[i >> 2] = lw;
    }
    return finite ? sbyte : 255;
}

// The same split on plain rows: hi and lo [rows, k] e4m3 codes, scales [rows, k/32].
// One thread per 32-block.  (Check of the split by itself.)
__global__ void mx_split_rows_kernel(const __nv_bfloat16* __restrict__ src, int rows, int k, uint8_t* __restrict__ hi,
                                     uint8_t* __restrict__ lo, uint8_t* __restrict__ scales)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * (k / 32)) return;
    float v[32];
    mx_load32(src + size_t(idx) * 32, v);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    if (!(amax == amax)) amax = __uint_as_float(0x7f800000u);   // a NaN in the block: fmaxf drops it
#pragma unroll
    for (int i = 0; i < 32; ++i)
        if (v[i] != v[i]) amax = __uint_as_float(0x7f800000u);
    uint32_t hi_w[8], lo_w[8];
    scales[idx] = uint8_t(mx_split_block(v, amax, hi_w, lo_w));
    uint4* dh = reinterpret_cast<uint4*>(hi + size_t(idx) * 32);
    uint4* dl = reinterpret_cast<uint4*>(lo + size_t(idx) * 32);
    dh[0] = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
    dh[1] = make_uint4(hi_w[4], hi_w[5], hi_w[6], hi_w[7]);
    dl[0] = make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
    dl[1] = make_uint4(lo_w[4], lo_w[5], lo_w[6], lo_w[7]);
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
    const int kslabs = kp / kMxSlab;
    for (int b = threadIdx.x; b < kp / 32; b += blockDim.x) {
        float v[32];
        float amax = 0.f;
        if (b * 32 < k) {
            mx_load32(row + b * 32, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                amax = fmaxf(amax, fabsf(v[i]));
                if (v[i] != v[i]) amax = __uint_as_float(0x7f800000u);   // fmaxf drops a NaN: mark the block non-finite
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        uint32_t hi_w[8], lo_w[8];
        const int sbyte = mx_split_block(v, amax, hi_w, lo_w);
        uint8_t* dst_hi = q + (size_t(tile) * nt + r) * kp + b * 32;
        uint8_t* dst_lo = dst_hi + size_t(q_rows) * kp;
        *reinterpret_cast<uint4*>(dst_hi) = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
        *reinterpret_cast<uint4*>(dst_hi + 16) = make_uint4(hi_w[4], hi_w[5], hi_w[6], hi_w[7]);
        *reinterpret_cast<uint4*>(dst_lo) = make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
        *reinterpret_cast<uint4*>(dst_lo + 16) = make_uint4(lo_w[4], lo_w[5], lo_w[6], lo_w[7]);
        // both pieces of the row carry the same scale: one byte of the tile's scale atom
        uint8_t* atom = sf + (size_t(tile) * kslabs + (b >> 2)) * kMxAtom;
        atom[(r & 31) * 16 + ((r >> 5) & 3) * 4 + (b & 3)] = uint8_t(sbyte);
    }
}

// ------------------------------------------------------------------ host side

// GARNET_B200_MOE_MX: 0 keeps the experts on the streaming kernel at every size, 2
// uses the block-scaled path at every size (for tests), anything else lets the row
// count per expert decide.  Read once.
static int moe_mx_mode()
{
    static const int mode = [] {
        const char* e = getenv("GARNET_B200_MOE_MX");
        return (e && e[0] == '0') ? 0 : (e && e[0] == '2') ? 2 : 1;
    }();
    return mode;
}
int moe_mx_mode_of(const garnet_b200_moe_options& o)
{
    if (o.layouts == GARNET_B200_MOE_LAYOUT_STREAM) return 0;
    if (o.layouts == GARNET_B200_MOE_LAYOUT_BLOCK) return 2;
    return moe_mx_mode();
}

MoeMxPlan moe_mx_plan(const garnet_b200_moe_options& o, int tokens, int slots)
{
    (void)tokens;
    MoeMxPlan m;
    m.nt = kMxRowsPerTile;
    m.tiles_max = slots / m.nt + std::min(slots, o.experts) + 1;   // full tiles + one partial tile per expert that has rows
    m.q_rows = m.tiles_max * m.nt;
    const int kmax = std::max(o.hidden, o.intermediate);
    m.kp_max = (kmax + kMxSlab - 1) / kMxSlab * kMxSlab;
    m.q_bytes = size_t(2) * m.q_rows * m.kp_max;
    m.sf_bytes = size_t(m.tiles_max) * (m.kp_max / kMxSlab) * kMxAtom;
    return m;
}

int mx_encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base, const cuuint64_t* dims,
                         const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle)
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

// Second copy of the expert weights in the block-scaled path's layout.  `blocks` and
// `scales` are the tensors of the stored experts, in stored order.
int Moe::finish_mx()
{
    mx_ok = false;
    if (!tensor_map_encoder() || opt.experts > kMxMaxExperts) return GARNET_B200_OK;
    if ((opt.hidden % 32) || (opt.intermediate % 32)) return GARNET_B200_OK;
    if (int rc = finish_mxr()) return rc;
    mx_ok = true;
    return GARNET_B200_OK;
}

// Quantises the rows (layer input for the gate/up projection, activations for the
// down projection) and runs the grouped GEMM of one projection.
//   x: layer input [tokens, hidden] in the operator's io dtype (gate/up only)
int Moe::launch_mx(bool up, const MoeWorkspacePtrs& w, const void* x, int x_is_sorted, int tokens, int slots, int topk,
                   cudaStream_t stream)
{
    const int pass = up ? 0 : 1;
    const PackGeom& geo = up ? geo_up : geo_down;
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

    // The view of the quantised rows depends only on the buffer, the padded K and the
    // row capacity: encoded once per such triple, not on every call.
    QMapCache& c = q_map_cache[pass];
    if (c.base != w.mx_q || c.kp != kp || c.q_rows != plan.q_rows) {
        const cuuint64_t dims[2] = {cuuint64_t(kp), cuuint64_t(2) * plan.q_rows};
        const cuuint64_t strides[1] = {cuuint64_t(kp)};
        const cuuint32_t box[2] = {kMxSlab, cuuint32_t(nt)};
        if (int rc = mx_encode_tensor_map(reinterpret_cast<CUtensorMap*>(&c.map), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.mx_q, dims,
                                          strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return rc;
        c.base = w.mx_q;
        c.kp = kp;
        c.q_rows = plan.q_rows;
    }
    return launch_mxr_gemm(up, w, &c.map, plan.q_rows, plan.tiles_max, stream);
}

}  // namespace gb200

extern "C" int garnet_b200_mx_split_rows(const void* d_x_bf16, int rows, int k, uint8_t* d_hi, uint8_t* d_lo, uint8_t* d_scales,
                                         void* stream)
{
    using namespace gb200;
    if (!d_x_bf16 || !d_hi || !d_lo || !d_scales || rows <= 0 || k <= 0 || k % 32)
        return fail(GARNET_B200_INVALID_VALUE, "mx_split_rows: bad argument");
    if ((reinterpret_cast<uintptr_t>(d_x_bf16) | reinterpret_cast<uintptr_t>(d_hi) | reinterpret_cast<uintptr_t>(d_lo)) & 15)
        return fail(GARNET_B200_INVALID_VALUE, "mx_split_rows: pointers must be 16-byte aligned");
    const int blocks = rows * (k / 32);
    mx_split_rows_kernel<<<(blocks + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(d_x_bf16), rows, k, d_hi, d_lo, d_scales);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}
