// Weight-only int4 linear for sm_100a: repackers, dequant check kernel, the
// small-batch streaming kernel (M <= 16 per launch) and the C ABI around them.
//
// Numerics: y[m,n] = bf16( sum_k x[m,k] * q[n,k] * s[n,k/group] ) with fp32
// accumulation.  In the streaming kernel q is expanded to an exact bf16 integer,
// each group's partial sum is accumulated by the tensor core in fp32 and the
// group scale is applied to that partial sum in fp32, so no product is rounded
// before the final bf16 store.
#include <algorithm>
#include <memory>
#include <vector>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"
#include "layout.h"
#include "w4a16.h"

namespace gb200 {

// ------------------------------------------------------------------ repack

// One thread per packed 32-bit word (8 codes of one row).
__global__ void w4_repack_codes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, PackGeom geo,
                                       long long src_row0)
{
    const size_t words_per_chunk = geo.chunk_data / 4;
    const size_t total = size_t(geo.strips_padded) * geo.chunks * words_per_chunk;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t chunk_lin = idx / words_per_chunk;
    const int w = int(idx % words_per_chunk);
    const int strip = int(chunk_lin / geo.chunks), chunk = int(chunk_lin % geo.chunks);
    // invert locate(): word index -> (row, first column)
    const int tile = w >> 7, unit = (w >> 2) & 31, word = w & 3;      // 128 words per 512-byte tile
    const int g = unit >> 2, t = unit & 3, h = word & 1, j = word >> 1;
    const int n = strip * 16 + row_of_g(g) + 8 * h;
    const int k0 = chunk * geo.chunk_k + tile * 64 + (t + 4 * j) * 8;
    uint32_t out = 0;
    if (n < geo.rows && k0 < geo.cols) {
        // K is a multiple of 8, so the 8 codes are 4 aligned source bytes.
        const size_t sb = ((size_t(src_row0) + n) * size_t(geo.cols) + k0) / 2;
        const uint32_t in = *reinterpret_cast<const uint32_t*>(src + sb);
        if (geo.format == kFormatInt4) {
#pragma unroll
            for (int e = 0; e < 8; ++e) out |= ((in >> (4 * e)) & 15u) << (4 * ((e >> 1) + 4 * (e & 1)));
        } else {
            out = in;
        }
    }
    const size_t ob = (size_t(strip) * geo.chunks + chunk) * geo.chunk_bytes + size_t(w) * 4;
    *reinterpret_cast<uint32_t*>(dst + ob) = out;
}

// int4 scales: one thread per (padded row, chunk).  The 16 scale bits are kept as
// they are (fp16 or bf16); the kernels widen them to fp32 according to the
// handle's scale_dtype.
__global__ void w4_repack_scales_int4_kernel(const uint16_t* __restrict__ src, uint8_t* __restrict__ dst,
                                             PackGeom geo, long long src_row0)
{
    const size_t total = size_t(geo.strips_padded) * 16 * geo.chunks;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int n = int(idx / geo.chunks), chunk = int(idx % geo.chunks);
    uint16_t bits = 0;
    if (n < geo.rows) {
        const int groups = geo.cols / geo.group;
        bits = src[(size_t(src_row0) + n) * groups + (chunk * geo.chunk_k) / geo.group];
    }
    *reinterpret_cast<uint16_t*>(dst + locate_scale(geo, n, chunk * geo.chunk_k)) = bits;
}

// ------------------------------------------------------------------ dequant

// fp32 q*s of every logical element, decoded from the packed tiles with the same
// device function the GEMM kernels use.
__device__ __forceinline__ float scale16_to_float(uint32_t bits16, int scale_dtype)
{
    return scale_dtype == GARNET_B200_BF16 ? __uint_as_float(bits16 << 16)
                                           : __half2float(__ushort_as_half(uint16_t(bits16)));
}

__global__ void w4_dequant_kernel(const uint8_t* __restrict__ packed, float* __restrict__ out, PackGeom geo,
                                  int scale_dtype)
{
    const size_t total = size_t(geo.rows) * geo.cols / 2;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int n = int(idx / (geo.cols / 2)), k = int(idx % (geo.cols / 2)) * 2;   // elements k, k+1
    const PackPos p = locate(geo, n, k);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(packed + p.word_byte);
    const int pair = (k & 7) >> 1;
    const uint32_t v = int4x2_to_bf16x2(w >> (4 * pair));
    const float s = scale16_to_float(*reinterpret_cast<const uint16_t*>(packed + locate_scale(geo, n, k)), scale_dtype);
    out[size_t(n) * geo.cols + k] = __bfloat162float(__ushort_as_bfloat16(uint16_t(v & 0xffff))) * s;
    out[size_t(n) * geo.cols + k + 1] = __bfloat162float(__ushort_as_bfloat16(uint16_t(v >> 16))) * s;
}

// --------------------------------------------------------------- quantizer

// One warp per (row, group).  weight_quantization.cpp:220-266.
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, size_t i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, size_t i)
{
    return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p, size_t i) { return __half2float(p[i]); }

template <typename T>
__global__ void int4_quantize_kernel(const T* __restrict__ src, long long rows, long long cols, int group,
                                     int scale_dtype, uint8_t* __restrict__ nibbles, uint16_t* __restrict__ scales)
{
    const long long groups = cols / group;
    const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= rows * groups) return;
    const long long row = wid / groups, grp = wid % groups;
    const size_t start = size_t(row) * cols + size_t(grp) * group;
    float lo = 0.f, hi = 0.f;
    for (int o = lane; o < group; o += 32) {
        const float v = load_as_float(src, start + o);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    for (int off = 16; off; off >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
    }
    float scale = fmaxf(__fdiv_rn(-lo, 8.0f), __fdiv_rn(hi, 7.0f));
    if (!isfinite(scale) || scale <= 0.f) scale = 1.0f;
    uint16_t bits;
    float stored;
    if (scale_dtype == GARNET_B200_FP16) {
        const __half hs = __float2half_rn(scale);
        bits = __half_as_ushort(hs);
        stored = __half2float(hs);
    } else {
        const __nv_bfloat16 bs = __float2bfloat16_rn(scale);
        bits = __bfloat16_as_ushort(bs);
        stored = __bfloat162float(bs);
    }
    if (lane == 0) scales[row * groups + grp] = bits;
    // each lane packs pairs of elements: byte index (start + 2i) / 2
    for (int o = 2 * lane; o < group; o += 64) {
        int q0 = __float2int_rn(__fdiv_rn(load_as_float(src, start + o), stored));
        int q1 = __float2int_rn(__fdiv_rn(load_as_float(src, start + o + 1), stored));
        q0 = max(-8, min(7, q0));
        q1 = max(-8, min(7, q1));
        nibbles[(start + o) >> 1] = uint8_t((q0 & 15) | ((q1 & 15) << 4));
    }
}

// ------------------------------------------------------- streaming kernel

// Two shapes of CTA, both with 16-chunk segments: 8 consumer warps with two chunks
// each (many strips per CTA) and 16 consumer warps with one chunk each (few strips,
// e.g. a 2048-row projection: more warps share one strip, lower latency).
constexpr int kInt4ChunkBytes = 1024 + 32;
constexpr int kWideMaxStripsPerSm = 1;    // at most this many strips per SM: 16-warp CTAs
constexpr int kStreamCtasPerSm = 3;       // 8-warp CTAs per SM (shared memory allows 3 at K = 2048)
// A 16-warp CTA asks for more than half of the SM's shared memory so that it has the
// SM to itself: with programmatic dependent launch the next launch's CTAs otherwise
// move in beside it, two of them land on some SMs, and the launch takes as long as
// those (down_proj at batch 1: 5.0 us with sharing, 3.8 us without).
constexpr size_t kWideSmemFloor = 120000;
__host__ __device__ constexpr int stream_stages(int) { return 3; }
__host__ __device__ constexpr int chunks_per_warp(int warps) { return warps == 16 ? 1 : 2; }
__host__ __device__ constexpr int seg_chunks(int warps) { return chunks_per_warp(warps) * warps; }
__host__ __device__ constexpr int seg_bytes(int warps) { return seg_chunks(warps) * kInt4ChunkBytes; }

constexpr int kMaxGroup = 4;   // linears that share one input and one launch (q/k/v, gate/up)

struct StreamParams {
    const uint8_t* packed[kMaxGroup];
    __nv_bfloat16* y[kMaxGroup];
    int n[kMaxGroup];         // logical weight rows of each matrix
    int ldy[kMaxGroup];       // row stride of each y in elements
    int strip_end[kMaxGroup]; // cumulative strip count: matrix g owns strips [strip_end[g-1], strip_end[g])
    int group;                // matrices in this launch
    const __nv_bfloat16* x;
    int* fault;               // mapped host word; non-zero = a bounded wait gave up
    int m, k;                 // batch rows, logical K
    int strips, chunks;       // total real strips over the group, chunks per strip
    int scale_dtype;          // GARNET_B200_FP16 / GARNET_B200_BF16
};

// Strip of the concatenated list -> (matrix, strip inside it).
__device__ __forceinline__ int stream_matrix_of(const StreamParams& p, int strip, int& local)
{
    int g = 0;
#pragma unroll
    for (int q = 0; q < kMaxGroup - 1; ++q)
        if (q + 1 < p.group && strip >= p.strip_end[q]) g = q + 1;
    local = strip - (g ? p.strip_end[g - 1] : 0);
    return g;
}

// Two int4 codes -> bf16x2 {128 + (q+8), ...}: the biased form, without the
// subtraction.  The bias is removed once per (batch row, chunk) from the
// accumulated sum: sum_k (136 + q_k) x_k - 136 * sum_k x_k.
__device__ __forceinline__ uint32_t int4x2_to_bf16x2_biased(uint32_t word_shifted)
{
    return lop3_and_xor(word_shifted, 0x000F000Fu, 0x43084308u);
}

template <bool kBiased>
__device__ __forceinline__ uint32_t int4x2_expand(uint32_t word_shifted)
{
    return kBiased ? int4x2_to_bf16x2_biased(word_shifted) : int4x2_to_bf16x2(word_shifted);
}

// Shared-memory plan of the streaming kernel (bytes).
struct StreamSmem {
    int ring, red, bars, sx, xs, total;
    int x_rows, x_stride;
};
__host__ __device__ inline StreamSmem stream_smem_plan(int warps, int mb, int m, int k, int chunks)
{
    const int kStreamStages = stream_stages(warps), kSegBytes = seg_bytes(warps), kStreamWarps = warps;
    StreamSmem p;
    p.x_rows = min(m, 8 * mb) + 1;                 // one shared all-zero row for the padded batch columns
    p.x_stride = k * 2 + 64;                       // 64 mod 128: conflict-free 16-byte reads across rows
    p.ring = 0;
    p.red = p.ring + kStreamStages * kSegBytes;    // [2][warps][mb*4][32] fp32
    p.bars = p.red + 2 * kStreamWarps * mb * 128 * 4;
    p.sx = p.bars + 2 * kStreamStages * 8 + 8;         // [chunks][8*mb] fp32: -136 * sum of x over the chunk
    p.xs = (p.sx + chunks * 8 * mb * 4 + 127) & ~127;
    p.total = p.xs + p.x_rows * p.x_stride;
    return p;
}

// Persistent CTAs; each owns a contiguous range of 16-row strips.  A strip is one
// linear byte range of the packed matrix; the producer warp streams it in
// segments of 16 chunks (16.5 KiB) through a ring of bulk copies.  The consumer
// warps split each segment along K (two chunks or one each), expand int4 -> bf16 in
// registers and feed m16n8k16 MMAs whose N dimension is the (padded) batch; at
// the end of a strip their partial sums meet in shared memory.  No global
// scratch, no atomics: the summation order is fixed.
template <int MB, bool kBiased, int kStreamWarps>
__global__ void __launch_bounds__((kStreamWarps + 1) * 32) w4a16_stream_kernel(const StreamParams p)
{
    constexpr int kStreamStages = stream_stages(kStreamWarps);
    constexpr int kSegChunks = seg_chunks(kStreamWarps);
    constexpr int kSegBytes = seg_bytes(kStreamWarps);
    extern __shared__ __align__(128) uint8_t smem[];
    const StreamSmem plan = stream_smem_plan(kStreamWarps, MB, p.m, p.k, p.chunks);
    uint8_t* ring = smem + plan.ring;
    float* red = reinterpret_cast<float*>(smem + plan.red);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + plan.bars);
    uint64_t* empty = full + kStreamStages;
    uint64_t* xbar = empty + kStreamStages;   // completion of the batch-row copies
    float* sx = reinterpret_cast<float*>(smem + plan.sx);
    uint8_t* xs = smem + plan.xs;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s0 = int((long long)blockIdx.x * p.strips / gridDim.x);
    const int s1 = int((long long)(blockIdx.x + 1) * p.strips / gridDim.x);
    const int nseg = (p.chunks + kSegChunks - 1) / kSegChunks;
    const int items = (s1 - s0) * nseg;
    const size_t strip_bytes = size_t(p.chunks) * kInt4ChunkBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStreamStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kStreamWarps);
        }
        mbar_init(xbar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kStreamWarps) {
        // ---- producer: weights are constants, so streaming starts before the
        // previous kernel in the stream has finished.
        if (lane == 0) {
            for (int i = 0; i < items; ++i) {
                const int s = i % kStreamStages;
                if (i >= kStreamStages && !mbar_wait(&empty[s], ((i / kStreamStages) - 1) & 1)) {
                    atomicExch(p.fault, 1);
                    break;
                }
                const int strip = s0 + i / nseg, seg = i % nseg;
                const int nch = min(kSegChunks, p.chunks - seg * kSegChunks);
                const uint32_t bytes = uint32_t(nch) * kInt4ChunkBytes;
                mbar_expect_tx(&full[s], bytes);
                int local;
                const int g = stream_matrix_of(p, strip, local);
                bulk_g2s(ring + size_t(s) * kSegBytes,
                         p.packed[g] + size_t(local) * strip_bytes + size_t(seg) * kSegBytes, bytes, &full[s]);
            }
        }
        return;
    }

    // ---- consumers
    pdl_wait();   // x is produced by the previous kernel; y may still be read by it
    bool ok = true;
    {
        // Stage the batch rows (bf16) with one bulk copy per row - a single round trip
        // to L2 however long the rows are - and then, per (row, chunk), -136 * the sum of
        // the row's 128 values (the bias term of the int4 expansion).  16 consecutive
        // threads cover one chunk of one row.
        const int rows = plan.x_rows - 1;
        const int vec_per_row = p.k / 8;
        const int total = rows * vec_per_row;
        if (threadIdx.x == 0) {
            mbar_expect_tx(xbar, uint32_t(rows) * uint32_t(p.k) * 2u);
            for (int m = 0; m < rows; ++m)
                bulk_g2s(xs + size_t(m) * plan.x_stride, p.x + size_t(m) * p.k, uint32_t(p.k) * 2u, xbar);
        }
        for (int i = threadIdx.x; i < vec_per_row; i += kStreamWarps * 32)
            *reinterpret_cast<uint4*>(xs + size_t(rows) * plan.x_stride + i * 16) = make_uint4(0, 0, 0, 0);
        if (kBiased)
            for (int i = threadIdx.x; i < p.chunks * 8 * MB; i += kStreamWarps * 32)
                if ((i % (8 * MB)) >= rows) sx[i] = 0.f;
        if (!mbar_wait(xbar, 0)) {
            atomicExch(p.fault, 3);
            ok = false;
        }
        if (kBiased) {
            for (int i0 = 0; i0 < total; i0 += kStreamWarps * 32) {
                const int i = i0 + threadIdx.x;
                const int m = i / vec_per_row, v = i % vec_per_row;
                uint4 val = make_uint4(0, 0, 0, 0);
                if (i < total) val = *reinterpret_cast<const uint4*>(xs + size_t(m) * plan.x_stride + v * 16);
                float part = 0.f;
                const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    part += __uint_as_float(w4[q] << 16) + __uint_as_float(w4[q] & 0xffff0000u);
#pragma unroll
                for (int off = 8; off; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
                if ((lane & 15) == 0 && i < total) sx[(v >> 4) * (8 * MB) + m] = -136.f * part;
            }
        }
    }
    named_barrier_sync(1, kStreamWarps * 32);

    const int g = lane >> 2, t = lane & 3;
    // Per-lane x row pointers: batch row g (and 8+g), or the zero row.
    const uint8_t* xrow[MB];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        const int r = mb * 8 + g;
        xrow[mb] = xs + size_t(r < p.m ? r : plan.x_rows - 1) * plan.x_stride + t * 16;
    }
    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mb][i] = 0.f;
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};

    int s = 0, phase = 0, strip = s0, seg = 0;
    for (int i = 0; i < items; ++i) {
        if (ok && !mbar_wait(&full[s], phase)) {
            atomicExch(p.fault, 2);
            ok = false;
        }
        const int nch = min(kSegChunks, p.chunks - seg * kSegChunks);
        if (ok) {
#pragma unroll
            for (int cc = 0; cc < chunks_per_warp(kStreamWarps); ++cc) {
                const int c = chunks_per_warp(kStreamWarps) * warp + cc;
                if (c >= nch) break;
                const uint8_t* st = ring + s * kSegBytes + c * kInt4ChunkBytes;
                const uint32_t sc = *reinterpret_cast<const uint32_t*>(st + 1024 + g * 4);
                const int chunk = seg * kSegChunks + c;
                const uint4 u0 = *reinterpret_cast<const uint4*>(st + lane * 16);
                const uint4 u1 = *reinterpret_cast<const uint4*>(st + 512 + lane * 16);
                float tmp[MB][4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {   // q = 2*tile + half: octets t, t+4 of tile 0, then of tile 1
                    const uint32_t wlo = q == 0 ? u0.x : q == 1 ? u0.z : q == 2 ? u1.x : u1.z;
                    const uint32_t whi = q == 0 ? u0.y : q == 1 ? u0.w : q == 2 ? u1.y : u1.w;
                    const uint32_t a0[4] = {int4x2_expand<kBiased>(wlo), int4x2_expand<kBiased>(whi),
                                            int4x2_expand<kBiased>(wlo >> 4), int4x2_expand<kBiased>(whi >> 4)};
                    const uint32_t a1[4] = {int4x2_expand<kBiased>(wlo >> 8), int4x2_expand<kBiased>(whi >> 8),
                                            int4x2_expand<kBiased>(wlo >> 12), int4x2_expand<kBiased>(whi >> 12)};
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) {
                        const uint4 xb = *reinterpret_cast<const uint4*>(xrow[mb] + chunk * 256 + q * 64);
                        if (q == 0)
                            mma_bf16_16816(tmp[mb], a0, xb.x, xb.y, zero4);
                        else
                            mma_bf16_16816(tmp[mb], a0, xb.x, xb.y, tmp[mb]);
                        mma_bf16_16816(tmp[mb], a1, xb.z, xb.w, tmp[mb]);
                    }
                }

                const float s_lo = scale16_to_float(sc & 0xffffu, p.scale_dtype);
                const float s_hi = scale16_to_float(sc >> 16, p.scale_dtype);
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    if (kBiased) {
                        const float2 b = *reinterpret_cast<const float2*>(sx + chunk * (8 * MB) + mb * 8 + 2 * t);
                        tmp[mb][0] += b.x;
                        tmp[mb][1] += b.y;
                        tmp[mb][2] += b.x;
                        tmp[mb][3] += b.y;
                    }
                    acc[mb][0] = fmaf(tmp[mb][0], s_lo, acc[mb][0]);
                    acc[mb][1] = fmaf(tmp[mb][1], s_lo, acc[mb][1]);
                    acc[mb][2] = fmaf(tmp[mb][2], s_hi, acc[mb][2]);
                    acc[mb][3] = fmaf(tmp[mb][3], s_hi, acc[mb][3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        if (++s == kStreamStages) {
            s = 0;
            phase ^= 1;
        }
        if (++seg != nseg) continue;
        seg = 0;

        // ---- end of a strip: the warps' partial sums meet in shared memory (all
        // threads take part: leaving the sum to the few threads that batch 1 needs made
        // their warp the straggler and was measured slower).
        // acc[mb][0..1]: row R(g), batch columns 2t, 2t+1; [2..3]: row R(g)+8.
        float* slot = red + ((strip - s0) & 1) * (kStreamWarps * MB * 128);
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                slot[(warp * MB * 4 + mb * 4 + q) * 32 + lane] = acc[mb][q];
                acc[mb][q] = 0.f;
            }
        named_barrier_sync(1, kStreamWarps * 32);
        int local;
        const int grp = stream_matrix_of(p, strip, local);
        for (int idx = threadIdx.x; idx < MB * 128; idx += kStreamWarps * 32) {   // 128 outputs per 8 batch columns
            const int l = idx & 31, q = (idx >> 5) & 3, mb = idx >> 7;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kStreamWarps; ++w) v += slot[(w * MB * 4 + mb * 4 + q) * 32 + l];
            const int m = mb * 8 + 2 * (l & 3) + (q & 1);
            const int n = local * 16 + row_of_g(l >> 2) + 8 * (q >> 1);
            if (m < p.m && n < p.n[grp]) p.y[grp][size_t(m) * p.ldy[grp] + n] = __float2bfloat16_rn(v);
        }
        ++strip;
    }
    if (!ok) {
        // A wait gave up: give the copies still in flight a bounded chance to land
        // before this CTA's shared memory is released.
        for (int i = 0; i < min(items, kStreamStages); ++i) (void)mbar_wait(&full[i], 0);
    }
}

// ------------------------------------------------------------------ handle

constexpr size_t kMaxDynamicSmem = 227 * 1024;

static bool use_biased_expansion()
{
    // GARNET_B200_W4_EXACT_EXPAND=1 selects the variant that subtracts the int4
    // bias per element instead of once per chunk (A/B switch, read once).
    static const bool biased = [] {
        const char* e = getenv("GARNET_B200_W4_EXACT_EXPAND");
        return !(e && e[0] == '1');
    }();
    return biased;
}

template <int MB, bool B, int W>
static cudaError_t set_stream_attr()
{
    return cudaFuncSetAttribute(w4a16_stream_kernel<MB, B, W>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                int(kMaxDynamicSmem));
}

int W4A16::init_common()
{
    GB_CUDA(cudaGetDevice(&device));
    GB_CUDA(cudaHostAlloc(&fault_host, sizeof(int), cudaHostAllocMapped));
    *fault_host = 0;
    GB_CUDA(cudaHostGetDevicePointer(&fault_dev, fault_host, 0));
    if (size_t(stream_smem_plan(8, 1, 8, geo.cols, geo.chunks).total) > kMaxDynamicSmem)
        return fail(GARNET_B200_NOT_SUPPORTED, "w4a16: k=%d is too large for the streaming kernel", geo.cols);
    max_rows_per_launch = size_t(stream_smem_plan(8, 2, 16, geo.cols, geo.chunks).total) <= kMaxDynamicSmem ? 16 : 8;
    // The attribute is per kernel and per device, not per handle: always ask for the maximum.
    GB_CUDA((set_stream_attr<1, true, 16>()));
    GB_CUDA((set_stream_attr<2, true, 16>()));
    GB_CUDA((set_stream_attr<1, false, 16>()));
    GB_CUDA((set_stream_attr<2, false, 16>()));
    GB_CUDA((set_stream_attr<1, true, 8>()));
    GB_CUDA((set_stream_attr<2, true, 8>()));
    GB_CUDA((set_stream_attr<1, false, 8>()));
    GB_CUDA((set_stream_attr<2, false, 8>()));
    return init_tc();
}

static bool use_tensor_core_tiles()
{
    // GARNET_B200_W4_NO_TC=1 keeps every batch size on the streaming kernel (A/B switch).
    static const bool on = [] {
        const char* e = getenv("GARNET_B200_W4_NO_TC");
        return !(e && e[0] == '1');
    }();
    return on;
}

W4A16::~W4A16()
{
    if (owns_packed && packed) cudaFree(packed);
    if (fault_host) cudaFreeHost(fault_host);
    if (stage_x) cudaFree(stage_x);
    if (stage_y) cudaFree(stage_y);
    if (stage_ws) cudaFree(stage_ws);
}

size_t W4A16::workspace_bytes(int) const { return 0; }

int W4A16::launch_stream(const __nv_bfloat16* x, __nv_bfloat16* y, int m, int ldy, unsigned flags,
                         cudaStream_t stream)
{
    W4A16* one[1] = {this};
    __nv_bfloat16* ys[1] = {y};
    const int ldys[1] = {ldy};
    return launch_stream_group(one, 1, x, ys, ldys, m, flags, stream);
}

// One launch for up to kMaxGroup linears that read the same x (same K, same scale
// type): their strips are concatenated, so the small projections of a decoder layer
// share one kernel's launch latency.
int W4A16::launch_stream_group(W4A16* const* hs, int count, const __nv_bfloat16* x, __nv_bfloat16* const* ys,
                               const int* ldys, int m, unsigned flags, cudaStream_t stream)
{
    const PackGeom& geo0 = hs[0]->geo;
    StreamParams p;
    int total = 0;
    for (int g = 0; g < kMaxGroup; ++g) {
        const int src = g < count ? g : 0;
        p.packed[g] = hs[src]->packed;
        p.y[g] = ys[src];
        p.n[g] = hs[src]->geo.rows;
        p.ldy[g] = ldys[src];
        if (g < count) total += hs[g]->geo.strips;
        p.strip_end[g] = total;
    }
    p.group = count;
    p.x = x;
    p.fault = hs[0]->fault_dev;
    p.m = m;
    p.k = geo0.cols;
    p.strips = total;
    p.chunks = geo0.chunks;
    p.scale_dtype = hs[0]->scale_dtype;
    struct { int strips, cols, chunks; } geo = {total, geo0.cols, geo0.chunks};

    const int mb = m <= 8 ? 1 : 2;
    // Few strips per SM: 16 consumer warps per CTA so that more warps share each strip.
    const bool wide = geo.strips <= kWideMaxStripsPerSm * kSmCount &&
                      size_t(stream_smem_plan(16, mb, m, geo.cols, geo.chunks).total) <= kMaxDynamicSmem;
    const int warps = wide ? 16 : 8;
    const size_t smem = size_t(stream_smem_plan(warps, mb, m, geo.cols, geo.chunks).total);
    if (smem > kMaxDynamicSmem)
        return fail(GARNET_B200_NOT_SUPPORTED, "w4a16: batch %d with k=%d does not fit shared memory", m, geo.cols);
    const int ctas_per_sm = std::max(1, std::min(kStreamCtasPerSm, int(kMaxDynamicSmem / (smem + 1024))));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(std::min(geo.strips, kSmCount * ctas_per_sm)));
    cfg.blockDim = dim3((warps + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    if (wide) {
        cfg.dynamicSmemBytes = std::max(smem, kWideSmemFloor);
        cfg.gridDim = dim3(unsigned(std::min(geo.strips, kSmCount)));
    }
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & 1u) ? 1 : 0;
    const bool biased = use_biased_expansion();
#define GB_LAUNCH_STREAM(MB_, B_, W_) GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_stream_kernel<MB_, B_, W_>, p))
    if (warps == 16) {
        if (mb == 1 && biased) GB_LAUNCH_STREAM(1, true, 16);
        else if (mb == 1) GB_LAUNCH_STREAM(1, false, 16);
        else if (biased) GB_LAUNCH_STREAM(2, true, 16);
        else GB_LAUNCH_STREAM(2, false, 16);
    } else {
        if (mb == 1 && biased) GB_LAUNCH_STREAM(1, true, 8);
        else if (mb == 1) GB_LAUNCH_STREAM(1, false, 8);
        else if (biased) GB_LAUNCH_STREAM(2, true, 8);
        else GB_LAUNCH_STREAM(2, false, 8);
    }
#undef GB_LAUNCH_STREAM
    return GARNET_B200_OK;
}

int W4A16::run(const void* d_x, void* d_y, int m, void* ws, size_t ws_bytes, unsigned flags, cudaStream_t stream)
{
    if (m <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: m must be positive (got %d)", m);
    if (!d_x || !d_y) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: null x or y");
    if ((reinterpret_cast<uintptr_t>(d_x) & 15) || (reinterpret_cast<uintptr_t>(d_y) & 1))
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: x must be 16-byte aligned");
    if (ws_bytes < workspace_bytes(m) || (workspace_bytes(m) && !ws))
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: workspace too small (%zu < %zu)", ws_bytes,
                    workspace_bytes(m));
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(d_x);
    __nv_bfloat16* y = static_cast<__nv_bfloat16*>(d_y);
    // Above 16 rows the weights are worth expanding once per 128 rows for the tensor core.
    if (m > 16 && use_tensor_core_tiles()) return launch_tc(x, y, m, flags, stream);
    for (int m0 = 0; m0 < m; m0 += max_rows_per_launch) {
        const int rows = std::min(max_rows_per_launch, m - m0);
        const int rc = launch_stream(x + size_t(m0) * geo.cols, y + size_t(m0) * geo.rows, rows, geo.rows, flags,
                                     stream);
        if (rc) return rc;
    }
    return GARNET_B200_OK;
}

static int validate_shape(int n, int k, int group)
{
    if (n <= 0 || k <= 0 || group <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16: n, k, group must be positive");
    if (k % group) return fail(GARNET_B200_INVALID_VALUE, "w4a16: k (%d) is not a multiple of group (%d)", k, group);
    if (group % 128)
        return fail(GARNET_B200_NOT_SUPPORTED, "w4a16: group %d is not a multiple of 128", group);
    return GARNET_B200_OK;
}

int w4a16_repack_device(const uint8_t* d_nibbles, const uint16_t* d_scales, const PackGeom& geo, long long row0,
                        uint8_t* d_packed, cudaStream_t stream)
{
    const size_t words = size_t(geo.strips_padded) * geo.chunks * (geo.chunk_data / 4);
    w4_repack_codes_kernel<<<unsigned((words + 255) / 256), 256, 0, stream>>>(d_nibbles, d_packed, geo, row0);
    const size_t sc = size_t(geo.strips_padded) * 16 * geo.chunks;
    w4_repack_scales_int4_kernel<<<unsigned((sc + 255) / 256), 256, 0, stream>>>(d_scales, d_packed, geo, row0);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

// ---------------------------------------------------------- host-buffer batches

struct ScatterEntry {
    const uint8_t* src;   // device staging of one linear's output
    uint8_t* dst;         // device alias of the caller's pinned host buffer
    size_t bytes;
};

// Copies every entry's output to its host buffer: one launch at the end of a batch
// instead of one copy (or one flush of host-memory writes) per linear.
__global__ void w4_scatter_outputs_kernel(const ScatterEntry* __restrict__ table, int count)
{
    pdl_wait();
    for (int e = blockIdx.y; e < count; e += gridDim.y) {
        const ScatterEntry t = table[e];
        const size_t start = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 16, step = size_t(gridDim.x) * blockDim.x * 16;
        if (((reinterpret_cast<uintptr_t>(t.src) | reinterpret_cast<uintptr_t>(t.dst)) & 15) == 0) {
            for (size_t o = start; o + 16 <= t.bytes; o += step)
                *reinterpret_cast<uint4*>(t.dst + o) = *reinterpret_cast<const uint4*>(t.src + o);
            if (blockIdx.x == 0 && threadIdx.x < (t.bytes & 15)) t.dst[(t.bytes & ~size_t(15)) + threadIdx.x] = t.src[(t.bytes & ~size_t(15)) + threadIdx.x];
        } else {
            for (size_t o = start / 16; o < t.bytes; o += step / 16) t.dst[o] = t.src[o];
        }
    }
}

struct HostBatch {
    struct Call {
        W4A16* h;
        const void* h_x;
        void* h_y;
        int m;
        int x_slot;          // index into xs
        size_t y_off;        // offset of this call's output in y_stage
        void* y_alias;       // device alias of h_y, or nullptr (pageable: copied with cudaMemcpyAsync)
    };
    struct X {
        const void* host;
        size_t bytes, off;
    };
    std::vector<Call> calls;
    std::vector<X> xs;
    uint8_t* x_stage = nullptr;
    uint8_t* y_stage = nullptr;
    ScatterEntry* table = nullptr;
    int table_count = 0;
    ~HostBatch()
    {
        if (x_stage) cudaFree(x_stage);
        if (y_stage) cudaFree(y_stage);
        if (table) cudaFree(table);
    }
};

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_int4_quantize(const void* d_src, int src_dtype, int64_t rows, int64_t cols, int group,
                              int scale_dtype, uint8_t* d_nibbles, uint16_t* d_scales, void* stream)
{
    if (!d_src || !d_nibbles || !d_scales) return fail(GARNET_B200_INVALID_VALUE, "int4_quantize: null pointer");
    if (rows <= 0 || cols <= 0 || group <= 0 || cols % group || (group & 1))
        return fail(GARNET_B200_INVALID_VALUE, "int4_quantize: bad shape rows=%lld cols=%lld group=%d",
                    (long long)rows, (long long)cols, group);
    if (scale_dtype != GARNET_B200_FP16 && scale_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "int4_quantize: scale dtype must be fp16 or bf16");
    const long long warps = rows * (cols / group);
    const unsigned blocks = unsigned((warps * 32 + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (src_dtype) {
        case GARNET_B200_FP32:
            int4_quantize_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(d_src), rows, cols, group,
                                                              scale_dtype, d_nibbles, d_scales);
            break;
        case GARNET_B200_BF16:
            int4_quantize_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(d_src),
                                                                      rows, cols, group, scale_dtype, d_nibbles,
                                                                      d_scales);
            break;
        case GARNET_B200_FP16:
            int4_quantize_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(d_src), rows, cols,
                                                               group, scale_dtype, d_nibbles, d_scales);
            break;
        default:
            return fail(GARNET_B200_INVALID_VALUE, "int4_quantize: unknown source dtype %d", src_dtype);
    }
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_packed_bytes(int n, int k, int group, size_t* bytes)
{
    if (!bytes) return fail(GARNET_B200_INVALID_VALUE, "w4a16_packed_bytes: null output");
    if (int rc = validate_shape(n, k, group)) return rc;
    *bytes = make_geom(kFormatInt4, n, k, group).matrix_bytes();
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_pack_host(const uint8_t* nibbles, const uint16_t* scales, int scale_dtype, int n, int k,
                                int group, uint8_t* packed)
{
    if (!nibbles || !scales || !packed) return fail(GARNET_B200_INVALID_VALUE, "w4a16_pack_host: null pointer");
    if (int rc = validate_shape(n, k, group)) return rc;
    if (scale_dtype != GARNET_B200_FP16 && scale_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_pack_host: scale dtype must be fp16 or bf16");
    const PackGeom geo = make_geom(kFormatInt4, n, k, group);
    std::memset(packed, 0, geo.matrix_bytes());
    const int groups = k / group;
    for (int row = 0; row < n; ++row) {
        for (int col = 0; col < k; col += 8) {
            uint32_t in;
            std::memcpy(&in, nibbles + (size_t(row) * k + col) / 2, 4);
            uint32_t out = 0;
            for (int e = 0; e < 8; ++e) out |= ((in >> (4 * e)) & 15u) << (4 * ((e >> 1) + 4 * (e & 1)));
            std::memcpy(packed + locate(geo, row, col).word_byte, &out, 4);
        }
        for (int chunk = 0; chunk < geo.chunks; ++chunk) {
            const uint16_t s = scales[size_t(row) * groups + (chunk * 128) / group];
            std::memcpy(packed + locate_scale(geo, row, chunk * 128), &s, 2);
        }
    }
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_create(const uint8_t* d_nibbles, const void* d_scales, int scale_dtype, int n, int k,
                             int group, int shard_rank, int shard_world, void* stream,
                             garnet_b200_w4a16_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: null output handle");
    *out = nullptr;
    if (!d_nibbles || !d_scales) return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: null weight pointer");
    if (int rc = validate_shape(n, k, group)) return rc;
    if (scale_dtype != GARNET_B200_FP16 && scale_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: scale dtype must be fp16 or bf16");
    if (shard_world < 1) shard_world = 1;
    if (shard_rank < 0 || shard_rank >= shard_world || n % shard_world)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: bad shard %d of %d for n=%d", shard_rank, shard_world, n);
    const int n_local = n / shard_world;
    W4A16* h = new (std::nothrow) W4A16();
    if (!h) return fail(GARNET_B200_OUT_OF_MEMORY, "w4a16_create: host allocation failed");
    h->geo = make_geom(kFormatInt4, n_local, k, group);
    h->scale_dtype = scale_dtype;
    h->owns_packed = true;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = GARNET_B200_OK;
    do {
        if (cudaMalloc(&h->packed, h->geo.matrix_bytes()) != cudaSuccess) {
            rc = fail(GARNET_B200_OUT_OF_MEMORY, "w4a16_create: cudaMalloc of %zu bytes failed", h->geo.matrix_bytes());
            cudaGetLastError();
            break;
        }
        if ((rc = w4a16_repack_device(d_nibbles, static_cast<const uint16_t*>(d_scales), h->geo,
                                      (long long)shard_rank * n_local, h->packed, s)))
            break;
        if ((rc = h->init_common())) break;
        if (cudaStreamSynchronize(s) != cudaSuccess) {
            rc = cuda_fail(cudaGetLastError(), "w4a16_create: synchronize");
            break;
        }
    } while (false);
    if (rc) {
        delete h;
        return rc;
    }
    *out = reinterpret_cast<garnet_b200_w4a16_t>(h);
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_create_prepacked(const uint8_t* d_packed, int scale_dtype, int n, int k, int group,
                                       garnet_b200_w4a16_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "w4a16_create_prepacked: null output handle");
    *out = nullptr;
    if (!d_packed || (reinterpret_cast<uintptr_t>(d_packed) & 127))
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_create_prepacked: packed pointer must be 128-byte aligned");
    if (int rc = validate_shape(n, k, group)) return rc;
    W4A16* h = new (std::nothrow) W4A16();
    if (!h) return fail(GARNET_B200_OUT_OF_MEMORY, "w4a16_create_prepacked: host allocation failed");
    h->geo = make_geom(kFormatInt4, n, k, group);
    h->packed = const_cast<uint8_t*>(d_packed);
    h->scale_dtype = scale_dtype;
    h->owns_packed = false;
    if (int rc = h->init_common()) {
        delete h;
        return rc;
    }
    *out = reinterpret_cast<garnet_b200_w4a16_t>(h);
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_shape(garnet_b200_w4a16_t hh, int* n_local, int* k)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "w4a16_shape: null handle");
    if (n_local) *n_local = h->geo.rows;
    if (k) *k = h->geo.cols;
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_workspace(garnet_b200_w4a16_t hh, int m, size_t* bytes)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h || !bytes || m <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16_workspace: bad argument");
    *bytes = h->workspace_bytes(m);
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_run(garnet_b200_w4a16_t hh, const void* d_x, void* d_y, int m, void* d_workspace,
                          size_t workspace_bytes, unsigned flags, void* stream)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: null handle");
    return h->run(d_x, d_y, m, d_workspace, workspace_bytes, flags, static_cast<cudaStream_t>(stream));
}

int garnet_b200_w4a16_run_group(const garnet_b200_w4a16_t* handles, int count, const void* d_x, void* const* d_ys,
                                int m, unsigned flags, void* stream)
{
    if (!handles || !d_ys || !d_x || count <= 0 || m <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: bad argument");
    if (count > kMaxGroup) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: at most %d linears per group", kMaxGroup);
    if (reinterpret_cast<uintptr_t>(d_x) & 15) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: x must be 16-byte aligned");
    W4A16* hs[kMaxGroup];
    __nv_bfloat16* ys[kMaxGroup];
    int ldys[kMaxGroup];
    int max_rows = 16;
    for (int g = 0; g < count; ++g) {
        hs[g] = reinterpret_cast<W4A16*>(handles[g]);
        ys[g] = static_cast<__nv_bfloat16*>(d_ys[g]);
        if (!hs[g] || !ys[g]) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: null handle or output %d", g);
        if (hs[g]->geo.cols != hs[0]->geo.cols || hs[g]->scale_dtype != hs[0]->scale_dtype)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: linears of a group must share K and the scale type");
        ldys[g] = hs[g]->geo.rows;
        max_rows = std::min(max_rows, hs[g]->max_rows_per_launch);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (m > max_rows) {   // larger batches: one launch per linear (tile kernel or row blocks)
        for (int g = 0; g < count; ++g)
            if (int rc = hs[g]->run(d_x, ys[g], m, nullptr, 0, flags, s)) return rc;
        return GARNET_B200_OK;
    }
    return W4A16::launch_stream_group(hs, count, static_cast<const __nv_bfloat16*>(d_x), ys, ldys, m, flags, s);
}

// Device-visible alias of a host pointer (pinned and mapped memory), or nullptr.
static void* device_alias_of(const void* host_ptr)
{
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host_ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

// One linear with host buffers, enqueued on `s`.  `d_x_shared`: a device copy of h_x made
// by an earlier call of the same batch (then no copy is enqueued), or nullptr.
static int run_host_one(W4A16* h, const void* h_x, const void* d_x_shared, void* h_y, int m, cudaStream_t s)
{
    const size_t xb = size_t(m) * h->geo.cols * 2, yb = size_t(m) * h->geo.rows * 2, wb = h->workspace_bytes(m);
    if (m > h->stage_rows) {
        if (h->stage_x) cudaFree(h->stage_x);
        if (h->stage_y) cudaFree(h->stage_y);
        if (h->stage_ws) cudaFree(h->stage_ws);
        h->stage_x = h->stage_y = h->stage_ws = nullptr;
        h->stage_rows = 0;
        GB_CUDA(cudaMalloc(&h->stage_x, xb));
        GB_CUDA(cudaMalloc(&h->stage_y, yb));
        if (wb) GB_CUDA(cudaMalloc(&h->stage_ws, wb));
        h->stage_rows = m;
    }
    // y in pinned, mapped host memory is written by the kernel itself (one posted write per
    // output over the host link, no copy to enqueue); any other y goes through a staged copy.
    if (h_y != h->last_host_y) {
        h->last_host_y = h_y;
        h->last_host_y_alias = device_alias_of(h_y);
    }
    if (!d_x_shared) GB_CUDA(cudaMemcpyAsync(h->stage_x, h_x, xb, cudaMemcpyHostToDevice, s));
    void* y_dev = h->last_host_y_alias ? h->last_host_y_alias : h->stage_y;
    if (int rc = h->run(d_x_shared ? d_x_shared : h->stage_x, y_dev, m, h->stage_ws, wb, 0, s)) return rc;
    if (!h->last_host_y_alias) GB_CUDA(cudaMemcpyAsync(h_y, h->stage_y, yb, cudaMemcpyDeviceToHost, s));
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_run_host_async(garnet_b200_w4a16_t hh, const void* h_x, void* h_y, int m, void* stream)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h || !h_x || !h_y || m <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_host: bad argument");
    return run_host_one(h, h_x, nullptr, h_y, m, static_cast<cudaStream_t>(stream));
}

int garnet_b200_w4a16_batch_create(const garnet_b200_w4a16_t* handles, const void* const* h_xs, void* const* h_ys,
                                   const int* ms, int count, garnet_b200_w4a16_batch_t* out)
{
    if (!handles || !h_xs || !h_ys || !ms || !out || count <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_batch_create: bad argument");
    std::unique_ptr<HostBatch> b(new HostBatch);
    size_t x_total = 0, y_total = 0;
    for (int i = 0; i < count; ++i) {
        W4A16* h = reinterpret_cast<W4A16*>(handles[i]);
        if (!h || !h_xs[i] || !h_ys[i] || ms[i] <= 0)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_batch_create: bad argument at index %d", i);
        if (h->workspace_bytes(ms[i])) return fail(GARNET_B200_NOT_SUPPORTED, "w4a16_batch_create: linear needs a workspace");
        const size_t xb = size_t(ms[i]) * h->geo.cols * 2, yb = size_t(ms[i]) * h->geo.rows * 2;
        // inputs are read-only during a run: every distinct host buffer is copied once
        int slot = -1;
        for (size_t q = 0; q < b->xs.size(); ++q)
            if (b->xs[q].host == h_xs[i] && b->xs[q].bytes == xb) slot = int(q);
        if (slot < 0) {
            slot = int(b->xs.size());
            b->xs.push_back({h_xs[i], xb, x_total});
            x_total += (xb + 255) & ~size_t(255);
        }
        b->calls.push_back({h, h_xs[i], h_ys[i], ms[i], slot, y_total, device_alias_of(h_ys[i])});
        y_total += (yb + 255) & ~size_t(255);
    }
    GB_CUDA(cudaMalloc(&b->x_stage, x_total));
    GB_CUDA(cudaMalloc(&b->y_stage, y_total));
    std::vector<ScatterEntry> table;
    for (const HostBatch::Call& c : b->calls)
        if (c.y_alias)
            table.push_back({b->y_stage + c.y_off, static_cast<uint8_t*>(c.y_alias), size_t(c.m) * c.h->geo.rows * 2});
    b->table_count = int(table.size());
    if (b->table_count) {
        GB_CUDA(cudaMalloc(&b->table, table.size() * sizeof(ScatterEntry)));
        GB_CUDA(cudaMemcpy(b->table, table.data(), table.size() * sizeof(ScatterEntry), cudaMemcpyHostToDevice));
    }
    *out = reinterpret_cast<garnet_b200_w4a16_batch_t>(b.release());
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_batch_run(garnet_b200_w4a16_batch_t bb, void* stream)
{
    HostBatch* b = reinterpret_cast<HostBatch*>(bb);
    if (!b) return fail(GARNET_B200_INVALID_VALUE, "w4a16_batch_run: null batch");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (const HostBatch::X& x : b->xs)
        GB_CUDA(cudaMemcpyAsync(b->x_stage + x.off, x.host, x.bytes, cudaMemcpyHostToDevice, s));
    for (const HostBatch::Call& c : b->calls)
        if (int rc = c.h->run(b->x_stage + b->xs[c.x_slot].off, b->y_stage + c.y_off, c.m, nullptr, 0, 1, s)) return rc;
    if (b->table_count) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(8, unsigned(std::min(b->table_count, 1024)));
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        GB_CUDA(cudaLaunchKernelEx(&cfg, w4_scatter_outputs_kernel, (const ScatterEntry*)b->table, b->table_count));
    }
    for (const HostBatch::Call& c : b->calls)
        if (!c.y_alias)
            GB_CUDA(cudaMemcpyAsync(c.h_y, b->y_stage + c.y_off, size_t(c.m) * c.h->geo.rows * 2, cudaMemcpyDeviceToHost, s));
    return GARNET_B200_OK;
}

void garnet_b200_w4a16_batch_destroy(garnet_b200_w4a16_batch_t bb) { delete reinterpret_cast<HostBatch*>(bb); }

int garnet_b200_w4a16_run_host(garnet_b200_w4a16_t hh, const void* h_x, void* h_y, int m, void* stream)
{
    if (int rc = garnet_b200_w4a16_run_host_async(hh, h_x, h_y, m, stream)) return rc;
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    GB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    if (*h->fault_host) return fail(GARNET_B200_DEVICE_FAULT, "w4a16: device wait gave up (code %d)", *h->fault_host);
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_dequant(garnet_b200_w4a16_t hh, float* d_out, void* stream)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h || !d_out) return fail(GARNET_B200_INVALID_VALUE, "w4a16_dequant: bad argument");
    const size_t total = size_t(h->geo.rows) * h->geo.cols / 2;
    w4_dequant_kernel<<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        h->packed, d_out, h->geo, h->scale_dtype);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_fault(garnet_b200_w4a16_t hh)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    return h && h->fault_host ? *h->fault_host : -1;
}

void garnet_b200_w4a16_destroy(garnet_b200_w4a16_t hh) { delete reinterpret_cast<W4A16*>(hh); }

}  // extern "C"
