// gpt-oss MXFP4 mixture-of-experts operator (`gpt_oss_moe_mxfp4`) for sm_100a:
// repackers, router, top-k, slot bucketing, the streaming expert kernel used for
// small per-expert batches, the weighted combine, and the C ABI around them.
//
// Numerics follow the reference operator step by step
// (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:537-587, :681-726, :762-811, :907-921):
//   logit = bf(x . Wr + br); k rounds of arg-max, ties to the lowest index;
//   p_j = bf(exp(l_j - l_0) / sum_i exp(l_i - l_0));
//   g = min(bf(bf(x . w_gate) + b), limit); u = clamp(bf(bf(x . w_up) + b), +-limit);
//   h = bf(bf(g * bf(sigmoid(bf(1.702 g)))) * bf(u + 1));
//   y = bf(sum_j bf(bf(h . w_down) + bd) * p_j)   (router order j).
// Dot products accumulate in fp32.  MXFP4 codes are expanded by the hardware
// conversion cvt.rn.f16x2.e2m1x2 (exact) and the e8m0 group scale multiplies the
// fp32 partial sum of each 32-column group (exact power of two), so no weight
// value is ever rounded.  Activations enter the tensor core as fp16 after an
// exact per-token power-of-two normalisation (bf16 inputs have 8 significant
// bits, fp16 carries 11).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

#include "common.cuh"
#include "layout.h"
#include "moe.h"
#include "moe_pack.h"

namespace gb200 {

constexpr int kMxChunkBytes = 512 + 32;

// ------------------------------------------------------------------ repack

// Timing build (-DGB_MOE_TRACE): CTA 7 of each small-batch launch records global-timer stamps (router: slots
// 0..15, gate/up: 16..47, down: 48..79, combine: 80..83), read back with garnet_b200_moe_trace.  Absent from the
// normal build.
#ifdef GB_MOE_TRACE
__device__ unsigned long long g_moe_trace[96];
#define GB_MTRACE(slot) do { if (blockIdx.x == 7) g_moe_trace[(slot)] = global_timer_ns(); } while (0)
#define GB_MTRACE_ANY(slot) do { g_moe_trace[(slot)] = global_timer_ns(); } while (0)
#else
#define GB_MTRACE(slot) do {} while (0)
#define GB_MTRACE_ANY(slot) do {} while (0)
#endif

// One thread per packed 32-bit word (moe_pack.h says where each comes from).
__global__ void mx_repack_codes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, PackGeom geo,
                                       int interleaved)
{
    const int expert = blockIdx.y;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= mx_stream_words(geo)) return;
    size_t db, sb;
    uint32_t out = 0;
    if (mx_stream_word(geo, idx, interleaved, &db, &sb))
        out = *reinterpret_cast<const uint32_t*>(src + size_t(expert) * geo.rows * size_t(geo.cols / 2) + sb);
    *reinterpret_cast<uint32_t*>(dst + size_t(expert) * geo.matrix_bytes() + db) = out;
}

// One thread per (packed row, 32-column group).  Padding gets scale 127 (1.0).
__global__ void mx_repack_scales_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, PackGeom geo,
                                        int interleaved)
{
    const int expert = blockIdx.y;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= mx_stream_scale_count(geo)) return;
    size_t db, sb;
    uint8_t e = 127;
    if (mx_stream_scale(geo, idx, interleaved, &db, &sb)) e = src[size_t(expert) * geo.rows * size_t(geo.cols / 32) + sb];
    dst[size_t(expert) * geo.matrix_bytes() + db] = e;
}

// Flags e8m0 bytes 0 (2^-127, an fp32 subnormal) and 255 (NaN), which need the
// careful scale decode.
__global__ void mx_scan_scales_kernel(const uint8_t* __restrict__ scales, size_t count, int* flag)
{
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx < count && (scales[idx] == 0 || scales[idx] == 255)) atomicOr(flag, 1);
}

// 2^(e-127) as fp32.  The plain form is a shift; the careful form also covers
// e = 0 (subnormal 2^-127) and e = 255 (NaN), gpt_oss_kernels.cu:55-56.
template <bool kCareful>
__device__ __forceinline__ float e8m0_to_float(uint32_t e)
{
    if (kCareful) {
        if (e == 0) return __uint_as_float(0x00400000u);
        if (e == 255) return __uint_as_float(0x7fc00000u);
    }
    return __uint_as_float(e << 23);
}

// ------------------------------------------------------------ decode checks

// rows x 32 columns, one scale per row: the shape of the reference's exhaustive
// decode test (TestGptOssMxfp4Decode, gpt_oss_kernels.cu:71-76).  Uses the same
// conversion instruction and scale decode as the expert kernels.
__global__ void mx_decode_rows_kernel(const uint8_t* __restrict__ blocks, const uint8_t* __restrict__ scales,
                                      float* __restrict__ out, int rows)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;   // one 32-bit word = eight codes
    if (idx >= rows * 4) return;
    const int row = idx >> 2;
    // The conversion is fed from a full 32-bit word, as in the expert kernels.
    const uint32_t w = reinterpret_cast<const uint32_t*>(blocks)[idx];
    const float s = e8m0_to_float<true>(scales[row]);
    const uint32_t pairs[4] = {e2m1x2_to_f16x2(w, 0), e2m1x2_to_f16x2(w, 1), e2m1x2_to_f16x2(w, 2),
                               e2m1x2_to_f16x2(w, 3)};
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const __half2 hv = *reinterpret_cast<const __half2*>(&pairs[b]);
        out[8 * idx + 2 * b] = __half2float(__low2half(hv)) * s;
        out[8 * idx + 2 * b + 1] = __half2float(__high2half(hv)) * s;
    }
}

// fp32 value of every logical element of one packed expert matrix (row order of
// the ORIGINAL matrix), decoded from the packed tiles.
__global__ void mx_dequant_kernel(const uint8_t* __restrict__ packed, float* __restrict__ out, PackGeom geo,
                                  int interleaved, int expert)
{
    const size_t total = size_t(geo.rows) * geo.cols / 2;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int src_row = int(idx / (geo.cols / 2)), k = int(idx % (geo.cols / 2)) * 2;
    int n = src_row;
    if (interleaved) {
        const int i = src_row >> 1, up = src_row & 1;
        n = (i >> 3) * 16 + (i & 7) + 8 * up;
    }
    const uint8_t* base = packed + size_t(expert) * geo.matrix_bytes();
    const PackPos p = locate(geo, n, k);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(base + p.word_byte);
    const uint32_t pair = e2m1x2_to_f16x2(w >> (8 * ((k & 7) >> 1)), 0);
    const float s = e8m0_to_float<true>(base[locate_scale(geo, n, k)]);
    const __half2 hv = *reinterpret_cast<const __half2*>(&pair);
    out[size_t(src_row) * geo.cols + k] = __half2float(__low2half(hv)) * s;
    out[size_t(src_row) * geo.cols + k + 1] = __half2float(__high2half(hv)) * s;
}

// ------------------------------------------------------------------ router

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

constexpr int kRouteTokens = 8;     // tokens per CTA
constexpr int kRouteWarps = 8;      // one expert per warp at a time

// logits[t,e] = bf(sum_d x[t,d] * W[e,d] + b[e]) with fp32 accumulation
// (gpt_oss_kernels.cu:537-587).  A CTA stages 8 tokens in shared memory; each warp
// walks experts, its lanes striding the hidden dimension.  The CTA of expert
// group 0 also writes, per token, the fp16 copy of x used by the expert kernels
// (x rounded to bf16, then scaled by an exact power of two so that the largest
// magnitude lands in [2^13, 2^14)), and that exponent.
template <typename XT>
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_scores_kernel(const XT* __restrict__ x, const float* __restrict__ rw, const float* __restrict__ rb,
                        float* __restrict__ logits, __half* __restrict__ xh, int* __restrict__ xshift, int tokens,
                        int hidden, int experts, int experts_per_cta)
{
    extern __shared__ float xs[];   // [kRouteTokens][hidden]
    __shared__ float s_amax[kRouteTokens];
    const int t0 = blockIdx.x * kRouteTokens;
    const int nt = min(kRouteTokens, tokens - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < kRouteTokens * hidden; i += blockDim.x) {
        const int t = i / hidden, d = i % hidden;
        xs[i] = t < nt ? to_float(x[size_t(t0 + t) * hidden + d]) : 0.f;
    }
    __syncthreads();
    const int e0 = blockIdx.y * experts_per_cta, e1 = min(experts, e0 + experts_per_cta);
    // A warp takes four experts at a time: every activation value read from shared
    // memory feeds four FMAs (one per expert), every weight value eight (one per token).
    constexpr int kEx = 4;
    for (int eb = e0 + warp * kEx; eb < e1; eb += kRouteWarps * kEx) {
        float acc[kEx][kRouteTokens];
#pragma unroll
        for (int q = 0; q < kEx; ++q)
#pragma unroll
            for (int t = 0; t < kRouteTokens; ++t) acc[q][t] = 0.f;
        const float* w[kEx];
#pragma unroll
        for (int q = 0; q < kEx; ++q) w[q] = rw + size_t(min(eb + q, e1 - 1)) * hidden;
        for (int d = lane; d < hidden; d += 32) {
            float wv[kEx];
#pragma unroll
            for (int q = 0; q < kEx; ++q) wv[q] = w[q][d];
#pragma unroll
            for (int t = 0; t < kRouteTokens; ++t) {
                const float xv = xs[t * hidden + d];
#pragma unroll
                for (int q = 0; q < kEx; ++q) acc[q][t] = fmaf(xv, wv[q], acc[q][t]);
            }
        }
#pragma unroll
        for (int q = 0; q < kEx; ++q) {
            const int e = eb + q;
            if (e >= e1) break;
            const float b = rb[e];
#pragma unroll
            for (int t = 0; t < kRouteTokens; ++t) {
                const float v = warp_sum(acc[q][t]);
                if (lane == 0 && t < nt) logits[size_t(t0 + t) * experts + e] = bf16_round_f(v + b);
            }
        }
    }
    if (blockIdx.y != 0 || !xh) return;
    // fp16 copy of x: one warp per token
    for (int t = warp; t < nt; t += kRouteWarps) {
        float amax = 0.f;
        for (int d = lane; d < hidden; d += 32) amax = fmaxf(amax, fabsf(bf16_round_f(xs[t * hidden + d])));
#pragma unroll
        for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        if (lane == 0) s_amax[t] = amax;
    }
    __syncthreads();
    for (int t = warp; t < nt; t += kRouteWarps) {
        const float amax = s_amax[t];
        int shift = 0;   // x = xh * 2^shift
        if (amax > 0.f && isfinite(amax)) shift = int((__float_as_uint(amax) >> 23) & 0xff) - 127 - 13;
        shift = max(-100, min(100, shift));
        const float scale = __uint_as_float(uint32_t(127 - shift) << 23);   // 2^-shift
        for (int d = lane; d < hidden; d += 32)
            xh[size_t(t0 + t) * hidden + d] = __float2half_rn(bf16_round_f(xs[t * hidden + d]) * scale);
        if (lane == 0) xshift[t0 + t] = shift;
    }
}

__device__ __forceinline__ bool expert_is_local(int e, const MoeShard& sh)
{
    if (sh.world <= 1) return true;
    return sh.interleaved ? (e % sh.world) == sh.rank : (e >= sh.lo && e < sh.hi);
}

// Decode-sized batches (at most 8 tokens, at most 256 experts): top-k, counts, stable slot
// order, the task list and the row-tile prefix by one CTA of 256 threads - the last CTA of
// the router kernel to finish (same results as moe_topk_kernel + moe_count_kernel +
// moe_fill_kernel).
struct SmallMeta {
    int* selected;
    float* probs;
    int* counts;
    int* offsets;
    int* sorted;
    int4* tasks;
    int* ntasks;
    int* tile_prefix;
    unsigned* done;       // CTAs of the router kernel that have written their logits; nullptr: no bookkeeping here
    int topk, rows_per_task, tile_rows;
    MoeShard sh;
};

__device__ __forceinline__ void small_meta_body(const float* logits, const SmallMeta& mt, int tokens, int experts)
{
    __shared__ int s_sel[8 * 8];
    __shared__ int s_count[256], s_ntask[256], s_ntile[256], s_offset[257], s_task[257], s_tile[257];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int topk = mt.topk;
    // ---- top-k: one warp per token (8 warps); the logits were written by other CTAs: read them from L2,
    // once (a lane keeps its up to eight logits in registers over the k rounds)
    if (warp < tokens) {
        const float* l = logits + size_t(warp) * experts;
        float mine_v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) mine_v[u] = lane + 32 * u < experts ? __ldcg(&l[lane + 32 * u]) : -INFINITY;
        unsigned taken = 0;   // bit u: this lane's u-th logit has been selected
        // The rounds run through one copy of the code (this body runs once per call, cold: see the router kernel);
        // lane j keeps the j-th pick.
        float my_top = -INFINITY, top0 = 0.f;
        int my_pick = 0;
#pragma unroll 1
        for (int j = 0; j < topk; ++j) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int e = lane + 32 * u;
                if (e < experts && !(taken & (1u << u)) && (arg == 0x7fffffff || mine_v[u] > best)) {   // ascending e: ties keep the lower
                    best = mine_v[u];
                    arg = e;
                }
            }
#pragma unroll
            for (int off = 16; off; off >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, off);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
                if (oa != 0x7fffffff && (arg == 0x7fffffff || ov > best || (ov == best && oa < arg))) {
                    best = ov;
                    arg = oa;
                }
            }
            if ((arg & 31) == lane) taken |= 1u << (arg >> 5);
            if (lane == j) my_top = best, my_pick = arg;
            if (j == 0) top0 = best;
        }
        // the sum runs over j = 0, 1, ... in that order
        const float ex = lane < topk ? expf(my_top - top0) : 0.f;
        float total = 0.f;
#pragma unroll 1
        for (int j = 0; j < topk; ++j) total += __shfl_sync(0xffffffffu, ex, j);
        if (lane < topk) {
            mt.selected[warp * topk + lane] = my_pick;
            s_sel[warp * topk + lane] = my_pick;
            mt.probs[warp * topk + lane] = bf16_round_f(ex / total);
        }
    }
    __syncthreads();
    const int slots = tokens * topk;
    const int e = threadIdx.x;
    if (tokens == 1 && !mt.tile_rows) {
        // One token: its experts are distinct, so every local one of them is a task of one row, in ascending
        // expert order - no scan, no second barrier.
        if (e < experts) {
            int before = 0, mine_slot = -1;
            for (int j = 0; j < topk; ++j) {
                const int c = s_sel[j];
                if (!expert_is_local(c, mt.sh)) continue;
                before += c < e;
                if (c == e) mine_slot = j;
            }
            mt.counts[e] = mine_slot >= 0 ? 1 : 0;
            mt.offsets[e] = before;
            if (mine_slot >= 0) {
                mt.sorted[before] = mine_slot;
                mt.tasks[before] = make_int4(e, before, 1, 0);
            }
            if (e == experts - 1) {
                const int total = before + (mine_slot >= 0 ? 1 : 0);
                mt.offsets[experts] = total;
                *mt.ntasks = total;
            }
        }
        return;
    }
    // ---- rows per expert (thread e)
    int mine = 0;
    if (e < experts && expert_is_local(e, mt.sh))
        for (int i = 0; i < slots; ++i) mine += s_sel[i] == e;
    s_count[e] = e < experts ? mine : 0;
    // tasks and row tiles of this expert: the divisions run once per thread, side by side, not in the scan below
    s_ntask[e] = e < experts ? (mine + mt.rows_per_task - 1) / mt.rows_per_task : 0;
    s_ntile[e] = (e < experts && mt.tile_rows) ? (mine + mt.tile_rows - 1) / mt.tile_rows : 0;
    if (e < experts) mt.counts[e] = mine;
    __syncthreads();
    // ---- exclusive prefix sums of rows, tasks and row tiles: warp 0, eight experts per lane
    if (warp == 0) {
        int off = 0, tk = 0, tp = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            off += s_count[lane * 8 + q];
            tk += s_ntask[lane * 8 + q];
            tp += s_ntile[lane * 8 + q];
        }
        int xo = off, xt = tk, xp = tp;   // inclusive scan over the lanes
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int a = __shfl_up_sync(0xffffffffu, xo, d), b = __shfl_up_sync(0xffffffffu, xt, d),
                      c = __shfl_up_sync(0xffffffffu, xp, d);
            if (lane >= d) xo += a, xt += b, xp += c;
        }
        off = xo - off, tk = xt - tk, tp = xp - tp;   // exclusive start of this lane's eight experts
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int idx = lane * 8 + q;
            s_offset[idx] = off, s_task[idx] = tk, s_tile[idx] = tp;
            off += s_count[idx];
            tk += s_ntask[idx];
            tp += s_ntile[idx];
        }
        if (lane == 31) s_offset[256] = off, s_task[256] = tk, s_tile[256] = tp;
    }
    __syncthreads();
    if (e < experts) {
        mt.offsets[e] = s_offset[e];
        if (mt.tile_rows) mt.tile_prefix[e] = s_tile[e];
    }
    if (e == 0) {
        // experts beyond `experts` have no rows, so entry `experts` already holds the totals
        mt.offsets[experts] = s_offset[experts];
        *mt.ntasks = s_task[experts];
        if (mt.tile_rows) mt.tile_prefix[experts] = s_tile[experts];
    }
    if (e < experts && mine) {
        int n = 0;
        for (int i = 0; i < slots; ++i)
            if (s_sel[i] == e) mt.sorted[s_offset[e] + n++] = i;   // slot order kept: stable
        for (int b = 0; b * mt.rows_per_task < mine; ++b)
            mt.tasks[s_task[e] + b] = make_int4(e, s_offset[e] + b * mt.rows_per_task, min(mt.rows_per_task, mine - b * mt.rows_per_task), 0);
    }
}

// Router for at most 8 tokens (decode).  Latency is everything here, so: one expert per CTA with the
// hidden dimension split over the CTA's 256 threads (a thread's first twelve weights are requested
// before the wait on the preceding kernel: the router weights are constants); x arrives with 16-byte
// loads, all in flight together; the fp16 copy of x is written in slices by all CTAs.  Same results
// contract as moe_route_scores_kernel (fp32 accumulation, bf16-rounded logits).
constexpr int kSmallRouteSteps = 12;   // weights per thread held in registers (hidden <= 3072; a loop covers the rest)
template <typename XT>
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_small_kernel(const XT* __restrict__ x, const float* __restrict__ rw, const float* __restrict__ rb,
                       float* __restrict__ logits, __half* __restrict__ xh, int* __restrict__ xshift, int tokens,
                       int hidden, int experts, const SmallMeta mt)
{
    extern __shared__ __align__(16) uint8_t xs_raw[];
    XT* xs = reinterpret_cast<XT*>(xs_raw);   // [tokens][hidden], as it comes (converted where it is used: less code here)
    __shared__ float part[kRouteWarps][kRouteTokens];
    __shared__ float s_amax[kRouteWarps];
    __shared__ int s_last;
    constexpr int kThreads = kRouteWarps * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) GB_MTRACE(0);
    const int e = blockIdx.x;
    const float* wrow = rw + size_t(e) * hidden;
    float wv[kSmallRouteSteps];
#pragma unroll
    for (int i = 0; i < kSmallRouteSteps; ++i) {
        const int d = threadIdx.x + i * kThreads;
        wv[i] = d < hidden ? __ldg(&wrow[d]) : 0.f;
    }
    const float bias = __ldg(&rb[e]);
    pdl_launch_dependents();
    pdl_wait();   // x comes from the kernel before this one
    if (threadIdx.x == 0) GB_MTRACE(1);
    {
        constexpr int kPer = 16 / int(sizeof(XT));   // elements per 16-byte load
        const int total = tokens * hidden;
        if (hidden % kPer == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            const uint4* xv = reinterpret_cast<const uint4*>(x);
            const int nvec = total / kPer;
#pragma unroll 6
            for (int v = threadIdx.x; v < nvec; v += kThreads) reinterpret_cast<uint4*>(xs)[v] = __ldcg(&xv[v]);
        } else {
            for (int i = threadIdx.x; i < total; i += kThreads) xs[i] = x[i];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) GB_MTRACE(2);
    // One token after the other through the same few instructions: this code runs once per CTA, so every
    // instruction of it is fetched cold, and unrolled over eight tokens it spent more time being fetched than
    // running.
#pragma unroll 1
    for (int t = 0; t < tokens; ++t) {
        const XT* xt = xs + t * hidden;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < kSmallRouteSteps; ++i) {
            const int d = threadIdx.x + i * kThreads;
            if (d < hidden) acc = fmaf(to_float(xt[d]), wv[i], acc);
        }
        for (int d = threadIdx.x + kSmallRouteSteps * kThreads; d < hidden; d += kThreads)
            acc = fmaf(to_float(xt[d]), __ldg(&wrow[d]), acc);
        const float v = warp_sum(acc);
        if (lane == 0) part[warp][t] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) GB_MTRACE(3);
    if (threadIdx.x < tokens) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kRouteWarps; ++w) v += part[w][threadIdx.x];
        logits[size_t(threadIdx.x) * experts + e] = bf16_round_f(v + bias);
    }
    // fp16 copy of x: token t's row in `slices` pieces, piece (t, s) by CTA t * slices + s (mod the grid)
    if (xh) {
        const int slices = max(1, int(gridDim.x) / tokens);
        const int len = ((hidden + slices - 1) / slices + 7) & ~7;
        for (int u = blockIdx.x; u < tokens * slices; u += gridDim.x) {
            const int t = u / slices, sl = u % slices;
            float amax = 0.f;
            for (int d = threadIdx.x; d < hidden; d += kThreads) amax = fmaxf(amax, fabsf(bf16_round_f(to_float(xs[t * hidden + d]))));
#pragma unroll
            for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            __syncthreads();
            if (lane == 0) s_amax[warp] = amax;
            __syncthreads();
#pragma unroll
            for (int w = 0; w < kRouteWarps; ++w) amax = fmaxf(amax, s_amax[w]);
            int shift = 0;
            if (amax > 0.f && isfinite(amax)) shift = int((__float_as_uint(amax) >> 23) & 0xff) - 127 - 13;
            shift = max(-100, min(100, shift));
            const float scale = __uint_as_float(uint32_t(127 - shift) << 23);
            const int d1 = min(hidden, (sl + 1) * len);
            for (int d = sl * len + threadIdx.x; d < d1; d += kThreads)
                xh[size_t(t) * hidden + d] = __float2half_rn(bf16_round_f(to_float(xs[t * hidden + d])) * scale);
            if (sl == 0 && threadIdx.x == 0) xshift[t] = shift;
        }
    }
    if (!mt.done) return;
    if (threadIdx.x == 0) GB_MTRACE(4);
    // the CTA that finishes last has every logit in reach and does the call's bookkeeping
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(mt.done, 1u) == gridDim.x - 1;
    __syncthreads();
    if (threadIdx.x == 0) GB_MTRACE(5);
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) GB_MTRACE_ANY(6);
    small_meta_body(logits, mt, tokens, experts);
    if (threadIdx.x == 0) GB_MTRACE_ANY(7);
    if (threadIdx.x == 0) *mt.done = 0;   // for the next call
}

// k rounds of arg-max (ties to the lowest expert index), then the softmax over the
// selected logits only (gpt_oss_kernels.cu:681-726).  One warp per token.
__global__ void moe_topk_kernel(const float* __restrict__ logits, int* __restrict__ selected,
                                float* __restrict__ probs, int tokens, int experts, int topk, int* __restrict__ counts,
                                MoeShard sh)
{
    const int token = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (token >= tokens) return;
    const float* l = logits + size_t(token) * experts;
    float top[8];
    int chosen[8];
    for (int j = 0; j < topk; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;   // "none yet"
        for (int e = lane; e < experts; e += 32) {
            bool used = false;
            for (int q = 0; q < j; ++q) used |= chosen[q] == e;
            const float v = l[e];
            if (!used && (arg == 0x7fffffff || v > best || (v == best && e < arg))) {
                best = v;
                arg = e;
            }
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
            if (oa != 0x7fffffff && (arg == 0x7fffffff || ov > best || (ov == best && oa < arg))) {
                best = ov;
                arg = oa;
            }
        }
        chosen[j] = arg;
        top[j] = best;
    }
    if (lane == 0) {
        float total = 0.f;
        for (int j = 0; j < topk; ++j) total += expf(top[j] - top[0]);
        for (int j = 0; j < topk; ++j) {
            selected[token * topk + j] = chosen[j];
            probs[token * topk + j] = bf16_round_f(expf(top[j] - top[0]) / total);
            // rows per local expert (zeroed by the caller): integer adds, any order
            if (counts && expert_is_local(chosen[j], sh)) atomicAdd(&counts[chosen[j]], 1);
        }
    }
}

// After the tensor-core router, one warp per token: adds the K ranges' partial sums in order (+ bias, bf16
// rounding: the logits), picks the top k from registers (ties to the lowest expert index) with the softmax over
// the picked logits only (gpt_oss_kernels.cu:681-726), counts the rows of the local experts, and - when the
// streaming expert kernel follows - writes the token's fp16 row copy (same arithmetic as moe_prep_rows_kernel).
// At most 256 experts (eight logits per lane) and top 8.
template <typename XT>
__global__ void __launch_bounds__(256)
moe_route_finish_topk_kernel(const float* __restrict__ partial, int splits, const float* __restrict__ rb,
                             float* __restrict__ logits, int* __restrict__ selected, float* __restrict__ probs,
                             int* __restrict__ counts, MoeShard sh, const XT* __restrict__ x, __half* __restrict__ xh,
                             int* __restrict__ xshift, int tokens, int hidden, int experts, int topk)
{
    pdl_launch_dependents();
    pdl_wait();
    const int token = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (token >= tokens) return;
    const size_t plane = size_t(tokens) * experts;
    const float* p0 = partial + size_t(token) * experts;
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = lane + 32 * u < experts ? p0[lane + 32 * u] : 0.f;
#pragma unroll 2
    for (int z = 1; z < splits; ++z) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (lane + 32 * u < experts) v[u] += p0[z * plane + lane + 32 * u];
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int e = lane + 32 * u;
        if (e < experts) {
            v[u] = bf16_round_f(v[u] + rb[e]);
            logits[size_t(token) * experts + e] = v[u];
        } else {
            v[u] = -INFINITY;
        }
    }
    unsigned taken = 0;   // bit u: this lane's u-th logit has been picked
    // the rounds run through one copy of the code (a warp runs this once: every instruction is fetched cold);
    // lane j keeps the j-th pick
    float my_top = -INFINITY, top0 = 0.f;
    int my_pick = 0;
#pragma unroll 1
    for (int j = 0; j < topk; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int e = lane + 32 * u;
            if (e < experts && !(taken & (1u << u)) && (arg == 0x7fffffff || v[u] > best)) {   // ascending e: ties keep the lower
                best = v[u];
                arg = e;
            }
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
            if (oa != 0x7fffffff && (arg == 0x7fffffff || ov > best || (ov == best && oa < arg))) {
                best = ov;
                arg = oa;
            }
        }
        if ((arg & 31) == lane) taken |= 1u << (arg >> 5);
        if (lane == j) my_top = best, my_pick = arg;
        if (j == 0) top0 = best;
    }
    const float ex = lane < topk ? expf(my_top - top0) : 0.f;
    float total = 0.f;
#pragma unroll 1
    for (int j = 0; j < topk; ++j) total += __shfl_sync(0xffffffffu, ex, j);
    if (lane < topk) {
        selected[token * topk + lane] = my_pick;
        probs[token * topk + lane] = bf16_round_f(ex / total);
        // rows per local expert (zeroed by the caller): integer adds, any order
        if (counts && expert_is_local(my_pick, sh)) atomicAdd(&counts[my_pick], 1);
    }
    if (!xh) return;
    const XT* src = x + size_t(token) * hidden;
    __half* dst = xh + size_t(token) * hidden;
    auto shift_of = [](float amax) {
        int shift = 0;
        if (amax > 0.f && isfinite(amax)) shift = int((__float_as_uint(amax) >> 23) & 0xff) - 127 - 13;
        return max(-100, min(100, shift));
    };
    if constexpr (sizeof(XT) == 2) {
        // a bf16 row of up to 3072 columns in one round trip: twelve 16-byte loads per lane, kept in registers
        constexpr int kVec = 12;
        if (hidden % 8 == 0 && hidden <= kVec * 32 * 8 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            const uint4* sv = reinterpret_cast<const uint4*>(src);
            const int nvec = hidden / 8;
            uint4 r[kVec];
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < kVec; ++i) r[i] = lane + 32 * i < nvec ? sv[lane + 32 * i] : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int i = 0; i < kVec; ++i) {
                const uint32_t w[4] = {r[i].x, r[i].y, r[i].z, r[i].w};
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[q] << 16)), fabsf(__uint_as_float(w[q] & 0xffff0000u))));
            }
#pragma unroll
            for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            const int shift = shift_of(amax);
            const float scale = __uint_as_float(uint32_t(127 - shift) << 23);
#pragma unroll
            for (int i = 0; i < kVec; ++i) {
                if (lane + 32 * i < nvec) {
                    const uint32_t w[4] = {r[i].x, r[i].y, r[i].z, r[i].w};
                    uint32_t o[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const __half2 h = __floats2half2_rn(__uint_as_float(w[q] << 16) * scale, __uint_as_float(w[q] & 0xffff0000u) * scale);
                        o[q] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(dst + size_t(lane + 32 * i) * 8) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
            if (lane == 0) xshift[token] = shift;
            return;
        }
    }
    float amax = 0.f;
#pragma unroll 8
    for (int d = lane; d < hidden; d += 32) amax = fmaxf(amax, fabsf(bf16_round_f(to_float(src[d]))));
#pragma unroll
    for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const int shift = shift_of(amax);
    const float scale = __uint_as_float(uint32_t(127 - shift) << 23);
#pragma unroll 8
    for (int d = lane; d < hidden; d += 32) dst[d] = __float2half_rn(bf16_round_f(to_float(src[d])) * scale);
    if (lane == 0) xshift[token] = shift;
}

// fp16 copy of activation rows for the expert kernels, one warp per row: the row
// is rounded to bf16 and scaled by an exact power of two so that its largest
// magnitude lands in [2^13, 2^14); `xshift` keeps the exponent (x = xh * 2^shift).
// Same arithmetic as the tail of moe_route_scores_kernel.
template <typename XT>
__global__ void moe_prep_rows_kernel(const XT* __restrict__ x, __half* __restrict__ xh, int* __restrict__ xshift,
                                     int rows, int hidden)
{
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    const XT* src = x + size_t(row) * hidden;
    float amax = 0.f;
    for (int d = lane; d < hidden; d += 32) amax = fmaxf(amax, fabsf(bf16_round_f(to_float(src[d]))));
#pragma unroll
    for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    int shift = 0;
    if (amax > 0.f && isfinite(amax)) shift = int((__float_as_uint(amax) >> 23) & 0xff) - 127 - 13;
    shift = max(-100, min(100, shift));
    const float scale = __uint_as_float(uint32_t(127 - shift) << 23);
    for (int d = lane; d < hidden; d += 32)
        xh[size_t(row) * hidden + d] = __float2half_rn(bf16_round_f(to_float(src[d])) * scale);
    if (lane == 0) xshift[row] = shift;
}

// Activations of the routed rows between the two projections, exchanged with the
// caller in row order as fp32 (bf16-valued).  The kernels keep them as fp16 at
// the row's sorted position (block-scaled path) or at the row itself (streaming path).
__global__ void moe_act_to_rows_kernel(const __half* __restrict__ act, const int* __restrict__ sorted,
                                       const int* __restrict__ offsets, int experts, int inter, int by_position,
                                       float* __restrict__ out)
{
    const int pos = blockIdx.x;
    if (pos >= offsets[experts]) return;
    const int row = sorted[pos];
    const __half* src = act + size_t(by_position ? pos : row) * inter;
    for (int i = threadIdx.x; i < inter; i += blockDim.x) out[size_t(row) * inter + i] = __half2float(src[i]);
}
__global__ void moe_rows_to_act_kernel(const float* __restrict__ in, const int* __restrict__ sorted,
                                       const int* __restrict__ offsets, int experts, int inter, int by_position,
                                       __half* __restrict__ act)
{
    const int pos = blockIdx.x;
    if (pos >= offsets[experts]) return;
    const int row = sorted[pos];
    __half* dst = act + size_t(by_position ? pos : row) * inter;
    for (int i = threadIdx.x; i < inter; i += blockDim.x) dst[i] = __float2half_rn(in[size_t(row) * inter + i]);
}

// ------------------------------------------------------------ slot bucketing


// counts[e] = number of routed slots of expert e (0 for experts of other ranks).
__global__ void moe_count_kernel(const int* __restrict__ selected, int slots, int* __restrict__ counts, MoeShard sh)
{
    const int e = blockIdx.x;
    __shared__ int s_part[32];
    int c = 0;
    if (expert_is_local(e, sh))
        for (int i = threadIdx.x; i < slots; i += blockDim.x) c += selected[i] == e;
    for (int off = 16; off; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int w = 0; w < int(blockDim.x >> 5); ++w) total += s_part[w];
        counts[e] = total;
    }
}

// Stable counting sort of the slots by expert (slot order preserved inside an
// expert, like gpt_oss_marlin.cu:239-277) plus the task list: one task per block
// of up to `rows_per_task` slots of one expert.  One CTA per expert.
__global__ void __launch_bounds__(1024)
moe_fill_kernel(const int* __restrict__ selected, int slots, const int* __restrict__ counts,
                int* __restrict__ offsets, int* __restrict__ sorted, int4* __restrict__ tasks,
                int* __restrict__ ntasks, int experts, int rows_per_task, MoeShard sh, int tile_rows,
                int* __restrict__ tile_prefix)
{
    const int e = blockIdx.x;
    __shared__ int s_offset, s_warp[32];
    // rows, tasks and row tiles of the experts before this one: warp 0 adds them up, a slice per lane
    int off = 0, tk = 0, tp = 0;
    if (threadIdx.x < 32) {
        for (int q = threadIdx.x; q < e; q += 32) {
            const int c = counts[q];
            off += c;
            tk += (c + rows_per_task - 1) / rows_per_task;
            if (tile_rows) tp += (c + tile_rows - 1) / tile_rows;
        }
#pragma unroll
        for (int d = 16; d; d >>= 1) {
            off += __shfl_xor_sync(0xffffffffu, off, d);
            tk += __shfl_xor_sync(0xffffffffu, tk, d);
            tp += __shfl_xor_sync(0xffffffffu, tp, d);
        }
    }
    if (threadIdx.x == 0) {
        if (tile_rows) {
            // row tiles before each expert (block-scaled path)
            tile_prefix[e] = tp;
            if (e == experts - 1) tile_prefix[experts] = tp + (counts[e] + tile_rows - 1) / tile_rows;
        }
        s_offset = off;
        offsets[e] = off;
        const int mine = counts[e];
        for (int b = 0; b * rows_per_task < mine; ++b)
            tasks[tk + b] = make_int4(e, off + b * rows_per_task, min(rows_per_task, mine - b * rows_per_task), 0);
        if (e == experts - 1) {
            offsets[experts] = off + mine;
            *ntasks = tk + (mine + rows_per_task - 1) / rows_per_task;
        }
    }
    __syncthreads();
    if (counts[e] == 0) return;
    // Stable order of this expert's slots: a thread counts its own run of consecutive slots, one scan over the
    // threads gives every run its place, and the thread writes its run's hits in slot order.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per = (slots + int(blockDim.x) - 1) / int(blockDim.x);
    const int i0 = min(slots, int(threadIdx.x) * per), i1 = min(slots, i0 + per);
    int hits = 0;
    for (int i = i0; i < i1; ++i) hits += selected[i] == e;
    int incl = hits;   // inclusive scan over the warp's lanes
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int before = s_offset + incl - hits;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    for (int i = i0; i < i1; ++i)
        if (selected[i] == e) sorted[before++] = i;
}

// ------------------------------------------------- streaming expert kernel


#ifndef GB_MOE_WARPS
#define GB_MOE_WARPS 8
#endif
constexpr int kMoeWarps = GB_MOE_WARPS;                       // warps per CTA; each streams its own strips through its own ring
#ifndef GB_MOE_STAGES
#define GB_MOE_STAGES 2
#endif
constexpr int kMoeStages = GB_MOE_STAGES;          // ring slots per warp
#ifndef GB_MOE_CTAS
#define GB_MOE_CTAS 2
#endif
constexpr int kMoeCtasPerSm = GB_MOE_CTAS;
#ifndef GB_MOE_SEG
#define GB_MOE_SEG 9
#endif
constexpr int kMoeSegChunks = GB_MOE_SEG;          // chunks per bulk copy (a gpt-oss strip is 45 chunks = 5 copies; copies of 3 / 5 / 9
                                                   // chunks measured 275 / 244 / 221 us per 32-token call: the work around a copy is per copy)
constexpr int kMoeSegBytes = kMoeSegChunks * kMxChunkBytes;
constexpr int kMoeRows = 8;                        // slots per task (one MMA N-tile)
constexpr int kMoeListCache = 32;                  // leading task and slot-order entries a CTA keeps in shared memory

struct MoeStreamParams {
    const uint8_t* packed;      // [experts_local][matrix]
    const __half* act_in;       // up: xh [tokens, K]; down: act [slots, K]
    const int* xshift;          // up: per-token exponent of the fp16 copy; down: null
    const int4* tasks;
    const int* ntasks;
    const int* sorted;
    const float* bias;          // [experts_local, rows] fp32, original row order
    __half* act_out;            // up: [slots, inter]
    float* vals_out;            // down: [slots, hidden]
    int* fault;
    int k, rows;                // K columns, logical rows of one expert matrix
    int strips, chunks;
    int topk;
    int expert_base, expert_div;   // stored expert = (e - expert_base) / expert_div
    int bias_by_global;            // bias rows are indexed by the global expert id
    int tasks_early;               // the task list was complete before this grid could start (see kernel)
    int slots;                     // entries of `sorted` (tokens * topk)
    int tasks_cap;                 // entries the task list has room for
    int vals_bf16;                 // vals_out holds bf16
    float limit;
    size_t matrix_bytes;
};

struct MoeSmem {
    int ring, bars, total;
};
__host__ __device__ inline MoeSmem moe_smem_plan()
{
    MoeSmem p;
    p.ring = 0;
    p.bars = kMoeWarps * kMoeStages * kMoeSegBytes;
    p.total = p.bars + kMoeWarps * kMoeStages * 8;
    return p;
}

// m16n8k16 fp16 MMA, fp32 accumulation, as a plain (not volatile) statement: the compiler may interleave the
// independent MMAs of neighbouring column groups and chunks.
__device__ __forceinline__ void moe_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1, const float (&c)[4])
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// One chunk (16 rows x 64 columns: 512 bytes of codes, 32 scale bytes) times the task's slots.  xa/xb: this lane's
// activations of column groups 0 and 1.  acc[0..1]: strip row R(g), slots 2t and 2t+1; acc[2..3]: strip row R(g)+8.
template <bool kCareful>
__device__ __forceinline__ void moe_chunk_math(const uint8_t* st, int lane, int g, const uint4& xa, const uint4& xb,
                                               float (&acc)[4])
{
    const uint4 u = *reinterpret_cast<const uint4*>(st + lane * 16);
    const uint32_t sc = *reinterpret_cast<const uint32_t*>(st + 512 + g * 4);
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
    float t0[4], t1[4];
    // group 0: octets 0..3 (words x = row R, y = row R+8); group 1: octets 4..7 (words z, w)
    moe_mma(t0, e2m1x2_to_f16x2(u.x, 0), e2m1x2_to_f16x2(u.y, 0), e2m1x2_to_f16x2(u.x, 1), e2m1x2_to_f16x2(u.y, 1), xa.x, xa.y, zero4);
    moe_mma(t1, e2m1x2_to_f16x2(u.z, 0), e2m1x2_to_f16x2(u.w, 0), e2m1x2_to_f16x2(u.z, 1), e2m1x2_to_f16x2(u.w, 1), xb.x, xb.y, zero4);
    moe_mma(t0, e2m1x2_to_f16x2(u.x, 2), e2m1x2_to_f16x2(u.y, 2), e2m1x2_to_f16x2(u.x, 3), e2m1x2_to_f16x2(u.y, 3), xa.z, xa.w, t0);
    moe_mma(t1, e2m1x2_to_f16x2(u.z, 2), e2m1x2_to_f16x2(u.w, 2), e2m1x2_to_f16x2(u.z, 3), e2m1x2_to_f16x2(u.w, 3), xb.z, xb.w, t1);
    const float f0_lo = e8m0_to_float<kCareful>(sc & 0xff), f0_hi = e8m0_to_float<kCareful>((sc >> 8) & 0xff);
    const float f1_lo = e8m0_to_float<kCareful>((sc >> 16) & 0xff), f1_hi = e8m0_to_float<kCareful>(sc >> 24);
    acc[0] = fmaf(t0[0], f0_lo, acc[0]);
    acc[1] = fmaf(t0[1], f0_lo, acc[1]);
    acc[2] = fmaf(t0[2], f0_hi, acc[2]);
    acc[3] = fmaf(t0[3], f0_hi, acc[3]);
    acc[0] = fmaf(t1[0], f1_lo, acc[0]);
    acc[1] = fmaf(t1[1], f1_lo, acc[1]);
    acc[2] = fmaf(t1[2], f1_hi, acc[2]);
    acc[3] = fmaf(t1[3], f1_hi, acc[3]);
}

// What a lane keeps about the task (up to 8 routed slots of one expert) it is working on.
struct MoeTaskLane {
    int expert = 0, rows = 0;
    int slot0 = -1, slot1 = -1, shift0 = 0, shift1 = 0;   // the two slots (2t, 2t + 1) this lane finishes
    const uint8_t* xg = nullptr;                           // this lane's activation row (row g of the task), at column 8t
};

template <bool kUp>
__device__ __forceinline__ void moe_task_lane(const MoeStreamParams& p, const int4* s_tasks, const int* s_sorted, int task,
                                              int g, int t, MoeTaskLane& tl)
{
    const int4 tk = task < kMoeListCache ? s_tasks[task] : __ldcg(&p.tasks[task]);
    tl.expert = tk.x;
    tl.rows = tk.z;
    auto slot_at = [&](int m) {
        const int at = tk.y + m;
        return at < kMoeListCache ? s_sorted[at] : __ldcg(&p.sorted[at]);
    };
    // a lane whose slot g is beyond the task's rows reads the first row: the MMA column it feeds is never
    // stored, and the loop needs no test
    const int sg = slot_at(g < tl.rows ? g : 0);
    const size_t src_row = kUp ? size_t(sg / p.topk) : size_t(sg);
    tl.xg = reinterpret_cast<const uint8_t*>(p.act_in + src_row * p.k) + t * 16;
    tl.slot0 = 2 * t < tl.rows ? slot_at(2 * t) : -1;
    tl.slot1 = 2 * t + 1 < tl.rows ? slot_at(2 * t + 1) : -1;
    tl.shift0 = tl.shift1 = 0;
    if (kUp) {
        if (tl.slot0 >= 0) tl.shift0 = __ldg(&p.xshift[tl.slot0 / p.topk]);
        if (tl.slot1 >= 0) tl.shift1 = __ldg(&p.xshift[tl.slot1 / p.topk]);
    }
}

// The two bias values a lane needs at the end of a strip (requested at its start).
template <bool kUp>
__device__ __forceinline__ void moe_strip_bias(const MoeStreamParams& p, const MoeTaskLane& tl, int strip, int g, float& bias0,
                                               float& bias1)
{
    const int ebias = p.bias_by_global ? tl.expert : (tl.expert - p.expert_base) / p.expert_div;
    bias0 = bias1 = 0.f;
    if (kUp) {
        const int i = strip * 8 + row_of_g(g);
        if (2 * i + 1 < p.rows) {
            const float* b = p.bias + size_t(ebias) * p.rows + 2 * i;
            bias0 = __ldg(b), bias1 = __ldg(b + 1);
        }
    } else {
        const int d = strip * 16 + row_of_g(g);
        if (d < p.rows) bias0 = __ldg(&p.bias[size_t(ebias) * p.rows + d]);
        if (d + 8 < p.rows) bias1 = __ldg(&p.bias[size_t(ebias) * p.rows + d + 8]);
    }
}

// End of a strip.  acc[0..1]: strip row R(g), slots 2t, 2t+1; acc[2..3]: strip row R(g)+8.
template <bool kUp>
__device__ __forceinline__ void moe_strip_finish(const MoeStreamParams& p, const MoeTaskLane& tl, int strip, int g,
                                                 const float (&acc)[4], float bias0, float bias1)
{
    if (kUp) {
        // rows R(g) and R(g)+8 are the gate and the up value of one intermediate channel
        const int i = strip * 8 + row_of_g(g);
        if (2 * i + 1 < p.rows) {
#pragma unroll
            for (int par = 0; par < 2; ++par) {
                const int slot = par ? tl.slot1 : tl.slot0;
                if (slot < 0) continue;
                const float sc2 = __uint_as_float(uint32_t(127 + (par ? tl.shift1 : tl.shift0)) << 23);   // 2^shift
                float gate = fminf(bf16_round_f(bf16_round_f(acc[par] * sc2) + bias0), p.limit);
                const float up = fminf(p.limit, fmaxf(-p.limit, bf16_round_f(bf16_round_f(acc[par + 2] * sc2) + bias1)));
                const float sig = bf16_round_f(1.f / (1.f + expf(-bf16_round_f(1.702f * gate))));
                const float glu = bf16_round_f(gate * sig);
                p.act_out[size_t(slot) * (p.rows / 2) + i] = __float2half_rn(bf16_round_f(glu * bf16_round_f(up + 1.f)));
            }
        }
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int slot = (q & 1) ? tl.slot1 : tl.slot0;
            const int d = strip * 16 + row_of_g(g) + 8 * (q >> 1);
            if (slot >= 0 && d < p.rows)
            {
                    const float v = bf16_round_f(bf16_round_f(acc[q]) + ((q >> 1) ? bias1 : bias0));
                    if (p.vals_bf16) reinterpret_cast<__nv_bfloat16*>(p.vals_out)[size_t(slot) * p.rows + d] = __float2bfloat16_rn(v);
                    else p.vals_out[size_t(slot) * p.rows + d] = v;
                }
        }
    }
}

// The chunks of one ring slot (a copy of up to kMoeSegChunks chunks of a strip, starting at chunk seg * kMoeSegChunks)
// times the task's slots, added to acc.  The slots' activations are read where they are used, by plain loads (cached
// in L1; three CTAs per SM would leave an L1 too small for them): the rows were written by the kernel before this
// one, which may still have been running when this one started.
template <bool kCareful>
__device__ __forceinline__ void moe_seg_math(const uint8_t* sbase, const uint8_t* xg, int seg, int nch, int row_bytes, int lane,
                                             float (&acc)[4])
{
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* xseg = xg + size_t(seg) * (kMoeSegChunks * 128);   // 64 columns = 128 bytes of x
    if (nch == kMoeSegChunks && (seg + 1) * (kMoeSegChunks * 128) <= row_bytes) {   // the common case as one straight run
#pragma unroll
        for (int c = 0; c < kMoeSegChunks; ++c) {
            const uint4 xa = *reinterpret_cast<const uint4*>(xseg + c * 128);
            const uint4 xb = *reinterpret_cast<const uint4*>(xseg + c * 128 + 64);
            moe_chunk_math<kCareful>(sbase + c * kMxChunkBytes, lane, g, xa, xb, acc);
        }
    } else {
#pragma unroll
        for (int c = 0; c < kMoeSegChunks; ++c)
            if (c < nch) {
                uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
                const int off = (seg * kMoeSegChunks + c) * 128 + t * 16;
                if (off + 16 <= row_bytes) xa = *reinterpret_cast<const uint4*>(xseg + c * 128);
                if (off + 80 <= row_bytes) xb = *reinterpret_cast<const uint4*>(xseg + c * 128 + 64);
                moe_chunk_math<kCareful>(sbase + c * kMxChunkBytes, lane, g, xa, xb, acc);
            }
    }
}

// Persistent CTAs over the flattened list of (task, strip) items; a task is up to 8 routed slots of
// one expert, a strip 16 rows of that expert's matrix (codes and scales together, contiguous).  A CTA
// owns a contiguous range of items and its warps take them in turn; every warp works alone: lane 0
// requests the strip in 9-chunk bulk copies into the warp's own two-slot ring, the warp converts e2m1 pairs to
// fp16 pairs with one instruction each and runs m16n8k16 fp16 MMAs whose N dimension is the task's
// slots (the slots' activations come straight from global memory: a few rows that stay in L1), scales
// each 32-column group's fp32 partial sum by its e8m0 factor, and finishes the strip from its own
// registers.  No warp waits for another one (the kernel is bound by instruction issue, and barriers
// between warps were a third of its stalls).  kUp: epilogue = bias + clamped SwiGLU -> activation
// (bf16-valued, stored as fp16); else bias -> per-slot values for the combine.
template <bool kUp, bool kCareful>
__global__ void __launch_bounds__(kMoeWarps * 32, kMoeCtasPerSm) moe_stream_kernel(const MoeStreamParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const MoeSmem plan = moe_smem_plan();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* ring = smem + plan.ring + warp * (kMoeStages * kMoeSegBytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + plan.bars) + warp * kMoeStages;
    [[maybe_unused]] constexpr int kTr = kUp ? 16 : 48;   // first trace slot of this launch (timing build)
    if (threadIdx.x == 0) GB_MTRACE(kTr + 0);
    if (lane == 0) {
        for (int s = 0; s < kMoeStages; ++s) mbar_init(&full[s], 1);
        fence_barrier_init();
    }
    // Programmatic dependent launch.  The gate/up launch lets its dependent (the down
    // launch) start only after its own wait has returned, i.e. once the kernels that
    // wrote the task list have completed: the down launch can therefore read the task
    // list and request its expert weights before its own wait, while gate/up still runs.
    // It waits before it reads gate/up's activations.
    if (!p.tasks_early) pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x == 0) GB_MTRACE(kTr + 1);

    // The first entries of the task list and of the slot order, and the task count, in one round trip to L2
    // (three warps load side by side); a decode-sized call never needs more than these.
    __shared__ int4 s_tasks[kMoeListCache];
    __shared__ int s_sorted[kMoeListCache];
    __shared__ int s_ntasks;
    if (threadIdx.x < kMoeListCache) {
        if (int(threadIdx.x) < p.tasks_cap) s_tasks[threadIdx.x] = __ldcg(&p.tasks[threadIdx.x]);
    } else if (threadIdx.x < 2 * kMoeListCache) {
        const int i = threadIdx.x - kMoeListCache;
        if (i < p.slots) s_sorted[i] = __ldcg(&p.sorted[i]);
    } else if (threadIdx.x == 2 * kMoeListCache) {
        s_ntasks = __ldcg(p.ntasks);
    }
    __syncthreads();
    const int ntasks = s_ntasks;
    // this CTA's items [i0, i1): an even split of ntasks * strips
    const unsigned long long total = (unsigned long long)ntasks * unsigned(p.strips);
    unsigned long long i0, i1;
    if (total < (1ull << 31)) {
        const unsigned per = unsigned(total) / gridDim.x, rem = unsigned(total) % gridDim.x;
        i0 = (unsigned long long)blockIdx.x * per + min(blockIdx.x, rem);
        i1 = i0 + per + (blockIdx.x < rem ? 1u : 0u);
    } else {
        i0 = total * blockIdx.x / gridDim.x, i1 = total * (blockIdx.x + 1) / gridDim.x;
    }
    if (i0 + warp >= i1) return;   // nothing for this warp (it holds no copies and no barrier another warp uses)
    const int my_items = int((i1 - i0 - warp + kMoeWarps - 1) / kMoeWarps);
    const int nseg = (p.chunks + kMoeSegChunks - 1) / kMoeSegChunks;
    const size_t strip_bytes = size_t(p.chunks) * kMxChunkBytes;
    const int last_bytes = (p.chunks - (nseg - 1) * kMoeSegChunks) * kMxChunkBytes;
    const int total_segs = my_items * nseg;

    auto expert_of = [&](int task) { return task < kMoeListCache ? s_tasks[task].x : __ldcg(&p.tasks[task]).x; };
    auto advance = [&](int& task, int& strip) {   // the warp's next item: kMoeWarps strips further
        strip += kMoeWarps;
        while (strip >= p.strips) strip -= p.strips, ++task;
    };

    // ---- requests run kMoeStages copies ahead of the arithmetic; their state lives in every lane, lane 0 acts
    int iss = 0, iss_seg = 0, iss_stage = 0;
    int iss_task, iss_strip;
    {
        const unsigned long long first = i0 + warp;
        if (first < (1ull << 31))   // 32-bit division: this sits in front of the first request
            iss_task = int(unsigned(first) / unsigned(p.strips)), iss_strip = int(unsigned(first) % unsigned(p.strips));
        else
            iss_task = int(first / unsigned(p.strips)), iss_strip = int(first % unsigned(p.strips));
    }
    int task = iss_task, strip = iss_strip;   // the item the arithmetic is at
    const uint8_t* iss_src = p.packed + size_t((expert_of(iss_task) - p.expert_base) / p.expert_div) * p.matrix_bytes +
                             size_t(iss_strip) * strip_bytes;
    auto request = [&]() {
        const int bytes = iss_seg == nseg - 1 ? last_bytes : kMoeSegBytes;
        if (lane == 0) {
            mbar_expect_tx(&full[iss_stage], uint32_t(bytes));
            bulk_g2s(ring + iss_stage * kMoeSegBytes, iss_src + size_t(iss_seg) * kMoeSegBytes, uint32_t(bytes), &full[iss_stage]);
        }
        ++iss;
        if (++iss_stage == kMoeStages) iss_stage = 0;
        if (++iss_seg == nseg && iss < total_segs) {
            iss_seg = 0;
            advance(iss_task, iss_strip);
            iss_src = p.packed + size_t((expert_of(iss_task) - p.expert_base) / p.expert_div) * p.matrix_bytes +
                      size_t(iss_strip) * strip_bytes;
        }
    };
    for (int n = 0; n < kMoeStages && n < total_segs; ++n) request();
    if (threadIdx.x == 0) GB_MTRACE(kTr + 2);
    if (p.tasks_early) pdl_wait();   // the activations come from the launch before this one
    if (threadIdx.x == 0) GB_MTRACE(kTr + 5);

    const int g = lane >> 2, t = lane & 3;
    const int row_bytes = p.k * 2;
    bool ok = true;
    int stage = 0, phase = 0, con = 0;
    int cur_task = -1;
    MoeTaskLane tl;
    for (int item = 0; item < my_items && ok; ++item) {
#ifdef GB_MOE_TRACE
        const long long ti0 = clock64();
#endif
        if (task != cur_task) {
            moe_task_lane<kUp>(p, s_tasks, s_sorted, task, g, t, tl);
            cur_task = task;
        }
        // this strip's bias values are requested now and used in the epilogue
        float bias0, bias1;
        moe_strip_bias<kUp>(p, tl, strip, g, bias0, bias1);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#ifdef GB_MOE_TRACE
        if (threadIdx.x == 0 && blockIdx.x == 7) g_moe_trace[kUp ? 88 : 91] += (unsigned long long)(clock64() - ti0);
#endif
        for (int seg = 0; seg < nseg; ++seg, ++con) {
#ifdef GB_MOE_TRACE
            const long long ts0 = clock64();
#endif
            const int nch = min(kMoeSegChunks, p.chunks - seg * kMoeSegChunks);
#ifdef GB_MOE_TRACE
            const long long tw0 = clock64();
            if (threadIdx.x == 0 && blockIdx.x == 7) g_moe_trace[kUp ? 89 : 92] += (unsigned long long)(tw0 - ts0);
#endif
            if (!__all_sync(0xffffffffu, mbar_wait(&full[stage], phase))) {   // the whole warp gives up, or no lane
                atomicExch(p.fault, 2);
                ok = false;
                break;
            }
            if (threadIdx.x == 0 && con == 0) GB_MTRACE(kTr + 7);
#ifdef GB_MOE_TRACE
            const long long tw1 = clock64();
            if (threadIdx.x == 0 && blockIdx.x == 7) g_moe_trace[kUp ? 84 : 86] += (unsigned long long)(tw1 - tw0);
#endif
            moe_seg_math<kCareful>(ring + stage * kMoeSegBytes, tl.xg, seg, nch, row_bytes, lane, acc);
            // every lane has read this ring slot: lane 0 asks for the copy that reuses it
            __syncwarp();
            if (iss < total_segs) {
                if (lane == 0) fence_proxy_async_smem();
                request();
            }
            if (++stage == kMoeStages) stage = 0, phase ^= 1;
#ifdef GB_MOE_TRACE
            if (threadIdx.x == 0 && blockIdx.x == 7) g_moe_trace[kUp ? 85 : 87] += (unsigned long long)(clock64() - tw1);
#endif
        }
        if (!ok) break;

#ifdef GB_MOE_TRACE
        const long long te0 = clock64();
#endif
        moe_strip_finish<kUp>(p, tl, strip, g, acc, bias0, bias1);
        if (threadIdx.x == 0 && item < 20) GB_MTRACE(kTr + 8 + item);
#ifdef GB_MOE_TRACE
        if (threadIdx.x == 0 && blockIdx.x == 7) g_moe_trace[kUp ? 90 : 93] += (unsigned long long)(clock64() - te0);
#endif
        advance(task, strip);
    }
    if (threadIdx.x == 0) GB_MTRACE(kTr + 31);
    // after a give-up the copies already requested may still land: give each a short moment (the fault is
    // recorded already, nothing is read any more) before the CTA's shared memory is released
    if (!ok) {
        for (int n = con; n < iss; ++n) {
            (void)mbar_wait(&full[stage], phase, 2000000ull);
            if (++stage == kMoeStages) stage = 0, phase ^= 1;
        }
    }
}

// y[t,d] = bf(sum_j vals[t*k+j, d] * p[t,j]) over the local experts in router order
// (gpt_oss_kernels.cu:907-921); the partial of an expert-sharded rank is left
// unrounded (:920).
template <typename YT>
__global__ void moe_combine_kernel(const float* __restrict__ vals, const float* __restrict__ probs,
                                   const int* __restrict__ selected, YT* __restrict__ y, int tokens, int hidden,
                                   int topk, MoeShard sh, int round_output)
{
    if (threadIdx.x == 0) GB_MTRACE(80);
    pdl_launch_dependents();
    pdl_wait();   // the per-slot values come from the kernel before this one
    if (threadIdx.x == 0) GB_MTRACE(81);
    // grid = (tokens, column blocks): no division per element
    const int token = blockIdx.x, d = blockIdx.y * blockDim.x + threadIdx.x;
    if (token >= tokens || d >= hidden) return;
    const size_t idx = size_t(token) * hidden + d;
    float r = 0.f;
    for (int j = 0; j < topk; ++j) {
        const int slot = token * topk + j;
        if (sh.world > 1 && !expert_is_local(selected[slot], sh)) continue;
        r = __fmaf_rn(vals[size_t(slot) * hidden + d], probs[slot], r);   // one rounding per term, here and in the exchange's combine
    }
    if (round_output) r = bf16_round_f(r);
    if constexpr (sizeof(YT) == 4)
        y[idx] = r;
    else
        y[idx] = __float2bfloat16_rn(r);
    if (threadIdx.x == 0) GB_MTRACE(82);
}

// The same combine for Moe::run's own bf16 per-slot values: a CTA row per token, eight columns per thread (16-byte
// loads and stores, no division per element).  hidden is a multiple of 8.
template <typename YT>
__global__ void __launch_bounds__(256)
moe_combine_rows_kernel(const __nv_bfloat16* __restrict__ vals, const float* __restrict__ probs, const int* __restrict__ selected,
                        YT* __restrict__ y, int hidden, int topk, MoeShard sh, int round_output)
{
    pdl_launch_dependents();
    pdl_wait();   // the per-slot values come from the kernel before this one
    const int token = blockIdx.x;
    const int d0 = (blockIdx.y * 256 + threadIdx.x) * 8;
    if (d0 >= hidden) return;
    float r[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < topk; ++j) {
        const int slot = token * topk + j;
        if (sh.world > 1 && !expert_is_local(selected[slot], sh)) continue;
        const float pj = probs[slot];
        const uint4 v = *reinterpret_cast<const uint4*>(vals + size_t(slot) * hidden + d0);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {   // one rounding per term, in router order
            r[2 * q] = __fmaf_rn(__uint_as_float(w[q] << 16), pj, r[2 * q]);
            r[2 * q + 1] = __fmaf_rn(__uint_as_float(w[q] & 0xffff0000u), pj, r[2 * q + 1]);
        }
    }
    if (round_output) {
#pragma unroll
        for (int k = 0; k < 8; ++k) r[k] = bf16_round_f(r[k]);
    }
    YT* out = y + size_t(token) * hidden + d0;
    if constexpr (sizeof(YT) == 4) {
        *reinterpret_cast<float4*>(out) = make_float4(r[0], r[1], r[2], r[3]);
        *reinterpret_cast<float4*>(out + 4) = make_float4(r[4], r[5], r[6], r[7]);
    } else {
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * q], r[2 * q + 1]);
            o[q] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(out) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ------------------------------------------------------------------ handle


constexpr size_t kMaxDynamicSmem = 227 * 1024;

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

MoeWorkspace moe_workspace_plan(const garnet_b200_moe_options& o, int tokens)
{
    MoeWorkspace w;
    const size_t slots = size_t(tokens) * o.top_k;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off = align_up(off + bytes, 256);
        return at;
    };
    w.logits = take(size_t(tokens) * o.experts * 4);
    w.selected = take(slots * 4);
    w.probs = take(slots * 4);
    w.xshift = take(size_t(tokens) * 4);
    w.xh = take(size_t(tokens) * o.hidden * 2);
    w.counts = take(size_t(o.experts) * 4);
    w.offsets = take(size_t(o.experts + 1) * 4);
    w.sorted = take(slots * 4);
    w.ntasks = take(4);
    w.tasks = take((slots / kMoeRows + o.experts + 1) * 16);
    // the block-scaled path's buffers exist only at sizes that use it (see Moe::use_mx)
    const int mx_world = o.ep_world > 1 ? o.ep_world : 1;
    const int mx_local = mx_world <= 1 ? o.experts   // the same count as Moe::local_experts()
                         : o.ep_interleaved ? (o.experts - o.ep_rank + mx_world - 1) / mx_world : o.experts / mx_world;
    const int mx_mode = moe_mx_mode_of(o);
    const bool mx = mx_mode == 2 || (mx_mode == 1 && slots > size_t(kMxMinRowsPerExpert) * mx_local);
    const MoeMxPlan mxp = moe_mx_plan(o, tokens, int(slots));
    w.mx_tp = take(mx ? size_t(o.experts + 1) * 4 : 0);
    w.mx_q = take(mx ? mxp.q_bytes : 0);
    w.mx_sf = take(mx ? mxp.sf_bytes : 0);
    w.act = take(slots * o.intermediate * 2);
    // The tensor-core router (more than a decode batch) leaves its partial sums where the per-slot values go
    // later: the logits are final before any expert kernel writes.
    w.vals = take(std::max(slots * o.hidden * 4, tokens > 8 ? moe_route_partial_bytes(tokens, o.experts) : size_t(0)));
    w.route_partial = w.vals;
    w.total = off;
    return w;
}

int moe_resolve_options(const garnet_b200_moe_options* in, garnet_b200_moe_options* eff)
{
    if (!in) return fail(GARNET_B200_INVALID_VALUE, "moe: null options");
    // the struct as first published ends after `limit`; later fields default to zero
    const int first_size = int(offsetof(garnet_b200_moe_options, layouts));
    if (in->abi != GARNET_B200_ABI || (in->struct_size != first_size && in->struct_size != int(sizeof(garnet_b200_moe_options))))
        return fail(GARNET_B200_INVALID_VALUE, "moe: options abi/size mismatch (abi %d, size %d)", in->abi, in->struct_size);
    garnet_b200_moe_options o{};
    std::memcpy(&o, in, size_t(in->struct_size));
    o.struct_size = int(sizeof(garnet_b200_moe_options));
    if (o.hidden <= 0 || o.intermediate <= 0 || o.experts <= 0 || o.top_k <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "moe: hidden, intermediate, experts, top_k must be positive");
    if (o.hidden % 32 || o.intermediate % 32)
        return fail(GARNET_B200_INVALID_VALUE, "moe: hidden and intermediate must be multiples of 32");
    if (o.top_k > 8 || o.top_k > o.experts)
        return fail(GARNET_B200_INVALID_VALUE, "moe: top_k must be <= 8 and <= experts");
    if (o.experts > 1024) return fail(GARNET_B200_NOT_SUPPORTED, "moe: more than 1024 experts");
    if (o.io_dtype != GARNET_B200_FP32 && o.io_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "moe: io dtype must be fp32 or bf16");
    if (!(o.limit > 0.f) || o.limit * (o.limit + 1.f) > 60000.f)
        return fail(GARNET_B200_NOT_SUPPORTED, "moe: swiglu limit %g is outside the fp16 activation range", o.limit);
    if (o.ep_world > 1) {
        if (o.ep_rank < 0 || o.ep_rank >= o.ep_world)
            return fail(GARNET_B200_INVALID_VALUE, "moe: ep_rank %d outside ep_world %d", o.ep_rank, o.ep_world);
        if (!o.ep_interleaved && o.experts % o.ep_world)
            return fail(GARNET_B200_INVALID_VALUE, "moe: experts not divisible by ep_world");
    }
    if (o.layouts < 0 || o.layouts > GARNET_B200_MOE_LAYOUT_BLOCK)
        return fail(GARNET_B200_INVALID_VALUE, "moe: layouts must be 0 (both), 1 (stream) or 2 (block)");
    if (o.tp_world > 1) {
        if (o.tp_rank < 0 || o.tp_rank >= o.tp_world)
            return fail(GARNET_B200_INVALID_VALUE, "moe: tp_rank %d outside tp_world %d", o.tp_rank, o.tp_world);
        if (o.intermediate % (32 * o.tp_world))
            return fail(GARNET_B200_INVALID_VALUE, "moe: intermediate %d does not split into %d parts of whole 32-column groups",
                        o.intermediate, o.tp_world);
        o.intermediate /= o.tp_world;   // from here on: this rank's share
    } else {
        o.tp_world = 0;
        o.tp_rank = 0;
        o.tp_weights_sharded = 0;
    }
    *eff = o;
    return GARNET_B200_OK;
}

MoeShard Moe::shard() const
{
    MoeShard s{};
    s.world = opt.ep_world > 1 ? opt.ep_world : 1;
    s.rank = s.world > 1 ? opt.ep_rank : 0;
    s.interleaved = opt.ep_interleaved;
    const int per = opt.experts / s.world;
    s.lo = s.interleaved ? 0 : s.rank * per;
    s.hi = s.interleaved ? opt.experts : s.lo + per;
    return s;
}

int Moe::local_experts() const
{
    const MoeShard s = shard();
    if (s.world <= 1) return opt.experts;
    return s.interleaved ? (opt.experts - s.rank + s.world - 1) / s.world : opt.experts / s.world;
}

Moe::~Moe()
{
    if (router_w3) cudaFree(router_w3);
    if (owns_packed) {
        for (int i = 0; i < 2; ++i)
            if (mxr_w[i]) cudaFree(mxr_w[i]);   // blocks and scale atoms are one allocation
        if (packed_up) cudaFree(packed_up);
        if (packed_down) cudaFree(packed_down);
    }
    if (own_up_bias) cudaFree(own_up_bias);
    if (zero_down_bias) cudaFree(zero_down_bias);
    if (flag_dev) cudaFree(flag_dev);
    if (fault_host) cudaFreeHost(fault_host);
}

template <bool U, bool C>
static cudaError_t set_moe_attr()
{
    return cudaFuncSetAttribute(moe_stream_kernel<U, C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                int(kMaxDynamicSmem - 1024));   // the kernel also has under 1 KB of static shared memory
}

// weights[0..7] = in[1..8] of the reference operand list (gpt_oss_lowering.cpp:309-312):
// router W, router b, gate_up blocks, gate_up scales, gate_up bias, down blocks,
// down scales, down bias.  Expert tensors hold all experts, or only this rank's
// when expert_weights_sharded is set (gpt_oss_weight_shard.h:76-92).
// Scale bytes 0 and 255 in a packed blob (either layout): see mx_scan_scales_kernel.
__global__ void mx_scan_packed_kernel(const uint8_t* __restrict__ blob, size_t count, int stream_layout, int chunk_bytes,
                                      int* flag)
{
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= count) return;
    // streaming layout: the last 32 bytes of every chunk are scales; block layout: `blob` is the atom region
    const size_t at = stream_layout ? (idx / kScaleBytesPerChunk) * chunk_bytes + (chunk_bytes - kScaleBytesPerChunk) +
                                          idx % kScaleBytesPerChunk
                                    : idx;
    if (blob[at] == 0 || blob[at] == 255) atomicOr(flag, 1);
}

int Moe::setup_common(cudaStream_t stream)
{
    GB_CUDA(cudaGetDevice(&device));
    mx_mode = moe_mx_mode_of(opt);
    geo_up = make_geom(kFormatMxfp4, 2 * opt.intermediate, opt.hidden, 32);
    geo_down = make_geom(kFormatMxfp4, opt.hidden, opt.intermediate, 32);
    stored_experts = local_experts();
    GB_CUDA(cudaMalloc(&flag_dev, 2 * sizeof(int)));   // [0]: scale bytes that need the careful decode; [1]: router CTAs done
    GB_CUDA(cudaMemsetAsync(flag_dev, 0, 2 * sizeof(int), stream));
    GB_CUDA(cudaHostAlloc(&fault_host, sizeof(int), cudaHostAllocMapped));
    *fault_host = 0;
    GB_CUDA(cudaHostGetDevicePointer(&fault_dev, fault_host, 0));
    for (int pass = 0; pass < 2; ++pass) {
        const PackGeom& geo = pass == 0 ? geo_up : geo_down;
        mx_kp[pass] = (geo.cols + kMxBlockCols - 1) / kMxBlockCols * kMxBlockCols;
        mx_kslabs[pass] = mx_kp[pass] / kMxBlockCols;
    }
    return GARNET_B200_OK;
}

int Moe::prepare(const void* const* weights, cudaStream_t stream)
{
    if (int rc = setup_common(stream)) return rc;
    const bool want_stream = opt.layouts != GARNET_B200_MOE_LAYOUT_BLOCK;
    const bool want_block = mx_mode != 0;
    if (want_stream) {
        GB_CUDA(cudaMalloc(&packed_up, geo_up.matrix_bytes() * stored_experts));
        GB_CUDA(cudaMalloc(&packed_down, geo_down.matrix_bytes() * stored_experts));
    }
    const MoeShard sh = shard();
    // source expert index of stored expert s
    auto src_expert = [&](int s) {
        if (opt.expert_weights_sharded || sh.world <= 1) return s;
        return sh.interleaved ? s * sh.world + sh.rank : sh.lo + s;
    };
    const int src_experts = opt.expert_weights_sharded ? stored_experts : opt.experts;
    const uint8_t* src_blocks[2] = {static_cast<const uint8_t*>(weights[2]), static_cast<const uint8_t*>(weights[5])};
    const uint8_t* src_scales[2] = {static_cast<const uint8_t*>(weights[3]), static_cast<const uint8_t*>(weights[6])};
    up_bias_ptr = static_cast<const float*>(weights[4]);
    down_bias_ptr = static_cast<const float*>(weights[7]);
    // Intermediate-axis split over full tensors: gather this rank's gate/up row pairs and
    // down-projection K groups first (GatherGptOssIntermediateShard modes 1 and 2,
    // gpt_oss_weight_shard.h:48-57), into temporaries that are released after the repack.
    uint8_t* gathered[4] = {nullptr, nullptr, nullptr, nullptr};
    auto free_gathered = [&] {
        for (uint8_t*& g : gathered)
            if (g) cudaFree(g), g = nullptr;
    };
    if (opt.tp_world > 1 && !opt.tp_weights_sharded) {
        const size_t il = size_t(opt.intermediate), w = size_t(opt.tp_world), r = size_t(opt.tp_rank), hd = size_t(opt.hidden);
        struct Cut { const void* src; size_t width, height; void** dst; };   // rows of `width` bytes out of rows w times as long
        void* up_bias_tmp = nullptr;
        const Cut cuts[5] = {
            {src_blocks[0], 2 * il * hd / 2, size_t(src_experts), reinterpret_cast<void**>(&gathered[0])},
            {src_scales[0], 2 * il * hd / 32, size_t(src_experts), reinterpret_cast<void**>(&gathered[1])},
            {src_blocks[1], il / 2, size_t(src_experts) * hd, reinterpret_cast<void**>(&gathered[2])},
            {src_scales[1], il / 32, size_t(src_experts) * hd, reinterpret_cast<void**>(&gathered[3])},
            {up_bias_ptr, 2 * il * 4, size_t(src_experts), &up_bias_tmp},
        };
        for (const Cut& c : cuts) {
            cudaError_t e = cudaMalloc(c.dst, c.width * c.height);
            if (e == cudaSuccess)
                e = cudaMemcpy2DAsync(*c.dst, c.width, static_cast<const uint8_t*>(c.src) + r * c.width, c.width * w, c.width,
                                      c.height, cudaMemcpyDeviceToDevice, stream);
            if (e != cudaSuccess) {
                free_gathered();
                if (up_bias_tmp) cudaFree(up_bias_tmp);
                return fail(GARNET_B200_CUDA_ERROR, "moe_create: gathering the intermediate shard failed: %s", cudaGetErrorString(e));
            }
        }
        own_up_bias = static_cast<float*>(up_bias_tmp);
        up_bias_ptr = own_up_bias;
        src_blocks[0] = gathered[0], src_scales[0] = gathered[1], src_blocks[1] = gathered[2], src_scales[1] = gathered[3];
    }
    if (opt.tp_world > 1 && opt.tp_rank != 0) {
        // the down bias is added once, by rank 0 (mode 3 of the reference's gather, :42-47)
        const size_t n = size_t(src_experts) * opt.hidden * sizeof(float);
        GB_CUDA(cudaMalloc(&zero_down_bias, n));
        GB_CUDA(cudaMemsetAsync(zero_down_bias, 0, n, stream));
        down_bias_ptr = zero_down_bias;
    }
    for (int pass = 0; pass < 2; ++pass) {
        const PackGeom& geo = pass == 0 ? geo_up : geo_down;
        const uint8_t* blocks = src_blocks[pass];
        const uint8_t* scales = src_scales[pass];
        uint8_t* dst = pass == 0 ? packed_up : packed_down;
        const size_t words = mx_stream_words(geo), nsc = mx_stream_scale_count(geo);
        const size_t blk_per_expert = size_t(geo.rows) * geo.cols / 2, sc_per_expert = size_t(geo.rows) * geo.cols / 32;
        // contiguous runs of source experts are repacked with one launch each
        int s = 0;
        while (s < stored_experts) {
            int run = 1;
            while (s + run < stored_experts && src_expert(s + run) == src_expert(s) + run) ++run;
            const size_t e0 = size_t(src_expert(s));
            if (want_stream) {
                mx_repack_codes_kernel<<<dim3(unsigned((words + 255) / 256), run), 256, 0, stream>>>(
                    blocks + e0 * blk_per_expert, dst + size_t(s) * geo.matrix_bytes(), geo, pass == 0);
                mx_repack_scales_kernel<<<dim3(unsigned((nsc + 255) / 256), run), 256, 0, stream>>>(
                    scales + e0 * sc_per_expert, dst + size_t(s) * geo.matrix_bytes(), geo, pass == 0);
            }
            const size_t cnt = size_t(run) * sc_per_expert;
            mx_scan_scales_kernel<<<unsigned((cnt + 255) / 256), 256, 0, stream>>>(scales + e0 * sc_per_expert, cnt,
                                                                                 flag_dev);
            if (want_block)
                if (int rc = init_mxr(pass, blocks + e0 * blk_per_expert, scales + e0 * sc_per_expert, s, run, stream)) {
                    free_gathered();
                    return rc;
                }
            s += run;
        }
    }
    const cudaError_t launched = cudaGetLastError();
    const cudaError_t synced = cudaStreamSynchronize(stream);
    free_gathered();
    GB_CUDA(launched);
    GB_CUDA(synced);
    router_w_ptr = static_cast<const float*>(weights[0]);
    router_b_ptr = static_cast<const float*>(weights[1]);
    return finish_prepare(stream);
}

// The operator over packed blobs that the caller owns: nothing is copied or repacked.
int Moe::prepare_prepacked(const void* const* small, const void* const* packed, cudaStream_t stream)
{
    owns_packed = false;
    if (int rc = setup_common(stream)) return rc;
    const bool want_stream = opt.layouts != GARNET_B200_MOE_LAYOUT_BLOCK;
    const bool want_block = opt.layouts != GARNET_B200_MOE_LAYOUT_STREAM;
    for (int i = 0; i < 4; ++i) {
        const bool needed = i < 2 ? want_stream : want_block;
        if (needed && !packed[i]) return fail(GARNET_B200_INVALID_VALUE, "moe_create_prepacked: packed blob %d is null", i);
        if (needed && (reinterpret_cast<uintptr_t>(packed[i]) & 255))
            return fail(GARNET_B200_INVALID_VALUE, "moe_create_prepacked: packed blob %d must be 256-byte aligned", i);
    }
    if (want_stream) {
        packed_up = static_cast<uint8_t*>(const_cast<void*>(packed[0]));
        packed_down = static_cast<uint8_t*>(const_cast<void*>(packed[1]));
    }
    for (int pass = 0; pass < 2; ++pass) {
        const PackGeom& geo = pass == 0 ? geo_up : geo_down;
        const MxBlockGeom g = make_block_geom(geo.rows, geo.cols);
        if (want_block) {
            mxr_w[pass] = static_cast<uint8_t*>(const_cast<void*>(packed[2 + pass]));
            mxr_sf[pass] = mxr_w[pass] + size_t(stored_experts) * g.code_bytes();
            mxr_ntiles[pass] = g.ntiles;
        }
        // the streaming kernels decode scale bytes 0 and 255 on a slower path: find out whether there are any
        if (want_stream) {
            const size_t cnt = size_t(stored_experts) * geo.strips_padded * geo.chunks * kScaleBytesPerChunk;
            mx_scan_packed_kernel<<<unsigned((cnt + 255) / 256), 256, 0, stream>>>(pass == 0 ? packed_up : packed_down, cnt, 1,
                                                                                  geo.chunk_bytes, flag_dev);
        }
    }
    GB_CUDA(cudaGetLastError());
    router_w_ptr = static_cast<const float*>(small[0]);
    router_b_ptr = static_cast<const float*>(small[1]);
    up_bias_ptr = static_cast<const float*>(small[2]);
    down_bias_ptr = static_cast<const float*>(small[3]);
    if (opt.tp_world > 1 && opt.tp_rank != 0) {
        const size_t n = size_t(stored_experts) * opt.hidden * sizeof(float);
        GB_CUDA(cudaMalloc(&zero_down_bias, n));
        GB_CUDA(cudaMemsetAsync(zero_down_bias, 0, n, stream));
        down_bias_ptr = zero_down_bias;
    }
    return finish_prepare(stream);
}

int Moe::finish_prepare(cudaStream_t stream)
{
    int flag = 0;
    GB_CUDA(cudaMemcpyAsync(&flag, flag_dev, sizeof(int), cudaMemcpyDeviceToHost, stream));
    GB_CUDA(cudaStreamSynchronize(stream));
    careful_scales = flag != 0;
    if (mxr_w[0])
        if (int rc = finish_mx()) return rc;
    if (int rc = init_route_mma(stream)) return rc;
    GB_CUDA(cudaStreamSynchronize(stream));
    if (!packed_up && !mx_ok)
        return fail(GARNET_B200_NOT_SUPPORTED, "moe: the block-scaled layout alone was asked for, but this shape or driver does not support it");
    // the router kernels also have a little static shared memory: leave room for it
    GB_CUDA(cudaFuncSetAttribute(moe_route_small_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(kMaxDynamicSmem - 8192)));
    GB_CUDA(cudaFuncSetAttribute(moe_route_small_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(kMaxDynamicSmem - 8192)));
    GB_CUDA(cudaFuncSetAttribute(moe_route_scores_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(kMaxDynamicSmem - 1024)));
    GB_CUDA(cudaFuncSetAttribute(moe_route_scores_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(kMaxDynamicSmem - 1024)));
    GB_CUDA((set_moe_attr<true, true>()));
    GB_CUDA((set_moe_attr<true, false>()));
    GB_CUDA((set_moe_attr<false, true>()));
    GB_CUDA((set_moe_attr<false, false>()));
    return GARNET_B200_OK;
}

// Launch with (or without) the programmatic-dependent-launch attribute.  Kernels
// launched with it execute griddepcontrol.wait before they touch anything an
// earlier kernel produced.
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              bool pdl, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

int Moe::route(const void* x, float* logits, int* selected, float* probs, __half* xh, int* xshift, int tokens,
               cudaStream_t stream, bool skip_topk, float* route_partial, int* counts, const void* small_meta)
{
    SmallMeta mt{};   // no bookkeeping unless the caller (run, at most 8 tokens) hands its lists over
    if (small_meta) mt = *static_cast<const SmallMeta*>(small_meta);
    const size_t smem = size_t(kRouteTokens) * opt.hidden * sizeof(float);
    if (smem > kMaxDynamicSmem - 8192) return fail(GARNET_B200_NOT_SUPPORTED, "moe_route: hidden too large");
    // spread the experts over enough CTAs to fill the machine at small token counts
    const int token_ctas = (tokens + kRouteTokens - 1) / kRouteTokens;
    int per_cta = opt.experts;
    while (per_cta > 4 * kRouteWarps && token_ctas * ((opt.experts + per_cta - 1) / per_cta) < 2 * kSmCount) per_cta = (per_cta + 1) / 2;
    per_cta = std::max(per_cta, std::min(opt.experts, 4));
    const dim3 grid(token_ctas, (opt.experts + per_cta - 1) / per_cta);
    if (route_partial && route_mma_ok && tokens > kRouteTokens) {
        // more than a decode batch: tensor-core router; the streaming expert kernel (not the block-scaled one,
        // which quantises the rows itself) also wants the fp16 row copies
        const bool want_xh = xh && !use_mx(tokens * opt.top_k);
        if (!skip_topk && opt.experts <= 256 && opt.top_k <= 8) {
            // one more launch: the ranges' sum, the top k, the rows per expert and the fp16 row copies
            if (int rc = route_mma(x, logits, route_partial, tokens, stream, false)) return rc;
            if (counts) GB_CUDA(cudaMemsetAsync(counts, 0, size_t(opt.experts) * sizeof(int), stream));
            const unsigned blocks = unsigned((size_t(tokens) * 32 + 255) / 256);
            const int splits = moe_route_splits(tokens, opt.experts);
            if (opt.io_dtype == GARNET_B200_FP32)
                moe_route_finish_topk_kernel<float><<<blocks, 256, 0, stream>>>(
                    route_partial, splits, router_b_ptr, logits, selected, probs, counts, shard(), static_cast<const float*>(x),
                    want_xh ? xh : nullptr, xshift, tokens, opt.hidden, opt.experts, opt.top_k);
            else
                moe_route_finish_topk_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
                    route_partial, splits, router_b_ptr, logits, selected, probs, counts, shard(),
                    static_cast<const __nv_bfloat16*>(x), want_xh ? xh : nullptr, xshift, tokens, opt.hidden, opt.experts, opt.top_k);
            GB_CUDA(cudaGetLastError());
            return GARNET_B200_OK;
        }
        if (int rc = route_mma(x, logits, route_partial, tokens, stream)) return rc;
        if (want_xh) {
            const unsigned blocks = unsigned((size_t(tokens) * 32 + 255) / 256);
            if (opt.io_dtype == GARNET_B200_FP32)
                moe_prep_rows_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), xh, xshift, tokens, opt.hidden);
            else
                moe_prep_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), xh, xshift,
                                                                                tokens, opt.hidden);
        }
    } else if (tokens <= kRouteTokens) {
        const unsigned ctas = unsigned(opt.experts);   // one expert per CTA
        const size_t small_smem = size_t(tokens) * opt.hidden * sizeof(float);
        if (opt.io_dtype == GARNET_B200_FP32)
            GB_CUDA(launch_pdl(moe_route_small_kernel<float>, dim3(ctas), dim3(kRouteWarps * 32), small_smem, stream, true,
                               static_cast<const float*>(x), router_w_ptr, router_b_ptr, logits, xh, xshift, tokens,
                               opt.hidden, opt.experts, mt));
        else
            GB_CUDA(launch_pdl(moe_route_small_kernel<__nv_bfloat16>, dim3(ctas), dim3(kRouteWarps * 32), small_smem, stream,
                               true, static_cast<const __nv_bfloat16*>(x), router_w_ptr, router_b_ptr, logits, xh,
                               xshift, tokens, opt.hidden, opt.experts, mt));
    } else if (opt.io_dtype == GARNET_B200_FP32) {
        moe_route_scores_kernel<float><<<grid, kRouteWarps * 32, smem, stream>>>(
            static_cast<const float*>(x), router_w_ptr, router_b_ptr, logits, xh, xshift, tokens, opt.hidden,
            opt.experts, per_cta);
    } else {
        moe_route_scores_kernel<__nv_bfloat16><<<grid, kRouteWarps * 32, smem, stream>>>(
            static_cast<const __nv_bfloat16*>(x), router_w_ptr, router_b_ptr, logits, xh, xshift, tokens,
            opt.hidden, opt.experts, per_cta);
    }
    if (!skip_topk) {
        if (counts) GB_CUDA(cudaMemsetAsync(counts, 0, size_t(opt.experts) * sizeof(int), stream));
        moe_topk_kernel<<<(tokens * 32 + 255) / 256, 256, 0, stream>>>(logits, selected, probs, tokens, opt.experts,
                                                                     opt.top_k, counts, shard());
    }
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int Moe::launch_stream(bool up, const MoeWorkspacePtrs& w, int tokens, cudaStream_t stream, int topk)
{
    if (topk <= 0) topk = opt.top_k;
    const PackGeom& geo = up ? geo_up : geo_down;
    const MoeShard sh = shard();
    MoeStreamParams p;
    p.packed = up ? packed_up : packed_down;
    p.act_in = up ? w.xh : w.act;
    p.xshift = up ? w.xshift : nullptr;
    p.tasks = w.tasks;
    p.ntasks = w.ntasks;
    p.sorted = w.sorted;
    p.bias = up ? up_bias_ptr : down_bias_ptr;
    p.act_out = w.act;
    p.vals_out = w.vals;
    p.vals_bf16 = w.vals_bf16;
    p.fault = fault_dev;
    p.k = geo.cols;
    p.rows = geo.rows;
    p.strips = geo.strips;
    p.chunks = geo.chunks;
    p.topk = topk;
    // stored expert index of global expert e; biases follow the same indexing as
    // the expert tensors the caller handed over
    p.expert_base = (sh.world > 1 && !sh.interleaved) ? sh.lo : (sh.world > 1 ? sh.rank : 0);
    p.expert_div = (sh.world > 1 && sh.interleaved) ? sh.world : 1;
    p.limit = opt.limit;
    p.matrix_bytes = geo.matrix_bytes();
    p.bias_by_global = (!opt.expert_weights_sharded && sh.world > 1) ? 1 : 0;
    // The down launch always follows the gate/up launch of the same call directly.
    p.tasks_early = up ? 0 : 1;
    p.slots = tokens * topk;
    p.tasks_cap = p.slots / kMoeRows + opt.experts + 1;   // as sized in moe_workspace_plan

    const size_t smem = size_t(moe_smem_plan().total);
    const int ctas_per_sm = kMoeCtasPerSm;   // as the kernel's launch bounds say
    // upper bound of (task, strip) items: every slot its own task
    const long long max_items = (long long)tokens * topk * geo.strips;
    const long long grid = std::max<long long>(1, std::min<long long>(max_items, (long long)kSmCount * ctas_per_sm));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(kMoeWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (up && careful_scales) GB_CUDA(cudaLaunchKernelEx(&cfg, moe_stream_kernel<true, true>, p));
    else if (up) GB_CUDA(cudaLaunchKernelEx(&cfg, moe_stream_kernel<true, false>, p));
    else if (careful_scales) GB_CUDA(cudaLaunchKernelEx(&cfg, moe_stream_kernel<false, true>, p));
    else GB_CUDA(cudaLaunchKernelEx(&cfg, moe_stream_kernel<false, false>, p));
    return GARNET_B200_OK;
}

// The kernels read and write rows with 16-byte vector accesses.
static bool misaligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }
// Row counts above this are rejected before any size arithmetic (2^24 rows of the
// largest supported width still fit the 64-bit byte counts used below).
constexpr int kMoeMaxRows = 1 << 24;

int Moe::run(const void* x, void* y, void* ws, size_t ws_bytes, int tokens, cudaStream_t stream)
{
    if (tokens <= 0 || tokens > kMoeMaxRows / opt.top_k)
        return fail(GARNET_B200_INVALID_VALUE, "moe_run: tokens must be in 1..%d (got %d)", kMoeMaxRows / opt.top_k, tokens);
    if (!x || !y || !ws) return fail(GARNET_B200_INVALID_VALUE, "moe_run: null pointer");
    if (misaligned16(x) || misaligned16(y)) return fail(GARNET_B200_INVALID_VALUE, "moe_run: x and y must be 16-byte aligned");
    {
        int dev = -1;
        GB_CUDA(cudaGetDevice(&dev));
        if (dev != device) return fail(GARNET_B200_INVALID_VALUE, "moe_run: the handle was created on device %d, the current device is %d", device, dev);
    }
    const MoeWorkspace plan = moe_workspace_plan(opt, tokens);
    if (ws_bytes < plan.total) return fail(GARNET_B200_INVALID_VALUE, "moe_run: workspace too small (%zu < %zu)", ws_bytes, plan.total);
    if (reinterpret_cast<uintptr_t>(ws) & 255) return fail(GARNET_B200_INVALID_VALUE, "moe_run: workspace must be 256-byte aligned");
    uint8_t* b = static_cast<uint8_t*>(ws);
    MoeWorkspacePtrs w;
    w.logits = reinterpret_cast<float*>(b + plan.logits);
    w.selected = reinterpret_cast<int*>(b + plan.selected);
    w.probs = reinterpret_cast<float*>(b + plan.probs);
    w.xshift = reinterpret_cast<int*>(b + plan.xshift);
    w.xh = reinterpret_cast<__half*>(b + plan.xh);
    w.counts = reinterpret_cast<int*>(b + plan.counts);
    w.offsets = reinterpret_cast<int*>(b + plan.offsets);
    w.sorted = reinterpret_cast<int*>(b + plan.sorted);
    w.ntasks = reinterpret_cast<int*>(b + plan.ntasks);
    w.tasks = reinterpret_cast<int4*>(b + plan.tasks);
    w.mx_tp = reinterpret_cast<int*>(b + plan.mx_tp);
    w.mx_q = b + plan.mx_q;
    w.mx_sf = b + plan.mx_sf;
    w.route_partial = reinterpret_cast<float*>(b + plan.route_partial);
    w.act = reinterpret_cast<__half*>(b + plan.act);
    w.vals = reinterpret_cast<float*>(b + plan.vals);
    w.vals_bf16 = 1;   // between this call's own kernels the per-slot values (bf16-valued) travel as bf16

    const int slots = tokens * opt.top_k;
    const MoeShard sh = shard();
    const bool small = tokens <= 8 && opt.experts <= 256;
    const int tile_rows = use_mx(slots) ? moe_mx_plan(opt, tokens, slots).nt : 0;
    SmallMeta mt{};
    if (small) {
        // at most 8 tokens: the router kernel's last CTA also selects, counts and builds the lists
        mt.selected = w.selected, mt.probs = w.probs, mt.counts = w.counts, mt.offsets = w.offsets, mt.sorted = w.sorted;
        mt.tasks = w.tasks, mt.ntasks = w.ntasks, mt.tile_prefix = w.mx_tp;
        mt.done = reinterpret_cast<unsigned*>(flag_dev + 1);
        mt.topk = opt.top_k, mt.rows_per_task = kMoeRows, mt.tile_rows = tile_rows, mt.sh = sh;
    }
    if (int rc = route(x, w.logits, w.selected, w.probs, w.xh, w.xshift, tokens, stream, small, w.route_partial, w.counts,
                       small ? &mt : nullptr))
        return rc;
    if (!small) {
        // the counts come from the top-k kernel
        moe_fill_kernel<<<opt.experts, 1024, 0, stream>>>(w.selected, slots, w.counts, w.offsets, w.sorted, w.tasks,
                                                         w.ntasks, opt.experts, kMoeRows, sh, tile_rows, w.mx_tp);
    }
    GB_CUDA(cudaGetLastError());
    if (use_mx(slots)) {
        if (int rc = launch_mx(true, w, x, 0, tokens, slots, opt.top_k, stream)) return rc;
        if (int rc = launch_mx(false, w, x, 0, tokens, slots, opt.top_k, stream)) return rc;
    } else {
#ifdef GB_MOE_PROBE
        // timing build only: leave launches out (the results are then meaningless) to read each one's share of a call
        static const int probe_skip = getenv("GB_MOE_SKIP") ? atoi(getenv("GB_MOE_SKIP")) : 0;
        if (!(probe_skip & 2))
#endif
        if (int rc = launch_stream(true, w, tokens, stream)) return rc;
#ifdef GB_MOE_PROBE
        if (!(probe_skip & 4))
#endif
        if (int rc = launch_stream(false, w, tokens, stream)) return rc;
#ifdef GB_MOE_PROBE
        if (probe_skip & 8) return GARNET_B200_OK;
#endif
    }
    const int round_output = partial_output() ? 0 : 1;
    const bool streamed = true;   // both expert paths end in kernels that support a programmatic dependent launch
    const __nv_bfloat16* vals16 = reinterpret_cast<const __nv_bfloat16*>(w.vals);
    const dim3 cgrid(unsigned(tokens), unsigned((opt.hidden + 2047) / 2048));
    if (opt.io_dtype == GARNET_B200_FP32)
        GB_CUDA(launch_pdl(moe_combine_rows_kernel<float>, cgrid, dim3(256), 0, stream, streamed, vals16, (const float*)w.probs,
                           (const int*)w.selected, static_cast<float*>(y), opt.hidden, opt.top_k, sh, round_output));
    else
        GB_CUDA(launch_pdl(moe_combine_rows_kernel<__nv_bfloat16>, cgrid, dim3(256), 0, stream, streamed, vals16,
                           (const float*)w.probs, (const int*)w.selected, static_cast<__nv_bfloat16*>(y), opt.hidden, opt.top_k, sh,
                           round_output));
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

static MoeWorkspacePtrs bind_workspace(void* ws, const MoeWorkspace& plan)
{
    uint8_t* b = static_cast<uint8_t*>(ws);
    MoeWorkspacePtrs w;
    w.logits = reinterpret_cast<float*>(b + plan.logits);
    w.selected = reinterpret_cast<int*>(b + plan.selected);
    w.probs = reinterpret_cast<float*>(b + plan.probs);
    w.xshift = reinterpret_cast<int*>(b + plan.xshift);
    w.xh = reinterpret_cast<__half*>(b + plan.xh);
    w.counts = reinterpret_cast<int*>(b + plan.counts);
    w.offsets = reinterpret_cast<int*>(b + plan.offsets);
    w.sorted = reinterpret_cast<int*>(b + plan.sorted);
    w.ntasks = reinterpret_cast<int*>(b + plan.ntasks);
    w.tasks = reinterpret_cast<int4*>(b + plan.tasks);
    w.mx_tp = reinterpret_cast<int*>(b + plan.mx_tp);
    w.mx_q = b + plan.mx_q;
    w.mx_sf = b + plan.mx_sf;
    w.route_partial = reinterpret_cast<float*>(b + plan.route_partial);
    w.act = reinterpret_cast<__half*>(b + plan.act);
    w.vals = reinterpret_cast<float*>(b + plan.vals);
    return w;
}

// Workspace plan of run_rows: every row is one routed slot (top_k = 1); the
// per-slot values go straight to the caller's buffer, so that region is empty.
MoeWorkspace moe_rows_workspace_plan(const garnet_b200_moe_options& o, int rows)
{
    garnet_b200_moe_options one = o;
    one.top_k = 1;
    one.experts = o.experts;
    MoeWorkspace plan = moe_workspace_plan(one, rows);
    plan.total = plan.vals;   // vals is the last region
    return plan;
}

// Experts only, on rows that have already been routed (and, in an expert-parallel
// run, already exchanged): row r goes through expert row_expert[r];
// vals[r, :] = bf(bf(h . w_down) + bd), unweighted.  Rows of experts that this
// handle does not hold are skipped (their vals are left untouched).
// `stage`: 0 = both projections (x_rows -> vals); 1 = gate/up + SwiGLU only (x_rows ->
// hidden_io [rows, intermediate] fp32); 2 = down projection only (hidden_io -> vals).
int Moe::run_rows(const void* x_rows, const int* row_expert, int rows, float* vals, void* ws, size_t ws_bytes,
                  cudaStream_t stream, int stage, float* hidden_io)
{
    if (rows <= 0 || rows > kMoeMaxRows) return fail(GARNET_B200_INVALID_VALUE, "moe_run_rows: rows must be in 1..%d (got %d)", kMoeMaxRows, rows);
    if (!row_expert || !ws || (stage != 2 && !x_rows) || (stage != 1 && !vals) || (stage != 0 && !hidden_io))
        return fail(GARNET_B200_INVALID_VALUE, "moe_run_rows: null pointer");
    if (misaligned16(x_rows) || misaligned16(vals) || misaligned16(hidden_io) || (reinterpret_cast<uintptr_t>(row_expert) & 3))
        return fail(GARNET_B200_INVALID_VALUE, "moe_run_rows: rows and values must be 16-byte aligned");
    const MoeWorkspace plan = moe_rows_workspace_plan(opt, rows);
    if (ws_bytes < plan.total) return fail(GARNET_B200_INVALID_VALUE, "moe_run_rows: workspace too small (%zu < %zu)", ws_bytes, plan.total);
    if (reinterpret_cast<uintptr_t>(ws) & 255) return fail(GARNET_B200_INVALID_VALUE, "moe_run_rows: workspace must be 256-byte aligned");
    MoeWorkspacePtrs w = bind_workspace(ws, plan);
    w.vals = vals;
    const bool mx = use_mx(rows);
    const unsigned blocks = unsigned((size_t(rows) * 32 + 255) / 256);
    if (mx || stage == 2) {
        // the block-scaled path quantises the rows itself and does not read the fp16 copies
    } else if (opt.io_dtype == GARNET_B200_FP32)
        moe_prep_rows_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x_rows), w.xh, w.xshift, rows, opt.hidden);
    else
        moe_prep_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x_rows), w.xh, w.xshift, rows, opt.hidden);
    const MoeShard sh = shard();
    moe_count_kernel<<<opt.experts, 256, 0, stream>>>(row_expert, rows, w.counts, sh);
    moe_fill_kernel<<<opt.experts, 1024, 0, stream>>>(row_expert, rows, w.counts, w.offsets, w.sorted, w.tasks, w.ntasks,
                                                     opt.experts, kMoeRows, sh, mx ? moe_mx_plan(opt, rows, rows).nt : 0, w.mx_tp);
    GB_CUDA(cudaGetLastError());
    if (stage != 2) {
        if (int rc = mx ? launch_mx(true, w, x_rows, 0, rows, rows, 1, stream) : launch_stream(true, w, rows, stream, 1)) return rc;
    }
    if (stage == 1) {
        moe_act_to_rows_kernel<<<rows, 128, 0, stream>>>(w.act, w.sorted, w.offsets, opt.experts, opt.intermediate, mx ? 1 : 0,
                                                        hidden_io);
        GB_CUDA(cudaGetLastError());
        return GARNET_B200_OK;
    }
    if (stage == 2) {
        moe_rows_to_act_kernel<<<rows, 128, 0, stream>>>(hidden_io, w.sorted, w.offsets, opt.experts, opt.intermediate, mx ? 1 : 0,
                                                        w.act);
        GB_CUDA(cudaGetLastError());
    }
    return mx ? launch_mx(false, w, x_rows, 0, rows, rows, 1, stream) : launch_stream(false, w, rows, stream, 1);
}

// y[t, :] = bf(sum_j vals[t*k + j, :] * probs[t, j]) in router order, all slots.
int Moe::combine(const float* vals, const float* probs, void* y, int tokens, cudaStream_t stream)
{
    if (tokens <= 0 || tokens > kMoeMaxRows / opt.top_k || !vals || !probs || !y) return fail(GARNET_B200_INVALID_VALUE, "moe_combine: bad argument");
    if (misaligned16(vals) || misaligned16(y) || (reinterpret_cast<uintptr_t>(probs) & 3))
        return fail(GARNET_B200_INVALID_VALUE, "moe_combine: values and y must be 16-byte aligned");
    MoeShard all{};
    all.world = 1;
    if (opt.io_dtype == GARNET_B200_FP32)
        moe_combine_kernel<float><<<dim3(unsigned(tokens), unsigned((opt.hidden + 255) / 256)), 256, 0, stream>>>(
            vals, probs, nullptr, static_cast<float*>(y), tokens, opt.hidden, opt.top_k, all, 1);
    else
        moe_combine_kernel<__nv_bfloat16><<<dim3(unsigned(tokens), unsigned((opt.hidden + 255) / 256)), 256, 0, stream>>>(
            vals, probs, nullptr, static_cast<__nv_bfloat16*>(y), tokens, opt.hidden, opt.top_k, all, 1);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

// ------------------------------------------- built-in scratch (no allocation)

// Scratch for garnet_b200_moe_run_static().  It lives in the library image: every
// GPU that loads the library holds these 8 MiB until the process exits.  The
// name below is only a host-side stand-in for the array; the device address is
// looked up once per device with cudaGetSymbolAddress and handed to the kernels.
constexpr size_t kMoeStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_moe_static_scratch[kMoeStaticScratchBytes];

constexpr int kMaxDevices = 64;

// Device address of the built-in scratch on the current device.  The first call
// on a device performs the symbol lookup (with that device current); it is made from
// garnet_b200_moe_create, so that garnet_b200_moe_run_static itself never does it.
int moe_static_scratch(void** out)
{
    static std::mutex mu;
    static void* address[kMaxDevices] = {};
    int dev = 0;
    GB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(GARNET_B200_NOT_SUPPORTED, "moe_run_static: device index %d", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!address[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_moe_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "moe_run_static: cudaGetSymbolAddress");
        if (!p) return fail(GARNET_B200_CUDA_ERROR, "moe_run_static: scratch symbol has no device address");
        address[dev] = p;
    }
    *out = address[dev];
    return GARNET_B200_OK;
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_moe_run_static(garnet_b200_moe_t hh, const void* d_x, void* d_y, int tokens, void* stream)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "moe_run_static: null handle");
    if (tokens <= 0) return fail(GARNET_B200_INVALID_VALUE, "moe_run_static: tokens must be positive");
    if (tokens > kMoeMaxRows / h->opt.top_k)
        return fail(GARNET_B200_INVALID_VALUE, "moe_run_static: %d tokens is far beyond what the built-in scratch holds", tokens);
    const size_t need = moe_workspace_plan(h->opt, tokens).total;
    if (need > kMoeStaticScratchBytes) {
        // the plan grows with the token count: bisect for the largest count that fits
        int lo = 0, hi = tokens;   // fits(lo), !fits(hi)
        while (hi - lo > 1) {
            const int mid = lo + (hi - lo) / 2;
            if (moe_workspace_plan(h->opt, mid).total <= kMoeStaticScratchBytes) lo = mid;
            else hi = mid;
        }
        return fail(GARNET_B200_INVALID_VALUE,
                    "moe_run_static: %d tokens need %zu bytes of scratch but the built-in array holds %zu "
                    "(at most %d tokens for this layer); use garnet_b200_moe_run with a caller workspace",
                    tokens, need, kMoeStaticScratchBytes, lo);
    }
    void* scratch = h->static_scratch;   // looked up when the handle was created, on the handle's device
    if (!scratch) return fail(GARNET_B200_CUDA_ERROR, "moe_run_static: the handle has no scratch address");
    // Nothing in the scratch has to start at zero: every region the kernels read
    // (logits, routing, counts, slot lists, activations, per-slot values) is fully
    // written earlier in the same call for the slots that are read.
    return h->run(d_x, d_y, scratch, kMoeStaticScratchBytes, tokens, static_cast<cudaStream_t>(stream));
}

int garnet_b200_mxfp4_decode(const uint8_t* d_blocks, const uint8_t* d_scales, float* d_out, int rows, void* stream)
{
    if (!d_blocks || !d_scales || !d_out || rows <= 0) return fail(GARNET_B200_INVALID_VALUE, "mxfp4_decode: bad argument");
    mx_decode_rows_kernel<<<(rows * 4 + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_blocks, d_scales,
                                                                                                d_out, rows);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_moe_workspace(const garnet_b200_moe_options* o, int tokens, size_t* bytes)
{
    garnet_b200_moe_options eff;
    if (int rc = moe_resolve_options(o, &eff)) return rc;
    if (!bytes || tokens <= 0) return fail(GARNET_B200_INVALID_VALUE, "moe_workspace: bad argument");
    *bytes = moe_workspace_plan(eff, tokens).total;
    return GARNET_B200_OK;
}

int garnet_b200_moe_create(const garnet_b200_moe_options* o, const void* const* weights, void* stream,
                           garnet_b200_moe_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "moe_create: null output handle");
    *out = nullptr;
    garnet_b200_moe_options eff;
    if (int rc = moe_resolve_options(o, &eff)) return rc;
    if (!weights) return fail(GARNET_B200_INVALID_VALUE, "moe_create: null weight list");
    for (int i = 0; i < 8; ++i)
        if (!weights[i]) return fail(GARNET_B200_INVALID_VALUE, "moe_create: weight operand %d is null", i + 1);
    Moe* h = new (std::nothrow) Moe();
    if (!h) return fail(GARNET_B200_OUT_OF_MEMORY, "moe_create: host allocation failed");
    h->opt = eff;
    int rc = h->prepare(weights, static_cast<cudaStream_t>(stream));
    // the address of the built-in scratch of garnet_b200_moe_run_static, so that no run call looks it up
    if (!rc) rc = moe_static_scratch(&h->static_scratch);
    if (rc) {
        delete h;
        return rc;
    }
    *out = reinterpret_cast<garnet_b200_moe_t>(h);
    return GARNET_B200_OK;
}

int garnet_b200_moe_create_prepacked(const garnet_b200_moe_options* o, const void* const* small, const void* const* packed,
                                     void* stream, garnet_b200_moe_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "moe_create_prepacked: null output handle");
    *out = nullptr;
    garnet_b200_moe_options eff;
    if (int rc = moe_resolve_options(o, &eff)) return rc;
    if (!small || !packed) return fail(GARNET_B200_INVALID_VALUE, "moe_create_prepacked: null operand list");
    for (int i = 0; i < 4; ++i)
        if (!small[i]) return fail(GARNET_B200_INVALID_VALUE, "moe_create_prepacked: small operand %d is null", i);
    Moe* h = new (std::nothrow) Moe();
    if (!h) return fail(GARNET_B200_OUT_OF_MEMORY, "moe_create_prepacked: host allocation failed");
    h->opt = eff;
    int rc = h->prepare_prepacked(small, packed, static_cast<cudaStream_t>(stream));
    if (!rc) rc = moe_static_scratch(&h->static_scratch);
    if (rc) {
        delete h;
        return rc;
    }
    *out = reinterpret_cast<garnet_b200_moe_t>(h);
    return GARNET_B200_OK;
}

int garnet_b200_moe_packed_view(garnet_b200_moe_t hh, int which, int layout, const void** d_blob, size_t* bytes)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h || !d_blob || !bytes || which < 0 || which > 1)
        return fail(GARNET_B200_INVALID_VALUE, "moe_packed_view: bad argument");
    const PackGeom& geo = which == 0 ? h->geo_up : h->geo_down;
    if (layout == GARNET_B200_MOE_LAYOUT_STREAM) {
        const uint8_t* p = which == 0 ? h->packed_up : h->packed_down;
        if (!p) return fail(GARNET_B200_NOT_SUPPORTED, "moe_packed_view: this handle does not hold the streaming layout");
        *d_blob = p;
        *bytes = geo.matrix_bytes() * size_t(h->stored_experts);
        return GARNET_B200_OK;
    }
    if (layout == GARNET_B200_MOE_LAYOUT_BLOCK) {
        if (!h->mxr_w[which]) return fail(GARNET_B200_NOT_SUPPORTED, "moe_packed_view: this handle does not hold the block layout");
        const MxBlockGeom g = make_block_geom(geo.rows, geo.cols);
        *d_blob = h->mxr_w[which];
        *bytes = size_t(h->stored_experts) * (g.code_bytes() + g.atom_bytes());
        return GARNET_B200_OK;
    }
    return fail(GARNET_B200_INVALID_VALUE, "moe_packed_view: layout must be 1 (stream) or 2 (block)");
}

int garnet_b200_moe_run(garnet_b200_moe_t hh, const void* d_x, void* d_y, void* d_workspace, size_t workspace_bytes,
                        int tokens, void* stream)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "moe_run: null handle");
    return h->run(d_x, d_y, d_workspace, workspace_bytes, tokens, static_cast<cudaStream_t>(stream));
}

int garnet_b200_moe_rows_workspace(const garnet_b200_moe_options* o, int rows, size_t* bytes)
{
    garnet_b200_moe_options eff;
    if (int rc = moe_resolve_options(o, &eff)) return rc;
    if (!bytes || rows <= 0) return fail(GARNET_B200_INVALID_VALUE, "moe_rows_workspace: bad argument");
    *bytes = moe_rows_workspace_plan(eff, rows).total;
    return GARNET_B200_OK;
}

int garnet_b200_moe_run_rows(garnet_b200_moe_t hh, const void* d_rows, const int* d_row_expert, int rows,
                             float* d_vals, void* d_workspace, size_t workspace_bytes, void* stream)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "moe_run_rows: null handle");
    return h->run_rows(d_rows, d_row_expert, rows, d_vals, d_workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int garnet_b200_moe_run_rows_stage(garnet_b200_moe_t hh, int stage, const void* d_rows, const int* d_row_expert, int rows,
                                   float* d_hidden, float* d_vals, void* d_workspace, size_t workspace_bytes, void* stream)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "moe_run_rows_stage: null handle");
    if (stage != 1 && stage != 2) return fail(GARNET_B200_INVALID_VALUE, "moe_run_rows_stage: stage must be 1 or 2");
    return h->run_rows(d_rows, d_row_expert, rows, d_vals, d_workspace, workspace_bytes, static_cast<cudaStream_t>(stream), stage,
                       d_hidden);
}

int garnet_b200_moe_combine(garnet_b200_moe_t hh, const float* d_vals, const float* d_probs, void* d_y, int tokens,
                            void* stream)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "moe_combine: null handle");
    return h->combine(d_vals, d_probs, d_y, tokens, static_cast<cudaStream_t>(stream));
}

int garnet_b200_moe_route(garnet_b200_moe_t hh, const void* d_x, int* d_selected, float* d_probs, float* d_logits,
                          int tokens, void* stream)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "moe_route: null handle");
    if (!d_x || !d_selected || !d_probs || !d_logits || tokens <= 0 || tokens > kMoeMaxRows / h->opt.top_k)
        return fail(GARNET_B200_INVALID_VALUE, "moe_route: bad argument");
    if (misaligned16(d_x) || ((reinterpret_cast<uintptr_t>(d_selected) | reinterpret_cast<uintptr_t>(d_probs) | reinterpret_cast<uintptr_t>(d_logits)) & 3))
        return fail(GARNET_B200_INVALID_VALUE, "moe_route: x must be 16-byte aligned");
    return h->route(d_x, d_logits, d_selected, d_probs, nullptr, nullptr, tokens, static_cast<cudaStream_t>(stream));
}

int garnet_b200_moe_route_workspace(const garnet_b200_moe_options* o, int tokens, size_t* bytes)
{
    garnet_b200_moe_options eff;
    if (int rc = moe_resolve_options(o, &eff)) return rc;
    if (!bytes || tokens <= 0 || tokens > kMoeMaxRows / o->top_k) return fail(GARNET_B200_INVALID_VALUE, "moe_route_workspace: bad argument");
    *bytes = std::max<size_t>(256, moe_route_partial_bytes(tokens, o->experts));
    return GARNET_B200_OK;
}

int garnet_b200_moe_route_ws(garnet_b200_moe_t hh, const void* d_x, int* d_selected, float* d_probs, float* d_logits,
                             int tokens, void* d_workspace, size_t workspace_bytes, void* stream)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "moe_route_ws: null handle");
    if (!d_x || !d_selected || !d_probs || !d_logits || !d_workspace || tokens <= 0 || tokens > kMoeMaxRows / h->opt.top_k)
        return fail(GARNET_B200_INVALID_VALUE, "moe_route_ws: bad argument");
    if (misaligned16(d_x) || (reinterpret_cast<uintptr_t>(d_workspace) & 255) ||
        ((reinterpret_cast<uintptr_t>(d_selected) | reinterpret_cast<uintptr_t>(d_probs) | reinterpret_cast<uintptr_t>(d_logits)) & 3))
        return fail(GARNET_B200_INVALID_VALUE, "moe_route_ws: x must be 16-byte and the workspace 256-byte aligned");
    if (workspace_bytes < moe_route_partial_need(tokens, h->opt.experts))
        return fail(GARNET_B200_INVALID_VALUE, "moe_route_ws: workspace too small");
    // the same call the one-call operator makes: identical logits, selection and probabilities
    return h->route(d_x, d_logits, d_selected, d_probs, nullptr, nullptr, tokens, static_cast<cudaStream_t>(stream), false,
                    static_cast<float*>(d_workspace), nullptr);
}

int garnet_b200_moe_dequant(garnet_b200_moe_t hh, int which, int stored_expert, float* d_out, void* stream)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    if (!h || !d_out || stored_expert < 0 || stored_expert >= h->stored_experts || which < 0 || which > 3)
        return fail(GARNET_B200_INVALID_VALUE, "moe_dequant: bad argument");
    if (which >= 2) return h->dequant_block_scaled(which - 2, stored_expert, d_out, static_cast<cudaStream_t>(stream));
    if (!h->packed_up) return fail(GARNET_B200_NOT_SUPPORTED, "moe_dequant: this handle does not hold the streaming layout");
    const PackGeom& geo = which == 0 ? h->geo_up : h->geo_down;
    const size_t total = size_t(geo.rows) * geo.cols / 2;
    mx_dequant_kernel<<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        which == 0 ? h->packed_up : h->packed_down, d_out, geo, which == 0, stored_expert);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_moe_fault(garnet_b200_moe_t hh)
{
    Moe* h = reinterpret_cast<Moe*>(hh);
    return h && h->fault_host ? *h->fault_host : -1;
}

void garnet_b200_moe_destroy(garnet_b200_moe_t hh) { delete reinterpret_cast<Moe*>(hh); }

#ifdef GB_MOE_TRACE
int garnet_b200_moe_trace(unsigned long long* out, int n)
{
    GB_CUDA(cudaMemcpyFromSymbol(out, g_moe_trace, sizeof(unsigned long long) * size_t(n)));
    static unsigned long long zeros[96];
    GB_CUDA(cudaMemcpyToSymbol(g_moe_trace, zeros, sizeof(zeros)));
    return 0;
}
#endif

}  // extern "C"
