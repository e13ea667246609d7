// The parts of a Qwen3 decode step that sit between its int4 linears and are not folded
// into them: the attention of one new token per sequence over a paged bf16 KV cache (with
// the per-head RMS norm of q and k, the rotary embedding and the cache append folded in),
// the embedding gather and the arg-max over the logits.
//
// Reference: the packed q/k/v lowering with q/k head norm and rotate-half RoPE
// (src/backends/tensorrt/trt_builder.cpp:7565-7726, :1815-1870), the paged KV cache and
// its split ("flash") decode attention (src/cuda/text_kv_attention_kernel.cu:640-840:
// cache row ((page * page_size + offset) * kv_heads + kv_head) * head_dim, page tables per
// sequence, partial (max, sum, output) per split merged afterwards, score scale
// 1/sqrt(head_dim)), and the greedy sampler (src/cuda/logits_sampler_kernel.cu, lowest
// index wins a tie).
//
// One launch per layer instead of the reference's four (RoPE engine, cache append,
// partials, reduce): CTA (q head, split, sequence) normalises and rotates its q head,
// the CTA whose split holds the new position does the same for the new k and appends k and
// v to the cache, every CTA walks its positions with an online softmax, and the last CTA
// of a head to finish merges the splits in order.
#include <cfloat>
#include <cstdint>

#include "common.cuh"

namespace gb200 {

namespace {

constexpr int kAttnHeadDim = 128;
constexpr int kAttnWarps = 8;
constexpr int kAttnSplitPositions = 128;   // positions per split: 16 per warp, all loaded at once (one wave of CTAs at 2048 positions)
constexpr int kAttnMaxSplits = 1024;       // contexts up to 65536 positions

struct AttnParams {
    const __nv_bfloat16* qkv;       // [batch, (q_heads + 2 kv_heads) * 128]: q | k | v
    const __nv_bfloat16* q_norm_w;  // [128]
    const __nv_bfloat16* k_norm_w;  // [128]
    const float* rope_cos;          // [positions, 64]
    const float* rope_sin;
    __nv_bfloat16* key_pages;
    __nv_bfloat16* value_pages;
    const int* page_tables;         // [batch, max_logical_pages]
    const int* positions;           // [batch]: slot of the new token; the context is positions 0 .. slot
    __nv_bfloat16* out;             // [batch, q_heads * 128]
    float* part_stats;              // [batch, q_heads, splits, 2]
    float* part_out;                // [batch, q_heads, splits, 128]
    unsigned* counters;             // [batch, q_heads], zero between launches
    int q_heads, kv_heads, page_size, max_logical_pages, splits, rope_positions;
    float eps;
};

__device__ __forceinline__ float warp_sum_f(float v)
{
#pragma unroll
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ float bf16r(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

// 8-byte asynchronous copy global -> shared (no registers in between), and the wait for a thread's own copies.
__device__ __forceinline__ void cp_async_8(void* dst_smem, const void* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(uint32_t(__cvta_generic_to_shared(dst_smem))), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Per-head RMS norm (weight w) and rotate-half RoPE of one 128-wide head held as dims
// lane, lane + 32, lane + 64, lane + 96; every step rounds to bf16 as a bf16 network does.
__device__ __forceinline__ void norm_rope_head(const __nv_bfloat16* head, const __nv_bfloat16* w, const float* cs, const float* sn,
                                               float eps, int lane, float (&o)[4])
{
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __bfloat162float(head[lane + 32 * i]);
    const float ss = warp_sum_f(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
    const float rs = 1.f / sqrtf(ss / float(kAttnHeadDim) + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = bf16r(__fmul_rn(__fmul_rn(v[i], rs), __bfloat162float(w[lane + 32 * i])));
    // out[d] = x[d] cos[d] - x[d + 64] sin[d];  out[d + 64] = x[d + 64] cos[d] + x[d] sin[d]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float c = cs[lane + 32 * i], s = sn[lane + 32 * i];
        o[i] = bf16r(__fsub_rn(__fmul_rn(v[i], c), __fmul_rn(v[i + 2], s)));
        o[i + 2] = bf16r(__fadd_rn(__fmul_rn(v[i + 2], c), __fmul_rn(v[i], s)));
    }
}

__global__ void __launch_bounds__(kAttnWarps * 32) attention_decode_kernel(const AttnParams p)
{
    __shared__ float q_s[kAttnHeadDim], k_new[kAttnHeadDim], v_new[kAttnHeadDim];
    __shared__ float w_max[kAttnWarps], w_sum[kAttnWarps], w_out[kAttnWarps][kAttnHeadDim];
    __shared__ int is_last;
    const int q_head = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = p.q_heads / p.kv_heads, kv_head = q_head / group;
    const int q_width = p.q_heads * kAttnHeadDim, kv_width = p.kv_heads * kAttnHeadDim;
    pdl_launch_dependents();
    pdl_wait();   // q, k, v come from the linear before this kernel
    const __nv_bfloat16* row = p.qkv + size_t(b) * (q_width + 2 * kv_width);
    const int* table = p.page_tables + size_t(b) * p.max_logical_pages;
    // the page of every position of this warp, one lane each: asked for together with the sequence's position
    // (it does not depend on it), so that the two look-ups cost one trip
    constexpr int kPer = kAttnSplitPositions / kAttnWarps;
    int page = 0;
    {
        const int pos = split * kAttnSplitPositions + warp + lane * kAttnWarps;
        if (lane < kPer && pos / p.page_size < p.max_logical_pages) page = __ldg(&table[pos / p.page_size]);
    }
    const int slot = p.positions[b];
    const int context = slot + 1;
    const int start = split * kAttnSplitPositions, end = min(context, start + kAttnSplitPositions);
    const bool valid = slot >= 0 && slot < p.rope_positions && slot / p.page_size < p.max_logical_pages;
    const float* cs = p.rope_cos + size_t(valid ? slot : 0) * (kAttnHeadDim / 2);
    const float* sn = p.rope_sin + size_t(valid ? slot : 0) * (kAttnHeadDim / 2);
    const bool holds_new = valid && slot >= start && slot < end;

    // A warp owns positions start + warp, + 8, ...: one per cache page of 16 when the pages are that size.  All
    // their rows are requested before the first is used, so the walk costs one trip to memory - as asynchronous
    // copies into shared memory issued from a loop, not as an unrolled run of loads into registers: this kernel
    // runs once per CTA, every instruction of it is fetched cold, and the unrolled form (sixteen address
    // computations, thirty-two loads, sixteen score steps) spent longer being fetched than running.
    extern __shared__ __align__(16) uint8_t kv_rows[];   // [warp][K, V][kPer][256 bytes]
    uint8_t* my_k = kv_rows + size_t(warp) * (2 * kPer * kAttnHeadDim * 2);
    uint8_t* my_v = my_k + kPer * kAttnHeadDim * 2;
    if (valid) {
#pragma unroll 1
        for (int u = 0; u < kPer; ++u) {
            const int pos = start + warp + u * kAttnWarps;
            const int pg = __shfl_sync(0xffffffffu, page, u);
            if (pos < end && pos != slot) {
                const size_t at = ((size_t(pg) * p.page_size + pos % p.page_size) * p.kv_heads + kv_head) * kAttnHeadDim;
                cp_async_8(my_k + u * (kAttnHeadDim * 2) + lane * 8, reinterpret_cast<const uint2*>(p.key_pages + at) + lane);
                cp_async_8(my_v + u * (kAttnHeadDim * 2) + lane * 8, reinterpret_cast<const uint2*>(p.value_pages + at) + lane);
            }
        }
        cp_async_commit();
    }

    if (warp == 0) {
        float o[4];
        norm_rope_head(row + q_head * kAttnHeadDim, p.q_norm_w, cs, sn, p.eps, lane, o);
#pragma unroll
        for (int i = 0; i < 4; ++i) q_s[lane + 32 * i] = o[i];
    } else if (warp == 1 && holds_new) {
        float o[4];
        norm_rope_head(row + q_width + kv_head * kAttnHeadDim, p.k_norm_w, cs, sn, p.eps, lane, o);
        const __nv_bfloat16* v_row = row + q_width + kv_width + kv_head * kAttnHeadDim;
        const size_t at = ((size_t(table[slot / p.page_size]) * p.page_size + slot % p.page_size) * p.kv_heads + kv_head) * kAttnHeadDim;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = lane + 32 * i;
            k_new[d] = o[i];
            v_new[d] = __bfloat162float(v_row[d]);
            if (q_head % group == 0) {   // one CTA per kv head appends to the cache
                p.key_pages[at + d] = __float2bfloat16_rn(o[i]);
                p.value_pages[at + d] = v_row[d];
            }
        }
    }
    __syncthreads();

    // ---- this warp's positions: dims 4 lane .. 4 lane + 3 of every row (8 bytes per lane)
    float qv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) qv[i] = q_s[4 * lane + i];
    const float scale = 0.08838834764831845f;   // 1 / sqrt(128)
    float run_max = -FLT_MAX, run_sum = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (valid) {
        cp_async_wait_all();   // a lane reads back only the bytes it copied itself
#pragma unroll 1
        for (int u = 0; u < kPer; ++u) {
            const int pos = start + warp + u * kAttnWarps;
            if (pos >= end) break;
            float kf[4], vf[4];
            if (pos == slot) {   // the new token's row is not read back from the cache
#pragma unroll
                for (int i = 0; i < 4; ++i) kf[i] = k_new[4 * lane + i], vf[i] = v_new[4 * lane + i];
            } else {
                const uint2 kr = *reinterpret_cast<const uint2*>(my_k + u * (kAttnHeadDim * 2) + lane * 8);
                const uint2 vr = *reinterpret_cast<const uint2*>(my_v + u * (kAttnHeadDim * 2) + lane * 8);
                kf[0] = __uint_as_float(kr.x << 16), kf[1] = __uint_as_float(kr.x & 0xffff0000u);
                kf[2] = __uint_as_float(kr.y << 16), kf[3] = __uint_as_float(kr.y & 0xffff0000u);
                vf[0] = __uint_as_float(vr.x << 16), vf[1] = __uint_as_float(vr.x & 0xffff0000u);
                vf[2] = __uint_as_float(vr.y << 16), vf[3] = __uint_as_float(vr.y & 0xffff0000u);
            }
            const float score = warp_sum_f(qv[0] * kf[0] + qv[1] * kf[1] + qv[2] * kf[2] + qv[3] * kf[3]) * scale;
            const float next_max = fmaxf(run_max, score);
            const float prev = run_sum == 0.f ? 0.f : __expf(run_max - next_max);
            const float wgt = __expf(score - next_max);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = acc[i] * prev + wgt * vf[i];
            run_sum = run_sum * prev + wgt;
            run_max = next_max;
        }
    }
    if (lane == 0) w_max[warp] = run_max, w_sum[warp] = run_sum;
#pragma unroll
    for (int i = 0; i < 4; ++i) w_out[warp][4 * lane + i] = acc[i];
    __syncthreads();

    // ---- the split's partial result, warps merged in order
    const size_t head_index = size_t(b) * p.q_heads + q_head;
    if (threadIdx.x < kAttnHeadDim) {
        const int d = threadIdx.x;
        float s_max = -FLT_MAX;
        for (int w = 0; w < kAttnWarps; ++w)
            if (w_sum[w] > 0.f) s_max = fmaxf(s_max, w_max[w]);
        float s_sum = 0.f, s_out = 0.f;
        for (int w = 0; w < kAttnWarps; ++w) {
            if (w_sum[w] <= 0.f) continue;
            const float m = __expf(w_max[w] - s_max);
            s_sum += m * w_sum[w];
            s_out += m * w_out[w][d];
        }
        const size_t si = head_index * p.splits + split;
        if (d == 0) p.part_stats[si * 2] = s_max, p.part_stats[si * 2 + 1] = s_sum;
        p.part_out[si * kAttnHeadDim + d] = s_out;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(&p.counters[head_index], 1u) == unsigned(p.splits) - 1u;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // ---- merge of the splits, in split order.  The statistics are fetched by one thread per split and the
    // partial outputs without a condition on them, so that the loads overlap instead of queueing behind one another.
    __shared__ float m_max[kAttnMaxSplits], m_sum[kAttnMaxSplits];
    for (int s = threadIdx.x; s < p.splits; s += blockDim.x) {
        m_max[s] = __ldcg(&p.part_stats[(head_index * p.splits + s) * 2]);
        m_sum[s] = __ldcg(&p.part_stats[(head_index * p.splits + s) * 2 + 1]);
    }
    __syncthreads();
    if (threadIdx.x < kAttnHeadDim) {
        const int d = threadIdx.x;
        float t_max = -FLT_MAX;
        for (int s = 0; s < p.splits; ++s)
            if (m_sum[s] > 0.f) t_max = fmaxf(t_max, m_max[s]);
        float t_sum = 0.f, t_out = 0.f;
        const float* po = p.part_out + head_index * p.splits * kAttnHeadDim + d;
        for (int s0 = 0; s0 < p.splits; s0 += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = s0 + u < p.splits ? __ldcg(po + size_t(s0 + u) * kAttnHeadDim) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int s = s0 + u;
                if (s >= p.splits || m_sum[s] <= 0.f) continue;
                const float m = __expf(m_max[s] - t_max);
                t_sum += m * m_sum[s];
                t_out += m * v[u];
            }
        }
        p.out[size_t(b) * q_width + q_head * kAttnHeadDim + d] = __float2bfloat16_rn(t_sum > 0.f ? t_out / t_sum : 0.f);
    }
    if (threadIdx.x == 0) p.counters[head_index] = 0;   // ready for the next launch
}

__global__ void embedding_gather_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                        __nv_bfloat16* __restrict__ out, int hidden, int vocab)
{
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    int id = ids[b];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(table + size_t(id) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + size_t(b) * hidden);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// One CTA per row; the largest value wins, the lowest index among equals; NaN never wins.
__global__ void __launch_bounds__(1024) argmax_bf16_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out, int vocab)
{
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_launch_dependents();
    pdl_wait();
    const __nv_bfloat16* row = logits + size_t(blockIdx.x) * vocab;
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = __bfloat162float(row[i]);
        if (v > best || (v == best && i < arg)) best = v, arg = i;
    }
    auto merge = [&](float ov, int oa) {
        if (ov > best || (ov == best && oa < arg)) best = ov, arg = oa;
    };
#pragma unroll
    for (int off = 16; off; off >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, off), __shfl_xor_sync(0xffffffffu, arg, off));
    if ((threadIdx.x & 31) == 0) s_val[threadIdx.x >> 5] = best, s_idx[threadIdx.x >> 5] = arg;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? s_val[threadIdx.x] : -INFINITY;
        arg = threadIdx.x < (blockDim.x >> 5) ? s_idx[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int off = 16; off; off >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, off), __shfl_xor_sync(0xffffffffu, arg, off));
        if (threadIdx.x == 0) out[blockIdx.x] = arg == 0x7fffffff ? 0 : arg;
    }
}

int attention_splits(const garnet_b200_attention_options& o) { return (o.max_context + kAttnSplitPositions - 1) / kAttnSplitPositions; }

int validate_attention(const garnet_b200_attention_options* o)
{
    if (!o) return fail(GARNET_B200_INVALID_VALUE, "attention: null options");
    if (o->abi != GARNET_B200_ABI || o->struct_size != int(sizeof(garnet_b200_attention_options)))
        return fail(GARNET_B200_INVALID_VALUE, "attention: options abi/size mismatch (abi %d, size %d)", o->abi, o->struct_size);
    if (o->head_dim != kAttnHeadDim) return fail(GARNET_B200_NOT_SUPPORTED, "attention: head_dim must be %d", kAttnHeadDim);
    if (o->q_heads <= 0 || o->kv_heads <= 0 || o->q_heads % o->kv_heads)
        return fail(GARNET_B200_INVALID_VALUE, "attention: q_heads must be a positive multiple of kv_heads");
    if (o->page_size <= 0 || o->max_logical_pages <= 0 || o->max_context <= 0 || o->rope_positions <= 0 || !(o->norm_eps > 0.f))
        return fail(GARNET_B200_INVALID_VALUE, "attention: page_size, max_logical_pages, max_context, rope_positions and norm_eps must be positive");
    if (o->max_context > kAttnMaxSplits * kAttnSplitPositions)
        return fail(GARNET_B200_NOT_SUPPORTED, "attention: max_context above %d", kAttnMaxSplits * kAttnSplitPositions);
    if (o->max_context > o->max_logical_pages * o->page_size || o->max_context > o->rope_positions)
        return fail(GARNET_B200_INVALID_VALUE, "attention: max_context exceeds the page table or the rope tables");
    return GARNET_B200_OK;
}

size_t attention_workspace(const garnet_b200_attention_options& o, int batch)
{
    const size_t heads = size_t(batch) * o.q_heads, splits = size_t(attention_splits(o));
    return 256 + ((heads * 4 + 255) & ~size_t(255)) + heads * splits * (2 + kAttnHeadDim) * 4;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_with_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, bool pdl, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_attention_decode_workspace(const garnet_b200_attention_options* o, int batch, size_t* bytes)
{
    if (int rc = validate_attention(o)) return rc;
    if (!bytes || batch <= 0) return fail(GARNET_B200_INVALID_VALUE, "attention_decode_workspace: bad argument");
    *bytes = attention_workspace(*o, batch);
    return GARNET_B200_OK;
}

int garnet_b200_attention_decode(const garnet_b200_attention_options* o, const void* d_qkv, const void* d_q_norm_weight,
                                 const void* d_k_norm_weight, const float* d_rope_cos, const float* d_rope_sin, void* d_key_pages,
                                 void* d_value_pages, const int* d_page_tables, const int* d_positions, void* d_out,
                                 void* d_workspace, size_t workspace_bytes, int batch, unsigned flags, void* stream)
{
    if (int rc = validate_attention(o)) return rc;
    if (!d_qkv || !d_q_norm_weight || !d_k_norm_weight || !d_rope_cos || !d_rope_sin || !d_key_pages || !d_value_pages ||
        !d_page_tables || !d_positions || !d_out || !d_workspace || batch <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "attention_decode: null pointer or bad batch");
    if (workspace_bytes < attention_workspace(*o, batch))
        return fail(GARNET_B200_INVALID_VALUE, "attention_decode: workspace too small (%zu < %zu)", workspace_bytes, attention_workspace(*o, batch));
    if ((reinterpret_cast<uintptr_t>(d_workspace) & 255) || (reinterpret_cast<uintptr_t>(d_key_pages) & 15) ||
        (reinterpret_cast<uintptr_t>(d_value_pages) & 15))
        return fail(GARNET_B200_INVALID_VALUE, "attention_decode: the workspace must be 256-byte and the cache pages 16-byte aligned");
    AttnParams p;
    p.qkv = static_cast<const __nv_bfloat16*>(d_qkv);
    p.q_norm_w = static_cast<const __nv_bfloat16*>(d_q_norm_weight);
    p.k_norm_w = static_cast<const __nv_bfloat16*>(d_k_norm_weight);
    p.rope_cos = d_rope_cos;
    p.rope_sin = d_rope_sin;
    p.key_pages = static_cast<__nv_bfloat16*>(d_key_pages);
    p.value_pages = static_cast<__nv_bfloat16*>(d_value_pages);
    p.page_tables = d_page_tables;
    p.positions = d_positions;
    p.out = static_cast<__nv_bfloat16*>(d_out);
    const size_t heads = size_t(batch) * o->q_heads;
    uint8_t* ws = static_cast<uint8_t*>(d_workspace);
    p.counters = reinterpret_cast<unsigned*>(ws);
    ws += (heads * 4 + 255) & ~size_t(255);
    p.splits = attention_splits(*o);
    p.part_stats = reinterpret_cast<float*>(ws);
    p.part_out = p.part_stats + heads * p.splits * 2;
    p.q_heads = o->q_heads;
    p.kv_heads = o->kv_heads;
    p.page_size = o->page_size;
    p.max_logical_pages = o->max_logical_pages;
    p.rope_positions = o->rope_positions;
    p.eps = o->norm_eps;
    {
        constexpr int kRowsBytes = kAttnWarps * 2 * (kAttnSplitPositions / kAttnWarps) * kAttnHeadDim * 2;   // 64 KB
        static bool attr_set[64] = {};
        int dev = 0;
        GB_CUDA(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            GB_CUDA(cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRowsBytes));
            attr_set[dev] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(o->q_heads), unsigned(p.splits), unsigned(batch));
        cfg.blockDim = dim3(kAttnWarps * 32);
        cfg.dynamicSmemBytes = kRowsBytes;
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = (flags & 1u) ? 1 : 0;
        GB_CUDA(cudaLaunchKernelEx(&cfg, attention_decode_kernel, p));
    }
    return GARNET_B200_OK;
}

int garnet_b200_embedding_gather(const void* d_table, const int* d_ids, void* d_out, int batch, int hidden, int vocab,
                                 unsigned flags, void* stream)
{
    if (!d_table || !d_ids || !d_out || batch <= 0 || hidden <= 0 || vocab <= 0 || (hidden % 8))
        return fail(GARNET_B200_INVALID_VALUE, "embedding_gather: bad argument (hidden must be a multiple of 8)");
    if ((reinterpret_cast<uintptr_t>(d_table) | reinterpret_cast<uintptr_t>(d_out)) & 15)
        return fail(GARNET_B200_INVALID_VALUE, "embedding_gather: table and output must be 16-byte aligned");
    GB_CUDA(launch_with_pdl(embedding_gather_kernel, dim3(unsigned(batch)), dim3(256), static_cast<cudaStream_t>(stream),
                            (flags & 1u) != 0, static_cast<const __nv_bfloat16*>(d_table), d_ids, static_cast<__nv_bfloat16*>(d_out),
                            hidden, vocab));
    return GARNET_B200_OK;
}

int garnet_b200_argmax_bf16(const void* d_logits, int* d_out, int batch, int vocab, unsigned flags, void* stream)
{
    if (!d_logits || !d_out || batch <= 0 || vocab <= 0) return fail(GARNET_B200_INVALID_VALUE, "argmax_bf16: bad argument");
    GB_CUDA(launch_with_pdl(argmax_bf16_kernel, dim3(unsigned(batch)), dim3(1024), static_cast<cudaStream_t>(stream),
                            (flags & 1u) != 0, static_cast<const __nv_bfloat16*>(d_logits), d_out, vocab));
    return GARNET_B200_OK;
}

}  // extern "C"
