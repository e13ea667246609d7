// The rest of a gpt-oss decoder layer around the MoE operator: RMS norm, YaRN rotary
// embedding, paged-KV attention with learned sinks and a sliding window, the bf16 GEMV of the
// q/k/v and output projections at decode, and the per-rank (score, token) pair of the sharded
// vocabulary.  x and y use the reference's fp32 carrier (fp32 tensors that hold bf16 values).
//
// Reference (plugins/gpt_oss/cuda/gpt_oss_kernels.cu): rmsNorm :22-48, rope :78-99,
// cacheOffset / writeKV :100-123, attention :125-160 (one warp per query head, the sink enters the
// softmax denominator only), decodeAttentionPartial / Merge :376-428,:513-535, vocabTop1 :430-455,
// the entry points RunGptOssRmsNorm / Rope / Attention / VocabTop1 :930-1210; decodeGemv
// (plugins/gpt_oss/cuda/gpt_oss_gemv.cu:7-39).
//
// Decode attention here: one CTA per (kv head, 64-position split, sequence) stages the split's K
// and V rows in shared memory once and serves all the q heads of the group from them (the
// reference's default path reads them once per q head); the last CTA of a (sequence, kv head)
// merges the splits and the sink.  With a sliding window of 128 a layer needs two splits.
#include <cfloat>
#include <cstdint>

#include "common.cuh"

namespace gb200 {

namespace {

__device__ __forceinline__ float bfr(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int off = 16; off; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// y = bf((bf(x) * rsqrt(mean(bf(x)^2) + eps)) * w), one CTA per row.
__global__ void __launch_bounds__(256) oss_rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                                                           int hidden, float eps)
{
    __shared__ float part[8];
    const float* xr = x + size_t(blockIdx.x) * hidden;
    float sum = 0.f;
    for (int d = threadIdx.x; d < hidden; d += 256) {
        const float v = bfr(xr[d]);
        sum += v * v;
    }
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sum;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += part[i];
    const float inv = rsqrtf(total / hidden + eps);
    for (int d = threadIdx.x; d < hidden; d += 256) y[size_t(blockIdx.x) * hidden + d] = bfr((bfr(xr[d]) * inv) * w[d]);
}

struct OssRope {
    int q_heads, kv_heads, head_dim;
    float theta, factor, initial_context, beta_fast, beta_slow;
};

// One thread per (token, rotated head, frequency): the pair (d, d + half) shares its angle.
__global__ void oss_rope_kernel(const float* __restrict__ x, const long long* __restrict__ positions, float* __restrict__ y, int tokens,
                                OssRope o)
{
    const int half = o.head_dim / 2, rot_heads = o.q_heads + o.kv_heads;
    const int packed = (o.q_heads + 2 * o.kv_heads) * o.head_dim;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t pairs = size_t(tokens) * rot_heads * half;
    if (idx < pairs) {
        const int frequency = int(idx % half), head = int((idx / half) % rot_heads), token = int(idx / (size_t(half) * rot_heads));
        const float pi = 3.14159265358979323846f;
        float inv = powf(o.theta, -2.f * frequency / o.head_dim), concentration = 1;
        if (o.factor > 1) {
            const float low = half * logf(o.initial_context / (o.beta_fast * 2 * pi)) / logf(o.theta);
            const float high = half * logf(o.initial_context / (o.beta_slow * 2 * pi)) / logf(o.theta);
            const float ramp = fminf(1, fmaxf(0, (frequency - low) / (high - low)));
            inv *= (1 - ramp) + ramp / o.factor;
            concentration = 1 + .1f * logf(o.factor);
        }
        const float angle = float(positions[token]) * inv;
        const float cosine = bfr(cosf(angle) * concentration), sine = bfr(sinf(angle) * concentration);
        const size_t at = size_t(token) * packed + size_t(head) * o.head_dim + frequency;
        const float a = x[at], b = x[at + half];
        y[at] = bfr(bfr(a * cosine) + bfr(-b * sine));
        y[at + half] = bfr(bfr(b * cosine) + bfr(a * sine));
    }
    // the v part passes through
    const size_t vcount = size_t(tokens) * o.kv_heads * o.head_dim;
    for (size_t i = idx; i < vcount; i += size_t(gridDim.x) * blockDim.x) {
        const size_t token = i / (size_t(o.kv_heads) * o.head_dim), c = i % (size_t(o.kv_heads) * o.head_dim);
        const size_t at = token * packed + size_t(rot_heads) * o.head_dim + c;
        y[at] = x[at];
    }
}

struct OssAttn {
    const float* qkv;             // [batch * tokens, (q + 2 kv) * d], already rotated
    __nv_bfloat16* keys;          // [layers][physical pages][page size][kv heads][d]
    __nv_bfloat16* values;
    const int* table;             // [batch, logical pages]
    const int* lengths;           // [batch]: positions visible at decode
    const int* starts;            // [batch]: position of the first new token
    const int* active;            // [batch]
    const float* sinks;           // [q heads]
    float* out;                   // [batch * tokens, q * d]
    float* part;                  // [batch, q heads, splits, 2 + d]
    unsigned* counters;           // [batch, kv heads]
    int batch, tokens, logical_pages, physical_pages;
    int q_heads, kv_heads, head_dim, layer, page_size, window, prefill, splits;
};

__device__ __forceinline__ size_t oss_cache_offset(const OssAttn& p, int b, int position, int head)
{
    if (position < 0 || position / p.page_size >= p.logical_pages) return SIZE_MAX;
    const int page = p.table[b * p.logical_pages + position / p.page_size];
    if (page < 0 || page >= p.physical_pages) return SIZE_MAX;
    return (((size_t(p.layer) * p.physical_pages + page) * p.page_size + position % p.page_size) * p.kv_heads + head) * p.head_dim;
}

__global__ void oss_write_kv_kernel(const OssAttn p)
{
    const int kv_width = p.kv_heads * p.head_dim, packed = (p.q_heads + 2 * p.kv_heads) * p.head_dim;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= size_t(p.batch) * p.tokens * kv_width) return;
    const int row = int(idx / kv_width), b = row / p.tokens, t = row % p.tokens, d = int(idx % kv_width);
    if (!p.active[b]) return;
    const size_t off = oss_cache_offset(p, b, p.starts[b] + t, d / p.head_dim);
    if (off == SIZE_MAX) return;
    p.keys[off + d % p.head_dim] = __float2bfloat16(p.qkv[size_t(row) * packed + p.q_heads * p.head_dim + d]);
    p.values[off + d % p.head_dim] = __float2bfloat16(p.qkv[size_t(row) * packed + (p.q_heads + p.kv_heads) * p.head_dim + d]);
}

// Any shape: one warp per (row, q head), online softmax in position order (the reference's baseline).
__global__ void oss_attention_generic_kernel(const OssAttn p)
{
    const int lane = threadIdx.x & 31;
    const int task = int((size_t(blockIdx.x) * blockDim.x + threadIdx.x) / 32);
    if (task >= p.batch * p.tokens * p.q_heads) return;
    const int head = task % p.q_heads, row = task / p.q_heads, b = row / p.tokens, t = row % p.tokens;
    const int packed = (p.q_heads + 2 * p.kv_heads) * p.head_dim;
    float accum[8] = {};
    const int end = p.prefill ? p.starts[b] + t + 1 : p.lengths[b];
    const int begin = p.window ? max(0, end - p.window) : 0;
    float maximum = p.sinks[head], sum = 1;
    const float* q = p.qkv + size_t(row) * packed + head * p.head_dim;
    if (p.active[b] && end > 0 && end <= p.logical_pages * p.page_size) {
        for (int pos = begin; pos < end; ++pos) {
            const size_t off = oss_cache_offset(p, b, pos, head / (p.q_heads / p.kv_heads));
            if (off == SIZE_MAX) continue;
            float score = 0;
            for (int d = lane; d < p.head_dim; d += 32) score += q[d] * __bfloat162float(p.keys[off + d]);
            score = warp_sum(score) * rsqrtf(float(p.head_dim));
            const float next = fmaxf(maximum, score);
            const float old = expf(maximum - next), weight = expf(score - next);
            sum = sum * old + weight;
            for (int d = lane, i = 0; d < p.head_dim; d += 32, ++i) accum[i] = accum[i] * old + weight * __bfloat162float(p.values[off + d]);
            maximum = next;
        }
    }
    for (int d = lane, i = 0; d < p.head_dim; d += 32, ++i)
        p.out[size_t(row) * p.q_heads * p.head_dim + head * p.head_dim + d] = bfr(accum[i] / sum);
}

constexpr int kOssSplit = 64;      // positions per split
constexpr int kOssDim = 64;        // head dimension of the grouped decode kernel
constexpr int kOssRowStride = 68;  // halves per staged row: 136 bytes (8-byte aligned), two-way bank conflicts at most

// Decode (one new token per sequence), head_dim 64: CTA (kv head, split, sequence); warp g serves q head kv * group + g.
__global__ void __launch_bounds__(512) oss_attention_decode_kernel(const OssAttn p)
{
    __shared__ __align__(16) __nv_bfloat16 ks[kOssSplit * kOssRowStride], vs[kOssSplit * kOssRowStride];
    __shared__ float qs[16][kOssDim];
    __shared__ unsigned char row_ok[kOssSplit];   // the row's page exists (looked up once, while staging)
    __shared__ int s_last;
    const int kv = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group = p.q_heads / p.kv_heads;
    const int head = kv * group + warp;
    const int packed = (p.q_heads + 2 * p.kv_heads) * kOssDim;
    const int end = p.lengths[b];
    const bool live = p.active[b] && end > 0 && end <= p.logical_pages * p.page_size;
    const int begin = p.window ? max(0, end - p.window) : 0;
    const int s0 = begin + split * kOssSplit, s1 = live ? min(end, s0 + kOssSplit) : s0;
    const int rows = max(0, s1 - s0);
    // ---- stage the split's K and V rows: 8 pieces of 16 bytes per row and tensor
    for (int i = threadIdx.x; i < rows * 16; i += blockDim.x) {
        const int r = i >> 4, piece = i & 7, is_v = (i >> 3) & 1;
        const size_t off = oss_cache_offset(p, b, s0 + r, kv);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (off != SIZE_MAX) v = __ldcg(reinterpret_cast<const uint4*>((is_v ? p.values : p.keys) + off) + piece);
        if ((i & 15) == 0) row_ok[r] = off != SIZE_MAX;
        // a staged row starts on an 8-byte boundary (136-byte rows): two 8-byte stores
        uint2* dst = reinterpret_cast<uint2*>((is_v ? vs : ks) + r * kOssRowStride + piece * 8);
        dst[0] = make_uint2(v.x, v.y);
        dst[1] = make_uint2(v.z, v.w);
    }
    {
        const float* qg = p.qkv + size_t(b) * packed + head * kOssDim;
        qs[warp][lane] = qg[lane];
        qs[warp][lane + 32] = qg[lane + 32];
    }
    __syncthreads();
    const float* q = qs[warp];
    const float scale = rsqrtf(float(kOssDim));
    // ---- scores: lane owns rows lane and lane + 32
    float sc[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int r = lane + 32 * u;
        float s = -FLT_MAX;
        if (r < rows && row_ok[r]) {
            float acc = 0.f;
            const __nv_bfloat162* kr = reinterpret_cast<const __nv_bfloat162*>(ks + r * kOssRowStride);
#pragma unroll 8
            for (int d = 0; d < kOssDim / 2; ++d) {
                const float2 kk = __bfloat1622float2(kr[d]);
                acc += q[2 * d] * kk.x + q[2 * d + 1] * kk.y;
            }
            s = acc * scale;
        }
        sc[u] = s;
    }
    const float m = warp_max(fmaxf(sc[0], sc[1]));
    float w[2], out0 = 0.f, out1 = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u) w[u] = sc[u] > -FLT_MAX ? __expf(sc[u] - m) : 0.f;
    const float total = warp_sum(w[0] + w[1]);
    // ---- weighted values: lane owns dims 2 lane, 2 lane + 1
    for (int r = 0; r < rows; ++r) {
        const float wr = __shfl_sync(0xffffffffu, w[r >> 5], r & 31);
        const float2 vv = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(vs + r * kOssRowStride)[lane]);
        out0 += wr * vv.x;
        out1 += wr * vv.y;
    }
    const size_t pi = ((size_t(b) * p.q_heads + head) * p.splits + split) * (2 + kOssDim);
    if (warp < group) {
        if (lane == 0) p.part[pi] = total > 0.f ? m : -FLT_MAX, p.part[pi + 1] = total;
        p.part[pi + 2 + 2 * lane] = out0;
        p.part[pi + 3 + 2 * lane] = out1;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&p.counters[b * p.kv_heads + kv], 1u) == unsigned(p.splits) - 1u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // ---- merge the splits of this group's heads, and the sink (denominator only)
    if (warp < group) {
        const size_t hb = (size_t(b) * p.q_heads + head) * p.splits * (2 + kOssDim);
        float mx = p.sinks[head];
        for (int s = lane; s < p.splits; s += 32) {   // both values requested at once
            const float pmax = __ldcg(&p.part[hb + size_t(s) * (2 + kOssDim)]), psum = __ldcg(&p.part[hb + size_t(s) * (2 + kOssDim) + 1]);
            if (psum > 0.f) mx = fmaxf(mx, pmax);
        }
        mx = warp_max(mx);
        float sum = __expf(p.sinks[head] - mx), o0 = 0.f, o1 = 0.f;
        // eight splits' values are requested together, without a condition on them, so that the loads overlap
        // instead of queueing behind one another (the order of the additions stays the order of the splits)
        for (int sb = 0; sb < p.splits; sb += 8) {
            float pm[8], psum[8], po0[8], po1[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool in = sb + u < p.splits;
                const float* ps = p.part + hb + size_t(in ? sb + u : sb) * (2 + kOssDim);
                pm[u] = __ldcg(ps), psum[u] = in ? __ldcg(ps + 1) : 0.f;
                po0[u] = __ldcg(ps + 2 + 2 * lane), po1[u] = __ldcg(ps + 3 + 2 * lane);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (psum[u] <= 0.f) continue;
                const float f = __expf(pm[u] - mx);
                sum += f * psum[u];
                o0 += f * po0[u];
                o1 += f * po1[u];
            }
        }
        float* o = p.out + size_t(b) * p.q_heads * kOssDim + head * kOssDim;
        o[2 * lane] = bfr(live ? o0 / sum : 0.f);
        o[2 * lane + 1] = bfr(live ? o1 / sum : 0.f);
    }
    if (threadIdx.x == 0) p.counters[b * p.kv_heads + kv] = 0;
}

__global__ void __launch_bounds__(256) oss_vocab_top1_kernel(const float* __restrict__ logits, float* __restrict__ pairs, int width, int rank)
{
    __shared__ float s_val[8];
    __shared__ int s_idx[8];
    const float* row = logits + size_t(blockIdx.x) * width;
    float best = -FLT_MAX;
    int arg = 0;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = row[i];
        if (v > best || (v == best && i < arg)) best = v, arg = i;
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
        if (ov > best || (ov == best && oa < arg)) best = ov, arg = oa;
    }
    if ((threadIdx.x & 31) == 0) s_val[threadIdx.x >> 5] = best, s_idx[threadIdx.x >> 5] = arg;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i)
            if (s_val[i] > best || (s_val[i] == best && s_idx[i] < arg)) best = s_val[i], arg = s_idx[i];
        pairs[size_t(blockIdx.x) * 2] = best;
        pairs[size_t(blockIdx.x) * 2 + 1] = float(rank * width + arg);
    }
}

// y[row] = bf16(sum_c w[weight_row(row), offset + c] * x[c]); one warp per row, 16-byte loads.
__global__ void __launch_bounds__(128) oss_gemv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                       __nv_bfloat16* __restrict__ y, int rows, int columns, int stride, int offset,
                                                       int q_heads, int kv_heads, int head_dim, int rank)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= rows) return;
    int wr = row;
    if (q_heads > 0) {   // this rank's half of the q, k and v rows of a packed q/k/v weight
        const int qp = (q_heads / 2) * head_dim, kp = (kv_heads / 2) * head_dim;
        wr = row < qp ? rank * qp + row : row < qp + kp ? q_heads * head_dim + rank * kp + row - qp : (q_heads + kv_heads) * head_dim + rank * kp + row - qp - kp;
    }
    const __nv_bfloat16* v = w + size_t(wr) * stride + offset;
    float sum = 0.f;
    if ((((reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) && columns % 8 == 0) {
        for (int c = lane * 8; c < columns; c += 256) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(v + c)), bx = __ldg(reinterpret_cast<const uint4*>(x + c));
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {bx.x, bx.y, bx.z, bx.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                sum = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), sum);
                sum = fmaf(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(bw[i] & 0xffff0000u), sum);
            }
        }
    } else {
        for (int c = lane; c < columns; c += 32) sum = fmaf(__bfloat162float(v[c]), __bfloat162float(x[c]), sum);
    }
    sum = warp_sum(sum);
    if (lane == 0) y[row] = __float2bfloat16_rn(sum);
}

int validate_oss(const garnet_b200_gpt_oss_options* o, bool attention)
{
    if (!o) return fail(GARNET_B200_INVALID_VALUE, "gpt_oss: null options");
    if (o->abi != GARNET_B200_ABI || o->struct_size != int(sizeof(garnet_b200_gpt_oss_options)))
        return fail(GARNET_B200_INVALID_VALUE, "gpt_oss: options abi/size mismatch (abi %d, size %d)", o->abi, o->struct_size);
    if (o->q_heads <= 0 || o->kv_heads <= 0 || o->q_heads % o->kv_heads || o->head_dim <= 0 || o->head_dim % 2 || o->head_dim > 256)
        return fail(GARNET_B200_INVALID_VALUE, "gpt_oss: bad head geometry");
    if (attention && (o->page_size <= 0 || o->layer < 0 || o->window < 0))
        return fail(GARNET_B200_INVALID_VALUE, "gpt_oss: page_size must be positive, layer and window non-negative");
    return GARNET_B200_OK;
}

int oss_splits(const garnet_b200_gpt_oss_options& o, int logical_pages)
{
    const int span = o.window ? std::min(o.window, logical_pages * o.page_size) : logical_pages * o.page_size;
    return std::max(1, (span + kOssSplit - 1) / kOssSplit);
}

size_t oss_workspace(const garnet_b200_gpt_oss_options& o, int batch, int logical_pages)
{
    const size_t counters = (size_t(batch) * o.kv_heads * 4 + 255) & ~size_t(255);
    return counters + size_t(batch) * o.q_heads * oss_splits(o, logical_pages) * (2 + kOssDim) * 4;
}

}  // namespace

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_gpt_oss_rms_norm(const float* d_x, const float* d_weight, float* d_y, int rows, int hidden, float epsilon, void* stream)
{
    if (!d_x || !d_weight || !d_y || rows <= 0 || hidden <= 0 || !(epsilon > 0.f))
        return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_rms_norm: bad argument");
    oss_rms_norm_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_weight, d_y, hidden, epsilon);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_gpt_oss_rope(const garnet_b200_gpt_oss_options* o, const float* d_x, const long long* d_positions, float* d_y, int tokens,
                             void* stream)
{
    if (int rc = validate_oss(o, false)) return rc;
    if (!d_x || !d_positions || !d_y || tokens <= 0) return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_rope: bad argument");
    OssRope r{o->q_heads, o->kv_heads, o->head_dim, o->theta, o->factor, o->initial_context, o->beta_fast, o->beta_slow};
    const size_t pairs = size_t(tokens) * (o->q_heads + o->kv_heads) * (o->head_dim / 2);
    oss_rope_kernel<<<unsigned((pairs + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_positions, d_y, tokens, r);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_gpt_oss_attention_workspace(const garnet_b200_gpt_oss_options* o, int batch, int logical_pages, size_t* bytes)
{
    if (int rc = validate_oss(o, true)) return rc;
    if (!bytes || batch <= 0 || logical_pages <= 0) return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_attention_workspace: bad argument");
    *bytes = oss_workspace(*o, batch, logical_pages);
    return GARNET_B200_OK;
}

int garnet_b200_gpt_oss_attention(const garnet_b200_gpt_oss_options* o, const void* const* in, float* d_y, void* d_workspace,
                                  size_t workspace_bytes, int batch, int tokens, int logical_pages, int physical_pages, void* stream)
{
    if (int rc = validate_oss(o, true)) return rc;
    if (!in || !d_y || batch <= 0 || tokens <= 0 || logical_pages <= 0 || physical_pages <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_attention: bad argument");
    for (int i = 0; i < 8; ++i)
        if (!in[i] && i != 4) return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_attention: operand %d is null", i);
    OssAttn p;
    p.qkv = static_cast<const float*>(in[0]);
    p.keys = static_cast<__nv_bfloat16*>(const_cast<void*>(in[1]));
    p.values = static_cast<__nv_bfloat16*>(const_cast<void*>(in[2]));
    p.table = static_cast<const int*>(in[3]);
    p.lengths = static_cast<const int*>(in[4]);
    p.starts = static_cast<const int*>(in[5]);
    p.active = static_cast<const int*>(in[6]);
    p.sinks = static_cast<const float*>(in[7]);
    p.out = d_y;
    p.batch = batch, p.tokens = tokens, p.logical_pages = logical_pages, p.physical_pages = physical_pages;
    p.q_heads = o->q_heads, p.kv_heads = o->kv_heads, p.head_dim = o->head_dim, p.layer = o->layer, p.page_size = o->page_size;
    p.window = o->window, p.prefill = o->prefill;
    p.splits = oss_splits(*o, logical_pages);
    p.part = nullptr, p.counters = nullptr;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t n = size_t(batch) * tokens * o->kv_heads * o->head_dim;
    oss_write_kv_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(p);
    GB_CUDA(cudaGetLastError());
    const int group = o->q_heads / o->kv_heads;
    const bool grouped = tokens == 1 && !o->prefill && o->head_dim == kOssDim && group <= 16 && in[4] &&
                         (reinterpret_cast<uintptr_t>(in[1]) & 15) == 0 && (reinterpret_cast<uintptr_t>(in[2]) & 15) == 0;
    if (grouped) {
        if (!d_workspace || workspace_bytes < oss_workspace(*o, batch, logical_pages) || (reinterpret_cast<uintptr_t>(d_workspace) & 255))
            return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_attention: the workspace is missing, too small or not 256-byte aligned");
        uint8_t* ws = static_cast<uint8_t*>(d_workspace);
        p.counters = reinterpret_cast<unsigned*>(ws);
        p.part = reinterpret_cast<float*>(ws + ((size_t(batch) * o->kv_heads * 4 + 255) & ~size_t(255)));
        oss_attention_decode_kernel<<<dim3(unsigned(o->kv_heads), unsigned(p.splits), unsigned(batch)), std::max(group, 1) * 32, 0, s>>>(p);
    } else {
        if (!in[4] && !o->prefill) return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_attention: decode needs the lengths operand");
        if (o->head_dim > 256) return fail(GARNET_B200_NOT_SUPPORTED, "gpt_oss_attention: head_dim above 256");
        const size_t tasks = size_t(batch) * tokens * o->q_heads;
        oss_attention_generic_kernel<<<unsigned((tasks * 32 + 255) / 256), 256, 0, s>>>(p);
    }
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_gpt_oss_vocab_top1(const float* d_logits, float* d_pairs, int rows, int width, int rank, void* stream)
{
    if (!d_logits || !d_pairs || rows <= 0 || width <= 0 || width > (1 << 23) || rank < 0)
        return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_vocab_top1: bad argument");
    oss_vocab_top1_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_logits, d_pairs, width, rank);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_gpt_oss_decode_gemv(const void* d_x, const void* d_weight, void* d_y, int rows, int columns, int weight_stride,
                                    int column_offset, int q_heads, int kv_heads, int head_dim, int rank, void* stream)
{
    if (!d_x || !d_weight || !d_y || rows <= 0 || columns <= 0 || columns % 32 != 0 || weight_stride < column_offset + columns ||
        column_offset < 0 ||
        (q_heads > 0 && (rank < 0 || rank > 1 || kv_heads <= 0 || head_dim <= 0 || q_heads % 2 || kv_heads % 2 ||
                         rows != (q_heads / 2 + kv_heads) * head_dim)))
        return fail(GARNET_B200_INVALID_VALUE, "gpt_oss_decode_gemv: bad argument");
    oss_gemv_kernel<<<unsigned((rows + 3) / 4), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(d_x), static_cast<const __nv_bfloat16*>(d_weight), static_cast<__nv_bfloat16*>(d_y), rows,
        columns, weight_stride, column_offset, q_heads, kv_heads, head_dim, rank);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

}  // extern "C"
