// Router logits for many tokens on the tensor cores (mma.sync m16n8k16, bf16 in, fp32
// accumulate): logits[t, e] = bf16(sum_k bf16(x[t, k]) * W[e, k] + b[e]), the
// arithmetic of gpt_oss_moe_mxfp4's router (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:
// 776-800: fp32 dot product of the bf16-rounded row with the router weight).
//
// The router weight is fp32.  It is split once, at create time, into three bf16
// terms w = w1 + w2 + w3 (w2 = bf16(w - w1), w3 = bf16(w - w1 - w2)), which together
// carry its 24 significant bits, so that every product x * w_i is exact in fp32 and
// the only difference from a serial fp32 dot product is the order of the additions.
// 3 GFLOP at 4096 tokens of gpt-oss-120b: 281 us on the fp32 pipe before, about a
// tenth of that here.
#include <algorithm>

#include "moe.h"
#include "common.cuh"

namespace gb200 {

constexpr int kRmTokens = 64;     // tokens per CTA: 4 warps x 16 rows
constexpr int kRmExperts = 64;    // experts per CTA: 8 MMA column tiles per warp
constexpr int kRmSlab = 64;       // K per staging step
constexpr int kRmStride = kRmSlab + 8;   // halves per staged row: bank-conflict-free fragment reads
// K is cut into moe_route_splits(tokens, experts) ranges (grid z): that many times the CTAs, partial sums added
// in a fixed order.  The ranges are chosen so that the CTAs about fill the GPU once (two CTAs of this kernel fit an
// SM): few tokens make few tiles and get up to nine ranges, 4096 tokens of 128 experts get two (256 CTAs; three
// ranges made 384 CTAs, a wave and a third).
constexpr int kRmMaxSplits = 9;
int moe_route_splits(int tokens, int experts)
{
    const long long tiles = (long long)((tokens + kRmTokens - 1) / kRmTokens) * ((experts + kRmExperts - 1) / kRmExperts);
    return int(std::max<long long>(1, std::min<long long>(kRmMaxSplits, (2 * kSmCount) / tiles)));
}

__global__ void moe_router_split_kernel(const float* __restrict__ w, __nv_bfloat16* __restrict__ w3, size_t count)
{
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float v = w[i];
    const __nv_bfloat16 a = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(a);
    const __nv_bfloat16 b = __float2bfloat16_rn(r1);
    const __nv_bfloat16 c = __float2bfloat16_rn(r1 - __bfloat162float(b));
    w3[i] = a;
    w3[count + i] = b;
    w3[2 * count + i] = c;
}

template <typename XT>
__device__ __forceinline__ uint32_t rm_pack2(const XT* p);
template <>
__device__ __forceinline__ uint32_t rm_pack2<float>(const float* p)
{
    const float2 f = *reinterpret_cast<const float2*>(p);
    const __nv_bfloat162 h = __floats2bfloat162_rn(f.x, f.y);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t rm_pack2<__nv_bfloat16>(const __nv_bfloat16* p)
{
    return *reinterpret_cast<const uint32_t*>(p);
}

// grid = (token tiles, expert tiles, K ranges); 128 threads.  hidden % 64 == 0.
// partial[z][t][e] = sum over K range z.
template <typename XT>
__global__ void __launch_bounds__(128)
moe_route_mma_kernel(const XT* __restrict__ x, const __nv_bfloat16* __restrict__ w3, float* __restrict__ partial,
                     int tokens, int hidden, int experts)
{
    __shared__ __align__(16) __nv_bfloat16 xs[kRmTokens * kRmStride];
    __shared__ __align__(16) __nv_bfloat16 ws[3 * kRmExperts * kRmStride];
    pdl_launch_dependents();
    pdl_wait();   // x comes from the kernel before this one
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int t0 = blockIdx.x * kRmTokens, e0 = blockIdx.y * kRmExperts;
    const size_t wcount = size_t(experts) * hidden;
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[n][q] = 0.f;

    const int slabs = hidden / kRmSlab;
    const int k_begin = int(blockIdx.z) * slabs / int(gridDim.z) * kRmSlab, k_end = int(blockIdx.z + 1) * slabs / int(gridDim.z) * kRmSlab;
    // The next slab's global loads are issued into registers before the current slab's
    // MMAs, so that their latency is covered by the math.
    constexpr int kXPer = kRmTokens * (kRmSlab / 2) / 128;          // 16 words of x per thread
    constexpr int kWPer = 3 * kRmExperts * (kRmSlab / 8) / 128;     // 12 x 16 bytes of W per thread
    uint32_t xr[kXPer];
    uint4 wr[kWPer];
    auto load_slab = [&](int k0) {
#pragma unroll
        for (int j = 0; j < kXPer; ++j) {
            const int i = threadIdx.x + j * 128;
            const int r = i / (kRmSlab / 2), c = (i % (kRmSlab / 2)) * 2;
            xr[j] = (t0 + r < tokens) ? rm_pack2<XT>(x + size_t(t0 + r) * hidden + k0 + c) : 0u;
        }
#pragma unroll
        for (int j = 0; j < kWPer; ++j) {
            const int i = threadIdx.x + j * 128;
            const int c = (i % (kRmSlab / 8)) * 8, r = (i / (kRmSlab / 8)) % kRmExperts, s = i / ((kRmSlab / 8) * kRmExperts);
            wr[j] = (e0 + r < experts) ? *reinterpret_cast<const uint4*>(w3 + s * wcount + size_t(e0 + r) * hidden + k0 + c)
                                       : make_uint4(0, 0, 0, 0);
        }
    };
    auto store_slab = [&]() {
#pragma unroll
        for (int j = 0; j < kXPer; ++j) {
            const int i = threadIdx.x + j * 128;
            const int r = i / (kRmSlab / 2), c = (i % (kRmSlab / 2)) * 2;
            *reinterpret_cast<uint32_t*>(&xs[r * kRmStride + c]) = xr[j];
        }
#pragma unroll
        for (int j = 0; j < kWPer; ++j) {
            const int i = threadIdx.x + j * 128;
            const int c = (i % (kRmSlab / 8)) * 8, r = (i / (kRmSlab / 8)) % kRmExperts, s = i / ((kRmSlab / 8) * kRmExperts);
            *reinterpret_cast<uint4*>(&ws[(s * kRmExperts + r) * kRmStride + c]) = wr[j];
        }
    };
    if (k_begin < k_end) load_slab(k_begin);
    for (int k0 = k_begin; k0 < k_end; k0 += kRmSlab) {
        __syncthreads();      // the previous slab's MMAs have read the staging buffers
        store_slab();
        __syncthreads();
        if (k0 + kRmSlab < k_end) load_slab(k0 + kRmSlab);
#pragma unroll
        for (int kk = 0; kk < kRmSlab; kk += 16) {
            const __nv_bfloat16* xa = xs + (warp * 16 + g) * kRmStride + kk + 2 * t;
            const uint32_t a[4] = {*reinterpret_cast<const uint32_t*>(xa), *reinterpret_cast<const uint32_t*>(xa + 8 * kRmStride),
                                   *reinterpret_cast<const uint32_t*>(xa + 8),
                                   *reinterpret_cast<const uint32_t*>(xa + 8 * kRmStride + 8)};
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int s = 0; s < 3; ++s) {
                    const __nv_bfloat16* wb = ws + (s * kRmExperts + n * 8 + g) * kRmStride + kk + 2 * t;
                    mma_bf16_16816(acc[n], a, *reinterpret_cast<const uint32_t*>(wb),
                                   *reinterpret_cast<const uint32_t*>(wb + 8), acc[n]);
                }
            }
        }
    }
    const int r0 = t0 + warp * 16 + g;
    float* out = partial + size_t(blockIdx.z) * tokens * experts;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const int e = e0 + n * 8 + 2 * t;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = r0 + 8 * h;
            if (row < tokens) {
                if (e < experts) out[size_t(row) * experts + e] = acc[n][2 * h];
                if (e + 1 < experts) out[size_t(row) * experts + e + 1] = acc[n][2 * h + 1];
            }
        }
    }
}

// logits = bf16(p0 + p1 + ... + b), the ranges added in this order.
__global__ void moe_route_finish_kernel(const float* __restrict__ partial, const float* __restrict__ rb,
                                        float* __restrict__ logits, int tokens, int experts, int splits)
{
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = size_t(tokens) * experts;
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = partial[i];
#pragma unroll
    for (int z = 1; z < splits; ++z) v += partial[z * n + i];
    logits[i] = bf16_round_f(v + rb[i % experts]);
}

// What a call with `tokens` tokens writes, and what a caller sizing for up to `tokens` tokens must provide (the
// number of K ranges drops above 512 tokens, so the second is kept monotone).
size_t moe_route_partial_need(int tokens, int experts)
{
    return size_t(moe_route_splits(tokens, experts)) * tokens * experts * sizeof(float);
}
size_t moe_route_partial_bytes(int tokens, int experts) { return size_t(kRmMaxSplits) * tokens * experts * sizeof(float); }

int Moe::init_route_mma(cudaStream_t stream)
{
    route_mma_ok = false;
    if (opt.hidden % kRmSlab) return GARNET_B200_OK;
    const size_t count = size_t(opt.experts) * opt.hidden;
    GB_CUDA(cudaMalloc(&router_w3, 3 * count * sizeof(__nv_bfloat16)));
    moe_router_split_kernel<<<unsigned((count + 255) / 256), 256, 0, stream>>>(router_w_ptr, router_w3, count);
    GB_CUDA(cudaGetLastError());
    route_mma_ok = true;
    return GARNET_B200_OK;
}

int Moe::route_mma(const void* x, float* logits, float* partial, int tokens, cudaStream_t stream, bool finish)
{
    const int splits = moe_route_splits(tokens, opt.experts);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned((tokens + kRmTokens - 1) / kRmTokens), unsigned((opt.experts + kRmExperts - 1) / kRmExperts),
                       unsigned(splits));
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (opt.io_dtype == GARNET_B200_FP32)
        GB_CUDA(cudaLaunchKernelEx(&cfg, moe_route_mma_kernel<float>, static_cast<const float*>(x),
                                   (const __nv_bfloat16*)router_w3, partial, tokens, opt.hidden, opt.experts));
    else
        GB_CUDA(cudaLaunchKernelEx(&cfg, moe_route_mma_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(x),
                                   (const __nv_bfloat16*)router_w3, partial, tokens, opt.hidden, opt.experts));
    if (!finish) return GARNET_B200_OK;   // the caller's own kernel adds the ranges up
    const size_t n = size_t(tokens) * opt.experts;
    cfg.gridDim = dim3(unsigned((n + 255) / 256));
    cfg.blockDim = dim3(256);
    GB_CUDA(cudaLaunchKernelEx(&cfg, moe_route_finish_kernel, (const float*)partial, router_b_ptr, logits, tokens,
                               opt.experts, splits));
    return GARNET_B200_OK;
}

}  // namespace gb200
