// C face of the reference's own GPU MoE, compiled from the reference's sources where they
// lie (see oracle/Makefile, target ref_gpu).  TEST AND MEASUREMENT INFRASTRUCTURE ONLY: it lets
// the GPU tests compare the product with the reference's kernels on the same inputs and lets
// bench.py's reference arm time them on the same box.  Nothing under garnet_b200/ uses it.
//
// Wrapped: size_t GptOssMoeWorkspace(int, const GptOssOptions&) / cudaError_t RunGptOssMoe(...)
// (plugins/gpt_oss/include/gpt_oss_kernels.h:41-43: the scalar path below 16 tokens, the
// grouped WMMA path from 16) and GptOssMarlin{ctor, Workspace, Run}
// (plugins/gpt_oss/include/gpt_oss_marlin.h:17-30: the production GEMM; 8 tokens at most
// unless GARNET_GPT_OSS_MARLIN_MAX_TOKENS raises the limit).
#include <cuda_runtime.h>

#include <new>

#include "gpt_oss_kernels.h"
#include "gpt_oss_marlin.h"

namespace {
Garnet::GptOssOptions make_options(int hidden, int intermediate, int experts, int top_k, float limit, int prefill)
{
    Garnet::GptOssOptions o;
    o.kind = 2;
    o.hidden = hidden;
    o.intermediate = intermediate;
    o.experts = experts;
    o.topK = top_k;
    o.limit = limit;
    o.prefill = prefill;
    return o;
}
}  // namespace

extern "C" {

// Workspace bytes of RunGptOssMoe (which = 0) or GptOssMarlin::Run (which = 1).
size_t ref_gpu_moe_workspace(int which, int tokens, int hidden, int intermediate, int experts, int top_k, float limit, int prefill)
{
    const Garnet::GptOssOptions o = make_options(hidden, intermediate, experts, top_k, limit, prefill);
    return which == 0 ? Garnet::GptOssMoeWorkspace(tokens, o) : Garnet::GptOssMarlin::Workspace(tokens, o);
}

// in[0..8]: x [tokens, hidden] f32, router W, router b, gate_up blocks, scales, bias, down blocks, scales, bias.
int ref_gpu_moe_run(const void* const* in, float* y, void* workspace, int tokens, int hidden, int intermediate, int experts,
                    int top_k, float limit, int prefill, void* stream)
{
    const Garnet::GptOssOptions o = make_options(hidden, intermediate, experts, top_k, limit, prefill);
    return int(Garnet::RunGptOssMoe(in, y, workspace, tokens, o, static_cast<cudaStream_t>(stream)));
}

void* ref_gpu_marlin_create(int hidden, int intermediate, int experts, int top_k, float limit, int prefill)
{
    return new (std::nothrow) Garnet::GptOssMarlin(make_options(hidden, intermediate, experts, top_k, limit, prefill));
}

int ref_gpu_marlin_run(void* handle, const void* const* in, float* y, void* workspace, int tokens, void* stream)
{
    if (!handle) return int(cudaErrorInvalidValue);
    return int(static_cast<Garnet::GptOssMarlin*>(handle)->Run(in, y, workspace, tokens, static_cast<cudaStream_t>(stream)));
}

void ref_gpu_marlin_destroy(void* handle) { delete static_cast<Garnet::GptOssMarlin*>(handle); }

// ---- the rest of the gpt-oss layer (gpt_oss_kernels.h:24-40)

int ref_gpu_rms_norm(const float* x, const float* weight, float* y, int rows, int hidden, float epsilon, int threads, void* stream)
{
    return int(Garnet::RunGptOssRmsNorm(x, weight, y, rows, hidden, epsilon, threads, static_cast<cudaStream_t>(stream)));
}

static Garnet::GptOssOptions attention_options(int kind, int q_heads, int kv_heads, int head_dim, int layer, int page_size, int window,
                                               int prefill, float theta, float factor, float initial_context, float beta_fast,
                                               float beta_slow)
{
    Garnet::GptOssOptions o;
    o.kind = kind;
    o.qHeads = q_heads, o.kvHeads = kv_heads, o.headDim = head_dim;
    o.layer = layer, o.pageSize = page_size, o.window = window, o.prefill = prefill;
    o.theta = theta, o.factor = factor, o.initialContext = initial_context, o.betaFast = beta_fast, o.betaSlow = beta_slow;
    return o;
}

int ref_gpu_rope(const float* x, const long long* positions, float* y, int tokens, int q_heads, int kv_heads, int head_dim, float theta,
                 float factor, float initial_context, float beta_fast, float beta_slow, void* stream)
{
    const Garnet::GptOssOptions o = attention_options(0, q_heads, kv_heads, head_dim, 0, 16, 0, 0, theta, factor, initial_context,
                                                      beta_fast, beta_slow);
    return int(Garnet::RunGptOssRope(x, reinterpret_cast<const std::int64_t*>(positions), y, tokens, o, static_cast<cudaStream_t>(stream)));
}

// in[0..7] as RunGptOssAttention takes them; the workspace holds batch * q_heads * 64 * (2 + head_dim) floats at least.
int ref_gpu_attention(const void* const* in, float* y, void* workspace, int batch, int tokens, int logical_pages, int physical_pages,
                      int q_heads, int kv_heads, int head_dim, int layer, int page_size, int window, int prefill, void* stream)
{
    const Garnet::GptOssOptions o = attention_options(1, q_heads, kv_heads, head_dim, layer, page_size, window, prefill, 150000, 32, 4096,
                                                      32, 1);
    return int(Garnet::RunGptOssAttention(in, y, workspace, batch, tokens, logical_pages, physical_pages, o,
                                          static_cast<cudaStream_t>(stream)));
}

int ref_gpu_vocab_top1(const float* logits, float* pairs, int rows, int width, int rank, void* stream)
{
    return int(Garnet::RunGptOssVocabTop1(logits, pairs, rows, width, rank, static_cast<cudaStream_t>(stream)));
}

int ref_gpu_decode_gemv(const void* x, const void* weight, void* y, int rows, int columns, int weight_stride, int column_offset,
                        int q_heads, int kv_heads, int head_dim, int rank, void* stream)
{
    return int(Garnet::RunGptOssDecodeGemv(x, weight, y, rows, columns, weight_stride, column_offset, q_heads, kv_heads, head_dim, rank,
                                           static_cast<cudaStream_t>(stream)));
}

}  // extern "C"
