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

}  // extern "C"
