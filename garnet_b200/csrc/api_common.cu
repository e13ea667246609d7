// Error reporting, manifest and symbol resolution of the C ABI.
#include <dlfcn.h>

#include <cstdarg>
#include <cstring>
#include <string>

#include "common.cuh"

namespace gb200 {

static thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int cuda_fail(cudaError_t e, const char* where)
{
    if (e == cudaErrorMemoryAllocation) return fail(GARNET_B200_OUT_OF_MEMORY, "%s: %s", where, cudaGetErrorString(e));
    return fail(GARNET_B200_CUDA_ERROR, "%s: %s", where, cudaGetErrorString(e));
}

// One warp waits on a shared-memory barrier that nothing ever arrives on, with the
// given limit, and reports through the status word the way every kernel of this
// library reports a wait that ran out.
__global__ void bounded_wait_probe_kernel(unsigned long long limit_ns, int* status)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    const bool completed = mbar_wait(&bar, 0, limit_ns);
    if (threadIdx.x == 0) *status = completed ? 0 : 77;
}

}  // namespace gb200

extern "C" {

const char* garnet_b200_last_error(void) { return gb200::g_last_error.c_str(); }

int garnet_b200_abi_version(void) { return GARNET_B200_ABI; }

// Same keys as the reference plugin manifest (gpt_oss_plugin.cpp:497-503); the
// operator list names the two operator families this library serves: the
// gpt-oss MoE operator under its reference name and the int4 linear family under
// the names the lowering treats as linear (trt_builder.cpp:6017-6022).
const char* garnet_b200_manifest_json(void)
{
    return "{\"id\":\"garnet_b200\",\"module\":\"garnet_b200\",\"abi\":1,\"version\":\"0.1.0\","
           "\"backend\":\"cuda\",\"arch\":\"sm_100a\","
           "\"operators\":[\"gpt_oss_moe_mxfp4\",\"linear\",\"q_proj\",\"k_proj\",\"v_proj\",\"o_proj\","
           "\"gate_proj\",\"up_proj\",\"down_proj\",\"lm_head\"],"
           "\"precisions\":[\"int4_bf16\",\"mxfp4\"]}";
}

void* garnet_b200_resolve(const char* symbol_name)
{
    if (!symbol_name || std::strncmp(symbol_name, "garnet_b200_", 12) != 0) return nullptr;
    Dl_info info;
    if (!dladdr(reinterpret_cast<const void*>(&garnet_b200_resolve), &info)) return nullptr;
    void* self = dlopen(info.dli_fname, RTLD_NOW | RTLD_NOLOAD);
    if (!self) return nullptr;
    void* sym = dlsym(self, symbol_name);
    dlclose(self);
    return sym;
}

int garnet_b200_is_int4_linear_weight(const char* name, const char* dtype, int rank, const int64_t* shape, int block)
{
    if (!name || !dtype || !shape || rank != 2) return 0;
    if (shape[0] <= 0 || shape[1] <= 0 || block <= 0 || shape[1] % block != 0) return 0;
    if (std::strcmp(dtype, "BF16") != 0 && std::strcmp(dtype, "F16") != 0 && std::strcmp(dtype, "F32") != 0) return 0;
    static const char* const kEndings[] = {
        ".self_attn.q_proj.weight",      ".self_attn.k_proj.weight",     ".self_attn.v_proj.weight",
        ".self_attn.o_proj.weight",      ".linear_attn.in_proj_qkv.weight", ".linear_attn.in_proj_z.weight",
        ".linear_attn.in_proj_b.weight", ".linear_attn.in_proj_a.weight", ".linear_attn.out_proj.weight",
        ".mlp.gate_proj.weight",         ".mlp.up_proj.weight",          ".mlp.down_proj.weight",
        "lm_head.weight"};
    const size_t len = std::strlen(name);
    for (const char* ending : kEndings) {
        const size_t el = std::strlen(ending);
        if (len >= el && std::memcmp(name + len - el, ending, el) == 0) return 1;
    }
    return 0;
}

int garnet_b200_selftest_bounded_wait(int limit_ms, void* stream)
{
    if (limit_ms <= 0 || limit_ms > 2000) return gb200::fail(GARNET_B200_INVALID_VALUE, "selftest_bounded_wait: limit must be 1..2000 ms");
    int* status_host = nullptr;
    int* status_dev = nullptr;
    GB_CUDA(cudaHostAlloc(&status_host, sizeof(int), cudaHostAllocMapped));
    *status_host = -1;
    cudaError_t e = cudaHostGetDevicePointer(&status_dev, status_host, 0);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (e == cudaSuccess) {
        gb200::bounded_wait_probe_kernel<<<1, 32, 0, s>>>((unsigned long long)limit_ms * 1000000ull, status_dev);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    const int status = *status_host;
    cudaFreeHost(status_host);
    if (e != cudaSuccess) return gb200::cuda_fail(e, "selftest_bounded_wait");
    if (status == 77) return gb200::fail(GARNET_B200_DEVICE_FAULT, "device wait gave up (code %d)", status);
    return status == 0 ? GARNET_B200_OK : gb200::fail(GARNET_B200_CUDA_ERROR, "selftest_bounded_wait: kernel did not report");
}

const char* garnet_b200_binary_path(void)
{
    static std::string path;
    if (path.empty()) {
        Dl_info info;
        if (dladdr(reinterpret_cast<const void*>(&garnet_b200_binary_path), &info) && info.dli_fname)
            path = info.dli_fname;
    }
    return path.c_str();
}

}  // extern "C"
