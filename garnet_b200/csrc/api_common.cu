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
