// C entry points over the reference's own int4 sources, compiled where they lie
// (see oracle/Makefile).  TEST INFRASTRUCTURE ONLY: this shim lets the tests
// and the benchmark's reference arm call Garnet::QuantizeSymmetricINT4
// (src/model/weight_quantization.cpp:188) and Garnet::Q4Q8Linear
// (src/backends/cpu/q4q8_linear.cpp:227-389) unchanged.  No reference source is
// copied; only its headers are included at build time.
#include "q4q8_linear.h"
#include "weight_quantization.h"

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

namespace {
struct RefLinear {
    Garnet::Q4Q8Linear owner;   // owns the reference's repacked nibbles
    Garnet::Q4Q8Linear view;    // same nibbles, caller-supplied fp32 scales
    std::vector<float> scales;
};
thread_local std::string g_error;
}

extern "C" {

const char* ref_last_error() { return g_error.c_str(); }

// Runs the reference quantizer on an fp32 [rows, cols] matrix.  Returns 0 on
// success and fills canonical nibbles (rows*cols/2 bytes) and fp16 scale bits.
int ref_quantize_int4(const float* weights, long long rows, long long cols, int block,
                      std::uint8_t* packed, std::uint16_t* fp16_scales, double* max_error)
{
    Garnet::SafeTensorMetadata meta;
    meta.dataType = "F32";
    meta.shape = {rows, cols};
    meta.dataSize = static_cast<std::uint64_t>(rows) * cols * sizeof(float);
    Garnet::QuantizedWeight q;
    if (!Garnet::QuantizeSymmetricINT4("model.layers.0.self_attn.q_proj.weight", meta,
                                       weights, block, q, g_error))
        return 1;
    std::memcpy(packed, q.packedValues.data(), q.packedValues.size());
    std::memcpy(fp16_scales, q.fp16Scales.data(), q.fp16Scales.size() * sizeof(std::uint16_t));
    if (max_error) *max_error = q.maximumAbsoluteError;
    return 0;
}

// Builds the reference CPU operator from canonical nibbles and fp32 scales.
// Prepare() performs the reference's own repack; BindPackedView() then rebinds
// the repacked nibbles with the caller's fp32 scales so that bf16-valued scales
// reach Forward() without an fp16 rounding step.
void* ref_q4q8_create(const std::uint8_t* packed, const float* scales, int rows, int cols,
                      int block)
{
    auto op = std::make_unique<RefLinear>();
    Garnet::QuantizedWeight q;
    q.shape = {rows, cols};
    q.blockSize = block;
    q.packedValues.assign(packed, packed + static_cast<std::size_t>(rows) * cols / 2);
    q.fp16Scales.assign(static_cast<std::size_t>(rows) * cols / block, 0x3c00);
    if (!op->owner.Prepare(q, g_error)) return nullptr;
    op->scales.assign(scales, scales + static_cast<std::size_t>(rows) * cols / block);
    if (!op->view.BindPackedView(rows, cols, block, op->owner.PackedWeightData(),
                                 op->owner.PackedWeightBytes(), op->scales.data(),
                                 op->scales.size(), g_error))
        return nullptr;
    return op.release();
}

int ref_q4q8_forward(void* handle, const float* x, float* y, int threads)
{
    auto* op = static_cast<RefLinear*>(handle);
    if (!op) { g_error = "null handle"; return 1; }
    return op->view.Forward(x, y, threads, g_error) ? 0 : 1;
}

void ref_q4q8_destroy(void* handle) { delete static_cast<RefLinear*>(handle); }

}  // extern "C"
