// Host-side state of one W4A16 linear operator (the object behind
// garnet_b200_w4a16_t).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "layout.h"

namespace gb200 {

struct W4A16 {
    PackGeom geo{};
    int scale_dtype = 1;             // GARNET_B200_FP16 or GARNET_B200_BF16: how the 16-bit scales are read
    uint8_t* packed = nullptr;       // packed tiles (device)
    bool owns_packed = false;
    int device = 0;
    struct alignas(64) TensorMapStorage { unsigned char bytes[128]; };
    TensorMapStorage tc_packed_map[2];   // TMA views of the packed matrix: 8 and 16 strips per box
    int max_rows_per_launch = 16;    // batch rows one launch of the streaming kernel takes
    int* fault_host = nullptr;       // mapped host word written by bounded device waits
    int* fault_dev = nullptr;
    // staging for the host-buffer entry point
    void* stage_x = nullptr;
    void* stage_y = nullptr;
    void* stage_ws = nullptr;
    int stage_rows = 0;

    ~W4A16();
    int init_common();
    size_t workspace_bytes(int m) const;
    int launch_stream(const __nv_bfloat16* x, __nv_bfloat16* y, int m, int ldy, unsigned flags,
                      cudaStream_t stream);
    static int launch_stream_group(W4A16* const* hs, int count, const __nv_bfloat16* x, __nv_bfloat16* const* ys,
                                   const int* ldys, int m, unsigned flags, cudaStream_t stream);
    int init_tc();
    int launch_tc(const __nv_bfloat16* x, __nv_bfloat16* y, int m, void* ws, size_t ws_bytes, unsigned flags, cudaStream_t stream);
    int run(const void* d_x, void* d_y, int m, void* ws, size_t ws_bytes, unsigned flags, cudaStream_t stream);
};

// Tiling of the tensor-core tile kernel for a batch of m rows.
struct TcPlan {
    int token_tiles, atiles, panels, kslices, chunks_per_slice;
    size_t workspace;   // bytes of fp32 partial sums the K slices need (0 without slices)
};
TcPlan tc_plan(const PackGeom& geo, int m);

int w4a16_repack_device(const uint8_t* d_nibbles, const uint16_t* d_scales, const PackGeom& geo, long long row0,
                        uint8_t* d_packed, cudaStream_t stream, int src_cols = 0, int col0 = 0);

}  // namespace gb200
