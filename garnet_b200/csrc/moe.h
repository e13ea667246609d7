// Host-side state of one gpt_oss_moe_mxfp4 operator (the object behind
// garnet_b200_moe_t).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/garnet_b200.h"
#include "layout.h"

namespace gb200 {

// Which experts this rank computes: all (world <= 1), a contiguous block
// [lo, hi), or every world-th expert (the reference's 2-way rule
// expert % 2 == rank, gpt_oss_kernels.cu:771).
struct MoeShard {
    int world, rank, interleaved, lo, hi;
};

// Byte offsets of the regions of the caller's workspace.
struct MoeWorkspace {
    size_t logits, selected, probs, xshift, xh, counts, offsets, sorted, ntasks, tasks, mx_tp, mx_q, mx_sf, route_partial,
        act, vals, total;
};

struct MoeWorkspacePtrs {
    float* logits;
    int* selected;
    float* probs;
    int* xshift;
    __half* xh;
    int* counts;
    int* offsets;
    int* sorted;
    int* ntasks;
    int4* tasks;
    int* mx_tp;        // row tiles before each expert (block-scaled path)
    uint8_t* mx_q;     // e4m3 row pieces at tile-aligned positions: [2][q_rows][kp]
    uint8_t* mx_sf;    // their scale atoms: [tiles][kslabs][512]
    float* route_partial;   // [K ranges][tokens][experts] partial router sums (tensor-core router)
    int vals_bf16 = 0;      // `vals` holds bf16 (the per-slot values are bf16-valued; Moe::run keeps them so between its own kernels)
    __half* act;
    float* vals;
};

MoeWorkspace moe_workspace_plan(const garnet_b200_moe_options& o, int tokens);
MoeWorkspace moe_rows_workspace_plan(const garnet_b200_moe_options& o, int rows);
// Sizes of the block-scaled path's per-call buffers.
struct MoeMxPlan {
    int nt;            // rows per tile (UMMA N)
    int tiles_max;     // upper bound of the row tiles of one call
    int q_rows;        // tiles_max * nt
    int kp_max;        // max(hidden, intermediate) padded to 128
    size_t q_bytes, sf_bytes;
};
MoeMxPlan moe_mx_plan(const garnet_b200_moe_options& o, int tokens, int slots);
// Which expert kernels an operator with these options uses: 0 = the streaming kernels at
// every size, 2 = the block-scaled tensor-core kernels at every size, 1 = by rows per expert.
int moe_mx_mode_of(const garnet_b200_moe_options& o);
// Checks caller options (either version of the struct) and writes the operator's own
// view of them: later fields zero-filled, `intermediate` = this rank's share of it.
int moe_resolve_options(const garnet_b200_moe_options* in, garnet_b200_moe_options* eff);
size_t moe_route_partial_bytes(int tokens, int experts);   // to provide for calls of up to `tokens` tokens
size_t moe_route_partial_need(int tokens, int experts);    // written by a call of exactly `tokens` tokens
int moe_route_splits(int tokens, int experts);   // K ranges (partial-sum planes) of the tensor-core router
constexpr int kMxMinRowsPerExpert = 8;   // routed rows per local expert above which the block-scaled path is used

struct Moe {
    garnet_b200_moe_options opt{};     // resolved: `intermediate` is this rank's share
    int mx_mode = 1;                   // moe_mx_mode_of(opt)
    bool owns_packed = true;           // false: the packed blobs are the caller's (create_prepacked)
    float* own_up_bias = nullptr;      // rank-local gate/up bias gathered at create time (intermediate-axis split)
    float* zero_down_bias = nullptr;   // down bias of the ranks that do not add it
    PackGeom geo_up{}, geo_down{};
    int stored_experts = 0;            // experts whose packed weights this handle holds
    uint8_t* packed_up = nullptr;      // [stored_experts][geo_up.matrix_bytes()]
    uint8_t* packed_down = nullptr;
    const float* router_w_ptr = nullptr;   // borrowed constants
    const float* router_b_ptr = nullptr;
    const float* up_bias_ptr = nullptr;
    const float* down_bias_ptr = nullptr;
    bool careful_scales = false;       // some e8m0 byte is 0 or 255
    struct alignas(64) TensorMapStorage { unsigned char bytes[128]; };
    int mx_kp[2] = {0, 0}, mx_kslabs[2] = {0, 0};   // block-scaled path: K padded to 128, and in slabs of 128
    bool mx_ok = false;
    struct QMapCache {                 // TMA view of the quantised rows of the last call
        TensorMapStorage map;
        const void* base = nullptr;
        int kp = 0, q_rows = 0;
    };
    QMapCache q_map_cache[2];
    uint8_t* mxr_w[2] = {nullptr, nullptr};    // rows-as-M form: 15 KiB blocks of 240 weight rows
    uint8_t* mxr_sf[2] = {nullptr, nullptr};   // and their scale atoms
    int mxr_ntiles[2] = {0, 0};
    TensorMapStorage mxr_w_map[2];
    __nv_bfloat16* router_w3 = nullptr;        // router weight split into three bf16 terms (tensor-core router)
    bool route_mma_ok = false;
    int device = 0;                    // device the handle was created on
    void* static_scratch = nullptr;    // device address of the library's built-in scratch (run_static)
    int* flag_dev = nullptr;
    int* fault_host = nullptr;
    int* fault_dev = nullptr;

    ~Moe();
    MoeShard shard() const;
    int local_experts() const;
    int prepare(const void* const* weights, cudaStream_t stream);
    int prepare_prepacked(const void* const* small, const void* const* packed, cudaStream_t stream);
    int setup_common(cudaStream_t stream);
    int finish_prepare(cudaStream_t stream);
    bool partial_output() const { return shard().world > 1 || opt.tp_world > 1; }
    int route(const void* x, float* logits, int* selected, float* probs, __half* xh, int* xshift, int tokens,
              cudaStream_t stream, bool skip_topk = false, float* route_partial = nullptr, int* counts = nullptr,
              const void* small_meta = nullptr);
    int launch_stream(bool up, const MoeWorkspacePtrs& w, int tokens, cudaStream_t stream, int topk = -1);
    int run_rows(const void* x_rows, const int* row_expert, int rows, float* vals, void* ws, size_t ws_bytes,
                 cudaStream_t stream, int stage = 0, float* hidden_io = nullptr);
    int finish_mx();
    int init_mxr(int pass, const uint8_t* blocks, const uint8_t* scales, int first_stored, int count, cudaStream_t stream);
    int finish_mxr();
    int dequant_block_scaled(int pass, int stored_expert, float* out, cudaStream_t stream);
    int launch_mxr_gemm(bool up, const MoeWorkspacePtrs& w, const void* q_map, int q_rows, int tiles_max,
                        cudaStream_t stream);
    int launch_mx(bool up, const MoeWorkspacePtrs& w, const void* x, int x_is_sorted, int tokens, int slots, int topk,
                  cudaStream_t stream);
    // The block-scaled path pays off once experts get several rows each (measured
    // crossover on the gpt-oss-120b layer: about 8 rows per expert); below that the
    // streaming kernel moves the weights faster.
    // A handle that holds one layout only runs every size on it.
    bool use_mx(int slots) const
    {
        if (!mx_ok || !mxr_w[0]) return false;
        return mx_mode == 2 || !packed_up || (mx_mode == 1 && slots > kMxMinRowsPerExpert * local_experts());
    }
    int init_route_mma(cudaStream_t stream);
    int route_mma(const void* x, float* logits, float* partial, int tokens, cudaStream_t stream, bool finish = true);
    int combine(const float* vals, const float* probs, void* y, int tokens, cudaStream_t stream);
    int run(const void* x, void* y, void* ws, size_t ws_bytes, int tokens, cudaStream_t stream);
};

}  // namespace gb200
