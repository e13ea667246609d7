// Host side of the packed expert constants: sizes, the host packer and the host
// gather of the intermediate-axis split.  The index arithmetic is shared with the device
// repackers through moe_pack.h.
//
// Reference: PackGptOssMarlinWeight (plugins/gpt_oss/include/gpt_oss_marlin_pack.h:74-193),
// which packs on up to 16 host threads (:85-99), and GatherGptOssIntermediateShard
// (src/backends/tensorrt/gpt_oss_weight_shard.h:25-60).
#include <algorithm>
#include <cstring>
#include <thread>
#include <vector>

#include "common.cuh"
#include "moe.h"
#include "moe_pack.h"

namespace gb200 {

namespace {

struct Projection {
    PackGeom geo;
    MxBlockGeom block;
    int interleaved;
};

int projection_of(const garnet_b200_moe_options* options, int which, Projection* out)
{
    garnet_b200_moe_options o;
    if (int rc = moe_resolve_options(options, &o)) return rc;
    if (which != 0 && which != 1) return fail(GARNET_B200_INVALID_VALUE, "moe packed blob: which must be 0 (gate_up) or 1 (down)");
    out->geo = which == 0 ? make_geom(kFormatMxfp4, 2 * o.intermediate, o.hidden, 32)
                          : make_geom(kFormatMxfp4, o.hidden, o.intermediate, 32);
    out->block = make_block_geom(out->geo.rows, out->geo.cols);
    out->interleaved = which == 0;
    return GARNET_B200_OK;
}

size_t blob_bytes(const Projection& p, int layout, int experts)
{
    return layout == GARNET_B200_MOE_LAYOUT_STREAM ? p.geo.matrix_bytes() * size_t(experts)
                                                   : size_t(experts) * (p.block.code_bytes() + p.block.atom_bytes());
}

void pack_stream_expert(const Projection& p, const uint8_t* blocks, const uint8_t* scales, uint8_t* dst)
{
    const size_t words = mx_stream_words(p.geo), nsc = mx_stream_scale_count(p.geo);
    for (size_t i = 0; i < words; ++i) {
        size_t db, sb;
        uint32_t w = 0;
        if (mx_stream_word(p.geo, i, p.interleaved, &db, &sb)) std::memcpy(&w, blocks + sb, 4);
        std::memcpy(dst + db, &w, 4);
    }
    for (size_t i = 0; i < nsc; ++i) {
        size_t db, sb;
        const bool real = mx_stream_scale(p.geo, i, p.interleaved, &db, &sb);
        dst[db] = real ? scales[sb] : uint8_t(127);
    }
}

void pack_block_expert(const Projection& p, const uint8_t* blocks, const uint8_t* scales, uint8_t* codes, uint8_t* atoms)
{
    const size_t pieces = p.block.code_bytes() / 16, nat = p.block.atom_bytes();
    for (size_t i = 0; i < pieces; ++i) {
        size_t sb;
        if (mx_block_piece(p.block, i, &sb)) std::memcpy(codes + i * 16, blocks + sb, 16);
        else std::memset(codes + i * 16, 0, 16);
    }
    for (size_t i = 0; i < nat; ++i) {
        size_t sb;
        atoms[i] = mx_block_atom(p.block, i, &sb) ? scales[sb] : uint8_t(127);
    }
}

}  // namespace

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_moe_packed_bytes(const garnet_b200_moe_options* options, int which, int layout, int experts, size_t* bytes)
{
    Projection p;
    if (int rc = projection_of(options, which, &p)) return rc;
    if (!bytes || experts <= 0 || (layout != GARNET_B200_MOE_LAYOUT_STREAM && layout != GARNET_B200_MOE_LAYOUT_BLOCK))
        return fail(GARNET_B200_INVALID_VALUE, "moe_packed_bytes: bad argument (layout must be 1 or 2)");
    *bytes = blob_bytes(p, layout, experts);
    return GARNET_B200_OK;
}

int garnet_b200_moe_pack_host(const garnet_b200_moe_options* options, int which, int layout, const uint8_t* blocks,
                              const uint8_t* scales, int experts, uint8_t* out)
{
    Projection p;
    if (int rc = projection_of(options, which, &p)) return rc;
    if (!blocks || !scales || !out || experts <= 0 ||
        (layout != GARNET_B200_MOE_LAYOUT_STREAM && layout != GARNET_B200_MOE_LAYOUT_BLOCK))
        return fail(GARNET_B200_INVALID_VALUE, "moe_pack_host: bad argument (layout must be 1 or 2)");
    const size_t blk = size_t(p.geo.rows) * p.geo.cols / 2, sc = size_t(p.geo.rows) * p.geo.cols / 32;
    auto one = [&](int e) {
        if (layout == GARNET_B200_MOE_LAYOUT_STREAM)
            pack_stream_expert(p, blocks + e * blk, scales + e * sc, out + size_t(e) * p.geo.matrix_bytes());
        else
            pack_block_expert(p, blocks + e * blk, scales + e * sc, out + size_t(e) * p.block.code_bytes(),
                              out + size_t(experts) * p.block.code_bytes() + size_t(e) * p.block.atom_bytes());
    };
    const int threads = std::max(1, std::min({16, experts, int(std::thread::hardware_concurrency())}));
    if (threads == 1) {
        for (int e = 0; e < experts; ++e) one(e);
        return GARNET_B200_OK;
    }
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([&, t] {
            for (int e = t; e < experts; e += threads) one(e);
        });
    for (std::thread& th : pool) th.join();
    return GARNET_B200_OK;
}

int garnet_b200_moe_gather_intermediate_shard(const void* source, size_t bytes, const long long* shape, int rank_dims,
                                              size_t element_bytes, int rank, int world, int mode, void* out)
{
    if (!source || !shape || !out || world < 2 || rank < 0 || rank >= world || mode < 1 || mode > 3 || rank_dims < 2 ||
        rank_dims > 4 || (element_bytes != 1 && element_bytes != 2 && element_bytes != 4) || (mode == 2 && rank_dims < 3) ||
        (mode == 3 && rank_dims != 2))
        return fail(GARNET_B200_INVALID_VALUE, "gather_intermediate_shard: invalid shard descriptor");
    size_t elements = 1;
    for (int i = 0; i < rank_dims; ++i) {
        if (shape[i] <= 0 || size_t(shape[i]) > SIZE_MAX / elements)
            return fail(GARNET_B200_INVALID_VALUE, "gather_intermediate_shard: shape overflow");
        elements *= size_t(shape[i]);
    }
    if (elements > SIZE_MAX / element_bytes || elements * element_bytes != bytes)
        return fail(GARNET_B200_INVALID_VALUE, "gather_intermediate_shard: byte count does not match the shape");
    if (mode == 3) {
        if (rank == 0) std::memcpy(out, source, bytes);
        else std::memset(out, 0, bytes);
        return GARNET_B200_OK;
    }
    const int axis = mode == 1 ? 1 : 2;
    if (shape[axis] % world)
        return fail(GARNET_B200_INVALID_VALUE, "gather_intermediate_shard: axis %d (%lld) does not divide into %d parts", axis,
                    shape[axis], world);
    size_t outer = 1, inner = element_bytes;
    for (int i = 0; i < axis; ++i) outer *= size_t(shape[i]);
    for (int i = axis + 1; i < rank_dims; ++i) inner *= size_t(shape[i]);
    const size_t stride = size_t(shape[axis]) * inner, part = stride / size_t(world);
    const uint8_t* data = static_cast<const uint8_t*>(source);
    uint8_t* dst = static_cast<uint8_t*>(out);
    for (size_t i = 0; i < outer; ++i) std::memcpy(dst + i * part, data + i * stride + size_t(rank) * part, part);
    return GARNET_B200_OK;
}

}  // extern "C"
