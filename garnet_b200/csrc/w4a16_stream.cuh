// Host/device description of the work the small-batch int4 kernel walks: a list
// of linears ("ops") that one persistent launch streams back to back.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace gb200 {

constexpr int kStreamConsumerWarps = 16;   // warps that multiply
constexpr int kStreamWarps = kStreamConsumerWarps + 1;   // + the weight producer
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kInt4ChunkBytes = 1024 + 32;   // 16 rows x 128 columns of codes + 16 scales
constexpr int kSlotChunks = 4;               // chunks per ring slot = the largest part one warp takes at a time
constexpr int kSlotBytes = kSlotChunks * kInt4ChunkBytes;
constexpr int kMaxRingSlots = 64;
constexpr int kMaxInlineOps = 4;
constexpr int kMaxSmemOps = 256;             // lists up to this long keep their op table in shared memory

enum : int {
    kOpSameX = 1,      // reads the same activation rows as the op before it: no restaging
    kOpSignal = 2,     // a later op reads this one's output: publish it in exchange packets
    kOpScaleFp16 = 4,  // 16-bit scales are fp16 (else bf16)
    kOpBuffer1 = 8,    // its activation rows live in the second buffer
    kOpNorm = 16,      // the input rows are RMS-normalised (and scaled by norm_w) before they are multiplied
    kOpSwiGLU = 32,    // the source rows are [m, 2k]: the input is silu(source[:, :k]) * source[:, k:]
    kOpResidual = 64,  // a bf16 matrix [m, ldy] in memory is added to the output before its rounding
    kOpResidualXch = 128,   // the same, taken from the exchange packets of an earlier op of the list
};

// Outputs that a later op of the same list consumes also travel as 8-byte packets
// {bf16 of row R(g), bf16 of row R(g)+8 | tag of the run}: data and "ready" flag in one
// store, so the consumer polls the data itself (one trip through L2 instead of a
// store, a counter update and a load).  Packet (m, strip, g) sits at
// [(m * strips + strip) * 8 + g].
struct StreamOp {
    const uint8_t* packed;        // strip-major packed matrix
    const __nv_bfloat16* x;       // [m, k]
    __nv_bfloat16* y;             // [m, ldy]
    uint2* xch_out;               // exchange packets this op writes (kOpSignal), else nullptr
    const uint2* xch_in;          // exchange packets of the op whose output is this op's x, else nullptr
    int n;                        // logical weight rows
    int ldy;
    int strips;                   // ceil(n / 16)
    int chunks;                   // k / 128
    int cpp;                      // chunks per part (1..kSlotChunks)
    int parts;                    // ceil(chunks / cpp)
    int dep;                      // index of the op whose outputs this op's x holds, or -1
    int flags;
    int first_cta;                // CTA that owns the first strips (rotates from op to op to even out the shares)
    int in_strips;                // strips of the op behind xch_in
    // precomputed for the launch grid, so that the consumer warps divide nothing
    int base_strips, rem_strips;  // strips / grid, strips % grid: the first rem_strips CTAs (from first_cta) take one more
    unsigned long long inv_parts; // ceil(2^40 / parts): x / parts = (x * inv_parts) >> 40
    const __nv_bfloat16* norm_w;  // kOpNorm: weight of the RMS norm, [k]
    const __nv_bfloat16* res;     // kOpResidual: [m, ldy]
    const uint2* res_xch;         // kOpResidualXch: packets of an op with the same n
    float norm_eps;
    int pad_;
};
static_assert(sizeof(StreamOp) % 16 == 0, "the op table is copied in 16-byte pieces");

struct StreamParams {
    const StreamOp* ops;          // device table; nullptr = use inline_ops
    StreamOp inline_ops[kMaxInlineOps];
    int count;
    int m;                        // batch rows of every op
    int max_chunks;               // largest chunks over the ops (sizes the activation buffers)
    int ring_slots;
    int nbuf;                     // activation buffers: with two, rows staged earlier stay usable (gate/up x, then down x, then back)
    int max_parts;                // largest parts over the ops (sizes the partial-sum slots)
    unsigned long long inv_ring;  // ceil(2^40 / ring_slots): q / ring_slots = (q * inv_ring) >> 40
    unsigned long long inv_pslots; // the same for the partial-sum slots
    int has_deps;
    int has_glue;                 // some op computes its input on the way in or adds a residual
    int table_in_smem;            // the op table is copied to shared memory at the start (short lists)
    int* epoch;                   // tag of this run's exchange packets; bumped by the last CTA (only with has_deps)
    int* finish;                  // CTAs that finished the list (only with has_deps)
    int* fault;                   // mapped host word
    unsigned long long wait_limit_ns;
};

// Shared-memory plan (byte offsets), the same on host and device.
struct StreamSmem {
    int bars, ctl, tags, sx, pcnt, pgen, optable, partial, xq, ring, total;
    int xq_stride, xq_rows, xq_bytes, mblk, part_slots, ring_slots;
};

__host__ __device__ inline int stream_mblk(int m) { return m <= 4 ? 1 : m <= 8 ? 2 : 4; }

__host__ __device__ inline StreamSmem stream_smem_plan(int m, int max_chunks, int ring_slots, int max_parts, int table_ops, int nbuf)
{
    StreamSmem p;
    p.mblk = stream_mblk(m);
    p.xq_rows = 2 * m + 1;                       // hi and lo piece of every batch row + one all-zero row
    p.xq_stride = max_chunks * 128 + 64;         // 64 mod 128: conflict-free 16-byte reads across rows
    p.xq_bytes = (p.xq_rows * p.xq_stride + 127) & ~127;
    p.ring_slots = ring_slots;
    p.part_slots = ring_slots + max_parts;   // a slot is reused only after every part of its strip has been added
    int off = 0;
    p.bars = off;   off += 2 * kMaxRingSlots * 8;
    p.ctl = off;    off += 128;                                      // abort flag, finished warps
    p.tags = off;   off += kMaxRingSlots * 4;                        // slot index each ring stage currently holds
    p.sx = off;     off += nbuf * max_chunks * p.mblk * 4 * 4;       // [buf][chunk][mblk][4] float
    p.pcnt = off;   off += p.part_slots * 4;                         // parts of a strip that have arrived
    p.pgen = off;   off += p.part_slots * 4;                         // times a partial-sum slot has been released
    off = (off + 15) & ~15;
    p.optable = off; off += table_ops * int(sizeof(StreamOp));       // copy of a short op table
    off = (off + 127) & ~127;
    p.partial = off; off += p.part_slots * p.mblk * 256;             // [slot][mblk][lane][2] float
    p.xq = off;     off += nbuf * p.xq_bytes;
    p.ring = off;   off += ring_slots * kSlotBytes;
    p.total = off;
    return p;
}

}  // namespace gb200
