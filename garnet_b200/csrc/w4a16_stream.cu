// Small-batch (M <= 16) int4 linear for sm_100a: one persistent launch walks a list
// of linears and streams their packed weights at HBM speed.
//
// Arithmetic.  Every 128-column group of an activation row becomes a 15-bit block
// fixed-point number: V = round(x * 2^(14-e)) with 2^e just above the group's largest
// magnitude, split into two signed bytes V = 128*hi + lo.  The int4 codes are widened
// to signed bytes 16 q with three logic operations per eight codes (a nibble moved to
// the top of its byte) and multiplied on the tensor cores in integers (mma.sync
// m16n8k32 s8 x s8 -> s32; the batch rows' hi and lo pieces are neighbouring MMA
// columns), so each group's sum sum_k q_k V_k is exact.  It is scaled by 2^(e-14) and the weight's group scale in
// fp32 and accumulated over the groups in fp32.  A bf16 activation within 2^-6 of its
// group's maximum is represented exactly; smaller ones carry an absolute error of at
// most 2^-15 of that maximum.
//
// Structure.  One CTA per SM.  A producer warp streams (strip, part-of-K) slots of at
// most four 1056-byte chunks through a ring of bulk copies that runs ahead across
// the boundaries of the linears - weights are constants, so the ring never waits for
// a dependency.  Sixteen consumer warps take the slots round-robin; the parts of a
// strip meet in shared memory, and the warp that delivers the last part adds them
// in a fixed order and stores bf16.  Before a linear with new activation rows the
// consumer warps turn those rows into int8 pieces together.  When a linear consumes
// an earlier one's output, that output also travels as 8-byte packets that carry the
// run's tag beside the data: the consumers poll the packets themselves (bounded), so
// a dependency costs one trip through L2 and no counter.  No atomics on the data
// path, no global scratch for sums: results do not depend on timing.
#include <algorithm>
#include <cstring>
#include <memory>
#include <new>
#include <vector>

#include "common.cuh"
#include "layout.h"
#include "w4a16.h"
#include "w4a16_stream.cuh"

namespace gb200 {

namespace {

__device__ __forceinline__ void imma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four two's-complement int4 codes in the HIGH nibbles of the bytes of `w` -> four signed
// bytes 16 q (a nibble moved to the top of its byte is the code times 16, sign and
// all); the factor 16 is taken out of the activation scale.
__device__ __forceinline__ uint32_t nib_to_s8x16(uint32_t w) { return w & 0xF0F0F0F0u; }

__device__ __forceinline__ uint4 ld_relaxed_gpu_v4(const void* p)
{
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint2 ld_relaxed_gpu_v2(const void* p)
{
    uint2 v;
    asm volatile("ld.relaxed.gpu.global.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu_v2(void* p, uint32_t a, uint32_t b)
{
    asm volatile("st.relaxed.gpu.global.v2.b32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

// Timing build (-DGB_STREAM_TRACE, see GARNET_B200_NVCC_FLAGS in _build.py): CTA 7 records when each op of a
// list reaches its stages (slots 0..6: arrive, rows free, staged, first and last weights ready, last part, last
// strip written), read back with garnet_b200_w4a16_trace.  Absent from the normal build.
#ifdef GB_STREAM_TRACE
__device__ unsigned long long g_trace[512];
#define GB_TRACE(op, slot) do { if (blockIdx.x == 7 && (op) < 63) g_trace[(op) * 8 + (slot)] = global_timer_ns(); } while (0)
#define GB_TRACE_MAX(op, slot) do { if (blockIdx.x == 7 && (op) < 63) atomicMax(&g_trace[(op) * 8 + (slot)], global_timer_ns()); } while (0)
#else
#define GB_TRACE(op, slot) do {} while (0)
#define GB_TRACE_MAX(op, slot) do {} while (0)
#endif

struct Ctl {
    volatile int abort_flag;
    int warps_done;   // consumer warps that have finished the list
    int next_slot;    // next slot of the CTA's sequence that no consumer warp has taken yet
    float row_sq[16]; // sum of squares of every batch row (RMS-normalised inputs)
};
static_assert(sizeof(Ctl) <= 128, "the control block has 128 bytes of shared memory");

// Waits on an mbarrier unless the CTA has been told to give up.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Ctl* ctl, unsigned long long limit)
{
    for (int spin = 0; spin < 64; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int spin = 0; spin < 128; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (ctl->abort_flag) return false;
        if (global_timer_ns() - t0 > limit) return false;
    }
}

__device__ __forceinline__ void give_up(const StreamParams& p, Ctl* ctl, int code)
{
    // the first code recorded stays: later ones are usually its consequences
    if (!ctl->abort_flag) *reinterpret_cast<volatile int*>(p.fault) = code;
    ctl->abort_flag = 1;
}

__device__ __forceinline__ void op_share(const StreamOp& op, int& s0, int& s1)
{
    int rb = int(blockIdx.x) - op.first_cta;
    if (rb < 0) rb += gridDim.x;
    s0 = rb * op.base_strips + min(rb, op.rem_strips);
    s1 = s0 + op.base_strips + (rb < op.rem_strips ? 1 : 0);
}

constexpr int kConsumerThreads = kStreamConsumerWarps * 32;
constexpr int kHalves = kStreamConsumerWarps * 2;   // half-warps that stage activation rows

// The 128 activations of one (batch row, chunk), eight per lane of a half-warp as fp32 bit
// patterns of bf16 values in `bits` (in the order of the MMA operand bytes), become the two
// int8 pieces and the scale factor of the group.
template <int MBLK>
__device__ __forceinline__ void quantise_group(const uint32_t (&bits)[8], uint32_t hmask, int at0, int at1, int m, int chunk, int hl,
                                               uint8_t* xb, float* sxb, const StreamSmem& plan)
{
    uint32_t amax = 0;
#pragma unroll
    for (int el = 0; el < 8; ++el) amax = max(amax, bits[el] & 0x7fffffffu);
#pragma unroll
    for (int off = 8; off; off >>= 1) amax = max(amax, __shfl_xor_sync(hmask, amax, off, 16));
    const int ef = int(amax >> 23);                   // biased exponent of the largest magnitude
    const int e = max(ef - 126, -100);                // 2^e > max |x|
    const float up = __uint_as_float(uint32_t(127 + 14 - e) << 23);      // 2^(14-e)
    float down = __uint_as_float(uint32_t(127 + e - 18) << 23);          // 2^(e-14) / 16: the codes enter the MMA as 16 q
    if (ef == 255) down = __uint_as_float(0x7fc00000u);                  // inf or NaN in the group: NaN out
    uint32_t hi_b[2] = {0, 0}, lo_b[2] = {0, 0};
#pragma unroll
    for (int el = 0; el < 8; ++el) {
        const float f = ef == 255 ? 0.f : __uint_as_float(bits[el]);
        const int V = __float2int_rn(f * up);
        const int hi = V >> 7, lo = V & 127;
        hi_b[el >> 2] |= uint32_t(hi & 0xff) << (8 * (el & 3));
        lo_b[el >> 2] |= uint32_t(lo) << (8 * (el & 3));
    }
    uint8_t* row_hi = xb + size_t(2 * m) * plan.xq_stride;
    uint8_t* row_lo = row_hi + plan.xq_stride;
    *reinterpret_cast<uint32_t*>(row_hi + at0) = hi_b[0];
    *reinterpret_cast<uint32_t*>(row_hi + at1) = hi_b[1];
    *reinterpret_cast<uint32_t*>(row_lo + at0) = lo_b[0];
    *reinterpret_cast<uint32_t*>(row_lo + at1) = lo_b[1];
    if (hl == 0) {
        const int mb = m >> 2, j = m & 3;
        sxb[(chunk * MBLK + mb) * 4 + j] = down;
    }
}

// The consumer threads turn the activation rows of `op` into the int8 pieces, scale
// factors that the MMAs read.  One half-warp per (batch row, chunk of
// 128 activations); each lane quantises eight of them against the chunk's largest
// magnitude.  Rows come from memory, or - when an earlier linear of the list
// produces them - from that linear's exchange packets, polled until they carry this
// run's tag.  Returns false if a poll ran out of time.
template <int MBLK>
__device__ __forceinline__ bool stage_rows(const StreamParams& p, const StreamOp& op, const StreamSmem& plan, Ctl* ctl,
                                           uint8_t* xb, float* sxb, uint32_t run_tag, int tid, int lane)
{
    const int half = tid >> 4, hl = tid & 15;
    const uint32_t hmask = 0xffffu << (lane & 16);   // the lanes of this half-warp
    const int k = op.chunks * 128;
    const int items = p.m * op.chunks;
    constexpr int kAhead = MBLK == 1 ? 2 : 4;   // items whose loads are in flight together (registers permitting)
    for (int item0 = half; item0 < items; item0 += kAhead * kHalves) {
        uint4 pre[kAhead], pre2[kAhead];
        if (!op.xch_in) {
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int item = item0 + u * kHalves;
                if (item < items) {
                    const int m = item / op.chunks, chunk = item - m * op.chunks;
                    pre[u] = __ldcg(reinterpret_cast<const uint4*>(op.x + size_t(m) * k + chunk * 128 + hl * 8));
                }
            }
        } else {
            // Packets of the producing op: strip `sidx` of the chunk, packets g = 4*gh .. 4*gh+3 (32 bytes).
            const int sidx = hl >> 1, gh = hl & 1;
            const unsigned long long t0 = global_timer_ns();
            uint32_t valid = 0;
            bool good = true;
            for (;;) {
#pragma unroll
                for (int u = 0; u < kAhead; ++u) {
                    const int item = item0 + u * kHalves;
                    if (item < items && !(valid & (1u << u))) {
                        const int m = item / op.chunks, chunk = item - m * op.chunks;
                        const uint2* src = op.xch_in + (size_t(m) * op.in_strips + size_t(chunk) * 8 + sidx) * 8 + gh * 4;
                        pre[u] = ld_relaxed_gpu_v4(src);
                        pre2[u] = ld_relaxed_gpu_v4(src + 2);
                    }
                }
#pragma unroll
                for (int u = 0; u < kAhead; ++u) {
                    const int item = item0 + u * kHalves;
                    if (item >= items || (pre[u].y == run_tag && pre[u].w == run_tag && pre2[u].y == run_tag && pre2[u].w == run_tag))
                        valid |= 1u << u;
                }
                if (__all_sync(hmask, valid == (1u << kAhead) - 1u)) break;
                if (ctl->abort_flag || global_timer_ns() - t0 > p.wait_limit_ns) good = false;
                if (!__all_sync(hmask, good)) return false;
            }
        }
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int item = item0 + u * kHalves;
            if (item < items) {
                const int m = item / op.chunks, chunk = item - m * op.chunks;
                uint32_t bits[8];   // the lane's eight activations, bf16 bits in the high half
                int at0, at1;       // where its two byte groups go in an activation row
                if (!op.xch_in) {
                    const uint32_t w4[4] = {pre[u].x, pre[u].y, pre[u].z, pre[u].w};
#pragma unroll
                    for (int el = 0; el < 8; ++el) {
                        // element el of the octet meets byte (el&3)*2 + (el>>2) of the MMA operand
                        const int pos = (el & 3) * 2 + (el >> 2);
                        bits[pos] = (el & 1) ? (w4[el >> 1] & 0xffff0000u) : (w4[el >> 1] << 16);
                    }
                    const int tile = hl >> 3, o = hl & 7;
                    at0 = chunk * 128 + tile * 64 + (o & 3) * 16 + (o >> 2) * 8;
                    at1 = at0 + 4;
                } else {
                    // Low halves of the packets are rows R(g) of the strip (octet 2*sidx), high halves rows
                    // R(g)+8 (octet 2*sidx+1); R(0..3) = 0,4,1,5 and R(4..7) = 2,6,3,7 are exactly the
                    // element orders of the two 4-byte groups of an octet.
                    const int sidx = hl >> 1, gh = hl & 1;
                    const uint32_t d[4] = {pre[u].x, pre[u].z, pre2[u].x, pre2[u].z};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        bits[j] = d[j] << 16;               // row R(g)
                        bits[4 + j] = d[j] & 0xffff0000u;   // row R(g) + 8
                    }
                    const int oa = 2 * sidx, ob = oa + 1;
                    at0 = chunk * 128 + (oa >> 3) * 64 + (oa & 3) * 16 + ((oa & 7) >> 2) * 8 + gh * 4;
                    at1 = chunk * 128 + (ob >> 3) * 64 + (ob & 3) * 16 + ((ob & 7) >> 2) * 8 + gh * 4;
                }
                quantise_group<MBLK>(bits, hmask, at0, at1, m, chunk, hl, xb, sxb, plan);
            }
        }
    }
    return true;
}

// ---- inputs that are computed on the way in (the glue between the linears of a decoder layer)

// The eight activations a lane holds of item (m, chunk), as fp32, with the columns they
// belong to.  From memory a lane has eight consecutive columns; from exchange packets it
// has rows R(4 gh .. 4 gh + 3) of two neighbouring octets (see stage_rows).  `col_shift`
// moves the source columns (the second half of a [m, 2k] source).  Packets are polled
// until they carry the run's tag; returns false when that ran out of time.
__device__ __forceinline__ bool load_lane_values(const StreamParams& p, const StreamOp& op, Ctl* ctl, uint32_t run_tag, uint32_t hmask,
                                                 int m, int chunk, int hl, int src_cols, int col_shift, float (&v)[8], int (&col)[8])
{
    if (!op.xch_in) {
        const uint4 w = __ldcg(reinterpret_cast<const uint4*>(op.x + size_t(m) * src_cols + col_shift + chunk * 128 + hl * 8));
        const uint32_t w4[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int el = 0; el < 8; ++el) {
            const int pos = (el & 3) * 2 + (el >> 2);
            v[pos] = __uint_as_float((el & 1) ? (w4[el >> 1] & 0xffff0000u) : (w4[el >> 1] << 16));
            col[pos] = chunk * 128 + hl * 8 + el;
        }
        return true;
    }
    const int sidx = hl >> 1, gh = hl & 1;
    const uint2* src = op.xch_in + (size_t(m) * op.in_strips + size_t(col_shift >> 4) + size_t(chunk) * 8 + sidx) * 8 + gh * 4;
    const unsigned long long t0 = global_timer_ns();
    uint4 a, b;
    for (;;) {
        a = ld_relaxed_gpu_v4(src);
        b = ld_relaxed_gpu_v4(src + 2);
        const bool have = a.y == run_tag && a.w == run_tag && b.y == run_tag && b.w == run_tag;
        if (__all_sync(hmask, have)) break;
        const bool stop = ctl->abort_flag || global_timer_ns() - t0 > p.wait_limit_ns;
        if (__any_sync(hmask, stop)) return false;
    }
    const uint32_t d[4] = {a.x, a.z, b.x, b.z};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int g = 4 * gh + j;
        v[j] = __uint_as_float(d[j] << 16);              // row R(g) of the strip
        v[4 + j] = __uint_as_float(d[j] & 0xffff0000u);  // row R(g) + 8
        col[j] = chunk * 128 + sidx * 16 + row_of_g(g);
        col[4 + j] = col[j] + 8;
    }
    return true;
}

// Where a lane's two 4-byte groups go in an activation row (see stage_rows).
__device__ __forceinline__ void lane_positions(bool from_packets, int chunk, int hl, int& at0, int& at1)
{
    if (!from_packets) {
        const int tile = hl >> 3, o = hl & 7;
        at0 = chunk * 128 + tile * 64 + (o & 3) * 16 + (o >> 2) * 8;
        at1 = at0 + 4;
    } else {
        const int sidx = hl >> 1, gh = hl & 1;
        const int oa = 2 * sidx, ob = oa + 1;
        at0 = chunk * 128 + (oa >> 3) * 64 + (oa & 3) * 16 + ((oa & 7) >> 2) * 8 + gh * 4;
        at1 = chunk * 128 + (ob >> 3) * 64 + (ob & 3) * 16 + ((ob & 7) >> 2) * 8 + gh * 4;
    }
}

__device__ __forceinline__ float bf16_round_dev(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

// One item's input values after the op's own activation: plain, or
// bf16(silu(gate) * up) with gate = source[:, c] and up = source[:, k + c].  The gate and up
// values are requested together, so that an item costs one trip to L2 and not two.
__device__ __forceinline__ bool load_item_values(const StreamParams& p, const StreamOp& op, Ctl* ctl, uint32_t run_tag, uint32_t hmask,
                                                 int m, int chunk, int hl, float (&v)[8], int (&col)[8])
{
    const int k = op.chunks * 128;
    if (!(op.flags & kOpSwiGLU)) return load_lane_values(p, op, ctl, run_tag, hmask, m, chunk, hl, k, 0, v, col);
    float up[8];
    if (!op.xch_in) {
        int col_up[8];
        if (!load_lane_values(p, op, ctl, run_tag, hmask, m, chunk, hl, 2 * k, 0, v, col)) return false;
        if (!load_lane_values(p, op, ctl, run_tag, hmask, m, chunk, hl, 2 * k, k, up, col_up)) return false;
    } else {
        const int sidx = hl >> 1, gh = hl & 1;
        const uint2* gate_src = op.xch_in + (size_t(m) * op.in_strips + size_t(chunk) * 8 + sidx) * 8 + gh * 4;
        const uint2* up_src = gate_src + size_t(k >> 4) * 8;
        const unsigned long long t0 = global_timer_ns();
        uint4 a, b, c, d;
        for (;;) {
            a = ld_relaxed_gpu_v4(gate_src);
            b = ld_relaxed_gpu_v4(gate_src + 2);
            c = ld_relaxed_gpu_v4(up_src);
            d = ld_relaxed_gpu_v4(up_src + 2);
            const bool have = a.y == run_tag && a.w == run_tag && b.y == run_tag && b.w == run_tag && c.y == run_tag &&
                              c.w == run_tag && d.y == run_tag && d.w == run_tag;
            if (__all_sync(hmask, have)) break;
            const bool stop = ctl->abort_flag || global_timer_ns() - t0 > p.wait_limit_ns;
            if (__any_sync(hmask, stop)) return false;
        }
        const uint32_t g4[4] = {a.x, a.z, b.x, b.z}, u4[4] = {c.x, c.z, d.x, d.z};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[j] = __uint_as_float(g4[j] << 16);
            v[4 + j] = __uint_as_float(g4[j] & 0xffff0000u);
            up[j] = __uint_as_float(u4[j] << 16);
            up[4 + j] = __uint_as_float(u4[j] & 0xffff0000u);
            col[j] = chunk * 128 + sidx * 16 + row_of_g(4 * gh + j);
            col[4 + j] = col[j] + 8;
        }
    }
#pragma unroll
    for (int el = 0; el < 8; ++el) {
        const float g = v[el];
        const float s = __fdividef(g, 1.f + __expf(-g));
        v[el] = bf16_round_dev(__fmul_rn(s, up[el]));
    }
    return true;
}

// stage_rows for ops whose input is computed on the way in: an RMS norm over the whole
// row (x * 1/sqrt(mean(x^2) + eps) * w, rounded to bf16) and/or the SwiGLU product.
// All consumer threads call it together: the norm needs two CTA-wide meetings.
template <int MBLK>
__device__ __forceinline__ bool stage_rows_glue(const StreamParams& p, const StreamOp& op, const StreamSmem& plan, Ctl* ctl,
                                                uint8_t* xb, float* sxb, uint32_t run_tag, int tid, int lane)
{
    const int half = tid >> 4, hl = tid & 15;
    const uint32_t hmask = 0xffffu << (lane & 16);
    const int k = op.chunks * 128;
    const int items = p.m * op.chunks;
    const bool norm = (op.flags & kOpNorm) != 0, from_packets = op.xch_in != nullptr;
    const bool single = items <= kHalves;   // every half-warp has at most one item: its values stay in registers
    bool good = true;
    float v[8];
    int col[8];
    if (norm) {
        // ---- first pass: the sum of squares of every row, added in a fixed order
        for (int item = half; item < items; item += kHalves) {
            const int m = item / op.chunks, chunk = item - m * op.chunks;
            if (good && !load_item_values(p, op, ctl, run_tag, hmask, m, chunk, hl, v, col)) good = false;
            float sq = 0.f;
            if (good) {
#pragma unroll
                for (int el = 0; el < 8; ++el) sq = __fmaf_rn(v[el], v[el], sq);
            }
#pragma unroll
            for (int off = 8; off; off >>= 1) sq += __shfl_xor_sync(hmask, sq, off, 16);
            if (hl == 0) sxb[(chunk * MBLK + (m >> 2)) * 4 + (m & 3)] = sq;   // the group's slot holds its share for now
        }
        named_barrier_sync(1, kConsumerThreads);
        if (half < p.m) {
            float total = 0.f;
            for (int c = hl; c < op.chunks; c += 16) total += sxb[(c * MBLK + (half >> 2)) * 4 + (half & 3)];
#pragma unroll
            for (int off = 8; off; off >>= 1) total += __shfl_xor_sync(hmask, total, off, 16);
            if (hl == 0) ctl->row_sq[half] = total;
        }
        named_barrier_sync(1, kConsumerThreads);
    }
    for (int item = half; item < items; item += kHalves) {
        const int m = item / op.chunks, chunk = item - m * op.chunks;
        if (good && !(norm && single) && !load_item_values(p, op, ctl, run_tag, hmask, m, chunk, hl, v, col)) good = false;
        if (!good) continue;
        uint32_t bits[8];
        if (norm) {
            const float rs = 1.f / sqrtf(ctl->row_sq[m] / float(k) + op.norm_eps);
#pragma unroll
            for (int el = 0; el < 8; ++el) {
                const float w = __bfloat162float(op.norm_w[col[el]]);
                bits[el] = __float_as_uint(bf16_round_dev(__fmul_rn(__fmul_rn(v[el], rs), w)));
            }
        } else {
#pragma unroll
            for (int el = 0; el < 8; ++el) bits[el] = __float_as_uint(v[el]);
        }
        int at0, at1;
        lane_positions(from_packets, chunk, hl, at0, at1);
        quantise_group<MBLK>(bits, hmask, at0, at1, m, chunk, hl, xb, sxb, plan);
    }
    return good;
}

}  // namespace

// kGlue: the list holds ops with computed inputs or residuals (the plain instantiation carries none of that code).
template <int MBLK, bool kGlue>
__global__ void __launch_bounds__(kStreamThreads, 1) w4a16_list_kernel(const __grid_constant__ StreamParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const StreamSmem plan = stream_smem_plan(p.m, p.max_chunks, p.ring_slots, p.max_parts, p.table_in_smem ? p.count : 0, p.nbuf);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + plan.bars);
    uint64_t* empty = full + kMaxRingSlots;
    Ctl* ctl = reinterpret_cast<Ctl*>(smem + plan.ctl);
    volatile int* tags = reinterpret_cast<volatile int*>(smem + plan.tags);
    float* sx = reinterpret_cast<float*>(smem + plan.sx);
    int* pcnt = reinterpret_cast<int*>(smem + plan.pcnt);
    volatile int* pgen = reinterpret_cast<volatile int*>(smem + plan.pgen);
    float* partial = reinterpret_cast<float*>(smem + plan.partial);
    uint8_t* xq = smem + plan.xq;
    uint8_t* ring = smem + plan.ring;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NS = p.ring_slots, PS = plan.part_slots;
    const StreamOp* ops = p.ops ? p.ops : p.inline_ops;
    const unsigned long long limit = p.wait_limit_ns;
    if (p.table_in_smem) {
        // every warp reads every entry: a short table is served from shared memory
        uint4* dst = reinterpret_cast<uint4*>(smem + plan.optable);
        const uint4* src = reinterpret_cast<const uint4*>(ops);
        for (int i = threadIdx.x; i < p.count * int(sizeof(StreamOp) / 16); i += blockDim.x) dst[i] = src[i];
        ops = reinterpret_cast<const StreamOp*>(smem + plan.optable);
    }

    if (int(threadIdx.x) < NS) {   // one thread per ring stage
        mbar_init(&full[threadIdx.x], 1);
        mbar_init(&empty[threadIdx.x], 1);
        fence_barrier_init();
    }
    // control words, part counters, the all-zero activation row (the scale factors and bias
    // terms need no clearing: every entry that is read has been staged)
    for (int i = threadIdx.x; i < int(sizeof(Ctl) / 4); i += blockDim.x) reinterpret_cast<int*>(ctl)[i] = 0;
    for (int i = threadIdx.x; i < PS; i += blockDim.x) {
        pcnt[i] = 0;
        pgen[i] = 0;
    }
    for (int b = 0; b < p.nbuf; ++b)
        for (int i = threadIdx.x; i < plan.xq_stride / 16; i += blockDim.x)
            *reinterpret_cast<uint4*>(xq + size_t(b) * plan.xq_bytes + size_t(2 * p.m) * plan.xq_stride + i * 16) = make_uint4(0, 0, 0, 0);
    __syncthreads();
    pdl_launch_dependents();

    // =============================================================== producer
    if (warp == kStreamConsumerWarps) {
        // Sixteen lanes issue sixteen consecutive slots at a time: one thread alone cannot
        // issue a 4 KiB copy often enough to keep HBM busy.  A lane's slot never needs a
        // slot of the same batch to be consumed first, because the ring is deeper than
        // the batch.
        constexpr int kBatch = 16;
        if (lane >= kBatch) return;
        int q_base = 0;
        bool ok = true;
        for (int i = 0; i < p.count && ok; ++i) {
            if (p.ops && !p.table_in_smem && i + 2 < p.count) {   // the table entry is needed the moment the previous op is issued
                prefetch_l1(p.ops + i + 2);
                prefetch_l1(reinterpret_cast<const char*>(p.ops + i + 3) - 4);
            }
            const StreamOp op = ops[i];
            int s0, s1;
            op_share(op, s0, s1);
            const int ntask = (s1 - s0) * op.parts;
            const size_t strip_bytes = size_t(op.chunks) * kInt4ChunkBytes;
            for (int base = 0; base < ntask; base += kBatch) {
                const int local = base + lane;
                if (local < ntask) {
                    const int q = q_base + local;
                    const int round = q / NS, stage = q - round * NS;
                    const int sl = local / op.parts, part = local - sl * op.parts;
                    if (round > 0 && !wait_or_abort(&empty[stage], (round - 1) & 1, ctl, limit)) {
                        give_up(p, ctl, 1);
                        ok = false;
                    } else {
                        const int c0 = part * op.cpp;
                        const uint32_t bytes = uint32_t(min(op.cpp, op.chunks - c0)) * kInt4ChunkBytes;
                        tags[stage] = q;   // published by the arrive below
                        mbar_expect_tx(&full[stage], bytes);
                        bulk_g2s(ring + size_t(stage) * kSlotBytes,
                                 op.packed + size_t(s0 + sl) * strip_bytes + size_t(c0) * kInt4ChunkBytes, bytes, &full[stage]);
                    }
                }
                ok = __all_sync((1u << kBatch) - 1, ok);
                if (!ok) break;
            }
            q_base += ntask;
        }
        if (!ok || ctl->abort_flag) {
            // Someone gave up: let the copies already issued land before the CTA's shared
            // memory is released (each wait is short; a copy takes microseconds).  A
            // stage whose last copy has been consumed passes at once.
            for (int stg = lane; stg < NS; stg += kBatch) {
                if (stg >= q_base) continue;
                const int last = ((q_base - 1 - stg) / NS);   // round of the last slot issued into this stage
                (void)mbar_wait(&full[stg], last & 1, 20000000ull);
            }
        }
        return;
    }

    // ============================================================== consumers
    pdl_wait();   // x is produced, and y may still be read, by earlier work in the stream
    const int g = lane >> 2, t = lane & 3;
    const uint32_t run_tag = p.has_deps ? uint32_t(*reinterpret_cast<volatile int*>(p.epoch)) : 0u;
    int q_base = 0;
    // Slots are handed out in order to whichever warp is free (a shared counter): a
    // slow warp then never holds up the ring while others idle.  my_q = the slot this
    // warp has taken and not yet processed, or -1.
    int my_q = -1;
    const uint8_t* xcol[MBLK];
    const float* sxb = sx;
    bool ok = true;
    for (int i = 0; i < p.count; ++i) {
        const StreamOp& op = ops[i];   // read where it lies (shared memory or the parameter bank): no registers held
        {
            const int buf = (op.flags & kOpBuffer1) ? 1 : 0;
            uint8_t* xb = xq + size_t(buf) * plan.xq_bytes;
            sxb = sx + size_t(buf) * p.max_chunks * MBLK * 4;
#pragma unroll
            for (int mb = 0; mb < MBLK; ++mb) {
                const int r = mb * 8 + g;
                xcol[mb] = xb + size_t(r < 2 * p.m ? r : 2 * p.m) * plan.xq_stride + t * 16;
            }
            if (!(op.flags & kOpSameX)) {
                // Every warp has finished with the rows this buffer held; then all stage the new
                // ones.  (A warp that gave up keeps meeting the others at these barriers.)
                if (threadIdx.x == 0) GB_TRACE(i, 0);
                named_barrier_sync(1, kConsumerThreads);
                if (threadIdx.x == 0) GB_TRACE(i, 1);
                if (kGlue && (op.flags & (kOpNorm | kOpSwiGLU))) {
                    // every thread takes part (the norm meets twice); one that has given up only keeps the meetings
                    if (!stage_rows_glue<MBLK>(p, op, plan, ctl, xb, const_cast<float*>(sxb), run_tag, threadIdx.x, lane) &&
                        (lane & 15) == 0)
                        give_up(p, ctl, 3);
                } else if (ok && !ctl->abort_flag &&
                           !stage_rows<MBLK>(p, op, plan, ctl, xb, const_cast<float*>(sxb), run_tag, threadIdx.x, lane)) {
                    if ((lane & 15) == 0) give_up(p, ctl, 3);
                }
                named_barrier_sync(1, kConsumerThreads);
                if (threadIdx.x == 0) GB_TRACE(i, 2);
                if (ctl->abort_flag) ok = false;
            }
        }
        int s0, s1;
        op_share(op, s0, s1);
        const int ntask = (s1 - s0) * op.parts, q_end = q_base + ntask;
        while (ok) {
            if (my_q < 0) {
                if (lane == 0) my_q = atomicAdd(&ctl->next_slot, 1);
                my_q = __shfl_sync(0xffffffffu, my_q, 0);
            }
            if (my_q >= q_end) break;   // a slot of a later linear: kept until this warp gets there
            const int local = my_q - q_base;
            const int sl = int((unsigned long long)(unsigned)local * op.inv_parts >> 40);
            const int part = local - sl * op.parts;
            const int round = int((unsigned long long)(unsigned)my_q * p.inv_ring >> 40), stage = my_q - round * NS;
            const int phase = round & 1;
            const int pround = int((unsigned long long)(unsigned)my_q * p.inv_pslots >> 40);
            const int pslot = my_q - pround * PS;
            // A parity wait alone cannot tell this slot's phase from the phase two rounds
            // earlier: the stage's tag says which slot the completed phase carried.
            if (!mbar_try_wait(&full[stage], phase) || tags[stage] != my_q) {
                const unsigned long long t0 = global_timer_ns();
                while (ok) {
                    if (!wait_or_abort(&full[stage], phase, ctl, limit)) ok = false;
                    else if (tags[stage] == my_q) break;
                    else if (global_timer_ns() - t0 > limit) ok = false;
                }
                if (!ok) {
                    if (lane == 0) give_up(p, ctl, 2);
                    break;
                }
            }
            if (lane == 0 && local == 0) GB_TRACE(i, 3);
            if (lane == 0 && local == ntask - 1) GB_TRACE(i, 6);
            const uint8_t* slot = ring + size_t(stage) * kSlotBytes;
            const int c_first = part * op.cpp;
            const int nch = min(op.cpp, op.chunks - c_first);
            // The residual that the strip's writer will add is requested now: by the time the
            // sums are complete it has arrived (only the warp that delivers the last part uses it).
            const int strip = s0 + sl;
            const int n_lo = strip * 16 + row_of_g(g), n_hi = n_lo + 8;
            float res_lo[MBLK], res_hi[MBLK];
            uint2 res_pk[MBLK];
            if (kGlue && (op.flags & kOpResidual)) {
#pragma unroll
                for (int mb = 0; mb < MBLK; ++mb) {
                    const int m = mb * 4 + t;
                    res_lo[mb] = (m < p.m && n_lo < op.n) ? __bfloat162float(op.res[size_t(m) * op.ldy + n_lo]) : 0.f;
                    res_hi[mb] = (m < p.m && n_hi < op.n) ? __bfloat162float(op.res[size_t(m) * op.ldy + n_hi]) : 0.f;
                }
            } else if (kGlue && (op.flags & kOpResidualXch)) {
#pragma unroll
                for (int mb = 0; mb < MBLK; ++mb) {
                    const int m = mb * 4 + t;
                    res_pk[mb] = m < p.m ? ld_relaxed_gpu_v2(op.res_xch + (size_t(m) * op.strips + strip) * 8 + g) : make_uint2(0, run_tag);
                }
            }
            // The fp32 sum over the chunks follows one fixed tree whatever the split into
            // parts: groups of four chunks G = (s0 + s1) + (s2 + s3), then the groups in
            // order.  pr[..][0] collects s0 + s1, pr[..][1] collects s2 + s3 of this part.
            float pr[MBLK][2][2];
#pragma unroll
            for (int mb = 0; mb < MBLK; ++mb) pr[mb][0][0] = pr[mb][0][1] = pr[mb][1][0] = pr[mb][1][1] = 0.f;
#pragma unroll
            for (int c = 0; c < kSlotChunks; ++c) {
                if (c >= nch) break;
                const uint8_t* ck = slot + c * kInt4ChunkBytes;
                const int chunk = c_first + c;
                const uint4 u0 = *reinterpret_cast<const uint4*>(ck + lane * 16);
                const uint4 u1 = *reinterpret_cast<const uint4*>(ck + 512 + lane * 16);
                const uint32_t sc = *reinterpret_cast<const uint32_t*>(ck + 1024 + g * 4);
                float s_lo, s_hi;
                if (op.flags & kOpScaleFp16) {
                    s_lo = __half2float(__ushort_as_half(uint16_t(sc & 0xffffu)));
                    s_hi = __half2float(__ushort_as_half(uint16_t(sc >> 16)));
                } else {
                    s_lo = __uint_as_float(sc << 16);
                    s_hi = __uint_as_float(sc & 0xffff0000u);
                }
                // the chunk's 128 codes as signed bytes, once; then one block of four batch rows after the
                // other (few registers live at a time: with several blocks in flight the kernel spilled)
                uint32_t a[2][2][4];
#pragma unroll
                for (int tile = 0; tile < 2; ++tile) {
                    const uint4 u = tile ? u1 : u0;
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const uint32_t w_lo = jj ? u.z : u.x, w_hi = jj ? u.w : u.y;
                        a[tile][jj][0] = nib_to_s8x16(w_lo << 4), a[tile][jj][1] = nib_to_s8x16(w_hi << 4);
                        a[tile][jj][2] = nib_to_s8x16(w_lo), a[tile][jj][3] = nib_to_s8x16(w_hi);
                    }
                }
#pragma unroll
                for (int mb = 0; mb < MBLK; ++mb) {
                    int acc_i[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int tile = 0; tile < 2; ++tile) {
                        const uint4 xv = *reinterpret_cast<const uint4*>(xcol[mb] + chunk * 128 + tile * 64);
                        imma_s8s8(acc_i, a[tile][0][0], a[tile][0][1], a[tile][0][2], a[tile][0][3], xv.x, xv.y);
                        imma_s8s8(acc_i, a[tile][1][0], a[tile][1][1], a[tile][1][2], a[tile][1][3], xv.z, xv.w);
                    }
                    const float f = sxb[(chunk * MBLK + mb) * 4 + t];
                    const int v0 = acc_i[0] * 128 + acc_i[1];   // hi and lo pieces of batch row 4*mb + t
                    const int v1 = acc_i[2] * 128 + acc_i[3];
                    // explicit roundings: no multiply-add contraction, so the bits do not depend on
                    // how the compiler arranges this loop
                    const float c_lo = __fmul_rn(__fmul_rn(float(v0), f), s_lo), c_hi = __fmul_rn(__fmul_rn(float(v1), f), s_hi);
                    pr[mb][0][c >> 1] = __fadd_rn(pr[mb][0][c >> 1], c_lo);
                    pr[mb][1][c >> 1] = __fadd_rn(pr[mb][1][c >> 1], c_hi);
                }
            }
            float acc[MBLK][2];
#pragma unroll
            for (int mb = 0; mb < MBLK; ++mb) {
                acc[mb][0] = __fadd_rn(pr[mb][0][0], pr[mb][0][1]);
                acc[mb][1] = __fadd_rn(pr[mb][1][0], pr[mb][1][1]);
            }

            // ---- the parts of a strip meet in shared memory
            bool writer = op.parts == 1;
            if (op.parts > 1) {
                int pbase = pslot - part;             // slot of the strip's first part
                int bround = pround;
                if (pbase < 0) {
                    pbase += PS;
                    --bround;
                }
                // A partial-sum slot (and the strip's counter) is taken again PS slots later.  The
                // ring's depth makes that far away in time, but only this generation count makes
                // it certain that the strip which used them before has been added up.
                if (!__all_sync(0xffffffffu, pgen[pslot] == pround && pgen[pbase] == bround)) {
                    const unsigned long long t0 = global_timer_ns();
                    for (;;) {
                        if (__all_sync(0xffffffffu, pgen[pslot] == pround && pgen[pbase] == bround)) break;
                        if (__any_sync(0xffffffffu, ctl->abort_flag || global_timer_ns() - t0 > limit)) {
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) {
                        if (lane == 0) give_up(p, ctl, 4);
                        break;
                    }
                }
                __threadfence_block();
                float* mine = partial + size_t(pslot) * (MBLK * 64);
#pragma unroll
                for (int mb = 0; mb < MBLK; ++mb)
                    *reinterpret_cast<float2*>(mine + mb * 64 + lane * 2) = make_float2(acc[mb][0], acc[mb][1]);
                __syncwarp();
                int arrived = 0;
                if (lane == 0) {
                    __threadfence_block();
                    arrived = atomicAdd(&pcnt[pbase], 1);
                }
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived == op.parts - 1) {
                    __threadfence_block();
#pragma unroll
                    for (int mb = 0; mb < MBLK; ++mb) acc[mb][0] = acc[mb][1] = 0.f;
                    // groups of 4 / cpp parts are added as a pair of pairs first (the same tree as
                    // inside a four-chunk part), then the groups in order
                    const int gs = kSlotChunks / op.cpp;
                    int pj = pbase;
                    for (int j0 = 0; j0 < op.parts; j0 += gs) {
                        float grp[MBLK][2][2];
#pragma unroll
                        for (int mb = 0; mb < MBLK; ++mb) grp[mb][0][0] = grp[mb][0][1] = grp[mb][1][0] = grp[mb][1][1] = 0.f;
                        for (int jj = 0; jj < gs && j0 + jj < op.parts; ++jj) {
                            const float* theirs = partial + size_t(pj) * (MBLK * 64);
                            if (++pj == PS) pj = 0;
                            const int side = gs == 4 ? (jj >> 1) : jj;   // which pair of the group this part belongs to
#pragma unroll
                            for (int mb = 0; mb < MBLK; ++mb) {
                                const float2 v = *reinterpret_cast<const float2*>(theirs + mb * 64 + lane * 2);
                                if (side) {
                                    grp[mb][0][1] = __fadd_rn(grp[mb][0][1], v.x);
                                    grp[mb][1][1] = __fadd_rn(grp[mb][1][1], v.y);
                                } else {
                                    grp[mb][0][0] = __fadd_rn(grp[mb][0][0], v.x);
                                    grp[mb][1][0] = __fadd_rn(grp[mb][1][0], v.y);
                                }
                            }
                        }
#pragma unroll
                        for (int mb = 0; mb < MBLK; ++mb) {
                            acc[mb][0] = __fadd_rn(acc[mb][0], __fadd_rn(grp[mb][0][0], grp[mb][0][1]));
                            acc[mb][1] = __fadd_rn(acc[mb][1], __fadd_rn(grp[mb][1][0], grp[mb][1][1]));
                        }
                    }
                    if (lane == 0) pcnt[pbase] = 0;
                    __threadfence_block();
                    __syncwarp();
                    for (int j = lane; j < op.parts; j += 32) {   // the strip's slots and counter may be taken again
                        int idx = pbase + j;
                        if (idx >= PS) idx -= PS;
                        pgen[idx] = pgen[idx] + 1;
                    }
                    writer = true;
                }
            }
            if (writer) {
#pragma unroll
                for (int mb = 0; mb < MBLK; ++mb) {
                    const int m = mb * 4 + t;
                    if (m < p.m) {
                        if (kGlue && (op.flags & kOpResidual)) {
                            acc[mb][0] = __fadd_rn(acc[mb][0], res_lo[mb]);
                            acc[mb][1] = __fadd_rn(acc[mb][1], res_hi[mb]);
                        } else if (kGlue && (op.flags & kOpResidualXch)) {
                            // the packet of (m, strip, g) holds exactly this lane's two columns
                            uint2 pk = res_pk[mb];
                            if (pk.y != run_tag) {
                                const uint2* src = op.res_xch + (size_t(m) * op.strips + strip) * 8 + g;
                                const unsigned long long t0 = global_timer_ns();
                                while (pk.y != run_tag && !ctl->abort_flag && global_timer_ns() - t0 <= limit) pk = ld_relaxed_gpu_v2(src);
                                if (pk.y != run_tag) give_up(p, ctl, 5);
                            }
                            acc[mb][0] = __fadd_rn(acc[mb][0], __uint_as_float(pk.x << 16));
                            acc[mb][1] = __fadd_rn(acc[mb][1], __uint_as_float(pk.x & 0xffff0000u));
                        }
                        const __nv_bfloat16 y_lo = __float2bfloat16_rn(acc[mb][0]), y_hi = __float2bfloat16_rn(acc[mb][1]);
                        if (n_lo < op.n) op.y[size_t(m) * op.ldy + n_lo] = y_lo;
                        if (n_hi < op.n) op.y[size_t(m) * op.ldy + n_hi] = y_hi;
                        if (op.xch_out)   // data and tag in one 8-byte store
                            st_relaxed_gpu_v2(op.xch_out + (size_t(m) * op.strips + strip) * 8 + g,
                                              uint32_t(__bfloat16_as_ushort(y_lo)) | (uint32_t(__bfloat16_as_ushort(y_hi)) << 16),
                                              run_tag);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) GB_TRACE_MAX(i, writer ? 5 : 4);
            if (lane == 0) mbar_arrive(&empty[stage]);
            my_q = -1;
        }
        q_base = q_end;
    }
    if (p.has_deps) {
        // The CTA whose last consumer warp finishes last of all moves the run tag on, so
        // that the next run does not take this run's packets for its own.  Every poll of
        // every CTA is over by then.
        __syncwarp();
        if (lane == 0 && atomicAdd(&ctl->warps_done, 1) == kStreamConsumerWarps - 1) {
            __threadfence();
            if (atomicAdd(p.finish, 1) == int(gridDim.x) - 1) {
                *reinterpret_cast<volatile int*>(p.epoch) = int(run_tag + 1u);
                *reinterpret_cast<volatile int*>(p.finish) = 0;
                __threadfence();
            }
        }
    }
}

// ------------------------------------------------------------------ host side

constexpr size_t kMaxDynamicSmem = 227 * 1024;

static unsigned long long stream_wait_limit_ns()
{
    // GARNET_B200_WAIT_LIMIT_MS shortens (or lengthens) the limit of every device-side
    // wait of this kernel; read once.
    static const unsigned long long ns = [] {
        const char* e = getenv("GARNET_B200_WAIT_LIMIT_MS");
        const long ms = e ? atol(e) : 0;
        return ms > 0 ? (unsigned long long)ms * 1000000ull : kWaitLimitNs;
    }();
    return ns;
}

// Largest batch one launch takes for a given K: the int8 pieces of the rows must leave
// room for a useful ring.
int stream_max_rows(int chunks)
{
    for (int m = 16; m >= 1; m >>= 1)
        if (size_t(2 * m + 1) * size_t(chunks * 128 + 64) <= 112 * 1024) return m;
    return 0;
}

// Chooses buffers and ring depth for a list; returns false when it does not fit.
static bool stream_fit(int m, int max_chunks, int max_parts, int table_ops, int nbuf, int* ring_slots)
{
    for (int slots = kMaxRingSlots; slots >= 20; --slots)
        if (size_t(stream_smem_plan(m, max_chunks, slots, max_parts, table_ops, nbuf).total) <= kMaxDynamicSmem) {
            *ring_slots = slots;
            return true;
        }
    return false;
}

// Splits the K dimension of an op into parts so that the list keeps every consumer
// warp of every SM busy: about eight slots per SM at least.
static void finish_op(StreamOp& op, int grid)
{
    op.base_strips = op.strips / grid;
    op.rem_strips = op.strips % grid;
    op.inv_parts = ((1ull << 40) + op.parts - 1) / op.parts;
}

static void choose_parts(StreamOp& op, int total_strips_hint)
{
    static const int per_sm = [] {
        const char* e = getenv("GARNET_B200_STREAM_TASKS_PER_SM");   // A/B switch, read once
        return e && atoi(e) > 0 ? atoi(e) : 8;
    }();
    const int want_tasks = kSmCount * per_sm;
    int cpp = kSlotChunks;
    while (cpp > 1 && (long long)total_strips_hint * ((op.chunks + cpp - 1) / cpp) < want_tasks) cpp >>= 1;
    op.cpp = cpp;
    op.parts = (op.chunks + cpp - 1) / cpp;
}

static int launch_list(StreamParams p, int grid, unsigned flags, cudaStream_t stream)
{
    const unsigned long long one = 1ull << 40;
    p.inv_ring = (one + p.ring_slots - 1) / p.ring_slots;
    p.inv_pslots = (one + (p.ring_slots + p.max_parts) - 1) / (p.ring_slots + p.max_parts);
    const size_t smem = size_t(stream_smem_plan(p.m, p.max_chunks, p.ring_slots, p.max_parts, p.table_in_smem ? p.count : 0, p.nbuf).total);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & 1u) ? 1 : 0;
    const int mblk = stream_mblk(p.m);
    if (p.has_glue) {
        if (mblk == 1) GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_list_kernel<1, true>, p));
        else if (mblk == 2) GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_list_kernel<2, true>, p));
        else GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_list_kernel<4, true>, p));
    } else {
        if (mblk == 1) GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_list_kernel<1, false>, p));
        else if (mblk == 2) GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_list_kernel<2, false>, p));
        else GB_CUDA(cudaLaunchKernelEx(&cfg, w4a16_list_kernel<4, false>, p));
    }
    return GARNET_B200_OK;
}

int stream_set_attributes()
{
    GB_CUDA(cudaFuncSetAttribute(w4a16_list_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMaxDynamicSmem)));
    GB_CUDA(cudaFuncSetAttribute(w4a16_list_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMaxDynamicSmem)));
    GB_CUDA(cudaFuncSetAttribute(w4a16_list_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMaxDynamicSmem)));
    GB_CUDA(cudaFuncSetAttribute(w4a16_list_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMaxDynamicSmem)));
    GB_CUDA(cudaFuncSetAttribute(w4a16_list_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMaxDynamicSmem)));
    GB_CUDA(cudaFuncSetAttribute(w4a16_list_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMaxDynamicSmem)));
    return GARNET_B200_OK;
}

static StreamOp make_op(const W4A16* h, const __nv_bfloat16* x, __nv_bfloat16* y, int ldy)
{
    StreamOp op = {};
    op.packed = h->packed;
    op.x = x;
    op.y = y;
    op.n = h->geo.rows;
    op.ldy = ldy;
    op.strips = h->geo.strips;
    op.chunks = h->geo.chunks;
    op.dep = -1;
    op.flags = h->scale_dtype == GARNET_B200_FP16 ? kOpScaleFp16 : 0;
    return op;
}

// One launch for up to kMaxInlineOps linears that read the same x.
int W4A16::launch_stream_group(W4A16* const* hs, int count, const __nv_bfloat16* x, __nv_bfloat16* const* ys,
                               const int* ldys, int m, unsigned flags, cudaStream_t stream)
{
    StreamParams p = {};
    int total_strips = 0, max_strips = 0;
    for (int g = 0; g < count; ++g) total_strips += hs[g]->geo.strips;
    int first = 0;
    for (int g = 0; g < count; ++g) {
        StreamOp op = make_op(hs[g], x, ys[g], ldys[g]);
        if (g > 0) op.flags |= kOpSameX;
        choose_parts(op, total_strips);
        op.first_cta = first % kSmCount;
        first += op.strips;
        max_strips = std::max(max_strips, op.strips);
        p.inline_ops[g] = op;
    }
    p.nbuf = 1;
    p.ops = nullptr;
    p.count = count;
    p.m = m;
    p.max_chunks = hs[0]->geo.chunks;
    p.fault = hs[0]->fault_dev;
    p.wait_limit_ns = stream_wait_limit_ns();
    for (int g = 0; g < count; ++g) p.max_parts = std::max(p.max_parts, p.inline_ops[g].parts);
    if (!stream_fit(m, p.max_chunks, p.max_parts, 0, 1, &p.ring_slots))
        return fail(GARNET_B200_NOT_SUPPORTED, "w4a16: batch %d with k=%d does not fit shared memory", m, hs[0]->geo.cols);
    const int grid = std::min(kSmCount, max_strips);
    for (int g = 0; g < count; ++g) {
        p.inline_ops[g].first_cta %= grid;
        finish_op(p.inline_ops[g], grid);
    }
    return launch_list(p, grid, flags, stream);
}

int W4A16::launch_stream(const __nv_bfloat16* x, __nv_bfloat16* y, int m, int ldy, unsigned flags, cudaStream_t stream)
{
    W4A16* one[1] = {this};
    __nv_bfloat16* ys[1] = {y};
    const int ldys[1] = {ldy};
    return launch_stream_group(one, 1, x, ys, ldys, m, flags, stream);
}

// ------------------------------------------------------------- prepared lists

struct LinearList {
    StreamParams params{};
    StreamOp* d_ops = nullptr;
    int* d_counters = nullptr;    // run tag (epoch) and finished-CTA counter
    uint2* d_exchange = nullptr;  // exchange packets of every op that a later op consumes
    int* fault_host = nullptr;
    int grid = 0;
    ~LinearList()
    {
        if (d_ops) cudaFree(d_ops);
        if (d_counters) cudaFree(d_counters);
        if (d_exchange) cudaFree(d_exchange);
        if (fault_host) cudaFreeHost(fault_host);
    }
};

}  // namespace gb200

using namespace gb200;

extern "C" {

static int list_create_impl(const garnet_b200_w4a16_list_item* items, int count, int m, garnet_b200_w4a16_list_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: null output");
    *out = nullptr;
    if (!items || count <= 0 || m <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: bad argument");
    std::vector<StreamOp> ops(static_cast<size_t>(count));
    std::vector<const void*> d_xs(static_cast<size_t>(count));
    int max_chunks = 0, max_strips = 0, l_nbuf = 1;
    bool has_deps = false, has_glue = false;
    for (int i = 0; i < count; ++i) {
        const garnet_b200_w4a16_list_item& it = items[i];
        const W4A16* h = reinterpret_cast<const W4A16*>(it.linear);
        if (!h || !it.d_x || !it.d_y)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: null handle, x or y at index %d", i);
        if (reinterpret_cast<uintptr_t>(it.d_x) & 15)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: x of linear %d must be 16-byte aligned", i);
        const int dep = it.dep;
        if (dep >= i || dep < -1)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: linear %d may only depend on an earlier linear (got %d)", i, dep);
        if (m > stream_max_rows(h->geo.chunks))
            return fail(GARNET_B200_NOT_SUPPORTED, "w4a16_list_create: batch %d is too large for k=%d in a list (at most %d)", m,
                        h->geo.cols, stream_max_rows(h->geo.chunks));
        if (it.activation != 0 && it.activation != 1)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: activation of linear %d must be 0 or 1", i);
        if (it.activation && it.d_norm_weight)
            return fail(GARNET_B200_NOT_SUPPORTED, "w4a16_list_create: linear %d asks for a norm and an activation on the same input", i);
        d_xs[i] = it.d_x;
        ops[i] = make_op(h, static_cast<const __nv_bfloat16*>(it.d_x), static_cast<__nv_bfloat16*>(it.d_y), h->geo.rows);
        ops[i].dep = dep;
        const int in_cols = it.activation ? 2 * h->geo.cols : h->geo.cols;   // columns of the source rows
        if (dep >= 0) {
            if (it.d_x != items[dep].d_y || ops[dep].n != in_cols)
                return fail(GARNET_B200_INVALID_VALUE,
                            "w4a16_list_create: linear %d depends on linear %d, so its x must be that linear's y (n=%d, needs %d)", i,
                            dep, ops[dep].n, in_cols);
            ops[dep].flags |= kOpSignal;
            has_deps = true;
        }
        if (it.activation) ops[i].flags |= kOpSwiGLU;
        if (it.d_norm_weight) {
            if (!(it.norm_eps > 0.f)) return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: norm_eps of linear %d must be positive", i);
            ops[i].flags |= kOpNorm;
            ops[i].norm_w = static_cast<const __nv_bfloat16*>(it.d_norm_weight);
            ops[i].norm_eps = it.norm_eps;
        }
        if (it.d_residual && it.residual_dep >= 0)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: linear %d names two residuals", i);
        if (it.d_residual) {
            ops[i].flags |= kOpResidual;
            ops[i].res = static_cast<const __nv_bfloat16*>(it.d_residual);
        } else if (it.residual_dep >= 0) {
            if (it.residual_dep >= i || ops[it.residual_dep].n != ops[i].n)
                return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: the residual of linear %d must be an earlier linear with the same n", i);
            ops[i].flags |= kOpResidualXch;
            ops[it.residual_dep].flags |= kOpSignal;
            has_deps = true;
        } else if (it.residual_dep < -1) {
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: residual_dep of linear %d must be -1 or an earlier index", i);
        }
        if (ops[i].flags & (kOpSwiGLU | kOpNorm | kOpResidual | kOpResidualXch)) has_glue = true;
        // (which activation buffer the rows go to, and whether they are already there, is decided below)
        max_chunks = std::max(max_chunks, ops[i].chunks);
        max_strips = std::max(max_strips, ops[i].strips);
    }
    // Two activation buffers (when they fit) hold the rows staged most recently: an op whose
    // rows - same pointer, same K, no dependency of their own to wait for - are still
    // in a buffer does not stage them again.  Rows that come from an earlier linear of
    // the list are always staged: they change from run to run.
    {
        const size_t xq_bytes = size_t(2 * m + 1) * size_t(max_chunks * 128 + 64);
        const int nbuf = 2 * xq_bytes <= 80 * 1024 ? 2 : 1;
        // what a buffer holds: the source rows, their width, and how they were transformed on the way in
        struct Held { const void* x; int chunks; const void* norm_w; int act; };
        Held held[2] = {{nullptr, 0, nullptr, 0}, {nullptr, 0, nullptr, 0}};
        int last_use[2] = {-1, -1};
        for (int i = 0; i < count; ++i) {
            int buf = -1;
            const Held want = {d_xs[i], ops[i].chunks, ops[i].norm_w, ops[i].flags & kOpSwiGLU};
            if (ops[i].dep < 0 || (i > 0 && ops[i].dep == ops[i - 1].dep && d_xs[i] == d_xs[i - 1]))
                for (int b = 0; b < nbuf; ++b)
                    if (held[b].x == want.x && held[b].chunks == want.chunks && held[b].norm_w == want.norm_w && held[b].act == want.act)
                        buf = b;
            if (buf >= 0) {
                ops[i].flags |= kOpSameX;
            } else {
                buf = (nbuf == 2 && last_use[1] < last_use[0]) ? 1 : 0;   // the buffer used longest ago
                held[buf] = want;
            }
            last_use[buf] = i;
            if (buf == 1) ops[i].flags |= kOpBuffer1;
        }
        l_nbuf = nbuf;
    }
    // ops that share their rows are one group for the purpose of splitting K
    for (int i = 0; i < count;) {
        int j = i + 1, strips = ops[i].strips;
        while (j < count && (ops[j].flags & kOpSameX)) strips += ops[j++].strips;
        for (int q = i; q < j; ++q) choose_parts(ops[q], strips);
        i = j;
    }
    std::unique_ptr<LinearList> l(new (std::nothrow) LinearList);
    if (!l) return fail(GARNET_B200_OUT_OF_MEMORY, "w4a16_list_create: host allocation failed");
    l->grid = std::min(kSmCount, max_strips);
    long long first = 0;
    for (int i = 0; i < count; ++i) {
        ops[i].first_cta = int(first % l->grid);
        first += ops[i].strips;
        finish_op(ops[i], l->grid);
    }
    StreamParams& p = l->params;
    p.count = count;
    p.m = m;
    p.max_chunks = max_chunks;
    p.has_deps = has_deps ? 1 : 0;
    p.has_glue = has_glue ? 1 : 0;
    p.nbuf = l_nbuf;
    p.wait_limit_ns = stream_wait_limit_ns();
    for (int i = 0; i < count; ++i) p.max_parts = std::max(p.max_parts, ops[i].parts);
    p.table_in_smem = count <= kMaxSmemOps ? 1 : 0;
    if (!stream_fit(m, max_chunks, p.max_parts, p.table_in_smem ? count : 0, p.nbuf, &p.ring_slots)) {
        p.table_in_smem = 0;   // a long K leaves no room for the table: read it from global memory
    }
    if (!p.table_in_smem && !stream_fit(m, max_chunks, p.max_parts, 0, p.nbuf, &p.ring_slots))
        return fail(GARNET_B200_NOT_SUPPORTED, "w4a16_list_create: batch %d with k=%d does not fit shared memory", m, max_chunks * 128);
    GB_CUDA(cudaMalloc(&l->d_counters, sizeof(int) * 2));
    const int counters_init[2] = {1, 0};   // first run tag 1 (the packets start as zeros), no CTA finished
    GB_CUDA(cudaMemcpy(l->d_counters, counters_init, sizeof(counters_init), cudaMemcpyHostToDevice));
    if (has_deps) {
        size_t packets = 0;
        std::vector<size_t> at(static_cast<size_t>(count), 0);
        for (int i = 0; i < count; ++i)
            if (ops[i].flags & kOpSignal) {
                at[i] = packets;
                packets += size_t(m) * ops[i].strips * 8;
            }
        GB_CUDA(cudaMalloc(&l->d_exchange, packets * sizeof(uint2)));
        GB_CUDA(cudaMemset(l->d_exchange, 0, packets * sizeof(uint2)));
        for (int i = 0; i < count; ++i) {
            if (ops[i].flags & kOpSignal) ops[i].xch_out = l->d_exchange + at[i];
            if (ops[i].dep >= 0) {
                ops[i].xch_in = l->d_exchange + at[ops[i].dep];
                ops[i].in_strips = ops[ops[i].dep].strips;
            }
            if (ops[i].flags & kOpResidualXch) ops[i].res_xch = l->d_exchange + at[items[i].residual_dep];
        }
    }
    GB_CUDA(cudaMalloc(&l->d_ops, sizeof(StreamOp) * size_t(count + 2)));   // two entries of slack for the table prefetch
    GB_CUDA(cudaMemset(l->d_ops, 0, sizeof(StreamOp) * size_t(count + 2)));
    GB_CUDA(cudaMemcpy(l->d_ops, ops.data(), sizeof(StreamOp) * size_t(count), cudaMemcpyHostToDevice));
    GB_CUDA(cudaHostAlloc(&l->fault_host, sizeof(int), cudaHostAllocMapped));
    *l->fault_host = 0;
    GB_CUDA(cudaHostGetDevicePointer(&p.fault, l->fault_host, 0));
    p.ops = l->d_ops;
    p.epoch = l->d_counters;
    p.finish = l->d_counters + 1;
    if (int rc = stream_set_attributes()) return rc;
    *out = reinterpret_cast<garnet_b200_w4a16_list_t>(l.release());
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_list_create(const garnet_b200_w4a16_t* handles, const void* const* d_xs, void* const* d_ys,
                                  const int* deps, int count, int m, garnet_b200_w4a16_list_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: null output");
    *out = nullptr;
    if (!handles || !d_xs || !d_ys || count <= 0 || m <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_create: bad argument");
    std::vector<garnet_b200_w4a16_list_item> items(static_cast<size_t>(count));
    for (int i = 0; i < count; ++i) {
        items[i] = garnet_b200_w4a16_list_item{};
        items[i].linear = handles[i];
        items[i].d_x = d_xs[i];
        items[i].d_y = d_ys[i];
        items[i].dep = deps ? deps[i] : -1;
        items[i].residual_dep = -1;
    }
    return list_create_impl(items.data(), count, m, out);
}

int garnet_b200_w4a16_list_create_ex(const garnet_b200_w4a16_list_item* items, int count, int m, garnet_b200_w4a16_list_t* out)
{
    return list_create_impl(items, count, m, out);
}

int garnet_b200_w4a16_list_run(garnet_b200_w4a16_list_t ll, unsigned flags, void* stream)
{
    LinearList* l = reinterpret_cast<LinearList*>(ll);
    if (!l) return fail(GARNET_B200_INVALID_VALUE, "w4a16_list_run: null list");
    // Linears that wait for one another need every CTA of the grid on the GPU at the same
    // time; with a programmatic dependent launch the grid may start while the previous
    // kernel still holds SMs, which only delays it (that kernel does not wait for this one).
    return launch_list(l->params, l->grid, flags, static_cast<cudaStream_t>(stream));
}

int garnet_b200_w4a16_list_fault(garnet_b200_w4a16_list_t ll)
{
    LinearList* l = reinterpret_cast<LinearList*>(ll);
    return l && l->fault_host ? *l->fault_host : -1;
}

#ifdef GB_STREAM_TRACE
int garnet_b200_w4a16_trace(unsigned long long* out, int n)
{
    GB_CUDA(cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * size_t(n)));
    static unsigned long long zeros[512];
    GB_CUDA(cudaMemcpyToSymbol(g_trace, zeros, sizeof(zeros)));
    return 0;
}
#endif

void garnet_b200_w4a16_list_destroy(garnet_b200_w4a16_list_t ll) { delete reinterpret_cast<LinearList*>(ll); }

}  // extern "C"
