// Expert-parallel gpt-oss MoE over the ranks of one node: tokens are split over the
// ranks, experts live in contiguous blocks (experts / world per rank), and the routed
// rows travel to the rank that owns their expert and back - all of it on the device.
//
//   route (this rank's tokens)  ->  plan: position of every routed row in the region this
//   rank owns inside its destination's receive buffer  ->  push: every row (bf16) and
//   its expert id are stored into the destination GPU's own memory, then the row count
//   and a "ready" flag  ->  the owner waits (bounded) for the flags of all sources,
//   marks the unused rows of the fixed-capacity regions, and runs the experts on what
//   it received (garnet_b200_moe_run_rows)  ->  the per-row values go back as bf16 the
//   same way (they are bf16-valued, so the wire format is exact)  ->  the source waits
//   for all owners and combines in router order.
//
// The receive regions have a fixed capacity per source (tokens_local_max * top_k rows),
// so no count has to be known before the data moves and there is no host
// synchronisation anywhere.  The GEMM operands are always in local memory; peers are
// only ever written to with plain stores.  A step's return flags double as the
// permission to overwrite the receive buffers in the next step (an owner has finished
// with its rows when its values arrive).
//
// The reference shards experts over two ranks with replicated tokens and an all-reduce
// (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:771,818; tp_collective.cpp:77-98); this is the
// token-exchanging form for up to eight ranks, with the single-GPU operator's results.
#include <algorithm>
#include <new>

#include "comm.h"
#include "common.cuh"
#include "moe.h"

namespace gb200 {

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool wait_epoch(const uint32_t* flag, uint32_t epoch, unsigned long long limit_ns)
{
    if (ld_acquire_sys(flag) == epoch) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int spin = 0; spin < 64; ++spin)
            if (ld_acquire_sys(flag) == epoch) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
}

}  // namespace

struct EpDev {
    uint8_t* peer_base[kCommMaxRanks];
    size_t flags_off;        // dispatch_ready[8], return_ready[8] (uint32), counts[8] (int): written by peers
    size_t rows_off;         // [world][cap][hidden] bf16: rows received from each source
    size_t expert_off;       // [world][cap] int32: their expert ids
    size_t ret_off;          // [world][cap][hidden] bf16: values returned by each owner
    uint32_t* seq;           // local: epoch of the last finished step
    uint32_t* counters;      // local: [0] CTAs done pushing, [1] CTAs done returning
    int* send_idx;           // local [slots]: position of a routed row in its destination region
    int* dest_count;         // local [world]
    int* fault;
    int rank, world, cap, hidden, topk, per;   // per = experts per rank
    unsigned long long limit_ns;
};

// Stable positions: CTA d scans the slots in order and numbers those bound for rank d.
// (The same arithmetic as garnet_b200_moe_ep_plan_host.)
__global__ void __launch_bounds__(1024) ep_plan_kernel(const EpDev ep, const int* __restrict__ selected, int slots)
{
    const int d = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ int warp_total[32];
    __shared__ int running;
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    for (int base = 0; base < slots; base += blockDim.x) {
        const int slot = base + threadIdx.x;
        const bool mine = slot < slots && selected[slot] / ep.per == d;
        const uint32_t ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_total[warp] = __popc(ballot);
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; ++w) before += warp_total[w];
        if (mine) ep.send_idx[slot] = before + __popc(ballot & ((1u << lane) - 1u));
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < int(blockDim.x >> 5); ++w) total += warp_total[w];
            running += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) ep.dest_count[d] = running;
}

// One CTA per routed row: the row and its expert id go to the owner's receive region.
template <typename XT>
__global__ void ep_push_kernel(const EpDev ep, const XT* __restrict__ x, const int* __restrict__ selected, int slots)
{
    const int slot = blockIdx.x;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ep.seq) + 1u;
    const int e = selected[slot], d = e / ep.per, idx = ep.send_idx[slot];
    const size_t at = size_t(ep.rank) * ep.cap + idx;
    uint8_t* dst = ep.peer_base[d] + ep.rows_off + at * ep.hidden * 2;
    const XT* src = x + size_t(slot / ep.topk) * ep.hidden;
    if constexpr (sizeof(XT) == 2) {
        const uint4* s = reinterpret_cast<const uint4*>(src);
        uint4* o = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < ep.hidden / 8; i += blockDim.x) o[i] = s[i];
    } else {
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(dst);
        for (int i = threadIdx.x; i < ep.hidden / 2; i += blockDim.x)
            o[i] = __floats2bfloat162_rn(float(src[2 * i]), float(src[2 * i + 1]));
    }
    if (threadIdx.x == 0) reinterpret_cast<int*>(ep.peer_base[d] + ep.expert_off)[at] = e;
    __threadfence_system();
    __syncthreads();
    // the CTA that finishes last publishes, to every rank, how many rows it got and "ready"
    if (threadIdx.x == 0 && atomicAdd(ep.counters, 1u) == gridDim.x - 1) {
        ep.counters[0] = 0;
        __threadfence_system();
        for (int r = 0; r < ep.world; ++r) {
            uint32_t* flags = reinterpret_cast<uint32_t*>(ep.peer_base[r] + ep.flags_off);
            reinterpret_cast<volatile int*>(flags + 2 * kCommMaxRanks)[ep.rank] = ep.dest_count[r];
            __threadfence_system();
            st_release_sys(flags + ep.rank, epoch);
        }
    }
}

// The owner: waits for every source, then marks the rows that nobody sent.
__global__ void ep_wait_dispatch_kernel(const EpDev ep, int* __restrict__ rows_received)
{
    __shared__ int failed;
    __shared__ int count[kCommMaxRanks];
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ep.seq) + 1u;
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(ep.peer_base[ep.rank] + ep.flags_off);
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    if (threadIdx.x < ep.world) {
        if (!wait_epoch(flags + threadIdx.x, epoch, ep.limit_ns)) failed = 1;
        count[threadIdx.x] = min(ep.cap, max(0, reinterpret_cast<const volatile int*>(flags + 2 * kCommMaxRanks)[threadIdx.x]));
    }
    __syncthreads();
    int* expert = reinterpret_cast<int*>(ep.peer_base[ep.rank] + ep.expert_off);
    if (failed) {
        if (threadIdx.x == 0) *reinterpret_cast<volatile int*>(ep.fault) = 71;
        for (int i = threadIdx.x; i < ep.world * ep.cap; i += blockDim.x) expert[i] = -1;   // nothing runs on a failed step
        return;
    }
    for (int i = threadIdx.x; i < ep.world * ep.cap; i += blockDim.x)
        if (i % ep.cap >= count[i / ep.cap]) expert[i] = -1;
    if (threadIdx.x == 0) {
        int total = 0;
        for (int s = 0; s < ep.world; ++s) total += count[s];
        *rows_received = total;
    }
}

// One CTA per receive slot: a row's values go back to its source as bf16.
__global__ void ep_return_kernel(const EpDev ep, const float* __restrict__ vals)
{
    const int s = blockIdx.x / ep.cap, r = blockIdx.x % ep.cap;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ep.seq) + 1u;
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(ep.peer_base[ep.rank] + ep.flags_off);
    const int count = min(ep.cap, max(0, reinterpret_cast<const volatile int*>(flags + 2 * kCommMaxRanks)[s]));
    if (r < count) {
        const float4* v = reinterpret_cast<const float4*>(vals + size_t(blockIdx.x) * ep.hidden);
        uint2* o = reinterpret_cast<uint2*>(ep.peer_base[s] + ep.ret_off + (size_t(ep.rank) * ep.cap + r) * ep.hidden * 2);
        for (int i = threadIdx.x; i < ep.hidden / 4; i += blockDim.x) {
            const float4 f = v[i];
            const __nv_bfloat162 a = __floats2bfloat162_rn(f.x, f.y), b = __floats2bfloat162_rn(f.z, f.w);
            o[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(ep.counters + 1, 1u) == gridDim.x - 1) {
        ep.counters[1] = 0;
        __threadfence_system();
        for (int p = 0; p < ep.world; ++p)
            st_release_sys(reinterpret_cast<uint32_t*>(ep.peer_base[p] + ep.flags_off) + kCommMaxRanks + ep.rank, epoch);
    }
}

// The source: waits for every owner's values, then the step is over (the epoch moves on).
__global__ void ep_wait_return_kernel(const EpDev ep)
{
    __shared__ int failed;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ep.seq) + 1u;
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(ep.peer_base[ep.rank] + ep.flags_off);
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    if (threadIdx.x < ep.world && !wait_epoch(flags + kCommMaxRanks + threadIdx.x, epoch, ep.limit_ns)) failed = 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (failed) *reinterpret_cast<volatile int*>(ep.fault) = 72;
        *reinterpret_cast<volatile uint32_t*>(ep.seq) = epoch;
    }
}

// y[t, :] = bf(sum_j value(t, j) * p[t, j]) in router order (combineExperts,
// gpt_oss_kernels.cu:907-921), the values read from the regions the owners filled.
template <typename YT>
__global__ void ep_combine_kernel(const EpDev ep, const int* __restrict__ selected, const float* __restrict__ probs,
                                  YT* __restrict__ y, int tokens)
{
    // grid = (tokens, blocks of column pairs): no division per element
    const int pairs = ep.hidden / 2;
    const int token = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;   // c: a pair of columns
    if (token >= tokens || c >= pairs) return;
    const size_t idx = size_t(token) * pairs + c;
    const uint8_t* ret = ep.peer_base[ep.rank] + ep.ret_off;
    float r0 = 0.f, r1 = 0.f;
    for (int j = 0; j < ep.topk; ++j) {
        const int slot = token * ep.topk + j;
        const int d = selected[slot] / ep.per;
        const uint32_t two = __ldcg(reinterpret_cast<const uint32_t*>(ret + (size_t(d) * ep.cap + ep.send_idx[slot]) * ep.hidden * 2) + c);
        const float p = probs[slot];
        r0 = __fmaf_rn(__uint_as_float(two << 16), p, r0);
        r1 = __fmaf_rn(__uint_as_float(two & 0xffff0000u), p, r1);
    }
    if constexpr (sizeof(YT) == 4) {
        reinterpret_cast<float2*>(y)[idx] = make_float2(bf16_round_f(r0), bf16_round_f(r1));
    } else {
        reinterpret_cast<__nv_bfloat162*>(y)[idx] = __floats2bfloat162_rn(r0, r1);
    }
}

struct MoeEp {
    Moe* moe = nullptr;
    Comm* comm = nullptr;
    EpDev dev{};
    int tokens_max = 0;
    // local buffers
    uint8_t* local = nullptr;
    float* logits = nullptr;
    int* selected = nullptr;
    float* probs = nullptr;
    void* route_ws = nullptr;
    size_t route_ws_bytes = 0;
    float* vals = nullptr;
    void* rows_ws = nullptr;
    size_t rows_ws_bytes = 0;
    int* rows_received = nullptr;   // mapped host word
    int* rows_received_dev = nullptr;
    ~MoeEp()
    {
        if (local) cudaFree(local);
        if (rows_received) cudaFreeHost(rows_received);
    }
};

static size_t ep_arena_bytes(int world, int cap, int hidden)
{
    const size_t rows = size_t(world) * cap * hidden * 2;
    return 256 + 256 + rows + 256 + size_t(world) * cap * 4 + 256 + rows + 1024;
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_moe_ep_plan_host(const int* selected, int slots, int experts_per_rank, int world, int* send_idx, int* dest_count)
{
    if (!selected || !send_idx || !dest_count || slots < 0 || experts_per_rank <= 0 || world <= 0 || world > kCommMaxRanks)
        return fail(GARNET_B200_INVALID_VALUE, "moe_ep_plan_host: bad argument");
    for (int d = 0; d < world; ++d) dest_count[d] = 0;
    for (int s = 0; s < slots; ++s) {
        const int d = selected[s] / experts_per_rank;
        if (selected[s] < 0 || d >= world) return fail(GARNET_B200_INVALID_VALUE, "moe_ep_plan_host: expert %d out of range", selected[s]);
        send_idx[s] = dest_count[d]++;
    }
    return GARNET_B200_OK;
}

int garnet_b200_moe_ep_arena_bytes(const garnet_b200_moe_options* o, int world, int tokens_local_max, size_t* bytes)
{
    if (!o || !bytes || world < 1 || world > kCommMaxRanks || tokens_local_max <= 0 || o->top_k <= 0 || o->hidden <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "moe_ep_arena_bytes: bad argument");
    *bytes = ep_arena_bytes(world, tokens_local_max * o->top_k, o->hidden);
    return GARNET_B200_OK;
}

int garnet_b200_moe_ep_create(garnet_b200_moe_t mm, garnet_b200_comm_t cc, int tokens_local_max, garnet_b200_moe_ep_t* out)
{
    Moe* moe = reinterpret_cast<Moe*>(mm);
    Comm* comm = reinterpret_cast<Comm*>(cc);
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "moe_ep_create: null output");
    *out = nullptr;
    if (!moe || !comm || tokens_local_max <= 0) return fail(GARNET_B200_INVALID_VALUE, "moe_ep_create: bad argument");
    const garnet_b200_moe_options& o = moe->opt;
    const int world = comm->world;
    if ((o.ep_world > 1 ? o.ep_world : 1) != world || (world > 1 && (o.ep_rank != comm->rank || o.ep_interleaved)))
        return fail(GARNET_B200_INVALID_VALUE, "moe_ep_create: the operator must be created for contiguous expert blocks with ep_rank/ep_world of the communicator");
    if (o.experts % world || (o.hidden % 8)) return fail(GARNET_B200_INVALID_VALUE, "moe_ep_create: experts must divide by the ranks");
    if (o.io_dtype != GARNET_B200_BF16) return fail(GARNET_B200_NOT_SUPPORTED, "moe_ep_create: the exchange carries bf16 rows: create the operator with io_dtype bf16");
    if (!comm->connected) return fail(GARNET_B200_INVALID_VALUE, "moe_ep_create: the communicator is not connected");
    MoeEp* ep = new (std::nothrow) MoeEp();
    if (!ep) return fail(GARNET_B200_OUT_OF_MEMORY, "moe_ep_create: host allocation failed");
    ep->moe = moe;
    ep->comm = comm;
    ep->tokens_max = tokens_local_max;
    EpDev& d = ep->dev;
    const int cap = tokens_local_max * o.top_k;
    const size_t rows_bytes = size_t(world) * cap * o.hidden * 2;
    int rc = comm->alloc(3 * kCommMaxRanks * 4, &d.flags_off);
    if (!rc) rc = comm->alloc(rows_bytes, &d.rows_off);
    if (!rc) rc = comm->alloc(size_t(world) * cap * 4, &d.expert_off);
    if (!rc) rc = comm->alloc(rows_bytes, &d.ret_off);
    void* counters = nullptr;
    if (!rc) rc = comm->alloc_local(4 * sizeof(uint32_t), &counters);
    if (!rc) {
        for (int r = 0; r < world; ++r) d.peer_base[r] = comm->peer_base[r];
        d.seq = static_cast<uint32_t*>(counters);
        d.counters = d.seq + 1;
        d.fault = comm->fault_dev;
        d.rank = comm->rank;
        d.world = world;
        d.cap = cap;
        d.hidden = o.hidden;
        d.topk = o.top_k;
        d.per = o.experts / world;
        d.limit_ns = comm->wait_limit_ns;
        // local buffers in one allocation
        size_t route_bytes = 0, rows_ws = 0;
        rc = garnet_b200_moe_route_workspace(&o, tokens_local_max, &route_bytes);
        if (!rc) rc = garnet_b200_moe_rows_workspace(&o, world * cap, &rows_ws);
        if (!rc) {
            size_t off = 0;
            auto take = [&](size_t bytes) {
                const size_t at = off;
                off = (off + bytes + 255) & ~size_t(255);
                return at;
            };
            const size_t a_logits = take(size_t(tokens_local_max) * o.experts * 4), a_sel = take(size_t(cap) * 4),
                         a_probs = take(size_t(cap) * 4), a_idx = take(size_t(cap) * 4), a_cnt = take(kCommMaxRanks * 4),
                         a_route = take(route_bytes), a_vals = take(size_t(world) * cap * o.hidden * 4), a_ws = take(rows_ws);
            if (cudaMalloc(&ep->local, off) != cudaSuccess) {
                cudaGetLastError();
                rc = fail(GARNET_B200_OUT_OF_MEMORY, "moe_ep_create: cudaMalloc of %zu bytes failed", off);
            } else {
                ep->logits = reinterpret_cast<float*>(ep->local + a_logits);
                ep->selected = reinterpret_cast<int*>(ep->local + a_sel);
                ep->probs = reinterpret_cast<float*>(ep->local + a_probs);
                d.send_idx = reinterpret_cast<int*>(ep->local + a_idx);
                d.dest_count = reinterpret_cast<int*>(ep->local + a_cnt);
                ep->route_ws = ep->local + a_route;
                ep->route_ws_bytes = route_bytes;
                ep->vals = reinterpret_cast<float*>(ep->local + a_vals);
                ep->rows_ws = ep->local + a_ws;
                ep->rows_ws_bytes = rows_ws;
            }
        }
    }
    if (!rc && cudaHostAlloc(&ep->rows_received, sizeof(int), cudaHostAllocMapped) != cudaSuccess) rc = cuda_fail(cudaGetLastError(), "moe_ep_create");
    if (!rc) {
        *ep->rows_received = 0;
        if (cudaHostGetDevicePointer(&ep->rows_received_dev, ep->rows_received, 0) != cudaSuccess) rc = cuda_fail(cudaGetLastError(), "moe_ep_create");
    }
    if (rc) {
        delete ep;
        return rc;
    }
    *out = reinterpret_cast<garnet_b200_moe_ep_t>(ep);
    return GARNET_B200_OK;
}

int garnet_b200_moe_ep_run(garnet_b200_moe_ep_t ee, const void* d_x, void* d_y, int tokens_local, void* stream)
{
    MoeEp* ep = reinterpret_cast<MoeEp*>(ee);
    if (!ep || !d_x || !d_y || tokens_local <= 0) return fail(GARNET_B200_INVALID_VALUE, "moe_ep_run: bad argument");
    if (tokens_local > ep->tokens_max)
        return fail(GARNET_B200_INVALID_VALUE, "moe_ep_run: %d tokens exceed the %d the exchange was created for", tokens_local, ep->tokens_max);
    if ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_y)) & 15)
        return fail(GARNET_B200_INVALID_VALUE, "moe_ep_run: x and y must be 16-byte aligned");
    Moe* moe = ep->moe;
    const EpDev& d = ep->dev;
    int dev = -1;
    GB_CUDA(cudaGetDevice(&dev));
    if (dev != ep->comm->device) return fail(GARNET_B200_INVALID_VALUE, "moe_ep_run: created on device %d, current device is %d", ep->comm->device, dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int slots = tokens_local * d.topk;
    if (int rc = garnet_b200_moe_route_ws(reinterpret_cast<garnet_b200_moe_t>(moe), d_x, ep->selected, ep->probs, ep->logits, tokens_local,
                                          ep->route_ws, ep->route_ws_bytes, stream))
        return rc;
    ep_plan_kernel<<<d.world, 1024, 0, s>>>(d, ep->selected, slots);
    if (moe->opt.io_dtype == GARNET_B200_BF16)
        ep_push_kernel<__nv_bfloat16><<<slots, 128, 0, s>>>(d, static_cast<const __nv_bfloat16*>(d_x), ep->selected, slots);
    else
        ep_push_kernel<float><<<slots, 128, 0, s>>>(d, static_cast<const float*>(d_x), ep->selected, slots);
    ep_wait_dispatch_kernel<<<1, 1024, 0, s>>>(d, ep->rows_received_dev);
    GB_CUDA(cudaGetLastError());
    // the experts on everything this rank received: regions of fixed capacity, unused rows marked -1
    const void* rows = d.peer_base[d.rank] + d.rows_off;
    const int* row_expert = reinterpret_cast<const int*>(d.peer_base[d.rank] + d.expert_off);
    if (int rc = moe->run_rows(rows, row_expert, d.world * d.cap, ep->vals, ep->rows_ws, ep->rows_ws_bytes, s)) return rc;
    ep_return_kernel<<<d.world * d.cap, 128, 0, s>>>(d, ep->vals);
    ep_wait_return_kernel<<<1, 32, 0, s>>>(d);
    const dim3 cgrid(unsigned(tokens_local), unsigned((d.hidden / 2 + 255) / 256));
    if (moe->opt.io_dtype == GARNET_B200_BF16)
        ep_combine_kernel<__nv_bfloat16><<<cgrid, 256, 0, s>>>(d, ep->selected, ep->probs, static_cast<__nv_bfloat16*>(d_y), tokens_local);
    else
        ep_combine_kernel<float><<<cgrid, 256, 0, s>>>(d, ep->selected, ep->probs, static_cast<float*>(d_y), tokens_local);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_moe_ep_rows_received(garnet_b200_moe_ep_t ee)
{
    MoeEp* ep = reinterpret_cast<MoeEp*>(ee);
    return ep && ep->rows_received ? *ep->rows_received : -1;
}

void garnet_b200_moe_ep_destroy(garnet_b200_moe_ep_t ee) { delete reinterpret_cast<MoeEp*>(ee); }

}  // extern "C"
