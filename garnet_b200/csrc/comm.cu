// Collectives over NVLink for the ranks of one node, written as peer stores: every rank
// owns an arena of device memory that its peers map (CUDA IPC); data and flags are
// written straight into the destination GPU's own memory with plain stores, and every
// wait polls local memory only, with a time limit.  No library collective, no host
// synchronisation, no multicast load; the kernels of different ranks run on different
// GPUs at the same time (never two waiting kernels on one GPU).
//
// Replaces the reference's two-rank collectives (plugins/gpt_oss/cuda/tp_collective.cpp:
// 77-148: GptOssTpAllReduce, GptOssTpAllReduceBf16, GptOssTpAllGather) and its
// peer-memory all-reduce with bounded waits and a fault word
// (plugins/gpt_oss/cuda/tp_peer_owner.cuh:30-106), for up to eight ranks.
//
// Protocol of a channel (all_gather / all_reduce).  Every call has an epoch (a device
// counter, so a captured graph replays correctly).  Regions are double-buffered by
// epoch parity.  A rank first tells every peer that it has arrived at the epoch (so
// whatever it read of the epoch before last is over), waits until the peer it
// writes to has arrived at the previous epoch at least, stores its contribution into
// the peer's region, publishes "ready", and finally waits for the ready flags of
// all ranks in its own memory.
#include <algorithm>
#include <cstring>
#include <new>

#include "comm.h"
#include "common.cuh"

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
__device__ __forceinline__ uint4 ld_cg_v4(const void* p)
{
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Polls a local flag until `done(value)`; false when the limit runs out.
template <typename Pred>
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, Pred done, unsigned long long limit_ns)
{
    if (done(ld_acquire_sys(flag))) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int spin = 0; spin < 64; ++spin)
            if (done(ld_acquire_sys(flag))) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
}

}  // namespace

// -------------------------------------------------------------- channel kernel

struct ChannelDev {
    uint8_t* peer_base[kCommMaxRanks];   // arenas of all ranks (own included), as mapped here
    size_t flags_off;                    // arrived[kCommMaxRanks], ready[kCommMaxRanks] (uint32 each)
    size_t region_off;                   // [2][world][slot_bytes]
    size_t slot_bytes;
    uint32_t* seq;                       // local epoch counter
    uint32_t* finished;                  // local counter of CTAs done with the call
    int* fault;
    int rank, world;
    unsigned long long limit_ns;
};

// mode 0: gather (the result is the local region); 1: sum of fp32 contributions;
// 2: contributions travel as bf16, are summed in fp32 in rank order and rounded to bf16
// (for two ranks: exactly bf16(a + b), the reference's wire format,
// plugins/gpt_oss/cuda/tp_peer_math.cuh:10-14); 3: the same with bf16 source and result.
__global__ void comm_exchange_kernel(const ChannelDev ch, const void* __restrict__ src, size_t bytes, int mode,
                                     void* __restrict__ dst_any, size_t count)
{
    __shared__ int failed;
    const int peer = blockIdx.x % ch.world, part = blockIdx.x / ch.world, parts = gridDim.x / ch.world;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ch.seq) + 1u;
    const int parity = int(epoch & 1u);
    uint32_t* my_flags = reinterpret_cast<uint32_t*>(ch.peer_base[ch.rank] + ch.flags_off);
    uint32_t* peer_flags = reinterpret_cast<uint32_t*>(ch.peer_base[peer] + ch.flags_off);
    if (threadIdx.x == 0) {
        failed = 0;
        if (part == 0) st_release_sys(peer_flags + ch.rank, epoch);   // arrived
        if (!wait_flag(my_flags + peer, [&](uint32_t v) { return int32_t(v - (epoch - 1u)) >= 0; }, ch.limit_ns)) failed = 1;
    }
    __syncthreads();
    if (!failed) {
        // my contribution -> slot `rank` of the peer's region of this parity
        uint8_t* slot = ch.peer_base[peer] + ch.region_off + (size_t(parity) * ch.world + ch.rank) * ch.slot_bytes;
        if (mode == 2) {
            const float* s = static_cast<const float*>(src);
            __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(slot);
            for (size_t i = size_t(part) * blockDim.x + threadIdx.x; i < count; i += size_t(parts) * blockDim.x)
                d[i] = __float2bfloat16_rn(s[i]);
        } else {
            const size_t vecs = bytes / 16;
            const uint4* s = static_cast<const uint4*>(src);
            uint4* d = reinterpret_cast<uint4*>(slot);
            for (size_t i = size_t(part) * blockDim.x + threadIdx.x; i < vecs; i += size_t(parts) * blockDim.x) d[i] = s[i];
            if (part == 0 && threadIdx.x < (bytes & 15))
                slot[vecs * 16 + threadIdx.x] = static_cast<const uint8_t*>(src)[vecs * 16 + threadIdx.x];
        }
    }
    __threadfence_system();
    __syncthreads();
    // the parts of one peer's push meet at a local counter; the last publishes "ready"
    if (threadIdx.x == 0 && !failed) {
        uint32_t* pushed = ch.finished + 1 + peer;
        if (atomicAdd(pushed, 1u) == uint32_t(parts) - 1u) {
            *pushed = 0;
            __threadfence_system();
            st_release_sys(peer_flags + kCommMaxRanks + ch.rank, epoch);   // ready
        }
    }
    if (threadIdx.x < ch.world && !failed) {
        if (!wait_flag(my_flags + kCommMaxRanks + threadIdx.x, [&](uint32_t v) { return v == epoch; }, ch.limit_ns)) failed = 2;
    }
    __syncthreads();
    if (failed) {
        if (threadIdx.x == 0) *reinterpret_cast<volatile int*>(ch.fault) = 60 + failed;
    } else if (mode == 0) {
        // the gathered contributions, rank after rank, to the caller's buffer
        const uint8_t* region = ch.peer_base[ch.rank] + ch.region_off + size_t(parity) * ch.world * ch.slot_bytes;
        uint8_t* dst = static_cast<uint8_t*>(dst_any);
        const size_t vecs = bytes / 16;
        for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs * ch.world; i += size_t(gridDim.x) * blockDim.x) {
            const size_t s = i / vecs, v = i - s * vecs;
            *reinterpret_cast<uint4*>(dst + s * bytes + v * 16) = ld_cg_v4(region + s * ch.slot_bytes + v * 16);
        }
    } else if (mode == 3) {
        const uint8_t* region = ch.peer_base[ch.rank] + ch.region_off + size_t(parity) * ch.world * ch.slot_bytes;
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(dst_any);
        for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x) {
            float sum = 0.f;
            for (int s = 0; s < ch.world; ++s)
                sum += __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(region + size_t(s) * ch.slot_bytes) + i)));
            dst[i] = __float2bfloat16_rn(sum);
        }
    } else {
        const uint8_t* region = ch.peer_base[ch.rank] + ch.region_off + size_t(parity) * ch.world * ch.slot_bytes;
        float* dst = static_cast<float*>(dst_any);
        for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x) {
            float sum = 0.f;
            for (int s = 0; s < ch.world; ++s) {
                const uint8_t* slot = region + size_t(s) * ch.slot_bytes;
                sum += mode == 1 ? __ldcg(reinterpret_cast<const float*>(slot) + i)
                                 : __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(slot) + i)));
            }
            dst[i] = mode == 2 ? bf16_round_f(sum) : sum;
        }
    }
    __syncthreads();
    // the CTA that finishes last moves the epoch on (every CTA has read it by then)
    if (threadIdx.x == 0 && atomicAdd(ch.finished, 1u) == gridDim.x - 1) {
        *ch.finished = 0;
        *reinterpret_cast<volatile uint32_t*>(ch.seq) = epoch;
    }
}

// One thread waits on a flag of this rank's arena that no peer ever writes.
__global__ void comm_wait_probe_kernel(const uint32_t* flag, unsigned long long limit_ns, int* fault)
{
    if (!wait_flag(flag, [](uint32_t v) { return v == 0xfeedu; }, limit_ns)) *reinterpret_cast<volatile int*>(fault) = 69;
}

// ------------------------------------------------------------------- host side

Comm::~Comm()
{
    for (int r = 0; r < world; ++r)
        if (r != rank && peer_base[r]) cudaIpcCloseMemHandle(peer_base[r]);
    if (arena) cudaFree(arena);
    if (local) cudaFree(local);
    if (fault_host) cudaFreeHost(fault_host);
}

int Comm::alloc(size_t bytes, size_t* offset)
{
    const size_t at = (used + 255) & ~size_t(255);
    if (at + bytes > arena_bytes)
        return fail(GARNET_B200_OUT_OF_MEMORY, "comm: arena of %zu bytes is full (%zu in use, %zu more asked for)", arena_bytes, at, bytes);
    *offset = at;
    used = at + bytes;
    return GARNET_B200_OK;
}

int Comm::alloc_local(size_t bytes, void** ptr)
{
    const size_t at = (local_used + 255) & ~size_t(255);
    if (at + bytes > kCommLocalBytes) return fail(GARNET_B200_OUT_OF_MEMORY, "comm: local counter block is full");
    *ptr = local + at;
    local_used = at + bytes;
    return GARNET_B200_OK;
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_comm_create(int rank, int world, size_t arena_bytes, garnet_b200_comm_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "comm_create: null output");
    *out = nullptr;
    if (world < 1 || world > kCommMaxRanks || rank < 0 || rank >= world || arena_bytes < 4096)
        return fail(GARNET_B200_INVALID_VALUE, "comm_create: rank %d of %d, arena %zu bytes", rank, world, arena_bytes);
    Comm* c = new (std::nothrow) Comm();
    if (!c) return fail(GARNET_B200_OUT_OF_MEMORY, "comm_create: host allocation failed");
    c->rank = rank;
    c->world = world;
    c->arena_bytes = (arena_bytes + 255) & ~size_t(255);
    int rc = GARNET_B200_OK;
    do {
        if (cudaGetDevice(&c->device) != cudaSuccess) { rc = cuda_fail(cudaGetLastError(), "comm_create: cudaGetDevice"); break; }
        if (cudaMalloc(&c->arena, c->arena_bytes) != cudaSuccess) {
            cudaGetLastError();
            rc = fail(GARNET_B200_OUT_OF_MEMORY, "comm_create: cudaMalloc of %zu bytes failed", c->arena_bytes);
            break;
        }
        if (cudaMemset(c->arena, 0, c->arena_bytes) != cudaSuccess || cudaMalloc(&c->local, kCommLocalBytes) != cudaSuccess ||
            cudaMemset(c->local, 0, kCommLocalBytes) != cudaSuccess ||
            cudaHostAlloc(&c->fault_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) {
            rc = cuda_fail(cudaGetLastError(), "comm_create: allocation");
            break;
        }
        *c->fault_host = 0;
        if (cudaHostGetDevicePointer(&c->fault_dev, c->fault_host, 0) != cudaSuccess) { rc = cuda_fail(cudaGetLastError(), "comm_create"); break; }
        if (world > 1 && cudaIpcGetMemHandle(&c->handle, c->arena) != cudaSuccess) { rc = cuda_fail(cudaGetLastError(), "comm_create: cudaIpcGetMemHandle"); break; }
        if (cudaDeviceSynchronize() != cudaSuccess) { rc = cuda_fail(cudaGetLastError(), "comm_create: synchronize"); break; }
        c->peer_base[rank] = c->arena;
        c->connected = world == 1;
    } while (false);
    if (rc) {
        delete c;
        return rc;
    }
    *out = reinterpret_cast<garnet_b200_comm_t>(c);
    return GARNET_B200_OK;
}

int garnet_b200_comm_export(garnet_b200_comm_t cc, void* blob, size_t blob_bytes)
{
    Comm* c = reinterpret_cast<Comm*>(cc);
    if (!c || !blob || blob_bytes < GARNET_B200_COMM_BLOB_BYTES) return fail(GARNET_B200_INVALID_VALUE, "comm_export: bad argument");
    std::memset(blob, 0, GARNET_B200_COMM_BLOB_BYTES);
    std::memcpy(blob, &c->handle, sizeof(c->handle));
    std::memcpy(static_cast<char*>(blob) + 64, &c->arena_bytes, sizeof(size_t));
    return GARNET_B200_OK;
}

int garnet_b200_comm_connect(garnet_b200_comm_t cc, const void* blobs)
{
    Comm* c = reinterpret_cast<Comm*>(cc);
    if (!c || (!blobs && c->world > 1)) return fail(GARNET_B200_INVALID_VALUE, "comm_connect: bad argument");
    if (c->connected) return GARNET_B200_OK;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        const char* b = static_cast<const char*>(blobs) + size_t(r) * GARNET_B200_COMM_BLOB_BYTES;
        size_t their_bytes = 0;
        std::memcpy(&their_bytes, b + 64, sizeof(size_t));
        if (their_bytes != c->arena_bytes)
            return fail(GARNET_B200_INVALID_VALUE, "comm_connect: rank %d has an arena of %zu bytes, this rank %zu", r, their_bytes, c->arena_bytes);
        cudaIpcMemHandle_t h;
        std::memcpy(&h, b, sizeof(h));
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
            return cuda_fail(cudaGetLastError(), "comm_connect: cudaIpcOpenMemHandle");
        c->peer_base[r] = static_cast<uint8_t*>(p);
    }
    c->connected = true;
    return GARNET_B200_OK;
}

int garnet_b200_comm_fault(garnet_b200_comm_t cc)
{
    Comm* c = reinterpret_cast<Comm*>(cc);
    return c && c->fault_host ? *c->fault_host : -1;
}

void garnet_b200_comm_destroy(garnet_b200_comm_t cc) { delete reinterpret_cast<Comm*>(cc); }

int garnet_b200_comm_channel_create(garnet_b200_comm_t cc, size_t slot_bytes, garnet_b200_channel_t* out)
{
    Comm* c = reinterpret_cast<Comm*>(cc);
    if (!c || !out || slot_bytes == 0) return fail(GARNET_B200_INVALID_VALUE, "comm_channel_create: bad argument");
    *out = nullptr;
    Channel* ch = new (std::nothrow) Channel();
    if (!ch) return fail(GARNET_B200_OUT_OF_MEMORY, "comm_channel_create: host allocation failed");
    ch->comm = c;
    ch->slot_bytes = (slot_bytes + 255) & ~size_t(255);
    int rc = c->alloc(2 * kCommMaxRanks * sizeof(uint32_t), &ch->flags_off);
    if (!rc) rc = c->alloc(2 * size_t(c->world) * ch->slot_bytes, &ch->region_off);
    void* counters = nullptr;
    if (!rc) rc = c->alloc_local((2 + kCommMaxRanks) * sizeof(uint32_t), &counters);
    if (rc) {
        delete ch;
        return rc;
    }
    ch->seq = static_cast<uint32_t*>(counters);
    ch->finished = ch->seq + 1;
    *out = reinterpret_cast<garnet_b200_channel_t>(ch);
    return GARNET_B200_OK;
}

void garnet_b200_comm_channel_destroy(garnet_b200_channel_t hh) { delete reinterpret_cast<Channel*>(hh); }

static int channel_launch(Channel* ch, const void* d_src, size_t bytes, int mode, void* d_dst, size_t count, cudaStream_t stream)
{
    Comm* c = ch->comm;
    if (!c->connected) return fail(GARNET_B200_INVALID_VALUE, "comm: garnet_b200_comm_connect has not been called");
    int dev = -1;
    GB_CUDA(cudaGetDevice(&dev));
    if (dev != c->device) return fail(GARNET_B200_INVALID_VALUE, "comm: created on device %d, current device is %d", c->device, dev);
    ChannelDev d = {};
    for (int r = 0; r < c->world; ++r) d.peer_base[r] = c->peer_base[r];
    d.flags_off = ch->flags_off;
    d.region_off = ch->region_off;
    d.slot_bytes = ch->slot_bytes;
    d.seq = ch->seq;
    d.finished = ch->finished;
    d.fault = c->fault_dev;
    d.rank = c->rank;
    d.world = c->world;
    d.limit_ns = c->wait_limit_ns;
    const int parts = int(std::max<size_t>(1, std::min<size_t>(16, bytes / 16384)));
    comm_exchange_kernel<<<c->world * parts, 256, 0, stream>>>(d, d_src, bytes, mode, d_dst, count);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_comm_all_gather(garnet_b200_channel_t hh, const void* d_src, size_t bytes, void* d_dst, void* stream)
{
    Channel* ch = reinterpret_cast<Channel*>(hh);
    if (!ch || !d_src || !d_dst || bytes == 0) return fail(GARNET_B200_INVALID_VALUE, "comm_all_gather: bad argument");
    if (bytes > ch->slot_bytes) return fail(GARNET_B200_INVALID_VALUE, "comm_all_gather: %zu bytes exceed the channel's slot of %zu", bytes, ch->slot_bytes);
    if (reinterpret_cast<uintptr_t>(d_src) & 15) return fail(GARNET_B200_INVALID_VALUE, "comm_all_gather: source must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(d_dst) & 15) || (bytes & 15))
        return fail(GARNET_B200_INVALID_VALUE, "comm_all_gather: destination must be 16-byte aligned and the size a multiple of 16");
    return channel_launch(ch, d_src, bytes, 0, d_dst, 0, static_cast<cudaStream_t>(stream));
}

int garnet_b200_comm_all_reduce(garnet_b200_channel_t hh, const float* d_src, float* d_dst, size_t count, int wire_dtype,
                                void* stream)
{
    Channel* ch = reinterpret_cast<Channel*>(hh);
    if (!ch || !d_src || !d_dst || count == 0) return fail(GARNET_B200_INVALID_VALUE, "comm_all_reduce: bad argument");
    if (wire_dtype != GARNET_B200_FP32 && wire_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "comm_all_reduce: wire dtype must be fp32 or bf16");
    const size_t bytes = count * (wire_dtype == GARNET_B200_FP32 ? 4 : 2);
    if (bytes > ch->slot_bytes) return fail(GARNET_B200_INVALID_VALUE, "comm_all_reduce: %zu bytes exceed the channel's slot of %zu", bytes, ch->slot_bytes);
    if (reinterpret_cast<uintptr_t>(d_src) & 15) return fail(GARNET_B200_INVALID_VALUE, "comm_all_reduce: source must be 16-byte aligned");
    return channel_launch(ch, d_src, bytes, wire_dtype == GARNET_B200_FP32 ? 1 : 2, d_dst, count, static_cast<cudaStream_t>(stream));
}

int garnet_b200_comm_all_reduce_bf16(garnet_b200_channel_t hh, const void* d_src, void* d_dst, size_t count, void* stream)
{
    Channel* ch = reinterpret_cast<Channel*>(hh);
    if (!ch || !d_src || !d_dst || count == 0) return fail(GARNET_B200_INVALID_VALUE, "comm_all_reduce_bf16: bad argument");
    const size_t bytes = count * 2;
    if (bytes > ch->slot_bytes) return fail(GARNET_B200_INVALID_VALUE, "comm_all_reduce_bf16: %zu bytes exceed the channel's slot of %zu", bytes, ch->slot_bytes);
    if ((reinterpret_cast<uintptr_t>(d_src) & 15) || (reinterpret_cast<uintptr_t>(d_dst) & 1))
        return fail(GARNET_B200_INVALID_VALUE, "comm_all_reduce_bf16: source must be 16-byte aligned");
    return channel_launch(ch, d_src, bytes, 3, d_dst, count, static_cast<cudaStream_t>(stream));
}

int garnet_b200_comm_selftest_wait(garnet_b200_comm_t cc, int limit_ms, void* stream)
{
    Comm* c = reinterpret_cast<Comm*>(cc);
    if (!c || limit_ms <= 0 || limit_ms > 2000) return fail(GARNET_B200_INVALID_VALUE, "comm_selftest_wait: bad argument");
    size_t off = 0;
    if (int rc = c->alloc(256, &off)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    comm_wait_probe_kernel<<<1, 1, 0, s>>>(reinterpret_cast<const uint32_t*>(c->arena + off), (unsigned long long)limit_ms * 1000000ull,
                                           c->fault_dev);
    GB_CUDA(cudaGetLastError());
    GB_CUDA(cudaStreamSynchronize(s));
    if (*c->fault_host) {
        const int code = *c->fault_host;
        *c->fault_host = 0;
        return fail(GARNET_B200_DEVICE_FAULT, "comm: device wait gave up (code %d)", code);
    }
    return GARNET_B200_OK;
}

}  // extern "C"
