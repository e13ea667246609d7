// Host-side state of a communicator (garnet_b200_comm_t) and of a collective channel.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/garnet_b200.h"

namespace gb200 {

constexpr int kCommMaxRanks = 8;
constexpr size_t kCommLocalBytes = 64 * 1024;   // epoch counters and the like: local, never mapped by peers

struct Comm {
    int rank = 0, world = 1, device = 0;
    uint8_t* arena = nullptr;          // this rank's arena: peers write into it
    size_t arena_bytes = 0, used = 0;  // bump allocation; every rank allocates in the same order, so offsets agree
    uint8_t* peer_base[kCommMaxRanks] = {};
    uint8_t* local = nullptr;
    size_t local_used = 0;
    cudaIpcMemHandle_t handle{};
    int* fault_host = nullptr;
    int* fault_dev = nullptr;
    bool connected = false;
    unsigned long long wait_limit_ns = 2000000000ull;

    ~Comm();
    int alloc(size_t bytes, size_t* offset);
    int alloc_local(size_t bytes, void** ptr);
};

struct Channel {
    Comm* comm = nullptr;
    size_t flags_off = 0, region_off = 0, slot_bytes = 0;
    uint32_t* seq = nullptr;
    uint32_t* finished = nullptr;
};

}  // namespace gb200
