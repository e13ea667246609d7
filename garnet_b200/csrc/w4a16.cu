// Weight-only int4 linear for sm_100a: repackers, dequant check kernel, the
// small-batch streaming kernel (M <= 16 per launch) and the C ABI around them.
//
// Numerics: y[m,n] = bf16( sum_k x[m,k] * q[n,k] * s[n,k/group] ) with fp32
// accumulation.  In the streaming kernel q is expanded to an exact bf16 integer,
// each group's partial sum is accumulated by the tensor core in fp32 and the
// group scale is applied to that partial sum in fp32, so no product is rounded
// before the final bf16 store.
#include <algorithm>
#include <memory>
#include <vector>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"
#include "layout.h"
#include "w4a16.h"

namespace gb200 {

// ------------------------------------------------------------------ repack

// One thread per packed 32-bit word (8 codes of one row).
__global__ void w4_repack_codes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, PackGeom geo,
                                       long long src_row0, int src_cols, int src_col0)
{
    const size_t words_per_chunk = geo.chunk_data / 4;
    const size_t total = size_t(geo.strips_padded) * geo.chunks * words_per_chunk;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t chunk_lin = idx / words_per_chunk;
    const int w = int(idx % words_per_chunk);
    const int strip = int(chunk_lin / geo.chunks), chunk = int(chunk_lin % geo.chunks);
    // invert locate(): word index -> (row, first column)
    const int tile = w >> 7, unit = (w >> 2) & 31, word = w & 3;      // 128 words per 512-byte tile
    const int g = unit >> 2, t = unit & 3, h = word & 1, j = word >> 1;
    const int n = strip * 16 + row_of_g(g) + 8 * h;
    const int k0 = chunk * geo.chunk_k + tile * 64 + (t + 4 * j) * 8;
    uint32_t out = 0;
    if (n < geo.rows && k0 < geo.cols) {
        // K is a multiple of 8, so the 8 codes are 4 aligned source bytes.
        const size_t sb = ((size_t(src_row0) + n) * size_t(src_cols) + size_t(src_col0) + k0) / 2;
        const uint32_t in = *reinterpret_cast<const uint32_t*>(src + sb);
        if (geo.format == kFormatInt4) {
#pragma unroll
            for (int e = 0; e < 8; ++e) out |= ((in >> (4 * e)) & 15u) << (4 * ((e >> 1) + 4 * (e & 1)));
        } else {
            out = in;
        }
    }
    const size_t ob = (size_t(strip) * geo.chunks + chunk) * geo.chunk_bytes + size_t(w) * 4;
    *reinterpret_cast<uint32_t*>(dst + ob) = out;
}

// int4 scales: one thread per (padded row, chunk).  The 16 scale bits are kept as
// they are (fp16 or bf16); the kernels widen them to fp32 according to the
// handle's scale_dtype.
__global__ void w4_repack_scales_int4_kernel(const uint16_t* __restrict__ src, uint8_t* __restrict__ dst,
                                             PackGeom geo, long long src_row0, int src_cols, int src_col0)
{
    const size_t total = size_t(geo.strips_padded) * 16 * geo.chunks;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int n = int(idx / geo.chunks), chunk = int(idx % geo.chunks);
    uint16_t bits = 0;
    if (n < geo.rows) {
        const int groups = src_cols / geo.group;
        bits = src[(size_t(src_row0) + n) * groups + (src_col0 + chunk * geo.chunk_k) / geo.group];
    }
    *reinterpret_cast<uint16_t*>(dst + locate_scale(geo, n, chunk * geo.chunk_k)) = bits;
}

// ------------------------------------------------------------------ dequant

// fp32 q*s of every logical element, decoded from the packed tiles with the same
// device function the GEMM kernels use.
__device__ __forceinline__ float scale16_to_float(uint32_t bits16, int scale_dtype)
{
    return scale_dtype == GARNET_B200_BF16 ? __uint_as_float(bits16 << 16)
                                           : __half2float(__ushort_as_half(uint16_t(bits16)));
}

__global__ void w4_dequant_kernel(const uint8_t* __restrict__ packed, float* __restrict__ out, PackGeom geo,
                                  int scale_dtype)
{
    const size_t total = size_t(geo.rows) * geo.cols / 2;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int n = int(idx / (geo.cols / 2)), k = int(idx % (geo.cols / 2)) * 2;   // elements k, k+1
    const PackPos p = locate(geo, n, k);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(packed + p.word_byte);
    const int pair = (k & 7) >> 1;
    const uint32_t v = int4x2_to_bf16x2(w >> (4 * pair));
    const float s = scale16_to_float(*reinterpret_cast<const uint16_t*>(packed + locate_scale(geo, n, k)), scale_dtype);
    out[size_t(n) * geo.cols + k] = __bfloat162float(__ushort_as_bfloat16(uint16_t(v & 0xffff))) * s;
    out[size_t(n) * geo.cols + k + 1] = __bfloat162float(__ushort_as_bfloat16(uint16_t(v >> 16))) * s;
}

// --------------------------------------------------------------- quantizer

// One warp per (row, group).  weight_quantization.cpp:220-266.
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, size_t i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, size_t i)
{
    return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p, size_t i) { return __half2float(p[i]); }

template <typename T>
__global__ void int4_quantize_kernel(const T* __restrict__ src, long long rows, long long cols, int group,
                                     int scale_dtype, uint8_t* __restrict__ nibbles, uint16_t* __restrict__ scales)
{
    const long long groups = cols / group;
    const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= rows * groups) return;
    const long long row = wid / groups, grp = wid % groups;
    const size_t start = size_t(row) * cols + size_t(grp) * group;
    float lo = 0.f, hi = 0.f;
    for (int o = lane; o < group; o += 32) {
        const float v = load_as_float(src, start + o);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    for (int off = 16; off; off >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
    }
    float scale = fmaxf(__fdiv_rn(-lo, 8.0f), __fdiv_rn(hi, 7.0f));
    if (!isfinite(scale) || scale <= 0.f) scale = 1.0f;
    uint16_t bits;
    float stored;
    if (scale_dtype == GARNET_B200_FP16) {
        const __half hs = __float2half_rn(scale);
        bits = __half_as_ushort(hs);
        stored = __half2float(hs);
    } else {
        const __nv_bfloat16 bs = __float2bfloat16_rn(scale);
        bits = __bfloat16_as_ushort(bs);
        stored = __bfloat162float(bs);
    }
    if (lane == 0) scales[row * groups + grp] = bits;
    // each lane packs pairs of elements: byte index (start + 2i) / 2
    for (int o = 2 * lane; o < group; o += 64) {
        int q0 = __float2int_rn(__fdiv_rn(load_as_float(src, start + o), stored));
        int q1 = __float2int_rn(__fdiv_rn(load_as_float(src, start + o + 1), stored));
        q0 = max(-8, min(7, q0));
        q1 = max(-8, min(7, q1));
        nibbles[(start + o) >> 1] = uint8_t((q0 & 15) | ((q1 & 15) << 4));
    }
}

// ------------------------------------------------------------------ handle

int stream_set_attributes();
int stream_max_rows(int chunks);

int W4A16::init_common()
{
    GB_CUDA(cudaGetDevice(&device));
    GB_CUDA(cudaHostAlloc(&fault_host, sizeof(int), cudaHostAllocMapped));
    *fault_host = 0;
    GB_CUDA(cudaHostGetDevicePointer(&fault_dev, fault_host, 0));
    max_rows_per_launch = stream_max_rows(geo.chunks);
    if (max_rows_per_launch < 1)
        return fail(GARNET_B200_NOT_SUPPORTED, "w4a16: k=%d is too large for the streaming kernel", geo.cols);
    if (int rc = stream_set_attributes()) return rc;
    return init_tc();
}

W4A16::~W4A16()
{
    if (owns_packed && packed) cudaFree(packed);
    if (fault_host) cudaFreeHost(fault_host);
    if (stage_x) cudaFree(stage_x);
    if (stage_y) cudaFree(stage_y);
    if (stage_ws) cudaFree(stage_ws);
}

// Only the tile kernel (more than 16 rows) uses a workspace: the partial sums of its K slices.
size_t W4A16::workspace_bytes(int m) const { return (m > 16 || m > max_rows_per_launch) ? tc_plan(geo, m).workspace : 0; }

int W4A16::run(const void* d_x, void* d_y, int m, void* ws, size_t ws_bytes, unsigned flags, cudaStream_t stream)
{
    if (m <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: m must be positive (got %d)", m);
    if (!d_x || !d_y) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: null x or y");
    if ((reinterpret_cast<uintptr_t>(d_x) & 15) || (reinterpret_cast<uintptr_t>(d_y) & 1))
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: x must be 16-byte aligned");
    // A workspace smaller than garnet_b200_w4a16_workspace asks for (or none) is allowed: the
    // tile kernel then does not cut K into slices (slower on small matrices, same results
    // up to the order of the fp32 sums).
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(d_x);
    __nv_bfloat16* y = static_cast<__nv_bfloat16*>(d_y);
    // Above 16 rows the weights are worth expanding once per 128 rows for the tensor core.
    // (also when the rows do not fit one launch of the streaming kernel: a very long K)
    if ((m > 16 || m > max_rows_per_launch)) return launch_tc(x, y, m, ws, ws_bytes, flags, stream);
    for (int m0 = 0; m0 < m; m0 += max_rows_per_launch) {
        const int rows = std::min(max_rows_per_launch, m - m0);
        const int rc = launch_stream(x + size_t(m0) * geo.cols, y + size_t(m0) * geo.rows, rows, geo.rows, flags,
                                     stream);
        if (rc) return rc;
    }
    return GARNET_B200_OK;
}

static int validate_shape(int n, int k, int group)
{
    if (n <= 0 || k <= 0 || group <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16: n, k, group must be positive");
    if (k % group) return fail(GARNET_B200_INVALID_VALUE, "w4a16: k (%d) is not a multiple of group (%d)", k, group);
    if (group % 128)
        return fail(GARNET_B200_NOT_SUPPORTED, "w4a16: group %d is not a multiple of 128", group);
    return GARNET_B200_OK;
}

// Rows [row0, row0 + geo.rows) and columns [col0, col0 + geo.cols) of a canonical [*, src_cols] matrix.
int w4a16_repack_device(const uint8_t* d_nibbles, const uint16_t* d_scales, const PackGeom& geo, long long row0,
                        uint8_t* d_packed, cudaStream_t stream, int src_cols, int col0)
{
    if (src_cols <= 0) src_cols = geo.cols;
    const size_t words = size_t(geo.strips_padded) * geo.chunks * (geo.chunk_data / 4);
    w4_repack_codes_kernel<<<unsigned((words + 255) / 256), 256, 0, stream>>>(d_nibbles, d_packed, geo, row0, src_cols, col0);
    const size_t sc = size_t(geo.strips_padded) * 16 * geo.chunks;
    w4_repack_scales_int4_kernel<<<unsigned((sc + 255) / 256), 256, 0, stream>>>(d_scales, d_packed, geo, row0, src_cols, col0);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

// ---------------------------------------------------------- host-buffer batches

struct ScatterEntry {
    const uint8_t* src;   // device staging of one linear's output
    uint8_t* dst;         // device alias of the caller's pinned host buffer
    size_t bytes;
};

// Copies every entry's output to its host buffer: one launch at the end of a batch
// instead of one copy (or one flush of host-memory writes) per linear.
__global__ void w4_scatter_outputs_kernel(const ScatterEntry* __restrict__ table, int count)
{
    pdl_wait();
    for (int e = blockIdx.y; e < count; e += gridDim.y) {
        const ScatterEntry t = table[e];
        const size_t start = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 16, step = size_t(gridDim.x) * blockDim.x * 16;
        if (((reinterpret_cast<uintptr_t>(t.src) | reinterpret_cast<uintptr_t>(t.dst)) & 15) == 0) {
            for (size_t o = start; o + 16 <= t.bytes; o += step)
                *reinterpret_cast<uint4*>(t.dst + o) = *reinterpret_cast<const uint4*>(t.src + o);
            if (blockIdx.x == 0 && threadIdx.x < (t.bytes & 15)) t.dst[(t.bytes & ~size_t(15)) + threadIdx.x] = t.src[(t.bytes & ~size_t(15)) + threadIdx.x];
        } else {
            for (size_t o = start / 16; o < t.bytes; o += step / 16) t.dst[o] = t.src[o];
        }
    }
}

struct HostBatch {
    struct Call {
        W4A16* h;
        const void* h_x;
        void* h_y;
        int m;
        int x_slot;          // index into xs
        size_t y_off;        // offset of this call's output in y_stage
        void* y_alias;       // device alias of h_y, or nullptr (pageable: copied with cudaMemcpyAsync)
    };
    struct X {
        const void* host;
        size_t bytes, off;
    };
    std::vector<Call> calls;
    std::vector<X> xs;
    uint8_t* x_stage = nullptr;
    uint8_t* y_stage = nullptr;
    void* ws = nullptr;
    size_t ws_bytes = 0;
    ScatterEntry* table = nullptr;
    int table_count = 0;
    garnet_b200_w4a16_list_t list = nullptr;   // the calls as one persistent launch, when they all share one small batch
    ~HostBatch()
    {
        if (list) garnet_b200_w4a16_list_destroy(list);
        if (x_stage) cudaFree(x_stage);
        if (y_stage) cudaFree(y_stage);
        if (ws) cudaFree(ws);
        if (table) cudaFree(table);
    }
};

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_int4_quantize(const void* d_src, int src_dtype, int64_t rows, int64_t cols, int group,
                              int scale_dtype, uint8_t* d_nibbles, uint16_t* d_scales, void* stream)
{
    if (!d_src || !d_nibbles || !d_scales) return fail(GARNET_B200_INVALID_VALUE, "int4_quantize: null pointer");
    if (rows <= 0 || cols <= 0 || group <= 0 || cols % group || (group & 1))
        return fail(GARNET_B200_INVALID_VALUE, "int4_quantize: bad shape rows=%lld cols=%lld group=%d",
                    (long long)rows, (long long)cols, group);
    if (scale_dtype != GARNET_B200_FP16 && scale_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "int4_quantize: scale dtype must be fp16 or bf16");
    const long long warps = rows * (cols / group);
    const unsigned blocks = unsigned((warps * 32 + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (src_dtype) {
        case GARNET_B200_FP32:
            int4_quantize_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(d_src), rows, cols, group,
                                                              scale_dtype, d_nibbles, d_scales);
            break;
        case GARNET_B200_BF16:
            int4_quantize_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(d_src),
                                                                      rows, cols, group, scale_dtype, d_nibbles,
                                                                      d_scales);
            break;
        case GARNET_B200_FP16:
            int4_quantize_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(d_src), rows, cols,
                                                               group, scale_dtype, d_nibbles, d_scales);
            break;
        default:
            return fail(GARNET_B200_INVALID_VALUE, "int4_quantize: unknown source dtype %d", src_dtype);
    }
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_packed_bytes(int n, int k, int group, size_t* bytes)
{
    if (!bytes) return fail(GARNET_B200_INVALID_VALUE, "w4a16_packed_bytes: null output");
    if (int rc = validate_shape(n, k, group)) return rc;
    *bytes = make_geom(kFormatInt4, n, k, group).matrix_bytes();
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_pack_host(const uint8_t* nibbles, const uint16_t* scales, int scale_dtype, int n, int k,
                                int group, uint8_t* packed)
{
    if (!nibbles || !scales || !packed) return fail(GARNET_B200_INVALID_VALUE, "w4a16_pack_host: null pointer");
    if (int rc = validate_shape(n, k, group)) return rc;
    if (scale_dtype != GARNET_B200_FP16 && scale_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_pack_host: scale dtype must be fp16 or bf16");
    const PackGeom geo = make_geom(kFormatInt4, n, k, group);
    std::memset(packed, 0, geo.matrix_bytes());
    const int groups = k / group;
    for (int row = 0; row < n; ++row) {
        for (int col = 0; col < k; col += 8) {
            uint32_t in;
            std::memcpy(&in, nibbles + (size_t(row) * k + col) / 2, 4);
            uint32_t out = 0;
            for (int e = 0; e < 8; ++e) out |= ((in >> (4 * e)) & 15u) << (4 * ((e >> 1) + 4 * (e & 1)));
            std::memcpy(packed + locate(geo, row, col).word_byte, &out, 4);
        }
        for (int chunk = 0; chunk < geo.chunks; ++chunk) {
            const uint16_t s = scales[size_t(row) * groups + (chunk * 128) / group];
            std::memcpy(packed + locate_scale(geo, row, chunk * 128), &s, 2);
        }
    }
    return GARNET_B200_OK;
}

// shard_axis 0: rows [rank n / world, ...) (N-sharded, "vocab" / "qkv"); 1: columns
// [rank k / world, ...) (K-sharded, "row").
static int create_sharded(const uint8_t* d_nibbles, const void* d_scales, int scale_dtype, int n, int k, int group,
                          int shard_axis, int shard_rank, int shard_world, void* stream, garnet_b200_w4a16_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: null output handle");
    *out = nullptr;
    if (!d_nibbles || !d_scales) return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: null weight pointer");
    if (int rc = validate_shape(n, k, group)) return rc;
    if (scale_dtype != GARNET_B200_FP16 && scale_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: scale dtype must be fp16 or bf16");
    if (shard_world < 1) shard_world = 1;
    if (shard_rank < 0 || shard_rank >= shard_world)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: bad shard %d of %d", shard_rank, shard_world);
    if (shard_axis == 0 && n % shard_world)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: bad shard %d of %d for n=%d", shard_rank, shard_world, n);
    if (shard_axis == 1 && k % (shard_world * group))
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_create: k=%d does not split into %d parts of whole groups of %d", k,
                    shard_world, group);
    const int n_local = shard_axis == 0 ? n / shard_world : n;
    const int k_local = shard_axis == 1 ? k / shard_world : k;
    W4A16* h = new (std::nothrow) W4A16();
    if (!h) return fail(GARNET_B200_OUT_OF_MEMORY, "w4a16_create: host allocation failed");
    h->geo = make_geom(kFormatInt4, n_local, k_local, group);
    h->scale_dtype = scale_dtype;
    h->owns_packed = true;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = GARNET_B200_OK;
    do {
        if (cudaMalloc(&h->packed, h->geo.matrix_bytes()) != cudaSuccess) {
            rc = fail(GARNET_B200_OUT_OF_MEMORY, "w4a16_create: cudaMalloc of %zu bytes failed", h->geo.matrix_bytes());
            cudaGetLastError();
            break;
        }
        if ((rc = w4a16_repack_device(d_nibbles, static_cast<const uint16_t*>(d_scales), h->geo,
                                      shard_axis == 0 ? (long long)shard_rank * n_local : 0, h->packed, s, k,
                                      shard_axis == 1 ? shard_rank * k_local : 0)))
            break;
        if ((rc = h->init_common())) break;
        if (cudaStreamSynchronize(s) != cudaSuccess) {
            rc = cuda_fail(cudaGetLastError(), "w4a16_create: synchronize");
            break;
        }
    } while (false);
    if (rc) {
        delete h;
        return rc;
    }
    *out = reinterpret_cast<garnet_b200_w4a16_t>(h);
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_create(const uint8_t* d_nibbles, const void* d_scales, int scale_dtype, int n, int k,
                             int group, int shard_rank, int shard_world, void* stream,
                             garnet_b200_w4a16_t* out)
{
    return create_sharded(d_nibbles, d_scales, scale_dtype, n, k, group, 0, shard_rank, shard_world, stream, out);
}

int garnet_b200_w4a16_create_k_shard(const uint8_t* d_nibbles, const void* d_scales, int scale_dtype, int n, int k,
                                     int group, int shard_rank, int shard_world, void* stream,
                                     garnet_b200_w4a16_t* out)
{
    return create_sharded(d_nibbles, d_scales, scale_dtype, n, k, group, 1, shard_rank, shard_world, stream, out);
}

int garnet_b200_w4a16_create_prepacked(const uint8_t* d_packed, int scale_dtype, int n, int k, int group,
                                       garnet_b200_w4a16_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "w4a16_create_prepacked: null output handle");
    *out = nullptr;
    if (!d_packed || (reinterpret_cast<uintptr_t>(d_packed) & 127))
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_create_prepacked: packed pointer must be 128-byte aligned");
    if (int rc = validate_shape(n, k, group)) return rc;
    W4A16* h = new (std::nothrow) W4A16();
    if (!h) return fail(GARNET_B200_OUT_OF_MEMORY, "w4a16_create_prepacked: host allocation failed");
    h->geo = make_geom(kFormatInt4, n, k, group);
    h->packed = const_cast<uint8_t*>(d_packed);
    h->scale_dtype = scale_dtype;
    h->owns_packed = false;
    if (int rc = h->init_common()) {
        delete h;
        return rc;
    }
    *out = reinterpret_cast<garnet_b200_w4a16_t>(h);
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_shape(garnet_b200_w4a16_t hh, int* n_local, int* k)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "w4a16_shape: null handle");
    if (n_local) *n_local = h->geo.rows;
    if (k) *k = h->geo.cols;
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_workspace(garnet_b200_w4a16_t hh, int m, size_t* bytes)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h || !bytes || m <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16_workspace: bad argument");
    *bytes = h->workspace_bytes(m);
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_run(garnet_b200_w4a16_t hh, const void* d_x, void* d_y, int m, void* d_workspace,
                          size_t workspace_bytes, unsigned flags, void* stream)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run: null handle");
    return h->run(d_x, d_y, m, d_workspace, workspace_bytes, flags, static_cast<cudaStream_t>(stream));
}

int garnet_b200_w4a16_run_group(const garnet_b200_w4a16_t* handles, int count, const void* d_x, void* const* d_ys,
                                int m, unsigned flags, void* stream)
{
    if (!handles || !d_ys || !d_x || count <= 0 || m <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: bad argument");
    constexpr int kMaxGroup = 4;
    if (count > kMaxGroup) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: at most %d linears per group", kMaxGroup);
    if (reinterpret_cast<uintptr_t>(d_x) & 15) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: x must be 16-byte aligned");
    W4A16* hs[kMaxGroup];
    __nv_bfloat16* ys[kMaxGroup];
    int ldys[kMaxGroup];
    int max_rows = 16;
    for (int g = 0; g < count; ++g) {
        hs[g] = reinterpret_cast<W4A16*>(handles[g]);
        ys[g] = static_cast<__nv_bfloat16*>(d_ys[g]);
        if (!hs[g] || !ys[g]) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: null handle or output %d", g);
        if (hs[g]->geo.cols != hs[0]->geo.cols || hs[g]->scale_dtype != hs[0]->scale_dtype)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_group: linears of a group must share K and the scale type");
        ldys[g] = hs[g]->geo.rows;
        max_rows = std::min(max_rows, hs[g]->max_rows_per_launch);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (m > max_rows) {   // larger batches: one launch per linear (tile kernel or row blocks)
        for (int g = 0; g < count; ++g)
            if (int rc = hs[g]->run(d_x, ys[g], m, nullptr, 0, flags, s)) return rc;
        return GARNET_B200_OK;
    }
    return W4A16::launch_stream_group(hs, count, static_cast<const __nv_bfloat16*>(d_x), ys, ldys, m, flags, s);
}

// Device-visible alias of a host pointer (pinned and mapped memory), or nullptr.
static void* device_alias_of(const void* host_ptr)
{
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host_ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

// Device staging for the host-buffer calls of one handle (x, y and workspace for up to
// `m` rows).  Allocates; the run calls do not.
static int reserve_host(W4A16* h, int m)
{
    if (m <= h->stage_rows) return GARNET_B200_OK;
    if (h->stage_x) cudaFree(h->stage_x);
    if (h->stage_y) cudaFree(h->stage_y);
    if (h->stage_ws) cudaFree(h->stage_ws);
    h->stage_x = h->stage_y = h->stage_ws = nullptr;
    h->stage_rows = 0;
    const size_t xb = size_t(m) * h->geo.cols * 2, yb = size_t(m) * h->geo.rows * 2, wb = h->workspace_bytes(m);
    GB_CUDA(cudaMalloc(&h->stage_x, xb));
    GB_CUDA(cudaMalloc(&h->stage_y, yb));
    if (wb) GB_CUDA(cudaMalloc(&h->stage_ws, wb));
    h->stage_rows = m;
    return GARNET_B200_OK;
}

// One linear with host buffers, enqueued on `s`.
static int run_host_one(W4A16* h, const void* h_x, void* h_y, int m, cudaStream_t s)
{
    if (m > h->stage_rows)
        return fail(GARNET_B200_INVALID_VALUE,
                    "w4a16_run_host: %d rows but staging is reserved for %d: call garnet_b200_w4a16_reserve_host first", m,
                    h->stage_rows);
    const size_t xb = size_t(m) * h->geo.cols * 2, yb = size_t(m) * h->geo.rows * 2, wb = h->workspace_bytes(m);
    // y in pinned, mapped host memory is written by the kernel itself (one posted write per
    // output over the host link, no copy to enqueue); any other y goes through a staged copy.
    // The lookup is a host-side query and is repeated on every call: the same address may be
    // pinned in one call and pageable in the next.
    void* alias = device_alias_of(h_y);
    GB_CUDA(cudaMemcpyAsync(h->stage_x, h_x, xb, cudaMemcpyHostToDevice, s));
    void* y_dev = alias ? alias : h->stage_y;
    if (int rc = h->run(h->stage_x, y_dev, m, h->stage_ws, wb, 0, s)) return rc;
    if (!alias) GB_CUDA(cudaMemcpyAsync(h_y, h->stage_y, yb, cudaMemcpyDeviceToHost, s));
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_reserve_host(garnet_b200_w4a16_t hh, int max_m)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h || max_m <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16_reserve_host: bad argument");
    return reserve_host(h, max_m);
}

int garnet_b200_w4a16_run_host_async(garnet_b200_w4a16_t hh, const void* h_x, void* h_y, int m, void* stream)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h || !h_x || !h_y || m <= 0) return fail(GARNET_B200_INVALID_VALUE, "w4a16_run_host: bad argument");
    return run_host_one(h, h_x, h_y, m, static_cast<cudaStream_t>(stream));
}

int garnet_b200_w4a16_batch_create(const garnet_b200_w4a16_t* handles, const void* const* h_xs, void* const* h_ys,
                                   const int* ms, int count, garnet_b200_w4a16_batch_t* out)
{
    if (!handles || !h_xs || !h_ys || !ms || !out || count <= 0)
        return fail(GARNET_B200_INVALID_VALUE, "w4a16_batch_create: bad argument");
    std::unique_ptr<HostBatch> b(new HostBatch);
    size_t x_total = 0, y_total = 0, ws_max = 0;
    for (int i = 0; i < count; ++i) {
        W4A16* h = reinterpret_cast<W4A16*>(handles[i]);
        if (!h || !h_xs[i] || !h_ys[i] || ms[i] <= 0)
            return fail(GARNET_B200_INVALID_VALUE, "w4a16_batch_create: bad argument at index %d", i);
        ws_max = std::max(ws_max, h->workspace_bytes(ms[i]));
        const size_t xb = size_t(ms[i]) * h->geo.cols * 2, yb = size_t(ms[i]) * h->geo.rows * 2;
        // inputs are read-only during a run: every distinct host buffer is copied once
        int slot = -1;
        for (size_t q = 0; q < b->xs.size(); ++q)
            if (b->xs[q].host == h_xs[i] && b->xs[q].bytes == xb) slot = int(q);
        if (slot < 0) {
            slot = int(b->xs.size());
            b->xs.push_back({h_xs[i], xb, x_total});
            x_total += (xb + 255) & ~size_t(255);
        }
        b->calls.push_back({h, h_xs[i], h_ys[i], ms[i], slot, y_total, device_alias_of(h_ys[i])});
        y_total += (yb + 255) & ~size_t(255);
    }
    GB_CUDA(cudaMalloc(&b->x_stage, x_total));
    GB_CUDA(cudaMalloc(&b->y_stage, y_total));
    if (ws_max) GB_CUDA(cudaMalloc(&b->ws, ws_max));   // the calls run one after the other: one workspace serves them all
    b->ws_bytes = ws_max;
    // Calls that all have the same small batch run as one list (one launch for the lot).
    bool one_list = true;
    for (const HostBatch::Call& c : b->calls)
        if (c.m != b->calls[0].m || c.m > c.h->max_rows_per_launch) one_list = false;
    // The list kernel writes pinned, mapped output buffers itself, strip by strip while the pass runs (the
    // writes cross PCIe under the rest of the pass); the other launches write device staging that one kernel
    // copies out at the end.
    const bool direct = one_list;
    std::vector<ScatterEntry> table;
    for (const HostBatch::Call& c : b->calls)
        if (c.y_alias && !direct)
            table.push_back({b->y_stage + c.y_off, static_cast<uint8_t*>(c.y_alias), size_t(c.m) * c.h->geo.rows * 2});
    b->table_count = int(table.size());
    if (b->table_count) {
        GB_CUDA(cudaMalloc(&b->table, table.size() * sizeof(ScatterEntry)));
        GB_CUDA(cudaMemcpy(b->table, table.data(), table.size() * sizeof(ScatterEntry), cudaMemcpyHostToDevice));
    }
    if (one_list) {
        std::vector<garnet_b200_w4a16_t> hs;
        std::vector<const void*> dxs;
        std::vector<void*> dys;
        for (const HostBatch::Call& c : b->calls) {
            hs.push_back(reinterpret_cast<garnet_b200_w4a16_t>(c.h));
            dxs.push_back(b->x_stage + b->xs[c.x_slot].off);
            dys.push_back(c.y_alias ? c.y_alias : static_cast<void*>(b->y_stage + c.y_off));
        }
        if (int rc = garnet_b200_w4a16_list_create(hs.data(), dxs.data(), dys.data(), nullptr, count, b->calls[0].m, &b->list))
            return rc;
    }
    *out = reinterpret_cast<garnet_b200_w4a16_batch_t>(b.release());
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_batch_run(garnet_b200_w4a16_batch_t bb, void* stream)
{
    HostBatch* b = reinterpret_cast<HostBatch*>(bb);
    if (!b) return fail(GARNET_B200_INVALID_VALUE, "w4a16_batch_run: null batch");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (const HostBatch::X& x : b->xs)
        GB_CUDA(cudaMemcpyAsync(b->x_stage + x.off, x.host, x.bytes, cudaMemcpyHostToDevice, s));
    if (b->list) {
        if (int rc = garnet_b200_w4a16_list_run(b->list, 0, stream)) return rc;
    } else {
        for (const HostBatch::Call& c : b->calls)
            if (int rc = c.h->run(b->x_stage + b->xs[c.x_slot].off, b->y_stage + c.y_off, c.m, b->ws, b->ws_bytes, 1, s)) return rc;
    }
    if (b->table_count) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(8, unsigned(std::min(b->table_count, 1024)));
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        GB_CUDA(cudaLaunchKernelEx(&cfg, w4_scatter_outputs_kernel, (const ScatterEntry*)b->table, b->table_count));
    }
    for (const HostBatch::Call& c : b->calls)
        if (!c.y_alias)
            GB_CUDA(cudaMemcpyAsync(c.h_y, b->y_stage + c.y_off, size_t(c.m) * c.h->geo.rows * 2, cudaMemcpyDeviceToHost, s));
    return GARNET_B200_OK;
}

void garnet_b200_w4a16_batch_destroy(garnet_b200_w4a16_batch_t bb) { delete reinterpret_cast<HostBatch*>(bb); }

int garnet_b200_w4a16_run_host(garnet_b200_w4a16_t hh, const void* h_x, void* h_y, int m, void* stream)
{
    if (int rc = garnet_b200_w4a16_run_host_async(hh, h_x, h_y, m, stream)) return rc;
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    GB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    if (*h->fault_host) return fail(GARNET_B200_DEVICE_FAULT, "w4a16: device wait gave up (code %d)", *h->fault_host);
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_dequant(garnet_b200_w4a16_t hh, float* d_out, void* stream)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    if (!h || !d_out) return fail(GARNET_B200_INVALID_VALUE, "w4a16_dequant: bad argument");
    const size_t total = size_t(h->geo.rows) * h->geo.cols / 2;
    w4_dequant_kernel<<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        h->packed, d_out, h->geo, h->scale_dtype);
    GB_CUDA(cudaGetLastError());
    return GARNET_B200_OK;
}

int garnet_b200_w4a16_fault(garnet_b200_w4a16_t hh)
{
    W4A16* h = reinterpret_cast<W4A16*>(hh);
    return h && h->fault_host ? *h->fault_host : -1;
}

void garnet_b200_w4a16_destroy(garnet_b200_w4a16_t hh) { delete reinterpret_cast<W4A16*>(hh); }

}  // extern "C"
