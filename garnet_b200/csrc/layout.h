// Packed-weight tile layout shared by the repackers (GPU and host), the unpack
// kernels and the GEMV / GEMM kernels.
//
// Input contract (what the caller hands over) is the reference's canonical form:
//   int4  : row-major [N, K], two's-complement nibbles, element i in bits
//           4*(i&1) of byte i/2, one scale per (row, K-group)
//           (src/model/weight_quantization.h:14-25, weight_quantization.cpp:253-259);
//   MXFP4 : row-major [rows, K/2] bytes, low nibble = even column, one e8m0 byte
//           per 32 columns (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:50-54).
//
// Packed form ("strip / chunk / tile"), designed for sm_100a streaming:
//   * rows are grouped into strips of 16 (one MMA M-tile); the strip count is
//     padded to a multiple of 8 so that 8 consecutive strips form a complete
//     128-row panel (one tcgen05 A tile);
//   * K is cut into chunks (128 columns for int4 = one scale group, 64 columns
//     for MXFP4 = two scale groups).  A strip-chunk is one contiguous block
//     [nibble data][32 bytes of scales] (1056 bytes int4, 544 bytes MXFP4), and all
//     chunks of a strip are contiguous: a strip is one linear byte range, so the
//     memory-bound kernels stream whole strips with a few large bulk copies
//     (cp.async.bulk) and the tensor-core kernel fetches the 8 strip-chunks of a
//     panel per pipeline stage;
//   * nibble data is cut into 512-byte tiles of 16 rows x 64 columns; a tile
//     holds 32 units of 16 bytes, unit L = 4*g + t being exactly what lane L of
//     a warp needs for four m16n8k16 MMAs: words {row R(g), octet t},
//     {R(g)+8, t}, {R(g), t+4}, {R(g)+8, t+4}, an octet being 8 consecutive K
//     columns;
//   * R(g) = (g>>1) + 4*(g&1) interleaves rows so that, when the same units are
//     expanded to 16-bit values and stored as 16-byte rows of a 128-byte-swizzled
//     K-major shared-memory tile for tcgen05.mma, the eight lanes of a
//     quarter-warp hit eight distinct bank groups;
//   * inside a 32-bit word, int4 element e sits in nibble (e>>1) + 4*(e&1) so that
//     one mask extracts the pair (2j, 2j+1) into the two halves of a bf16x2;
//     MXFP4 keeps the natural order, byte b = pair (2b, 2b+1), which is the
//     operand form of cvt.rn.f16x2.e2m1x2.
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define GB_HD __host__ __device__ __forceinline__
#else
#define GB_HD inline
#endif

namespace gb200 {

enum PackFormat : int { kFormatInt4 = 0, kFormatMxfp4 = 1 };

struct PackGeom {
    int format;        // PackFormat
    int rows, cols;    // logical N, K of one matrix
    int strips;        // ceil(rows / 16)
    int strips_padded; // strips rounded up to a multiple of 8
    int chunk_k;       // 128 (int4) or 64 (MXFP4)
    int chunks;        // ceil(cols / chunk_k)
    int chunk_data;    // bytes of nibble data per strip-chunk (16 * chunk_k / 2)
    int chunk_bytes;   // chunk_data + 32 bytes of scales
    int group;         // K columns per scale (int4: >= 128, multiple of 128; MXFP4: 32)

    GB_HD size_t strip_bytes() const { return size_t(chunks) * chunk_bytes; }
    GB_HD size_t matrix_bytes() const { return size_t(strips_padded) * strip_bytes(); }
    GB_HD int padded_cols() const { return chunks * chunk_k; }
    GB_HD int padded_rows() const { return strips_padded * 16; }
};

constexpr int kScaleBytesPerChunk = 32;

GB_HD PackGeom make_geom(int format, int rows, int cols, int group)
{
    PackGeom g;
    g.format = format;
    g.rows = rows;
    g.cols = cols;
    g.strips = (rows + 15) / 16;
    g.strips_padded = (g.strips + 7) / 8 * 8;
    g.chunk_k = format == kFormatInt4 ? 128 : 64;
    g.chunks = (cols + g.chunk_k - 1) / g.chunk_k;
    g.chunk_data = 16 * g.chunk_k / 2;
    g.chunk_bytes = g.chunk_data + kScaleBytesPerChunk;
    g.group = group;
    return g;
}

// Row interleave inside a 16-row strip: MMA row g (0..7) <-> storage row R(g).
GB_HD int row_of_g(int g) { return (g >> 1) + 4 * (g & 1); }
GB_HD int g_of_row(int r8) { return ((r8 & 3) << 1) | (r8 >> 2); }

// Position of element (row n, column k) inside the packed matrix.
struct PackPos {
    size_t word_byte;   // byte offset of the 32-bit word holding the element
    int nibble;         // nibble index (0..7) inside that word
};

GB_HD PackPos locate(const PackGeom& geo, int n, int k)
{
    const int strip = n >> 4, r16 = n & 15, h = r16 >> 3, g = g_of_row(r16 & 7);
    const int chunk = k / geo.chunk_k, kl = k % geo.chunk_k;
    const int tile = kl >> 6, kk = kl & 63;
    const int oct = kk >> 3, t = oct & 3, j = oct >> 2, e = kk & 7;
    PackPos p;
    p.word_byte = (size_t(strip) * geo.chunks + chunk) * geo.chunk_bytes + size_t(tile) * 512 +
                  size_t(4 * g + t) * 16 + size_t(h + 2 * j) * 4;
    p.nibble = geo.format == kFormatInt4 ? (e >> 1) + 4 * (e & 1) : e;
    return p;
}

// Byte offset of the scale that covers (row n, column k).  int4: one 16-bit scale
// per (row, chunk), laid out [g][h] so that a lane reads rows R(g), R(g)+8 as one
// 32-bit word.  MXFP4: one byte per (row, 32 columns), laid out
// [g][h + 2*group_in_chunk] so that a lane reads its four scales as one word.
GB_HD size_t locate_scale(const PackGeom& geo, int n, int k)
{
    const int strip = n >> 4, r16 = n & 15, h = r16 >> 3, g = g_of_row(r16 & 7);
    const int chunk = k / geo.chunk_k, kl = k % geo.chunk_k;
    const size_t base = (size_t(strip) * geo.chunks + chunk) * geo.chunk_bytes + geo.chunk_data;
    if (geo.format == kFormatInt4) return base + size_t(g) * 4 + size_t(h) * 2;
    return base + size_t(g) * 4 + size_t(h + 2 * (kl >> 5));
}

}  // namespace gb200
