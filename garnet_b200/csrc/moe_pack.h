// Where every byte of the packed expert constants comes from.  The device repackers
// and the host packer (garnet_b200_moe_pack_host) both call these functions, so a blob
// packed on the host is byte for byte the one a handle builds on the device (the
// property the reference checks for its own packer, test2026/gpt_oss/marlin_weight_pack.cpp:33-111).
//
// Source layout (one projection of one expert, checkpoint order): blocks [rows, K/2]
// bytes, low nibble = even column; scales [rows, K/32] e8m0 bytes
// (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:50-54).  For the gate/up projection row 2i is
// gate_i and row 2i+1 is up_i (:776).
#pragma once
#include "layout.h"

namespace gb200 {

constexpr int kMxBlockRows = 240;                        // weight rows per block of the block-scaled layout (UMMA N)
constexpr int kMxBlockCols = 128;                        // K columns per block (one pipeline stage)
constexpr int kMxBlockBytes = kMxBlockRows * kMxBlockCols / 2;   // 15360
constexpr int kMxAtomBytes = 512;                        // one scale atom: 128 rows x 4 groups of 32 columns

// ---- streaming layout: strips of 16 rows, 544-byte chunks of 64 columns ----------

GB_HD size_t mx_stream_words(const PackGeom& geo) { return size_t(geo.strips_padded) * geo.chunks * (geo.chunk_data / 4); }
GB_HD size_t mx_stream_scale_count(const PackGeom& geo) { return size_t(geo.strips_padded) * 16 * geo.chunks * 2; }

// 32-bit word `idx` of an expert's packed matrix: byte offset in the packed matrix, and
// the byte offset of its 8 codes in the source (false: padding, the word is zero).  In
// the gate/up matrix gate_i sits at strip row r and up_i at strip row r + 8
// (i = 8 * strip + r), so that one MMA accumulator lane holds both of a channel.
GB_HD bool mx_stream_word(const PackGeom& geo, size_t idx, int interleaved, size_t* dst_byte, size_t* src_byte)
{
    const size_t words_per_chunk = size_t(geo.chunk_data / 4);
    const size_t chunk_lin = idx / words_per_chunk;
    const int w = int(idx % words_per_chunk);
    const int strip = int(chunk_lin / geo.chunks), chunk = int(chunk_lin % geo.chunks);
    const int unit = (w >> 2) & 31, word = w & 3;          // one 512-byte tile per chunk
    const int g = unit >> 2, t = unit & 3, h = word & 1, j = word >> 1;
    const int r16 = row_of_g(g) + 8 * h;
    const int n = strip * 16 + r16;                          // packed row
    const int k0 = chunk * 64 + (t + 4 * j) * 8;
    *dst_byte = (size_t(strip) * geo.chunks + chunk) * geo.chunk_bytes + size_t(w) * 4;
    if (n >= geo.rows || k0 >= geo.cols) return false;
    const int src_row = interleaved ? 2 * (strip * 8 + (r16 & 7)) + (r16 >> 3) : n;
    *src_byte = size_t(src_row) * size_t(geo.cols / 2) + k0 / 2;
    return true;
}

// Scale `idx` = (packed row, group of 32 columns); false: padding, the byte is 127 (1.0).
GB_HD bool mx_stream_scale(const PackGeom& geo, size_t idx, int interleaved, size_t* dst_byte, size_t* src_byte)
{
    const int groups = geo.chunks * 2;
    const int n = int(idx / groups), grp = int(idx % groups);
    *dst_byte = locate_scale(geo, n, grp * 32);
    if (n >= geo.rows || grp * 32 >= geo.cols) return false;
    const int strip = n >> 4, r16 = n & 15;
    const int src_row = interleaved ? 2 * (strip * 8 + (r16 & 7)) + (r16 >> 3) : n;
    *src_byte = size_t(src_row) * size_t(geo.cols / 32) + grp;
    return true;
}

// ---- block-scaled layout: [row tile][K slab] blocks of 240 rows x 128 columns in the
// checkpoint's own row order, then all scale atoms [row tile][K slab][2][512] ---------

struct MxBlockGeom {
    int rows, k;        // the matrix
    int ntiles, kslabs; // blocks along the rows and along K
    GB_HD size_t code_bytes() const { return size_t(ntiles) * kslabs * kMxBlockBytes; }
    GB_HD size_t atom_bytes() const { return size_t(ntiles) * kslabs * 2 * kMxAtomBytes; }
};

GB_HD MxBlockGeom make_block_geom(int rows, int k)
{
    MxBlockGeom g;
    g.rows = rows;
    g.k = k;
    g.ntiles = (rows + kMxBlockRows - 1) / kMxBlockRows;
    g.kslabs = (k + kMxBlockCols - 1) / kMxBlockCols;
    return g;
}

// 16-byte piece `idx` of an expert's blocks (dst byte = 16 idx): source byte offset, or
// false for rows and columns beyond the matrix (zero codes).
GB_HD bool mx_block_piece(const MxBlockGeom& g, size_t idx, size_t* src_byte)
{
    const int piece = int(idx % 4);
    const int r = int((idx / 4) % kMxBlockRows);
    const size_t tile = idx / (4 * size_t(kMxBlockRows));
    const int ks = int(tile % g.kslabs);
    const int nt = int(tile / g.kslabs);
    const int row = nt * kMxBlockRows + r, col = ks * kMxBlockCols + piece * 32;
    if (row >= g.rows || col >= g.k) return false;
    *src_byte = size_t(row) * (g.k / 2) + col / 2;
    return true;
}

// Byte `idx` of an expert's scale atoms: atom a of a block covers its rows 128 a ..;
// inside an atom byte (r % 32) * 16 + (r / 32) * 4 + group.  false: 127.
GB_HD bool mx_block_atom(const MxBlockGeom& g, size_t idx, size_t* src_byte)
{
    const int byte = int(idx % kMxAtomBytes);
    const int atom = int((idx / kMxAtomBytes) % 2);
    const size_t tile = idx / (2 * size_t(kMxAtomBytes));
    const int ks = int(tile % g.kslabs);
    const int nt = int(tile / g.kslabs);
    const int r = atom * 128 + (byte >> 4) + 32 * ((byte >> 2) & 3), kb = byte & 3;
    const int row = nt * kMxBlockRows + r, blk = ks * 4 + kb;
    if (r >= kMxBlockRows || row >= g.rows || blk >= g.k / 32) return false;
    *src_byte = size_t(row) * (g.k / 32) + blk;
    return true;
}

}  // namespace gb200
